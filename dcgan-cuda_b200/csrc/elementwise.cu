// Memory-bound operators around the convolutions: bias add + activation,
// activation gradients, element-wise add / axpy, column and row sums, losses.
//
// All of them are HBM-bound streaming kernels: 128-bit loads and stores where
// the pointers and sizes allow it, grid-stride loops, grids sized as a multiple
// of the SM count.  Reductions use a fixed tree so results are deterministic.
#include <mutex>

#include <atomic>

#include "common.cuh"

namespace dcg {
namespace {

constexpr int kThreads = 256;

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int stream_grid(size_t work_items, int per_block = kThreads, int waves = 8)
{
    size_t blocks = (work_items + per_block - 1) / per_block;
    size_t cap = (size_t)sm_count() * waves;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

// ---- z = a + bias[col]; act(z) ---------------------------------------------
template <bool VEC>
__global__ void __launch_bounds__(kThreads)
bias_act_kernel(const float* __restrict__ a, const float* __restrict__ bias,
                float* __restrict__ z_out, float* __restrict__ act_out,
                size_t total, unsigned cols, int act, float alpha)
{
    pdl_enter();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (VEC) {
        const size_t n4 = total >> 2;
        for (; i < n4; i += stride) {
            float4 v = __ldg(reinterpret_cast<const float4*>(a) + i);
            if (bias) {
                const unsigned col = (unsigned)((i << 2) % cols);
                const float4 b = __ldg(reinterpret_cast<const float4*>(bias + col));
                v.x = __fadd_rn(v.x, b.x); v.y = __fadd_rn(v.y, b.y);
                v.z = __fadd_rn(v.z, b.z); v.w = __fadd_rn(v.w, b.w);
            }
            if (z_out) reinterpret_cast<float4*>(z_out)[i] = v;
            if (act_out) {
                v.x = act_apply(v.x, act, alpha); v.y = act_apply(v.y, act, alpha);
                v.z = act_apply(v.z, act, alpha); v.w = act_apply(v.w, act, alpha);
                reinterpret_cast<float4*>(act_out)[i] = v;
            }
        }
    } else {
        for (; i < total; i += stride) {
            float v = __ldg(a + i);
            if (bias) v = __fadd_rn(v, __ldg(bias + (i % cols)));
            if (z_out) z_out[i] = v;
            if (act_out) act_out[i] = act_apply(v, act, alpha);
        }
    }
}

// ---- out = dout * act'(gate) -----------------------------------------------
template <bool VEC>
__global__ void __launch_bounds__(kThreads)
act_grad_kernel(const float* __restrict__ gate, const float* __restrict__ dout,
                float* __restrict__ out, size_t total, int act, float alpha)
{
    pdl_enter();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (VEC) {
        const size_t n4 = total >> 2;
        for (; i < n4; i += stride) {
            const float4 g = __ldg(reinterpret_cast<const float4*>(gate) + i);
            const float4 d = __ldg(reinterpret_cast<const float4*>(dout) + i);
            float4 r;
            r.x = act_grad_apply(g.x, d.x, act, alpha); r.y = act_grad_apply(g.y, d.y, act, alpha);
            r.z = act_grad_apply(g.z, d.z, act, alpha); r.w = act_grad_apply(g.w, d.w, act, alpha);
            reinterpret_cast<float4*>(out)[i] = r;
        }
    } else {
        for (; i < total; i += stride)
            out[i] = act_grad_apply(__ldg(gate + i), __ldg(dout + i), act, alpha);
    }
}

// ---- out = a + b ; out += coeff * dv ----------------------------------------
template <bool VEC>
__global__ void __launch_bounds__(kThreads)
add_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
           size_t total)
{
    pdl_enter();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (VEC) {
        const size_t n4 = total >> 2;
        for (; i < n4; i += stride) {
            const float4 x = __ldg(reinterpret_cast<const float4*>(a) + i);
            const float4 y = __ldg(reinterpret_cast<const float4*>(b) + i);
            reinterpret_cast<float4*>(out)[i] =
                make_float4(__fadd_rn(x.x, y.x), __fadd_rn(x.y, y.y), __fadd_rn(x.z, y.z),
                            __fadd_rn(x.w, y.w));
        }
    } else {
        for (; i < total; i += stride) out[i] = __fadd_rn(__ldg(a + i), __ldg(b + i));
    }
}

__global__ void __launch_bounds__(kThreads)
update_kernel(const float* __restrict__ dv, float* __restrict__ out,
              const float* __restrict__ coeff, size_t total)
{
    pdl_enter();
    const float c = __ldg(coeff);
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride)
        out[i] = __fadd_rn(out[i], __fmul_rn(c, __ldg(dv + i)));
}

// ---- column sums (bias gradient) ---------------------------------------------
// Block (tx over column groups, ty over rows) reduces a slab of rows into
// partial[slab][cols].  VEC: a column group is one float4.  The slabs of one column tile are
// then added by whichever of its blocks finishes last (a ticket per column tile tells it so):
// lane l adds slabs l, l+L, ... and the lane sums are added in lane order, so the result depends
// on the launch shape only, never on which block came last.  `tickets` == nullptr leaves the
// slabs to colsum_final_kernel.
// The ticket words belong to whoever owns the scratch of the launch (they sit behind the partial
// sums in the caller's buffer, or at the tail of a context's scratch allocation), so two launches
// only ever share tickets if they share scratch - which already requires them to be stream-ordered.
// They must be zero when a launch starts; every adder resets the ticket it consumed.
constexpr int kTicketTiles = 16, kSlabGroup = 16, kMaxSlabs = 1008;
constexpr int kTicketsPerTile = 1 + kMaxSlabs / kSlabGroup;         // group-level ticket + one per slab group
constexpr size_t kTicketBytes = (size_t)kTicketTiles * kTicketsPerTile * sizeof(unsigned);
static_assert(kTicketBytes == dcg::kColsumTicketBytes, "ticket area size is part of the scratch contract");

// One block adds `nrows` rows of src ([nrows][cols]) for its column tile into dst: thread = (column
// group, lane); lane l adds rows l, l+L, ... through four independent accumulators (four loads in
// flight), combined in a fixed order; the lane sums are then added in lane order.  The result
// depends on the launch shape only.
template <bool VEC>
__device__ __forceinline__ void colsum_add_rows(const float* __restrict__ src, unsigned nrows, float* __restrict__ dst,
                                                unsigned cols, int tx_count, unsigned groups, float* smem)
{
    constexpr int W = VEC ? 4 : 1;
    const int lanes = blockDim.x / tx_count;     // >= 8
    const int g = threadIdx.x % tx_count, l = threadIdx.x / tx_count;
    const unsigned grp = blockIdx.x * tx_count + g;
    float4 t[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) t[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (grp < groups) {
        unsigned k = l;
        for (; k + 3 * lanes < nrows; k += 4 * lanes) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float* p = src + (size_t)(k + u * lanes) * cols + (size_t)grp * W;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (VEC) v = __ldcg(reinterpret_cast<const float4*>(p));
                else v.x = __ldcg(p);
                t[u].x += v.x; t[u].y += v.y; t[u].z += v.z; t[u].w += v.w;
            }
        }
        for (int u = 0; k < nrows; k += lanes, ++u) {   // at most three rows left per lane
            const float* p = src + (size_t)k * cols + (size_t)grp * W;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (VEC) v = __ldcg(reinterpret_cast<const float4*>(p));
            else v.x = __ldcg(p);
            t[u & 3].x += v.x; t[u & 3].y += v.y; t[u & 3].z += v.z; t[u & 3].w += v.w;
        }
    }
    float4 s4;
    s4.x = (t[0].x + t[1].x) + (t[2].x + t[3].x); s4.y = (t[0].y + t[1].y) + (t[2].y + t[3].y);
    s4.z = (t[0].z + t[1].z) + (t[2].z + t[3].z); s4.w = (t[0].w + t[1].w) + (t[2].w + t[3].w);
    __syncthreads();                             // smem is reused: [lane][group][W]
    float* slot = smem + ((size_t)l * tx_count + g) * W;
    slot[0] = s4.x;
    if (VEC) { slot[1] = s4.y; slot[2] = s4.z; slot[3] = s4.w; }
    __syncthreads();
    if (l == 0 && grp < groups) {
#pragma unroll
        for (int q = 0; q < W; ++q) {
            float r = smem[(size_t)g * W + q];
            for (int j = 1; j < lanes; ++j) r += smem[((size_t)j * tx_count + g) * W + q];
            dst[(size_t)grp * W + q] = r;
        }
    }
}

template <bool VEC>
__global__ void __launch_bounds__(kThreads)
colsum_partial_kernel(const float* __restrict__ a, float* __restrict__ partial,
                      size_t rows, unsigned cols, unsigned rows_per_slab, int tx_count,
                      float* __restrict__ out, unsigned* __restrict__ tickets)
{
    pdl_enter();
    extern __shared__ float smem[];  // [ty_count][tx_count * (VEC ? 4 : 1)]
    const int ty_count = blockDim.x / tx_count;
    const int tx = threadIdx.x % tx_count;
    const int ty = threadIdx.x / tx_count;
    const unsigned groups = VEC ? cols / 4 : cols;
    const unsigned group = blockIdx.x * tx_count + tx;
    const size_t r0 = (size_t)blockIdx.y * rows_per_slab;
    size_t r1 = r0 + rows_per_slab;
    if (r1 > rows) r1 = rows;

    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (group < groups) {
        size_t r = r0 + ty;
        if (VEC) {   // four rows in flight per thread
            for (; r + 3 * (size_t)ty_count < r1; r += 4 * (size_t)ty_count) {
                const float4 v0 = __ldg(reinterpret_cast<const float4*>(a + r * cols) + group);
                const float4 v1 = __ldg(reinterpret_cast<const float4*>(a + (r + ty_count) * cols) + group);
                const float4 v2 = __ldg(reinterpret_cast<const float4*>(a + (r + 2 * (size_t)ty_count) * cols) + group);
                const float4 v3 = __ldg(reinterpret_cast<const float4*>(a + (r + 3 * (size_t)ty_count) * cols) + group);
                acc.x += v0.x; acc.y += v0.y; acc.z += v0.z; acc.w += v0.w;
                acc.x += v1.x; acc.y += v1.y; acc.z += v1.z; acc.w += v1.w;
                acc.x += v2.x; acc.y += v2.y; acc.z += v2.z; acc.w += v2.w;
                acc.x += v3.x; acc.y += v3.y; acc.z += v3.z; acc.w += v3.w;
            }
        }
        for (; r < r1; r += ty_count) {
            if (VEC) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(a + r * cols) + group);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            } else {
                acc.x += __ldg(a + r * cols + group);
            }
        }
    }
    constexpr int W = VEC ? 4 : 1;
    float* mine = smem + ((size_t)ty * tx_count + tx) * W;
    mine[0] = acc.x;
    if (VEC) { mine[1] = acc.y; mine[2] = acc.z; mine[3] = acc.w; }
    __syncthreads();
    for (int s = ty_count >> 1; s > 0; s >>= 1) {
        if (ty < s) {
            const float* other = smem + ((size_t)(ty + s) * tx_count + tx) * W;
#pragma unroll
            for (int q = 0; q < W; ++q) mine[q] += other[q];
        }
        __syncthreads();
    }
    if (ty == 0 && group < groups) {
        float* dst = partial + (size_t)blockIdx.y * cols + (size_t)group * W;
#pragma unroll
        for (int q = 0; q < W; ++q) dst[q] = mine[q];
    }
    if (tickets == nullptr) return;
    // ---- two levels of "whoever finishes last adds": 16 slabs -> one group row, all group rows -> out ----
    // tickets of this column tile: [0] the group level, [1 + g] slab group g.  Each adder resets its
    // ticket, so a set is ready for the next launch that uses it.
    unsigned* my_tickets = tickets + (size_t)blockIdx.x * kTicketsPerTile;
    const unsigned slabs = gridDim.y, n_groups = (slabs + kSlabGroup - 1) / kSlabGroup;
    const unsigned g_idx = blockIdx.y / kSlabGroup;
    const unsigned g_first = g_idx * kSlabGroup;
    const unsigned g_count = slabs - g_first < (unsigned)kSlabGroup ? slabs - g_first : (unsigned)kSlabGroup;
    float* level2 = partial + (size_t)slabs * cols;      // [n_groups][cols], behind the slab rows
    __shared__ unsigned s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned t = atomicAdd(my_tickets + 1 + g_idx, 1u);
        s_last = (t == g_count - 1) ? 1u : 0u;
        if (s_last) my_tickets[1 + g_idx] = 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    colsum_add_rows<VEC>(partial + (size_t)g_first * cols, g_count, n_groups > 1 ? level2 + (size_t)g_idx * cols : out,
                         cols, tx_count, groups, smem);
    if (n_groups == 1) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned t = atomicAdd(my_tickets, 1u);
        s_last = (t == n_groups - 1) ? 1u : 0u;
        if (s_last) my_tickets[0] = 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    colsum_add_rows<VEC>(level2, n_groups, out, cols, tx_count, groups, smem);
}

// Stage 2: block = 32 columns x 8 slab lanes.  Lane ty adds slabs ty, ty+8, ... (four loads in
// flight at a time), then the eight lane sums are added in lane order: the result does not depend
// on the launch shape of anything else.
__global__ void __launch_bounds__(256)
colsum_final_kernel(const float* __restrict__ partial, float* __restrict__ out,
                    unsigned slabs, unsigned cols)
{
    pdl_enter();
    __shared__ float part[8][33];
    const unsigned tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const unsigned c = blockIdx.x * 32 + tx;
    float s = 0.f;
    if (c < cols) {
        unsigned k = ty;
        for (; k + 24 < slabs; k += 32) {
            const float v0 = __ldg(partial + (size_t)k * cols + c);
            const float v1 = __ldg(partial + (size_t)(k + 8) * cols + c);
            const float v2 = __ldg(partial + (size_t)(k + 16) * cols + c);
            const float v3 = __ldg(partial + (size_t)(k + 24) * cols + c);
            s += v0; s += v1; s += v2; s += v3;
        }
        for (; k < slabs; k += 8) s += __ldg(partial + (size_t)k * cols + c);
    }
    part[ty][tx] = s;
    __syncthreads();
    if (ty == 0 && c < cols) {
        float t = part[0][tx];
#pragma unroll
        for (int q = 1; q < 8; ++q) t += part[q][tx];
        out[c] = t;
    }
}

// ---- row sums: one warp per row -----------------------------------------------
__global__ void __launch_bounds__(kThreads)
rowsum_kernel(const float* __restrict__ a, float* __restrict__ out, size_t rows, size_t cols)
{
    pdl_enter();
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= rows) return;
    float s = 0.f;
    for (size_t c = lane; c < cols; c += 32) s += __ldg(a + warp * cols + c);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) out[warp] = s;
}

// ---- block-wide deterministic sum ----------------------------------------------
__device__ __forceinline__ float block_sum(float v, float* red /* [32] */)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    v = (threadIdx.x < nwarps) ? red[threadIdx.x] : 0.f;
    if (warp == 0) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    }
    __syncthreads();
    return v;  // valid in warp 0
}

// mean_i( x>=0 ? x - x*y + log(1+exp(-x)) : -x*y + log(1+exp(x)) ), src/cpu/ops.hxx:440-452
__global__ void __launch_bounds__(512)
sigmoid_xent_kernel(const float* __restrict__ y, const float* __restrict__ x,
                    float* __restrict__ out, size_t n)
{
    pdl_enter();
    __shared__ float red[32];
    float s = 0.f;
    for (size_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float xi = __ldg(x + i), yi = __ldg(y + i);
        s += xi >= 0.f ? xi - xi * yi + logf(1.f + expf(-xi)) : -xi * yi + logf(1.f + expf(xi));
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) out[0] = s / (float)n;
}

__global__ void __launch_bounds__(kThreads)
sigmoid_xent_grad_kernel(const float* __restrict__ y, const float* __restrict__ x,
                         float* __restrict__ out, size_t n)
{
    pdl_enter();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = (act_apply(__ldg(x + i), DCG_ACT_SIGMOID, 0.f) - __ldg(y + i)) / (float)n;
}

// Loss and its gradient in one launch (the two nodes are neighbours in a training list): the same
// expressions as the two kernels above, element for element, so the results are bit-identical.
__global__ void __launch_bounds__(512)
sigmoid_xent_both_kernel(const float* __restrict__ y, const float* __restrict__ x, float* __restrict__ loss,
                         float* __restrict__ grad, size_t n)
{
    pdl_enter();
    __shared__ float red[32];
    float s = 0.f;
    for (size_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float xi = __ldg(x + i), yi = __ldg(y + i);
        s += xi >= 0.f ? xi - xi * yi + logf(1.f + expf(-xi)) : -xi * yi + logf(1.f + expf(xi));
        grad[i] = (act_apply(xi, DCG_ACT_SIGMOID, 0.f) - yi) / (float)n;
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) loss[0] = s / (float)n;
}

__global__ void __launch_bounds__(512)
mse_kernel(const float* __restrict__ y, const float* __restrict__ y_hat, float* __restrict__ out,
           size_t n)
{
    pdl_enter();
    __shared__ float red[32];
    float s = 0.f;
    for (size_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float d = __ldg(y + i) - __ldg(y_hat + i);
        s += d * d;
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) out[0] = s / (float)n;
}

__global__ void __launch_bounds__(kThreads)
mse_grad_kernel(const float* __restrict__ y, const float* __restrict__ y_hat,
                float* __restrict__ out, size_t n, float coeff)
{
    pdl_enter();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = __fmul_rn(coeff, __fsub_rn(__ldg(y_hat + i), __ldg(y + i)));
}

// ---- softmax family: one warp per row (src/cpu/ops.hxx:129-186,418-430) ---------
// mode 0: softmax, 1: log_softmax, 2: (softmax - y)/rows
__global__ void __launch_bounds__(kThreads)
softmax_rows_kernel(const float* __restrict__ a, const float* __restrict__ y,
                    float* __restrict__ out, size_t rows, size_t cols, int mode)
{
    pdl_enter();
    const size_t row = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* ar = a + row * cols;
    float mx = -INFINITY;
    for (size_t c = lane; c < cols; c += 32) mx = fmaxf(mx, __ldg(ar + c));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float s = 0.f;
    for (size_t c = lane; c < cols; c += 32) s += expf(__ldg(ar + c) - mx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float logsum = mx + logf(s);
    for (size_t c = lane; c < cols; c += 32) {
        const float v = __ldg(ar + c);
        float r;
        if (mode == 0) r = expf(v - mx) / s;
        else if (mode == 1) r = v - logsum;
        else r = (expf(v - mx) / s - __ldg(y + row * cols + c)) / (float)rows;
        out[row * cols + c] = r;
    }
}

// -(1/rows) sum_ij y_ij (logit_ij - logsumexp_i)
__global__ void __launch_bounds__(512)
softmax_xent_kernel(const float* __restrict__ y, const float* __restrict__ logits,
                    float* __restrict__ out, size_t rows, size_t cols)
{
    pdl_enter();
    __shared__ float red[32];
    float acc = 0.f;
    for (size_t r = threadIdx.x; r < rows; r += blockDim.x) {
        const float* lr = logits + r * cols;
        float mx = lr[0];
        for (size_t c = 1; c < cols; ++c) mx = fmaxf(mx, lr[c]);
        float e = 0.f;
        for (size_t c = 0; c < cols; ++c) e += expf(lr[c] - mx);
        const float logsum = mx + logf(e);
        for (size_t c = 0; c < cols; ++c) acc += y[r * cols + c] * (lr[c] - logsum);
    }
    acc = block_sum(acc, red);
    if (threadIdx.x == 0) out[0] = -acc / (float)rows;
}

// Count of rows whose first maximum sits at the same column in both matrices.
// Integer counting keeps the result exact whatever the reduction order.
__global__ void __launch_bounds__(512)
argmax_acc_kernel(const float* __restrict__ a, const float* __restrict__ b,
                  float* __restrict__ out, size_t rows, size_t cols)
{
    pdl_enter();
    __shared__ unsigned count;
    if (threadIdx.x == 0) count = 0;
    __syncthreads();
    unsigned mine = 0;
    for (size_t r = threadIdx.x; r < rows; r += blockDim.x) {
        const float* ar = a + r * cols;
        const float* br = b + r * cols;
        size_t ia = 0, ib = 0;
        for (size_t c = 1; c < cols; ++c) {
            if (ar[c] > ar[ia]) ia = c;
            if (br[c] > br[ib]) ib = c;
        }
        mine += (ia == ib);
    }
    atomicAdd(&count, mine);
    __syncthreads();
    if (threadIdx.x == 0) out[0] = (float)count;
}

}  // namespace
}  // namespace dcg

using namespace dcg;

extern "C" int dcg_bias_act(const float* a, const float* bias, float* z_out, float* act_out,
                            size_t rows, size_t cols, int act, float alpha, dcg_stream_t stream)
{
    DCG_CHECK_ARG(a && (z_out || act_out), "dcg_bias_act: null input or no output");
    DCG_CHECK_ARG(cols > 0 && cols <= 0xffffffffu, "dcg_bias_act: bad cols %zu", cols);
    DCG_CHECK_ARG(act >= DCG_ACT_NONE && act <= DCG_ACT_SIGMOID, "dcg_bias_act: unknown act %d", act);
    const size_t total = rows * cols;
    if (total == 0) return DCG_OK;
    const bool vec = (cols % 4 == 0) && aligned16(a) && (!bias || aligned16(bias)) &&
                     (!z_out || aligned16(z_out)) && (!act_out || aligned16(act_out));
    if (vec)
        launch_pdl(bias_act_kernel<true>, stream_grid(total / 4), kThreads, 0, as_stream(stream), 
            a, bias, z_out, act_out, total, (unsigned)cols, act, alpha);
    else
        launch_pdl(bias_act_kernel<false>, stream_grid(total), kThreads, 0, as_stream(stream), 
            a, bias, z_out, act_out, total, (unsigned)cols, act, alpha);
    DCG_LAUNCH_CHECK("bias_act_kernel");
    return DCG_OK;
}

extern "C" int dcg_act_fwd(const float* a, float* out, size_t n, int act, float alpha,
                           dcg_stream_t stream)
{
    DCG_CHECK_ARG(a && out, "dcg_act_fwd: null pointer");
    return dcg_bias_act(a, nullptr, nullptr, out, n / 4 * 4 == n ? n / 4 : n, n / 4 * 4 == n ? 4 : 1,
                        act, alpha, stream);
}

extern "C" int dcg_act_grad(const float* gate, const float* dout, float* out, size_t n, int act,
                            float alpha, dcg_stream_t stream)
{
    DCG_CHECK_ARG(gate && dout && out, "dcg_act_grad: null pointer");
    DCG_CHECK_ARG(act >= DCG_ACT_NONE && act <= DCG_ACT_SIGMOID, "dcg_act_grad: unknown act %d", act);
    if (n == 0) return DCG_OK;
    const bool vec = (n % 4 == 0) && aligned16(gate) && aligned16(dout) && aligned16(out);
    if (vec)
        launch_pdl(act_grad_kernel<true>, stream_grid(n / 4), kThreads, 0, as_stream(stream), gate, dout, out, n, act, alpha);
    else
        launch_pdl(act_grad_kernel<false>, stream_grid(n), kThreads, 0, as_stream(stream), gate, dout, out, n, act, alpha);
    DCG_LAUNCH_CHECK("act_grad_kernel");
    return DCG_OK;
}

extern "C" int dcg_add(const float* a, const float* b, float* out, size_t n, dcg_stream_t stream)
{
    DCG_CHECK_ARG(a && b && out, "dcg_add: null pointer");
    if (n == 0) return DCG_OK;
    const bool vec = (n % 4 == 0) && aligned16(a) && aligned16(b) && aligned16(out);
    if (vec)
        launch_pdl(add_kernel<true>, stream_grid(n / 4), kThreads, 0, as_stream(stream), a, b, out, n);
    else
        launch_pdl(add_kernel<false>, stream_grid(n), kThreads, 0, as_stream(stream), a, b, out, n);
    DCG_LAUNCH_CHECK("add_kernel");
    return DCG_OK;
}

// ---- image decode: bytes -> [-1, 1] ---------------------------------------------------------
// The reference scales every pixel on the host, per step (src/datasets/celeba.cu:29):
//     img[j] = dbl_t(pixs[j]) / 127.5 - 1.;        (float -> double arithmetic -> float)
// Doing it on the device lets the input pipeline copy one byte per value instead of four.  The
// double-precision expression is kept, so the result is the reference's bit for bit.
namespace dcg { namespace {
__global__ void __launch_bounds__(kThreads) u8_to_unit_kernel(const unsigned char* __restrict__ in, float* __restrict__ out, size_t n)
{
    pdl_enter();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t n16 = n / 16;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(in) + i);
        const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
        float4* dst = reinterpret_cast<float4*>(out) + 4 * i;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float4 v;
            v.x = (float)((double)(float)(w[q] & 0xffu) / 127.5 - 1.);
            v.y = (float)((double)(float)((w[q] >> 8) & 0xffu) / 127.5 - 1.);
            v.z = (float)((double)(float)((w[q] >> 16) & 0xffu) / 127.5 - 1.);
            v.w = (float)((double)(float)(w[q] >> 24) / 127.5 - 1.);
            dst[q] = v;
        }
    }
    for (size_t i = n16 * 16 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = (float)((double)(float)in[i] / 127.5 - 1.);
}
} }

extern "C" int dcg_u8_to_unit(const unsigned char* in, float* out, size_t n, dcg_stream_t stream)
{
    DCG_CHECK_ARG(in && out, "dcg_u8_to_unit: null pointer");
    DCG_CHECK_ARG(aligned16(in) && aligned16(out), "dcg_u8_to_unit: buffers must be 16-byte aligned");
    if (n == 0) return DCG_OK;
    launch_pdl(u8_to_unit_kernel, stream_grid((n + 15) / 16), kThreads, 0, as_stream(stream), in, out, n);
    DCG_LAUNCH_CHECK("u8_to_unit_kernel");
    return DCG_OK;
}

extern "C" int dcg_update(const float* dv, float* out, const float* coeff, size_t n,
                          dcg_stream_t stream)
{
    DCG_CHECK_ARG(dv && out && coeff, "dcg_update: null pointer");
    if (n == 0) return DCG_OK;
    launch_pdl(update_kernel, stream_grid(n), kThreads, 0, as_stream(stream), dv, out, coeff, n);
    DCG_LAUNCH_CHECK("update_kernel");
    return DCG_OK;
}

namespace {
struct ColsumPlan {
    bool vec;
    int tx_count;       // threads along column groups
    unsigned groups;    // column groups (float4s or floats)
    unsigned grid_x;    // column-group tiles
    unsigned slabs;     // row slabs = grid_y
    unsigned rows_per_slab;
};

ColsumPlan colsum_plan(size_t rows, size_t cols, bool ptr_aligned)
{
    ColsumPlan p;
    p.vec = (cols % 4 == 0) && ptr_aligned;
    p.groups = (unsigned)(p.vec ? cols / 4 : cols);
    int tx = 1;
    while (tx < 32 && (unsigned)tx < p.groups) tx <<= 1;
    p.tx_count = tx;
    p.grid_x = (p.groups + tx - 1) / tx;
    const int ty = kThreads / tx;
    // enough blocks to fill the machine a few times over, each at least 4 row passes deep
    size_t want = ((size_t)sm_count() * 4 + p.grid_x - 1) / p.grid_x;
    if (want > (size_t)kMaxSlabs) want = kMaxSlabs;
    size_t max_slabs = (rows + (size_t)ty * 4 - 1) / ((size_t)ty * 4);
    if (max_slabs < 1) max_slabs = 1;
    if (want > max_slabs) want = max_slabs;
    if (want < 1) want = 1;
    p.rows_per_slab = (unsigned)((rows + want - 1) / want);
    if (p.rows_per_slab < 1) p.rows_per_slab = 1;
    p.slabs = (unsigned)((rows + p.rows_per_slab - 1) / p.rows_per_slab);
    if (p.slabs < 1) p.slabs = 1;
    return p;
}

// Bytes of partial sums a plan needs (0: a single slab writes the result directly).
size_t colsum_partial_bytes(const ColsumPlan& p, size_t cols)
{
    if (p.slabs <= 1) return 0;
    // slab rows plus one row per group of kSlabGroup slabs (the second level of the in-kernel sum)
    return (size_t)(p.slabs + (p.slabs + kSlabGroup - 1) / kSlabGroup) * cols * sizeof(float);
}
}  // namespace

namespace dcg {
// The launch behind dcg_colsum.  `tickets`: kColsumTicketBytes of zeroed device memory owned by the
// caller of this launch (see above), or nullptr to finish with a second kernel instead.
int colsum_launch(const float* a, float* out, size_t rows, size_t cols, void* workspace, size_t workspace_bytes,
                  unsigned* tickets, cudaStream_t stream)
{
    const ColsumPlan p = colsum_plan(rows, cols, aligned16(a) && aligned16(workspace));
    const size_t need = colsum_partial_bytes(p, cols);
    float* partial;
    if (p.slabs == 1) {
        partial = out;  // a single slab writes the result directly
    } else {
        if (!workspace || workspace_bytes < need)
            return fail(DCG_ERR_WORKSPACE, "dcg_colsum: workspace %zu < %zu bytes", workspace_bytes, need);
        DCG_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 3u) == 0, "dcg_colsum: workspace is not 4-byte aligned");
        partial = static_cast<float*>(workspace);
    }
    const dim3 grid(p.grid_x, p.slabs);
    const size_t smem = (size_t)kThreads * (p.vec ? 4 : 1) * sizeof(float);
    if (p.slabs <= 1 || p.grid_x > (unsigned)kTicketTiles) tickets = nullptr;   // nothing to add / too many column tiles
    if (p.vec)
        launch_pdl(colsum_partial_kernel<true>, grid, kThreads, smem, stream,
            a, partial, rows, (unsigned)cols, p.rows_per_slab, p.tx_count, out, tickets);
    else
        launch_pdl(colsum_partial_kernel<false>, grid, kThreads, smem, stream,
            a, partial, rows, (unsigned)cols, p.rows_per_slab, p.tx_count, out, tickets);
    DCG_LAUNCH_CHECK("colsum_partial_kernel");
    if (p.slabs > 1 && !tickets) {
        launch_pdl(colsum_final_kernel, (unsigned)((cols + 31) / 32), 256, 0, stream,
            partial, out, p.slabs, (unsigned)cols);
        DCG_LAUNCH_CHECK("colsum_final_kernel");
    }
    return DCG_OK;
}

size_t colsum_partial_bytes_max(size_t rows, size_t cols)
{
    // the larger of the vector / scalar plans (pointer alignment is unknown at query time)
    const size_t a = colsum_partial_bytes(colsum_plan(rows, cols, true), cols);
    const size_t b = colsum_partial_bytes(colsum_plan(rows, cols, false), cols);
    return a > b ? a : b;
}
}  // namespace dcg

extern "C" size_t dcg_colsum_workspace_bytes(size_t rows, size_t cols)
{
    const size_t partial = dcg::colsum_partial_bytes_max(rows, cols);
    if (partial == 0) return 0;
    return align_up(partial, 256) + kTicketBytes;   // partial sums, then the ticket words
}

extern "C" int dcg_colsum(const float* a, float* out, size_t rows, size_t cols, void* workspace,
                          size_t workspace_bytes, dcg_stream_t stream)
{
    DCG_CHECK_ARG(a && out, "dcg_colsum: null pointer");
    DCG_CHECK_ARG(cols > 0 && cols <= 0x7fffffffu && rows > 0, "dcg_colsum: bad shape %zu x %zu", rows, cols);
    const size_t need = dcg_colsum_workspace_bytes(rows, cols);
    unsigned* tickets = nullptr;
    if (need > 0) {
        if (!workspace || workspace_bytes < need)
            return fail(DCG_ERR_WORKSPACE, "dcg_colsum: workspace %zu < %zu bytes", workspace_bytes, need);
        DCG_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 3u) == 0, "dcg_colsum: workspace is not 4-byte aligned");
        // the caller's buffer may hold anything: clear the ticket words behind the partial sums on the
        // same stream (a memset node when the stream is being captured; never an allocation)
        tickets = reinterpret_cast<unsigned*>(static_cast<unsigned char*>(workspace) + need - kTicketBytes);
        DCG_CUDA(cudaMemsetAsync(tickets, 0, kTicketBytes, as_stream(stream)));
    }
    return dcg::colsum_launch(a, out, rows, cols, workspace, need ? need - kTicketBytes : 0, tickets, as_stream(stream));
}

extern "C" int dcg_rowsum(const float* a, float* out, size_t rows, size_t cols, dcg_stream_t stream)
{
    DCG_CHECK_ARG(a && out && rows > 0 && cols > 0, "dcg_rowsum: bad arguments");
    const size_t blocks = (rows * 32 + kThreads - 1) / kThreads;
    launch_pdl(rowsum_kernel, (unsigned)blocks, kThreads, 0, as_stream(stream), a, out, rows, cols);
    DCG_LAUNCH_CHECK("rowsum_kernel");
    return DCG_OK;
}

extern "C" int dcg_sigmoid_xent(const float* y, const float* logits, float* out, size_t n,
                                dcg_stream_t stream)
{
    DCG_CHECK_ARG(y && logits && out && n > 0, "dcg_sigmoid_xent: bad arguments");
    launch_pdl(sigmoid_xent_kernel, 1, 512, 0, as_stream(stream), y, logits, out, n);
    DCG_LAUNCH_CHECK("sigmoid_xent_kernel");
    return DCG_OK;
}

namespace dcg {
// dcg_sigmoid_xent and dcg_sigmoid_xent_grad as one launch (node fusion of the backend); n small enough for one block.
int sigmoid_xent_with_grad(const float* y, const float* logits, float* loss, float* grad, size_t n, cudaStream_t stream)
{
    DCG_CHECK_ARG(y && logits && loss && grad && n > 0, "sigmoid_xent_with_grad: bad arguments");
    launch_pdl(sigmoid_xent_both_kernel, 1, 512, 0, stream, y, logits, loss, grad, n);
    DCG_LAUNCH_CHECK("sigmoid_xent_both_kernel");
    return DCG_OK;
}
}  // namespace dcg

extern "C" int dcg_sigmoid_xent_grad(const float* y, const float* logits, float* out, size_t n,
                                     dcg_stream_t stream)
{
    DCG_CHECK_ARG(y && logits && out && n > 0, "dcg_sigmoid_xent_grad: bad arguments");
    launch_pdl(sigmoid_xent_grad_kernel, stream_grid(n), kThreads, 0, as_stream(stream), y, logits, out, n);
    DCG_LAUNCH_CHECK("sigmoid_xent_grad_kernel");
    return DCG_OK;
}

extern "C" int dcg_mse(const float* y, const float* y_hat, float* out, size_t rows, size_t cols,
                       dcg_stream_t stream)
{
    DCG_CHECK_ARG(y && y_hat && out && rows * cols > 0, "dcg_mse: bad arguments");
    launch_pdl(mse_kernel, 1, 512, 0, as_stream(stream), y, y_hat, out, rows * cols);
    DCG_LAUNCH_CHECK("mse_kernel");
    return DCG_OK;
}

extern "C" int dcg_mse_grad(const float* y, const float* y_hat, float* out, size_t n,
                            dcg_stream_t stream)
{
    DCG_CHECK_ARG(y && y_hat && out && n > 0, "dcg_mse_grad: bad arguments");
    launch_pdl(mse_grad_kernel, stream_grid(n), kThreads, 0, as_stream(stream), y, y_hat, out, n,
                                                                        (float)(2. / (double)n));
    DCG_LAUNCH_CHECK("mse_grad_kernel");
    return DCG_OK;
}

static int softmax_rows(const float* a, const float* y, float* out, size_t rows, size_t cols,
                        int mode, dcg_stream_t stream)
{
    DCG_CHECK_ARG(a && out && rows > 0 && cols > 0, "softmax: bad arguments");
    const size_t blocks = (rows * 32 + kThreads - 1) / kThreads;
    launch_pdl(softmax_rows_kernel, (unsigned)blocks, kThreads, 0, as_stream(stream), a, y, out, rows, cols, mode);
    DCG_LAUNCH_CHECK("softmax_rows_kernel");
    return DCG_OK;
}

extern "C" int dcg_softmax(const float* a, float* out, size_t rows, size_t cols, dcg_stream_t stream)
{
    return softmax_rows(a, nullptr, out, rows, cols, 0, stream);
}

extern "C" int dcg_log_softmax(const float* a, float* out, size_t rows, size_t cols,
                               dcg_stream_t stream)
{
    return softmax_rows(a, nullptr, out, rows, cols, 1, stream);
}

extern "C" int dcg_softmax_xent_grad(const float* y, const float* logits, float* out, size_t rows,
                                     size_t cols, dcg_stream_t stream)
{
    DCG_CHECK_ARG(y, "dcg_softmax_xent_grad: null labels");
    return softmax_rows(logits, y, out, rows, cols, 2, stream);
}

extern "C" int dcg_softmax_xent(const float* y, const float* logits, float* out, size_t rows,
                                size_t cols, dcg_stream_t stream)
{
    DCG_CHECK_ARG(y && logits && out && rows > 0 && cols > 0, "dcg_softmax_xent: bad arguments");
    launch_pdl(softmax_xent_kernel, 1, 512, 0, as_stream(stream), y, logits, out, rows, cols);
    DCG_LAUNCH_CHECK("softmax_xent_kernel");
    return DCG_OK;
}

extern "C" int dcg_argmax_acc(const float* y, const float* y_hat, float* out, size_t rows,
                              size_t cols, dcg_stream_t stream)
{
    DCG_CHECK_ARG(y && y_hat && out && rows > 0 && cols > 0, "dcg_argmax_acc: bad arguments");
    launch_pdl(argmax_acc_kernel, 1, 512, 0, as_stream(stream), y, y_hat, out, rows, cols);
    DCG_LAUNCH_CHECK("argmax_acc_kernel");
    return DCG_OK;
}

// ---- column sums with built-in scratch ---------------------------------------------------------
// Some callers have device memory for their operands and nothing else, and are not in a position
// to call cudaMalloc: the reference's runtime is the case in point - a node handler has the
// signature void(rt::Node*) (src/gpu/kernels.hh:8), the node carries operand pointers only, and
// the loop that calls it (src/gpu/runner.cu:10-18) may run where allocating is off the table
// (a memory budget fixed at start-up, a latency-critical loop that must not enter the driver's
// allocator).  For them the two-stage column sum can use a scratch area that is part of the
// library image: it exists on every GPU the library is loaded on, from load to exit, and costs
// kColsumStaticBytes of device memory there whether or not this entry point is ever called.
constexpr size_t kColsumStaticBytes = (size_t)256 << 10;   // 256 KiB: 65536 partial sums
static __device__ __align__(256) unsigned char g_colsum_static[kColsumStaticBytes];

// Device address of g_colsum_static per device ordinal.  In host code the array's name is only a
// handle for the runtime, not an address a kernel could use: the address is looked up once per
// device with cudaGetSymbolAddress while that device is current.
static void* g_colsum_static_ptr[64];
static std::mutex g_colsum_static_mutex;

extern "C" size_t dcg_colsum_noalloc_max_bytes(void) { return kColsumStaticBytes; }

extern "C" int dcg_colsum_noalloc(const float* a, float* out, size_t rows, size_t cols, dcg_stream_t stream)
{
    DCG_CHECK_ARG(a && out, "dcg_colsum_noalloc: null pointer");
    DCG_CHECK_ARG(cols > 0 && cols <= 0x7fffffffu && rows > 0, "dcg_colsum_noalloc: bad shape %zu x %zu", rows, cols);
    const size_t need = dcg_colsum_workspace_bytes(rows, cols);
    if (need > kColsumStaticBytes)
        return fail(DCG_ERR_WORKSPACE,
                    "dcg_colsum_noalloc: a %zu x %zu column sum needs %zu bytes of scratch, the built-in area holds %zu; "
                    "use dcg_colsum with caller-provided scratch",
                    rows, cols, need, kColsumStaticBytes);
    int dev = 0;
    DCG_CUDA(cudaGetDevice(&dev));
    DCG_CHECK_ARG(dev >= 0 && dev < 64, "dcg_colsum_noalloc: device ordinal %d out of range", dev);
    void* scratch;
    {
        std::lock_guard<std::mutex> lock(g_colsum_static_mutex);
        if (!g_colsum_static_ptr[dev]) {
            void* p = nullptr;
            DCG_CUDA(cudaGetSymbolAddress(&p, g_colsum_static));
            g_colsum_static_ptr[dev] = p;
        }
        scratch = g_colsum_static_ptr[dev];
    }
    // Stage 1 overwrites every partial sum stage 2 reads, so nothing in the area has to be
    // cleared between calls even though it keeps the previous call's contents.
    return dcg_colsum(a, out, rows, cols, scratch, kColsumStaticBytes, stream);
}
