// Dense-layer matrix products (src/gpu/matmul.cu:11-86): the generator's
// 100 -> 8192 projection, the discriminator's 8192 -> 1 head, and the MNIST MLP.
//
// These are small and HBM/latency bound (the largest operand is 3.3 MB), so they
// stay on CUDA cores: a shared-memory tiled kernel that accumulates each output
// over k in ascending order with unfused multiply/add - bit-identical to the
// reference CPU loops (src/cpu/ops.hxx:56-105,375-390) - plus three shape
// specialists for the DCGAN layers: short reduction / wide output (100 -> 8192 and
// its weight gradient), few outputs / long reduction (8192 -> 1), and tall output
// from a transposed operand (the head's weight gradient).
#include "common.cuh"

namespace dcg {
namespace {

constexpr int TILE = 64;  // output tile edge
constexpr int KT = 16;    // k-tile depth
constexpr int TPB = 256;  // 16 x 16 threads, 4 x 4 outputs each

// Operand views: element (row, col) of the logical [rows x cols] matrix.
// TRANS: the logical matrix is the transpose of the stored row-major one.
template <bool TRANS>
__device__ __forceinline__ float load_elem(const float* __restrict__ p, size_t r, size_t c,
                                           size_t rows, size_t cols)
{
    return TRANS ? __ldg(p + c * rows + r) : __ldg(p + r * cols + c);
}

// out[m,p] = A[m,n] * B[n,p] (+ bias[p]); A, B through the views above.
template <bool TA, bool TB>
__global__ void __launch_bounds__(TPB)
gemm_tiled_kernel(const float* __restrict__ a, const float* __restrict__ b,
                  const float* __restrict__ bias, float* __restrict__ out,
                  size_t m, size_t n, size_t p, const float* __restrict__ gate, float* __restrict__ gated_out,
                  int gate_act, float gate_alpha)
{
    pdl_enter();
    __shared__ float As[KT][TILE + 1];  // [k][row]
    __shared__ float Bs[KT][TILE + 1];  // [k][col]
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const size_t row0 = (size_t)blockIdx.y * TILE, col0 = (size_t)blockIdx.x * TILE;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (size_t k0 = 0; k0 < n; k0 += KT) {
        for (int e = threadIdx.x; e < KT * TILE; e += TPB) {
            // pick the fast-varying index along the contiguous memory direction
            int kk, rr;
            if (TA) { rr = e % TILE; kk = e / TILE; } else { kk = e % KT; rr = e / KT; }
            const size_t r = row0 + rr, k = k0 + kk;
            As[kk][rr] = (r < m && k < n) ? load_elem<TA>(a, r, k, m, n) : 0.f;
            int cc;
            if (TB) { kk = e % KT; cc = e / KT; } else { cc = e % TILE; kk = e / TILE; }
            const size_t c = col0 + cc, k2 = k0 + kk;
            Bs[kk][cc] = (c < p && k2 < n) ? load_elem<TB>(b, k2, c, n, p) : 0.f;
        }
        __syncthreads();
        const int klim = (n - k0 < (size_t)KT) ? (int)(n - k0) : KT;
        for (int kk = 0; kk < klim; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(av[i], bv[j]));
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const size_t r = row0 + ty * 4 + i;
        if (r >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const size_t c = col0 + tx * 4 + j;
            if (c >= p) continue;
            float v = acc[i][j];
            if (bias) v = __fadd_rn(v, __ldg(bias + c));
            out[r * p + c] = v;
            // the activation gradient that follows the product in a backward list, same expression as act_grad_kernel
            if (gate) gated_out[r * p + c] = act_grad_apply(__ldg(gate + r * p + c), v, gate_act, gate_alpha);
        }
    }
}

// One block per output element, for m*p small and n long: out = A[m,n] B[n,p] (+bias).
// Thread t adds elements t, t+256, ... in ascending order; the 256 thread sums are then added
// in a fixed tree, so the result is independent of scheduling.
__global__ void __launch_bounds__(TPB)
gemm_long_k_kernel(const float* __restrict__ a, const float* __restrict__ b,
                   const float* __restrict__ bias, float* __restrict__ out,
                   size_t m, size_t n, size_t p)
{
    pdl_enter();
    __shared__ float part[TPB];
    const size_t o = blockIdx.x;
    const size_t r = o / p, c = o % p;
    const float* ar = a + r * n;
    float s = 0.f;
    size_t k = threadIdx.x;
    for (; k + 3 * TPB < n; k += 4 * TPB) {
        const float a0 = __ldg(ar + k), a1 = __ldg(ar + k + TPB), a2 = __ldg(ar + k + 2 * TPB), a3 = __ldg(ar + k + 3 * TPB);
        const float b0 = __ldg(b + k * p + c), b1 = __ldg(b + (k + TPB) * p + c);
        const float b2 = __ldg(b + (k + 2 * TPB) * p + c), b3 = __ldg(b + (k + 3 * TPB) * p + c);
        s = fmaf(a0, b0, s); s = fmaf(a1, b1, s); s = fmaf(a2, b2, s); s = fmaf(a3, b3, s);
    }
    for (; k < n; k += TPB) s = fmaf(__ldg(ar + k), __ldg(b + k * p + c), s);
    part[threadIdx.x] = s;
    __syncthreads();
    for (int h = TPB / 2; h > 0; h >>= 1) {
        if ((int)threadIdx.x < h) part[threadIdx.x] += part[threadIdx.x + h];
        __syncthreads();
    }
    if (threadIdx.x == 0) out[o] = bias ? part[0] + __ldg(bias + c) : part[0];
}

// Short reduction, wide output (the generator's projection and its weight gradient):
// out[m,p] = A[m,n] B[n,p] (+bias) with n <= 256 and B row-major.  A block owns 128 columns and
// RB rows: the RB x n slab of A sits in shared memory, every thread walks one column of B
// (coalesced across the block) and keeps RB accumulators.  k ascends, multiply and add stay
// unfused: the same rounding sequence as the reference loops (src/cpu/ops.hxx:56-105).
constexpr int RB = 8;
template <bool TA>
__global__ void __launch_bounds__(128)
gemm_wide_kernel(const float* __restrict__ a, const float* __restrict__ b,
                 const float* __restrict__ bias, float* __restrict__ out,
                 size_t m, size_t n, size_t p)
{
    pdl_enter();
    __shared__ __align__(16) float As[256 * RB];   // [k][RB]
    const size_t row0 = (size_t)blockIdx.y * RB;
    for (int e = threadIdx.x; e < (int)n * RB; e += 128) {
        int kk, rr;
        if (TA) { rr = e % RB; kk = e / RB; } else { kk = e % (int)n; rr = e / (int)n; }
        const size_t r = row0 + rr;
        As[kk * RB + rr] = r < m ? load_elem<TA>(a, r, (size_t)kk, m, n) : 0.f;
    }
    __syncthreads();
    const size_t c = (size_t)blockIdx.x * 128 + threadIdx.x;
    if (c >= p) return;
    float acc[RB];
#pragma unroll
    for (int i = 0; i < RB; ++i) acc[i] = 0.f;
    const float* bc = b + c;
    int k = 0;
    // sixteen loads of B in flight per thread: the kernel is latency-bound otherwise (one warp walks
    // a column of B with nothing else to overlap the memory round trips)
    for (; k + 16 <= (int)n; k += 16) {
        float bv[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) bv[u] = __ldg(bc + (size_t)(k + u) * p);
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const float4* ak = reinterpret_cast<const float4*>(As + (k + u) * RB);
#pragma unroll
            for (int q = 0; q < RB / 4; ++q) {
                const float4 av = ak[q];
                acc[4 * q + 0] = __fadd_rn(acc[4 * q + 0], __fmul_rn(av.x, bv[u]));
                acc[4 * q + 1] = __fadd_rn(acc[4 * q + 1], __fmul_rn(av.y, bv[u]));
                acc[4 * q + 2] = __fadd_rn(acc[4 * q + 2], __fmul_rn(av.z, bv[u]));
                acc[4 * q + 3] = __fadd_rn(acc[4 * q + 3], __fmul_rn(av.w, bv[u]));
            }
        }
    }
    for (; k + 4 <= (int)n; k += 4) {
        float bv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) bv[u] = __ldg(bc + (size_t)(k + u) * p);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float4* ak = reinterpret_cast<const float4*>(As + (k + u) * RB);
#pragma unroll
            for (int q = 0; q < RB / 4; ++q) {
                const float4 av = ak[q];
                acc[4 * q + 0] = __fadd_rn(acc[4 * q + 0], __fmul_rn(av.x, bv[u]));
                acc[4 * q + 1] = __fadd_rn(acc[4 * q + 1], __fmul_rn(av.y, bv[u]));
                acc[4 * q + 2] = __fadd_rn(acc[4 * q + 2], __fmul_rn(av.z, bv[u]));
                acc[4 * q + 3] = __fadd_rn(acc[4 * q + 3], __fmul_rn(av.w, bv[u]));
            }
        }
    }
    for (; k < (int)n; ++k) {
        const float bv = __ldg(bc + (size_t)k * p);
#pragma unroll
        for (int i = 0; i < RB; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(As[k * RB + i], bv));
    }
    const float bb = bias ? __ldg(bias + c) : 0.f;
#pragma unroll
    for (int i = 0; i < RB; ++i) {
        const size_t r = row0 + i;
        if (r < m) out[r * p + c] = bias ? __fadd_rn(acc[i], bb) : acc[i];
    }
}

// Tall output with a handful of columns from a transposed left operand (the discriminator head's
// weight gradient, x^T dy): out[r,c] = sum_k A^T[k,r] B[k,c]; one thread per output, loads
// coalesced along r, k ascending, unfused.
__global__ void __launch_bounds__(TPB)
gemm_tall_tn_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                    size_t m, size_t n, size_t p)
{
    pdl_enter();
    const size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= m * p) return;
    const size_t c = o / m, r = o % m;   // r fastest across threads: coalesced reads of A^T
    float s = 0.f;
    size_t k = 0;
    for (; k + 16 <= n; k += 16) {
        float av[16], bw[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) { av[u] = __ldg(a + (k + u) * m + r); bw[u] = __ldg(b + (k + u) * p + c); }
#pragma unroll
        for (int u = 0; u < 16; ++u) s = __fadd_rn(s, __fmul_rn(av[u], bw[u]));
    }
    for (; k < n; ++k) s = __fadd_rn(s, __fmul_rn(__ldg(a + k * m + r), __ldg(b + k * p + c)));
    out[r * p + c] = s;
}

template <bool TA>
int launch_wide(const float* a, const float* b, const float* bias, float* out, size_t m, size_t n,
                size_t p, cudaStream_t stream)
{
    const dim3 grid((unsigned)((p + 127) / 128), (unsigned)((m + RB - 1) / RB));
    launch_pdl(gemm_wide_kernel<TA>, grid, 128, 0, stream, a, b, bias, out, m, n, p);
    DCG_LAUNCH_CHECK("gemm_wide_kernel");
    return DCG_OK;
}

inline bool wide_shape(size_t m, size_t n, size_t p) { return n <= 256 && p >= 512 && m <= 65535u * RB; }

template <bool TA, bool TB>
int launch_tiled(const float* a, const float* b, const float* bias, float* out, size_t m, size_t n,
                 size_t p, cudaStream_t stream, const char* name, const float* gate = nullptr, float* gated_out = nullptr,
                 int gate_act = 0, float gate_alpha = 0.f)
{
    const dim3 grid((unsigned)((p + TILE - 1) / TILE), (unsigned)((m + TILE - 1) / TILE));
    launch_pdl(gemm_tiled_kernel<TA, TB>, grid, TPB, 0, stream, a, b, bias, out, m, n, p, gate, gated_out, gate_act, gate_alpha);
    DCG_LAUNCH_CHECK(name);
    return DCG_OK;
}

}  // namespace
}  // namespace dcg

using namespace dcg;

extern "C" int dcg_matmul(const float* a, const float* b, const float* bias, float* out, size_t m,
                          size_t n, size_t p, dcg_stream_t stream)
{
    DCG_CHECK_ARG(a && b && out && m > 0 && n > 0 && p > 0, "dcg_matmul: bad arguments");
    if (m * p <= 4096 && n >= 1024) {
        launch_pdl(gemm_long_k_kernel, (unsigned)(m * p), TPB, 0, as_stream(stream), a, b, bias, out, m, n, p);
        DCG_LAUNCH_CHECK("gemm_long_k_kernel");
        return DCG_OK;
    }
    if (wide_shape(m, n, p)) return launch_wide<false>(a, b, bias, out, m, n, p, as_stream(stream));
    return launch_tiled<false, false>(a, b, bias, out, m, n, p, as_stream(stream), "gemm_tiled_kernel<nn>");
}

extern "C" int dcg_matmul_tn(const float* a, const float* b, float* out, size_t m, size_t n,
                             size_t p, dcg_stream_t stream)
{
    DCG_CHECK_ARG(a && b && out && m > 0 && n > 0 && p > 0, "dcg_matmul_tn: bad arguments");
    if (wide_shape(m, n, p)) return launch_wide<true>(a, b, nullptr, out, m, n, p, as_stream(stream));
    if (p <= 8 && m >= 1024) {
        launch_pdl(gemm_tall_tn_kernel, (unsigned)((m * p + 63) / 64), 64, 0, as_stream(stream), a, b, out, m, n, p);
        DCG_LAUNCH_CHECK("gemm_tall_tn_kernel");
        return DCG_OK;
    }
    return launch_tiled<true, false>(a, b, nullptr, out, m, n, p, as_stream(stream), "gemm_tiled_kernel<tn>");
}

namespace dcg {
// dcg_matmul_nt followed by dcg_act_grad(gate, out) -> gated_out as one launch (node fusion of the backend).
int matmul_nt_gated(const float* a, const float* b, float* out, size_t m, size_t n, size_t p, const float* gate,
                    float* gated_out, int gate_act, float gate_alpha, cudaStream_t stream)
{
    DCG_CHECK_ARG(a && b && out && gate && gated_out && m > 0 && n > 0 && p > 0, "matmul_nt_gated: bad arguments");
    return launch_tiled<false, true>(a, b, nullptr, out, m, n, p, stream, "gemm_tiled_kernel<nt>", gate, gated_out, gate_act,
                                     gate_alpha);
}
}  // namespace dcg

extern "C" int dcg_matmul_nt(const float* a, const float* b, float* out, size_t m, size_t n,
                             size_t p, dcg_stream_t stream)
{
    DCG_CHECK_ARG(a && b && out && m > 0 && n > 0 && p > 0, "dcg_matmul_nt: bad arguments");
    return launch_tiled<false, true>(a, b, nullptr, out, m, n, p, as_stream(stream), "gemm_tiled_kernel<nt>");
}
