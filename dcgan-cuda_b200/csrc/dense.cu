// Dense-layer matrix products (src/gpu/matmul.cu:11-86): the generator's
// 100 -> 8192 projection, the discriminator's 8192 -> 1 head, and the MNIST MLP.
//
// These are small and HBM/latency bound (the largest operand is 3.3 MB), so they
// stay on CUDA cores: a shared-memory tiled kernel that accumulates each output
// over k in ascending order with unfused multiply/add - bit-identical to the
// reference CPU loops (src/cpu/ops.hxx:56-105,375-390) - plus a warp-per-output
// kernel for the "few outputs, long reduction" head (64 x 8192 x 1).
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
                  size_t m, size_t n, size_t p)
{
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
        }
    }
}

// One warp per output element, for m*p small and n long: out = A[m,n] B[n,p] (+bias).
__global__ void __launch_bounds__(TPB)
gemm_warp_per_output_kernel(const float* __restrict__ a, const float* __restrict__ b,
                            const float* __restrict__ bias, float* __restrict__ out,
                            size_t m, size_t n, size_t p)
{
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= m * p) return;
    const size_t r = warp / p, c = warp % p;
    float s = 0.f;
    for (size_t k = lane; k < n; k += 32) s = fmaf(__ldg(a + r * n + k), __ldg(b + k * p + c), s);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) out[warp] = bias ? s + __ldg(bias + c) : s;
}

template <bool TA, bool TB>
int launch_tiled(const float* a, const float* b, const float* bias, float* out, size_t m, size_t n,
                 size_t p, cudaStream_t stream, const char* name)
{
    const dim3 grid((unsigned)((p + TILE - 1) / TILE), (unsigned)((m + TILE - 1) / TILE));
    gemm_tiled_kernel<TA, TB><<<grid, TPB, 0, stream>>>(a, b, bias, out, m, n, p);
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
        const size_t blocks = (m * p * 32 + TPB - 1) / TPB;
        gemm_warp_per_output_kernel<<<(unsigned)blocks, TPB, 0, as_stream(stream)>>>(a, b, bias, out, m, n, p);
        DCG_LAUNCH_CHECK("gemm_warp_per_output_kernel");
        return DCG_OK;
    }
    return launch_tiled<false, false>(a, b, bias, out, m, n, p, as_stream(stream), "gemm_tiled_kernel<nn>");
}

extern "C" int dcg_matmul_tn(const float* a, const float* b, float* out, size_t m, size_t n,
                             size_t p, dcg_stream_t stream)
{
    DCG_CHECK_ARG(a && b && out && m > 0 && n > 0 && p > 0, "dcg_matmul_tn: bad arguments");
    return launch_tiled<true, false>(a, b, nullptr, out, m, n, p, as_stream(stream), "gemm_tiled_kernel<tn>");
}

extern "C" int dcg_matmul_nt(const float* a, const float* b, float* out, size_t m, size_t n,
                             size_t p, dcg_stream_t stream)
{
    DCG_CHECK_ARG(a && b && out && m > 0 && n > 0 && p > 0, "dcg_matmul_nt: bad arguments");
    return launch_tiled<false, true>(a, b, nullptr, out, m, n, p, as_stream(stream), "gemm_tiled_kernel<nt>");
}
