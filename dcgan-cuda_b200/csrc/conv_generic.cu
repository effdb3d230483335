// CUDA-core fp32 convolution kernels for arbitrary shapes (DCG_PREC_FP32).
//
// These play the role of the reference's naive kernels (src/gpu/conv2d_naive.hh:
// one thread per output element) and are the path every shape the tensor-core
// kernels cannot take falls back to.  They are written for exactness, not speed:
// each output is accumulated in the order the reference's CPU code uses, with
// unfused IEEE multiplies and adds, so the results are bit-comparable with
// src/cpu/ops.hxx:
//   forward      : one accumulator over (channel, kernel row, kernel column), ops.hxx:227-246
//   input grad   : per output filter an inner sum over taps, filters added in order, ops.hxx:650-679
//   kernel grad  : per image an inner sum over output pixels, images added in order, ops.hxx:754-772
#include "common.cuh"
#include "conv.cuh"

namespace dcg {
namespace {

constexpr int kThreads = 128;

__global__ void __launch_bounds__(kThreads)
conv_fwd_generic_kernel(const float* __restrict__ x, const float* __restrict__ k,
                        float* __restrict__ y, const dcg_conv_desc d, const EpilogueArgs ep,
                        size_t total)
{
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int o = (int)(idx % d.o);
    size_t t = idx / d.o;
    const int j = (int)(t % d.wo); t /= d.wo;
    const int i = (int)(t % d.ho);
    const int n = (int)(t / d.ho);
    const int h0 = i * d.stride_h - d.pad_top, w0 = j * d.stride_w - d.pad_left;
    const float* xn = x + (size_t)n * d.h * d.w * d.c;
    float val = 0.f;
    for (int q = 0; q < d.c; ++q)
        for (int di = 0; di < d.kh; ++di) {
            const int h = h0 + di;
            if (h < 0 || h >= d.h) continue;
            for (int dj = 0; dj < d.kw; ++dj) {
                const int w = w0 + dj;
                if (w < 0 || w >= d.w) continue;
                const float xv = __ldg(xn + ((size_t)h * d.w + w) * d.c + q);
                const float kv = __ldg(k + (((size_t)di * d.kw + dj) * d.c + q) * d.o + o);
                val = __fadd_rn(val, __fmul_rn(xv, kv));
            }
        }
    y[idx] = epilogue_apply(ep, val, idx, o);
}

// dx[n,i,j,c] = sum_o ( sum_{di,dj} dyz[n,i+di-P,j+dj-Q,o] * k[KH-1-di,KW-1-dj,c,o] ), dyz the
// zero-inserted dy, P = KH-1-pad_top, Q = KW-1-pad_left (src/cpu/ops.hxx:618-629).
__global__ void __launch_bounds__(kThreads)
conv_dx_generic_kernel(const float* __restrict__ dy, const float* __restrict__ k,
                       float* __restrict__ dx, const dcg_conv_desc d, const EpilogueArgs ep,
                       size_t total)
{
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int c = (int)(idx % d.c);
    size_t t = idx / d.c;
    const int j = (int)(t % d.w); t /= d.w;
    const int i = (int)(t % d.h);
    const int n = (int)(t / d.h);
    const int P = d.kh - 1 - d.pad_top, Q = d.kw - 1 - d.pad_left;
    const float* dyn = dy + (size_t)n * d.ho * d.wo * d.o;
    float total_v = 0.f;
    for (int o = 0; o < d.o; ++o) {
        float val = 0.f;
        for (int di = 0; di < d.kh; ++di) {
            const int ph = i + di - P;
            if (ph < 0 || ph % d.stride_h != 0) continue;
            const int a = ph / d.stride_h;
            if (a >= d.ho) continue;
            for (int dj = 0; dj < d.kw; ++dj) {
                const int pw = j + dj - Q;
                if (pw < 0 || pw % d.stride_w != 0) continue;
                const int b = pw / d.stride_w;
                if (b >= d.wo) continue;
                const float g = __ldg(dyn + ((size_t)a * d.wo + b) * d.o + o);
                const float kv = __ldg(k + (((size_t)(d.kh - 1 - di) * d.kw + (d.kw - 1 - dj)) * d.c + c) * d.o + o);
                val = __fadd_rn(val, __fmul_rn(g, kv));
            }
        }
        total_v = (o == 0) ? val : __fadd_rn(total_v, val);
    }
    dx[idx] = epilogue_apply(ep, total_v, idx, c);
}

// dk[kh,kw,c,o] = sum_n ( sum_{a,b} x[n,kh+s*a-pt,kw+s*b-pl,c] * dy[n,a,b,o] )
__global__ void __launch_bounds__(kThreads)
conv_dk_generic_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                       float* __restrict__ dk, const dcg_conv_desc d, size_t total)
{
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int o = (int)(idx % d.o);
    size_t t = idx / d.o;
    const int c = (int)(t % d.c); t /= d.c;
    const int kw = (int)(t % d.kw);
    const int kh = (int)(t / d.kw);
    float total_v = 0.f;
    for (int n = 0; n < d.n; ++n) {
        const float* xn = x + (size_t)n * d.h * d.w * d.c;
        const float* dyn = dy + (size_t)n * d.ho * d.wo * d.o;
        float val = 0.f;
        for (int a = 0; a < d.ho; ++a) {
            const int h = kh + d.stride_h * a - d.pad_top;
            if (h < 0 || h >= d.h) continue;
            for (int b = 0; b < d.wo; ++b) {
                const int w = kw + d.stride_w * b - d.pad_left;
                if (w < 0 || w >= d.w) continue;
                const float xv = __ldg(xn + ((size_t)h * d.w + w) * d.c + c);
                const float g = __ldg(dyn + ((size_t)a * d.wo + b) * d.o + o);
                val = __fadd_rn(val, __fmul_rn(xv, g));
            }
        }
        total_v = (n == 0) ? val : __fadd_rn(total_v, val);
    }
    dk[idx] = total_v;
}

}  // namespace

int conv_fwd_generic(const dcg_conv_desc& d, const float* x, const float* k, float* y,
                     const EpilogueArgs& ep, cudaStream_t stream)
{
    const size_t total = (size_t)d.n * d.ho * d.wo * d.o;
    if (total == 0) return DCG_OK;
    conv_fwd_generic_kernel<<<(unsigned)((total + kThreads - 1) / kThreads), kThreads, 0, stream>>>(
        x, k, y, d, ep, total);
    DCG_LAUNCH_CHECK("conv_fwd_generic_kernel");
    return DCG_OK;
}

int conv_dx_generic(const dcg_conv_desc& d, const float* dy, const float* k, float* dx,
                    const EpilogueArgs& ep, cudaStream_t stream)
{
    const size_t total = (size_t)d.n * d.h * d.w * d.c;
    if (total == 0) return DCG_OK;
    conv_dx_generic_kernel<<<(unsigned)((total + kThreads - 1) / kThreads), kThreads, 0, stream>>>(
        dy, k, dx, d, ep, total);
    DCG_LAUNCH_CHECK("conv_dx_generic_kernel");
    return DCG_OK;
}

int conv_dk_generic(const dcg_conv_desc& d, const float* x, const float* dy, float* dk,
                    cudaStream_t stream)
{
    const size_t total = (size_t)d.kh * d.kw * d.c * d.o;
    if (total == 0) return DCG_OK;
    conv_dk_generic_kernel<<<(unsigned)((total + kThreads - 1) / kThreads), kThreads, 0, stream>>>(
        x, dy, dk, d, total);
    DCG_LAUNCH_CHECK("conv_dk_generic_kernel");
    return DCG_OK;
}

}  // namespace dcg
