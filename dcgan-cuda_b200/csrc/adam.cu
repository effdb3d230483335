// Fused multi-tensor Adam: one launch updates every variable of a network.
//
// Replaces the three launches per variable of the reference (moment_update,
// moment_update2, adam_update: src/gpu/update.cu:23-54,65-96).  HBM-bound:
// 28 bytes per parameter (read g, m, v, p; write m, v, p), 128-bit accesses.
// The arithmetic is written with explicit IEEE multiplies/adds in the order of
// src/cpu/ops.hxx:905-924, so with grad_scale == 1 the result is bit-identical
// to the reference's CPU path.
#include <cmath>

#include "adam.cuh"
#include "common.cuh"

namespace dcg {
namespace {

constexpr int kAdamThreads = 256;
constexpr int kAdamIlp = 4;                                       // float4s per thread
constexpr int kAdamChunk = kAdamThreads * kAdamIlp * 4;           // elements per block
constexpr int kAdamMaxTensors = 24;

struct AdamBatch {
    float* p[kAdamMaxTensors];
    const float* g[kAdamMaxTensors];
    const float* g2[kAdamMaxTensors];
    float* m[kAdamMaxTensors];
    float* v[kAdamMaxTensors];
    unsigned long long n[kAdamMaxTensors];
    unsigned block_begin[kAdamMaxTensors + 1];
    int count;
};

struct AdamCoeffs {
    float lr_t, a1, b1, a2, b2, eps, scale;
    const float* lr_t_dev;   // non-null: the step size is read from device memory instead (a captured
                             // launch then serves every step: the host only rewrites the scalar)
};

__device__ __forceinline__ void adam_one(float& p, float g, float& m, float& v, const AdamCoeffs& c)
{
    m = __fadd_rn(__fmul_rn(c.a1, m), __fmul_rn(c.b1, g));
    v = __fadd_rn(__fmul_rn(c.a2, v), __fmul_rn(__fmul_rn(c.b2, g), g));
    p = __fsub_rn(p, __fdiv_rn(__fmul_rn(c.lr_t, m), __fadd_rn(__fsqrt_rn(v), c.eps)));
}

__global__ void __launch_bounds__(kAdamThreads)
adam_multi_kernel(const __grid_constant__ AdamBatch batch, const AdamCoeffs c_in)
{
    pdl_enter();
    AdamCoeffs c = c_in;
    if (c.lr_t_dev) c.lr_t = __ldg(c.lr_t_dev);
    // which tensor does this block belong to?
    int t = 0;
    while (t + 1 < batch.count && blockIdx.x >= batch.block_begin[t + 1]) ++t;
    const unsigned long long n = batch.n[t];
    const unsigned long long base = (unsigned long long)(blockIdx.x - batch.block_begin[t]) * kAdamChunk;
    float* __restrict__ p = batch.p[t];
    const float* __restrict__ g = batch.g[t];
    const float* __restrict__ g2 = batch.g2[t];
    float* __restrict__ m = batch.m[t];
    float* __restrict__ v = batch.v[t];
    const bool scaled = c.scale != 1.f;

    const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                       reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                       reinterpret_cast<uintptr_t>(g2)) & 15u) == 0;
    if (vec && base + kAdamChunk <= n) {
        float4 pp[kAdamIlp], gg[kAdamIlp], mm[kAdamIlp], vv[kAdamIlp];
#pragma unroll
        for (int k = 0; k < kAdamIlp; ++k) {
            const unsigned long long i4 = (base >> 2) + (unsigned long long)k * kAdamThreads + threadIdx.x;
            gg[k] = __ldg(reinterpret_cast<const float4*>(g) + i4);
            if (g2) {
                const float4 h = __ldg(reinterpret_cast<const float4*>(g2) + i4);
                gg[k].x = __fadd_rn(gg[k].x, h.x); gg[k].y = __fadd_rn(gg[k].y, h.y);
                gg[k].z = __fadd_rn(gg[k].z, h.z); gg[k].w = __fadd_rn(gg[k].w, h.w);
            }
            pp[k] = reinterpret_cast<const float4*>(p)[i4];
            mm[k] = reinterpret_cast<const float4*>(m)[i4];
            vv[k] = reinterpret_cast<const float4*>(v)[i4];
        }
#pragma unroll
        for (int k = 0; k < kAdamIlp; ++k) {
            if (scaled) {
                gg[k].x = __fmul_rn(gg[k].x, c.scale); gg[k].y = __fmul_rn(gg[k].y, c.scale);
                gg[k].z = __fmul_rn(gg[k].z, c.scale); gg[k].w = __fmul_rn(gg[k].w, c.scale);
            }
            adam_one(pp[k].x, gg[k].x, mm[k].x, vv[k].x, c);
            adam_one(pp[k].y, gg[k].y, mm[k].y, vv[k].y, c);
            adam_one(pp[k].z, gg[k].z, mm[k].z, vv[k].z, c);
            adam_one(pp[k].w, gg[k].w, mm[k].w, vv[k].w, c);
            const unsigned long long i4 = (base >> 2) + (unsigned long long)k * kAdamThreads + threadIdx.x;
            reinterpret_cast<float4*>(m)[i4] = mm[k];
            reinterpret_cast<float4*>(v)[i4] = vv[k];
            reinterpret_cast<float4*>(p)[i4] = pp[k];
        }
    } else {
        unsigned long long end = base + kAdamChunk;
        if (end > n) end = n;
        for (unsigned long long i = base + threadIdx.x; i < end; i += kAdamThreads) {
            float gi = __ldg(g + i);
            if (g2) gi = __fadd_rn(gi, __ldg(g2 + i));
            if (scaled) gi = __fmul_rn(gi, c.scale);
            float pi = p[i], mi = m[i], vi = v[i];
            adam_one(pi, gi, mi, vi, c);
            m[i] = mi; v[i] = vi; p[i] = pi;
        }
    }
}

// Unfused forms, one per reference node type (src/gpu/update.cu:23-54); used when a
// node list is executed without fusion or a triple is incomplete.
__global__ void __launch_bounds__(kAdamThreads)
moment_kernel(const float* __restrict__ dv, float* __restrict__ out, float a, float b, size_t n,
              int squared)
{
    pdl_enter();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float g = __ldg(dv + i);
        const float bg = squared ? __fmul_rn(__fmul_rn(b, g), g) : __fmul_rn(b, g);
        out[i] = __fadd_rn(__fmul_rn(a, out[i]), bg);
    }
}

__global__ void __launch_bounds__(kAdamThreads)
adam_apply_kernel(const float* __restrict__ m, const float* __restrict__ v, float* __restrict__ out,
                  float lr_t, float eps, size_t n)
{
    pdl_enter();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = __fsub_rn(out[i], __fdiv_rn(__fmul_rn(lr_t, __ldg(m + i)),
                                             __fadd_rn(__fsqrt_rn(__ldg(v + i)), eps)));
}

inline unsigned flat_grid(size_t n)
{
    size_t blocks = (n + kAdamThreads - 1) / kAdamThreads;
    const size_t cap = (size_t)sm_count() * 8;
    return (unsigned)(blocks > cap ? cap : (blocks ? blocks : 1));
}

}  // namespace

int moment_update_launch(const float* dv, float* out, float a, float b, size_t n, bool squared,
                         cudaStream_t stream)
{
    DCG_CHECK_ARG(dv && out, "moment_update: null pointer");
    if (n == 0) return DCG_OK;
    launch_pdl(moment_kernel, flat_grid(n), kAdamThreads, 0, stream, dv, out, a, b, n, squared ? 1 : 0);
    DCG_LAUNCH_CHECK("moment_kernel");
    return DCG_OK;
}

int adam_apply_launch(const float* m, const float* v, float* out, float lr_t, float eps, size_t n,
                      cudaStream_t stream)
{
    DCG_CHECK_ARG(m && v && out, "adam_update: null pointer");
    if (n == 0) return DCG_OK;
    launch_pdl(adam_apply_kernel, flat_grid(n), kAdamThreads, 0, stream, m, v, out, lr_t, eps, n);
    DCG_LAUNCH_CHECK("adam_apply_kernel");
    return DCG_OK;
}

int adam_multi_launch(const dcg_adam_tensor* tensors, int count, float lr_t, float a1, float b1,
                      float a2, float b2, float eps, float grad_scale, cudaStream_t stream,
                      const float* lr_t_dev)
{
    DCG_CHECK_ARG(count >= 0 && (count == 0 || tensors), "adam: bad tensor list");
    AdamCoeffs c{lr_t, a1, b1, a2, b2, eps, grad_scale, lr_t_dev};
    int done = 0;
    while (done < count) {
        AdamBatch batch;
        batch.count = 0;
        unsigned blocks = 0;
        while (done < count && batch.count < kAdamMaxTensors) {
            const dcg_adam_tensor& t = tensors[done];
            DCG_CHECK_ARG(t.p && t.g && t.m && t.v, "adam: null pointer in tensor %d", done);
            if (t.n > 0) {
                const int k = batch.count++;
                batch.p[k] = t.p; batch.g[k] = t.g; batch.g2[k] = t.g2;
                batch.m[k] = t.m; batch.v[k] = t.v; batch.n[k] = t.n;
                batch.block_begin[k] = blocks;
                blocks += (unsigned)((t.n + kAdamChunk - 1) / kAdamChunk);
            }
            ++done;
        }
        if (batch.count == 0) continue;
        batch.block_begin[batch.count] = blocks;
        launch_pdl(adam_multi_kernel, blocks, kAdamThreads, 0, stream, batch, c);
        DCG_LAUNCH_CHECK("adam_multi_kernel");
    }
    return DCG_OK;
}

}  // namespace dcg

extern "C" float dcg_adam_lr_t(float* t_host, float lr, float beta1, float beta2)
{
    ++*t_host;
    return lr * std::sqrt(1 - std::pow(beta2, *t_host)) / (1 - std::pow(beta1, *t_host));
}

extern "C" int dcg_adam_multi(const dcg_adam_tensor* tensors, int count, float lr_t, float beta1,
                              float beta2, float eps, float grad_scale, dcg_stream_t stream)
{
    return dcg::adam_multi_launch(tensors, count, lr_t, beta1, 1.f - beta1, beta2, 1.f - beta2, eps,
                                  grad_scale, dcg::as_stream(stream));
}
