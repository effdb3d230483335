// Helper kernels of the <= 4-channel layers: partition finish of the kernel gradient, image / weight repacks, the
// stand-alone gather of the input gradient.  Included by conv_tc.cu only.
#pragma once

namespace dcg {
namespace {

// ---- narrow-channel DK: add the partitions' partial tiles -----------------------------------------
// partial[m tile][partition][col][row] (col = 32 * kernel row + window slot, row = output channel).
// Block = 32 rows x 8 lanes of one column: lane l adds partitions l, l+8, ... (all loads in
// flight), the eight lane sums are then added in lane order - a fixed order for a given partition
// count, so the result does not depend on timing.  blockIdx.x = column, blockIdx.y = 32-row group.
__global__ void __launch_bounds__(256)
dk_narrow_finish_kernel(const float* __restrict__ partial, float* __restrict__ dk, int parts, int bn,
                        int KH, int KW, int C, int O)
{
    pdl_enter();
    __shared__ float lane_sum[8][32];
    const int col = blockIdx.x;
    const int di = col >> 5, dj = (col & 31) >> 2, c = col & 3;
    if (di >= KH || dj >= KW || c >= C) return;   // padding slot (uniform over the block)
    const int r = threadIdx.x & 31, l = threadIdx.x >> 5;
    const int o = blockIdx.y * 32 + r;
    const int mt = o / BM, row = o % BM;
    float acc = 0.f;
    if (o < O) {
        const float* src = partial + ((size_t)mt * parts * bn + col) * BM + row;
        for (int sidx = l; sidx < parts; sidx += 8) acc = __fadd_rn(acc, __ldcg(src + (size_t)sidx * bn * BM));
    }
    lane_sum[l][r] = acc;
    __syncthreads();
    if (l == 0 && o < O) {
        float t = lane_sum[0][r];
#pragma unroll
        for (int q = 1; q < 8; ++q) t = __fadd_rn(t, lane_sum[q][r]);
        dk[((size_t)(di * KW + dj) * C + c) * O + o] = t;
    }
}

// ---- narrow-channel layers (<= 4 input channels: the RGB end of both networks) -------------------
// A 3-channel NHWC pixel is 12 bytes, which TMA cannot address (16-byte granularity), and a K of
// 3 per tap would waste the tensor core.  Such an input is first copied into a zero-bordered
// 4-channel image xp[n][h + pad_top][w + pad_left][4]; in that image the five taps of one kernel
// row that output pixel (i, j) needs are 32 CONTIGUOUS floats (8 pixels x 4 channels, the last 3
// pixels unused) starting at xp[n][s*i + di][s*j][0].  A tensor map whose pixel stride (s*16 bytes)
// is smaller than its 128-byte inner extent hands these overlapping windows to TMA directly, so a
// whole kernel row becomes one K = 32 step: FWD contracts it against the row's weights repacked as
// k4[di][4*dj + c][o]; DK contracts the window against dy over pixels and scatters the 32 slots
// back to dk[di][dj][c][o].
__global__ void __launch_bounds__(256)
repack_narrow_kernel(const float* __restrict__ x, float4* __restrict__ xp, int N, int H, int W, int C,
                     int Hp, int Wp, int pt, int pl)
{
    pdl_enter();
    const size_t total = (size_t)N * Hp * Wp;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int wp = (int)(i % Wp);
        const int hp = (int)((i / Wp) % Hp);
        const int n = (int)(i / ((size_t)Wp * Hp));
        const int h = hp - pt, w = wp - pl;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (h >= 0 && h < H && w >= 0 && w < W) {
            const float* src = x + (((size_t)n * H + h) * W + w) * C;
            for (int c = 0; c < C; ++c) v[c] = __ldg(src + c);
        }
        xp[i] = make_float4(v[0], v[1], v[2], v[3]);
    }
}

// Both repacks of a narrow-channel forward in one launch: blocks [0, gridDim.x - k4_blocks) build
// the padded 4-channel image, the last k4_blocks blocks the weights k4 [KH][32][O] (row 4*dj + c).
__global__ void __launch_bounds__(256)
repack_narrow_k4_kernel(const float* __restrict__ x, float4* __restrict__ xp, int N, int H, int W, int C,
                        int Hp, int Wp, int pt, int pl, const float* __restrict__ k, float* __restrict__ k4,
                        int KH, int KW, int O, int k4_blocks)
{
    pdl_enter();
    const int x_blocks = (int)gridDim.x - k4_blocks;
    if ((int)blockIdx.x >= x_blocks) {
        const int total = KH * 32 * O;
        for (int i = ((int)blockIdx.x - x_blocks) * blockDim.x + threadIdx.x; i < total; i += k4_blocks * blockDim.x) {
            const int o = i % O, slot = (i / O) % 32, di = i / (O * 32);
            const int dj = slot >> 2, c = slot & 3;
            k4[i] = (dj < KW && c < C) ? __ldg(k + (((size_t)di * KW + dj) * C + c) * O + o) : 0.f;
        }
        return;
    }
    const size_t total = (size_t)N * Hp * Wp;
    const size_t stride = (size_t)x_blocks * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int wp = (int)(i % Wp);
        const int hp = (int)((i / Wp) % Hp);
        const int n = (int)(i / ((size_t)Wp * Hp));
        const int h = hp - pt, w = wp - pl;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (h >= 0 && h < H && w >= 0 && w < W) {
            const float* src = x + (((size_t)n * H + h) * W + w) * C;
            for (int c = 0; c < C; ++c) v[c] = __ldg(src + c);
        }
        xp[i] = make_float4(v[0], v[1], v[2], v[3]);
    }
}

// ---- input gradient of a narrow-channel layer (<= 4 input channels) -------------------------------
// With C <= 4 the implicit GEMM of DX has N = C: every 128 x 32 tile of dy would be fetched for a
// sliver of tensor work, once per tap.  Instead dy is read ONCE by a plain GEMM against all taps,
//   ycol[tap][pixel of dy][c] = sum_o dy[pixel, o] * k[tap, c, o]      (N = 4 * KH*KW, padded to 32s)
// - the FWD kernel on a 1x1 "convolution" with the weights transposed to k2[o][4 * tap + c] - and a
// gather ("col2im") then adds, for every input pixel, the <= ceil(KH/s)*ceil(KW/s) products that
// land on it and applies the fused chain.
__global__ void __launch_bounds__(256)
repack_k2_kernel(const float* __restrict__ k, float* __restrict__ k2, int taps, int C, int Jp, int O)
{
    pdl_enter();
    const int total = O * Jp;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int j = i % Jp, o = i / Jp;
        const int tap = j >> 2, c = j & 3;   // four columns per tap, channels beyond C are zero
        k2[i] = (tap < taps && c < C) ? __ldg(k + ((size_t)tap * C + c) * O + o) : 0.f;
    }
}

// ycol is stored tap-major, [tap][pixel of dy][4 channels]: the threads of a warp walk adjacent
// pixels, so their 16-byte reads of one tap's plane are contiguous.  One thread per output pixel.
// KH_, KW_, S_ > 0 fix kernel extent and stride at compile time (the DCGAN layers: 5, 5, 2): the tap
// loops unroll, the divisions turn into shifts and all loads of a pixel are in flight together.
template <int KH_, int KW_, int S_>
__global__ void __launch_bounds__(256)
col2im_kernel(const float4* __restrict__ ycol, float* __restrict__ out, int N, int H, int W, int C, int Ho, int Wo,
              int KHr, int KWr, int shr, int swr, int pt, int pl, const EpilogueArgs ep)
{
    pdl_enter();
    const int KH = KH_ > 0 ? KH_ : KHr, KW = KW_ > 0 ? KW_ : KWr, sh = S_ > 0 ? S_ : shr, sw = S_ > 0 ? S_ : swr;
    const size_t total = (size_t)N * H * W;
    const size_t pixels = (size_t)N * Ho * Wo;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t pix = (size_t)blockIdx.x * blockDim.x + threadIdx.x; pix < total; pix += stride) {
        const int w = (int)(pix % W);
        const int h = (int)((pix / W) % H);
        const int n = (int)(pix / ((size_t)W * H));
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        const int di0 = (h + pt) % sh, dj0 = (w + pl) % sw;
        const float4* img = ycol + (size_t)n * Ho * Wo;
        if constexpr (KH_ > 0) {
            // all candidate taps of this pixel's parity class, loads first (zero where the tap falls outside)
            constexpr int SS = S_ > 0 ? S_ : 1;
            constexpr int TH = (KH_ + SS - 1) / SS, TW = (KW_ + SS - 1) / SS;
            float4 v[TH * TW];
#pragma unroll
            for (int a = 0; a < TH; ++a) {
                const int di = di0 + a * S_;
                const int hh = h + pt - di;
                const int i = hh / S_;
                const bool row_ok = di < KH_ && hh >= 0 && i < Ho;
#pragma unroll
                for (int b = 0; b < TW; ++b) {
                    const int dj = dj0 + b * S_;
                    const int ww = w + pl - dj;
                    const int j = ww / S_;
                    const bool ok = row_ok && dj < KW_ && ww >= 0 && j < Wo;
                    v[a * TW + b] = ok ? __ldg(img + (size_t)(di * KW_ + dj) * pixels + (size_t)i * Wo + j)
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            // same order as the run-time form: kernel rows ascending, columns ascending (absent taps add +0)
#pragma unroll
            for (int q = 0; q < TH * TW; ++q) {
                acc[0] = __fadd_rn(acc[0], v[q].x); acc[1] = __fadd_rn(acc[1], v[q].y);
                acc[2] = __fadd_rn(acc[2], v[q].z); acc[3] = __fadd_rn(acc[3], v[q].w);
            }
        } else {
            for (int di = di0; di < KH; di += sh) {      // taps whose row parity matches
                if (h + pt - di < 0) break;
                const int i = (h + pt - di) / sh;
                if (i >= Ho) continue;
                for (int dj = dj0; dj < KW; dj += sw) {
                    if (w + pl - dj < 0) break;
                    const int j = (w + pl - dj) / sw;
                    if (j >= Wo) continue;
                    const float4 v = __ldg(img + (size_t)(di * KW + dj) * pixels + (size_t)i * Wo + j);
                    acc[0] = __fadd_rn(acc[0], v.x); acc[1] = __fadd_rn(acc[1], v.y);
                    acc[2] = __fadd_rn(acc[2], v.z); acc[3] = __fadd_rn(acc[3], v.w);
                }
            }
        }
        for (int c = 0; c < C; ++c) {
            const size_t idx = pix * C + c;
            out[idx] = epilogue_apply(ep, acc[c], idx, c);
        }
    }
}

}  // namespace
}  // namespace dcg
