// conv_dx3_kernel: input gradient of a <= 4-channel layer, GEMM and gather in one persistent kernel.  Included by
// conv_tc.cu only.
#pragma once

namespace dcg {
namespace {

// ---- input gradient of a <= 4-channel layer: GEMM and gather in one persistent kernel -----------------
// dx[n, h, w, c] = sum over the taps of matching parity of ycol[tap][n, i, j][c], where ycol = dy x k^T is
// the plain GEMM of every dy pixel against all taps (N = 4 columns per tap).  Written to memory, ycol is
// 100 floats per dy pixel - 26 MB at batch 64 for a 3 MB result - and the gather is a second launch.
// Here a CTA owns 2R output rows of one image: it runs the GEMM for the R + 2 dy rows that contribute to
// them (two 128-pixel M tiles = 8 rows of 32 pixels, so the rows at the seams are computed twice), parks
// the products in shared memory as [tap][dy pixel][4] and gathers its own output pixels from there, fused
// chain included.  Nothing but dy, the weights and dx touches memory, and it is one launch.  Persistent:
// a CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...; the weights stay resident (read from k
// itself, K-major rows 4 * tap + c), the dy tiles of the next tile stream in and its MMAs run while this
// tile is being gathered (one TMEM accumulator per M tile, handed back as soon as it is in shared memory).
struct Dx3Args {
    int R;            // dy rows owned per tile (2R output rows)
    int lo;           // first dy row a tile needs, relative to its first owned row (<= 0)
    int tiles_per_img, tiles;
};
constexpr int kDx3Rows = 8;                               // dy rows per tile (two M tiles of 4 rows x 32 pixels)
constexpr int kDx3Stages = 4;
constexpr int kDx3Epi = 512;                              // epilogue threads: 16 warps, four per TMEM lane quadrant (one 32-column slab each)
constexpr int kDx3Threads = 64 + kDx3Epi;
constexpr int kDx3YcolBytes = 32 * kDx3Rows * 32 * 16;    // up to 32 taps x 256 dy pixels x 4 floats

template <int KH_, int KW_>   // 5, 5: tap loops unrolled, all loads of a pixel in flight; 0, 0: any kernel size
__global__ void __launch_bounds__(kDx3Threads, 1)
conv_dx3_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ Params p, const __grid_constant__ Dx3Args g)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem0 = smem_u32(smem_raw);
    const uint32_t b_res = (smem0 + 1023u) & ~1023u;
    const long long wait_limit = p.wait_cycles;
    const int ksteps = p.kchunks;
    const uint32_t b_bytes = 128u * BK * 4;                       // 128 rows (4 * tap + c) x 32 output channels
    const uint32_t ring = b_res + (uint32_t)ksteps * b_bytes;
    const uint32_t ycol_base = ring + (uint32_t)kDx3Stages * A_STAGE_BYTES;
    const int ntaps = p.KH * p.KW;
    const uint32_t bar_base = ycol_base + (uint32_t)ntaps * (kDx3Rows * 32 * 16);
    const uint32_t full_bar = bar_base;                           // [kDx3Stages]
    const uint32_t empty_bar = bar_base + 8u * kDx3Stages;        // [kDx3Stages]
    const uint32_t b_bar = bar_base + 16u * kDx3Stages;
    const uint32_t acc_full = b_bar + 8u;                         // [2] one per M tile
    const uint32_t acc_empty = acc_full + 16u;                    // [2]
    const uint32_t tmem_slot = acc_empty + 16u;
    uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem0));
    const float4* ycol = reinterpret_cast<const float4*>(smem_raw + (ycol_base - smem0));
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kDx3Stages; ++s) {
            mbar_init(full_bar + 8u * s, 1);
            mbar_init(empty_bar + 8u * s, 1);
        }
        mbar_init(b_bar, 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full + 8u * b, 1);
            mbar_init(acc_empty + 8u * b, kDx3Epi / 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    }
    constexpr int tmem_cols = 256;
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot_ptr;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        // ===== producer: the weights once; per tile two M tiles (4 dy rows x 32 pixels each) x the channel chunks =====
        if (elect_one()) {
            mbar_expect_tx(b_bar, (uint32_t)ksteps * b_bytes);
            for (int q = 0; q < ksteps; ++q) tma_load_3d(b_res + (uint32_t)q * b_bytes, &map_b, b_bar, q * BK, 0, 0);
        }
        int s = 0, it = 0;
        uint32_t phase = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < g.tiles && alive; tile += gridDim.x) {
            const int n = tile / g.tiles_per_img, t = tile - n * g.tiles_per_img;
            const int i_base = g.R * t + g.lo;
            for (int mt = 0; mt < 2 && alive; ++mt)
                for (int q = 0; q < ksteps; ++q, ++it) {
                    if (!mbar_wait_warp(empty_bar + 8u * s, phase ^ 1u, 0, it, wait_limit)) { alive = false; break; }
                    if (elect_one()) {
                        const uint32_t fb = full_bar + 8u * s;
                        mbar_expect_tx(fb, (uint32_t)A_STAGE_BYTES);
                        tma_load_4d(ring + (uint32_t)s * A_STAGE_BYTES, &map_a, fb, q * BK, 0, i_base + 4 * mt, n);
                    }
                    if (++s == kDx3Stages) { s = 0; phase ^= 1u; }
                }
        }
    } else if (warp == 1) {
        // ===== MMA issuer: both operands K-major =====
        const uint32_t idesc = make_idesc(0, 0, 128, BM);
        const uint64_t adesc0 = make_smem_desc(ring, 16u, 1024u, kLayoutSw128);
        const uint64_t bdesc0 = make_smem_desc(b_res, 16u, 1024u, kLayoutSw128);
        int s = 0, it = 0, n = 0;
        uint32_t phase = 0;
        bool alive = mbar_wait_warp(b_bar, 0, 1, -1, wait_limit);
        for (int tile = blockIdx.x; tile < g.tiles && alive; tile += gridDim.x, ++n) {
            for (int mt = 0; mt < 2 && alive; ++mt) {
                // the epilogue has copied this accumulator's previous tile to shared memory (first tile: passes at once)
                if (!mbar_wait_warp(acc_empty + 8u * mt, ((uint32_t)n & 1u) ^ 1u, 1, it, wait_limit)) { alive = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int q = 0; q < ksteps; ++q, ++it) {
                    if (!mbar_wait_warp(full_bar + 8u * s, phase, 1, it, wait_limit)) { alive = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (elect_one()) {
                        const uint64_t adesc = adesc0 + (uint64_t)((uint32_t)s * (A_STAGE_BYTES >> 4));
                        const uint64_t bdesc = bdesc0 + (uint64_t)((uint32_t)q * (b_bytes >> 4));
#pragma unroll
                        for (int kk = 0; kk < BK / 8; ++kk)
                            tcgen05_mma_tf32(tmem_d + (uint32_t)(mt * 128), adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc,
                                             (q > 0 || kk > 0) ? 1u : 0u);
                        tcgen05_commit(empty_bar + 8u * s);
                    }
                    if (++s == kDx3Stages) { s = 0; phase ^= 1u; }
                }
                if (elect_one()) tcgen05_commit(acc_full + 8u * mt);   // complete, or abandoned
            }
        }
    } else {
        // ===== epilogue: accumulators -> shared memory [tap][dy pixel][4], then gather the tile's own output pixels =====
        const int quad = warp & 3;
        const int row = quad * 32 + lane;                // dy pixel of the M tile: 32 * (row of the tile) + column
        const int slab = (warp - 2) >> 2;                // the four warps of a lane quadrant take one 32-column slab each
        const int tid_e = threadIdx.x - 64;
        const EpilogueArgs& e = p.ep;
        const int W = p.W, own = 2 * g.R * W;            // output pixels a tile owns
        int n_it = 0;
        for (int tile = blockIdx.x; tile < g.tiles; tile += gridDim.x, ++n_it) {
            const int n = tile / g.tiles_per_img, t = tile - n * g.tiles_per_img;
            const int i_base = g.R * t + g.lo;
            bool ok = true;
            for (int mt = 0; mt < 2; ++mt) {
                bool got = mbar_wait(acc_full + 8u * mt, (uint32_t)n_it & 1u, 2, n_it, wait_limit);
                got = __all_sync(0xffffffffu, got);
                ok = ok && got;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                {
                    const int c0 = slab * 32;
                    if (c0 < 4 * ntaps) {
                        uint32_t r[32];
                        tmem_ld_32x32b_x32(tmem_d + ((uint32_t)(quad * 32) << 16) + (uint32_t)(mt * 128 + c0), r);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const int tap = (c0 >> 2) + q;
                            if (tap < ntaps) {
                                const uint32_t addr = ycol_base + (uint32_t)(((tap * kDx3Rows * 32) + mt * 128 + row) * 16);
                                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(__uint_as_float(r[4 * q])),
                                             "f"(__uint_as_float(r[4 * q + 1])), "f"(__uint_as_float(r[4 * q + 2])),
                                             "f"(__uint_as_float(r[4 * q + 3])) : "memory");
                            }
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty + 8u * mt) : "memory");
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kDx3Epi) : "memory");
            // gather: consecutive threads take consecutive output pixels of the tile's 2R rows
            for (int px = tid_e; px < own; px += kDx3Epi) {
                const int hl = px / W, w = px - hl * W;
                const int h = 2 * g.R * t + hl;
                if (h >= p.H || !ok) continue;
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                const int di0 = (h + p.pt) & 1, dj0 = (w + p.pl) & 1;   // kernel rows / columns of matching parity, ascending
                if constexpr (KH_ > 0) {
                    constexpr int TH = (KH_ + 1) / 2, TW = (KW_ + 1) / 2;
                    float4 v[TH * TW];
#pragma unroll
                    for (int a = 0; a < TH; ++a) {
                        const int di = di0 + 2 * a;
                        const int hh = h + p.pt - di;
                        const int i = hh >> 1;
                        const bool row_ok = di < KH_ && hh >= 0 && i < p.Ho;
#pragma unroll
                        for (int b = 0; b < TW; ++b) {
                            const int dj = dj0 + 2 * b;
                            const int ww = w + p.pl - dj;
                            const int j = ww >> 1;
                            const bool in = row_ok && dj < KW_ && ww >= 0 && j < p.Wo;
                            v[a * TW + b] = in ? ycol[((di * KW_ + dj) * kDx3Rows + (i - i_base)) * 32 + j]
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    }
#pragma unroll
                    for (int q = 0; q < TH * TW; ++q) {
                        acc[0] = __fadd_rn(acc[0], v[q].x); acc[1] = __fadd_rn(acc[1], v[q].y);
                        acc[2] = __fadd_rn(acc[2], v[q].z); acc[3] = __fadd_rn(acc[3], v[q].w);
                    }
                } else {
                    for (int di = di0; di < p.KH; di += 2) {
                        const int i = (h + p.pt - di) >> 1;
                        if (h + p.pt - di < 0 || i >= p.Ho) continue;
                        const int rl = i - i_base;
                        for (int dj = dj0; dj < p.KW; dj += 2) {
                            const int j = (w + p.pl - dj) >> 1;
                            if (w + p.pl - dj < 0 || j >= p.Wo) continue;
                            const float4 v = ycol[((di * p.KW + dj) * kDx3Rows + rl) * 32 + j];
                            acc[0] = __fadd_rn(acc[0], v.x); acc[1] = __fadd_rn(acc[1], v.y);
                            acc[2] = __fadd_rn(acc[2], v.z); acc[3] = __fadd_rn(acc[3], v.w);
                        }
                    }
                }
                const size_t pix = ((size_t)n * p.H + h) * W + w;
                for (int c = 0; c < p.C; ++c) {
                    const size_t idx = pix * p.C + c;
                    p.out[idx] = epilogue_apply(e, acc[c], idx, c);
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kDx3Epi) : "memory");   // the products are consumed: the next tile may overwrite them
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(tmem_cols) : "memory");
    }
}

}  // namespace
}  // namespace dcg
