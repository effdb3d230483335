// conv_fwd_short_kernel: the short-K forward GEMMs of the 3-channel layers as persistent CTAs.  Included by conv_tc.cu only.
#pragma once

namespace dcg {
namespace {

// ---- short-K forward GEMMs as persistent CTAs ---------------------------------------------------------
// The two tensor-core launches of the 3-channel layers have almost no K: the forward contracts five
// 32-float row windows per tile (A through the overlapping-window map, B = k4), the GEMM of the input
// gradient two 32-channel chunks (a 1x1 convolution of dy against all taps, result in quad planes).
// With one tile per CTA such a CTA spends its life on set-up, pipeline fill and epilogue (2-5 stages
// of work against ~3 us of fixed cost) and fetches the same weights again for every tile.  Here a
// CTA (two per SM) walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...: the weights are loaded once and stay
// in shared memory, the A tiles of the next tiles stream through a ring while the tensor core works
// on this one, and the accumulator is double-buffered in TMEM so that the epilogue of tile i
// runs under the MMAs of tile i + 1.  The GEMM's result goes out straight from registers (thread = pixel
// row, and in the quad-plane layout consecutive pixels are consecutive 16-byte words); the forward's NHWC
// rows go through a small per-warp patch of shared memory (32 rows x 16 columns) so that every store
// instruction covers whole 64-byte row pieces.
constexpr int kShortMaxStages = 4;         // A ring depth (16 KB each): 4 for the GEMM, 3 next to the forward's patches
constexpr int kShortMaxB = 40 * 1024;      // resident weights
constexpr int kPatchPitch = 20;            // floats per patch row (16 columns + 4: keeps 16-byte alignment)
constexpr int kPatchBytes = 32 * kPatchPitch * 4;

template <bool NARROW>
__global__ void __launch_bounds__(kThreads, 2)
conv_fwd_short_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ Params p, const int tiles, const int ksteps)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem0 = smem_u32(smem_raw);
    const uint32_t b_res = (smem0 + 1023u) & ~1023u;
    const long long wait_limit = p.wait_cycles;
    const uint32_t b_bytes = (uint32_t)p.bn * BK * 4;
    const uint32_t ring = b_res + (uint32_t)ksteps * b_bytes;
    const int kShortStages = p.stages;
    const uint32_t patch_base = ring + (uint32_t)kShortStages * A_STAGE_BYTES;   // NARROW: one patch per epilogue warp
    const uint32_t bar_base = patch_base + (NARROW ? (uint32_t)(kEpi / 32) * kPatchBytes : 0u);
    const uint32_t full_bar = bar_base;                          // [kShortMaxStages]
    const uint32_t empty_bar = bar_base + 8u * kShortMaxStages;  // [kShortMaxStages]
    const uint32_t b_bar = bar_base + 16u * kShortMaxStages;     // weights have landed
    const uint32_t acc_full = b_bar + 8u;                        // [2] accumulator buffer complete
    const uint32_t acc_empty = acc_full + 16u;                   // [2] accumulator buffer drained (8 epilogue warps)
    const uint32_t tmem_slot = acc_empty + 16u;
    uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem0));
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kShortStages; ++s) {
            mbar_init(full_bar + 8u * s, 1);
            mbar_init(empty_bar + 8u * s, 1);
        }
        mbar_init(b_bar, 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full + 8u * b, 1);
            mbar_init(acc_empty + 8u * b, kEpi / 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    }
    int tmem_cols = 32;
    while (tmem_cols < 2 * p.bn) tmem_cols <<= 1;
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
    const int per_image = p.tiles_w * p.tiles_h;

    if (warp == 0) {
        // ===== producer: the weights once, then the A tiles of every tile of this CTA =====
        if (elect_one()) {
            mbar_expect_tx(b_bar, (uint32_t)ksteps * b_bytes);
            for (int q = 0; q < ksteps; ++q) {
                if (NARROW) tma_load_4d(b_res + (uint32_t)q * b_bytes, &map_b, b_bar, 0, 0, q, 0);
                else if (p.b_direct) tma_load_3d(b_res + (uint32_t)q * b_bytes, &map_b, b_bar, q * BK, 0, 0);
                else tma_load_4d(b_res + (uint32_t)q * b_bytes, &map_b, b_bar, 0, q * BK, 0, 0);
            }
        }
        int s = 0, it = 0;
        uint32_t phase = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
            const int j0 = (tile % p.tiles_w) * p.TW;
            const int i0 = ((tile / p.tiles_w) % p.tiles_h) * p.TH;
            const int n0 = (tile / per_image) * p.TN;
            for (int q = 0; q < ksteps; ++q, ++it) {
                if (!mbar_wait_warp(empty_bar + 8u * s, phase ^ 1u, 0, it, wait_limit)) { alive = false; break; }
                if (elect_one()) {
                    const uint32_t fb = full_bar + 8u * s;
                    const uint32_t dst = ring + (uint32_t)s * A_STAGE_BYTES;
                    mbar_expect_tx(fb, (uint32_t)A_STAGE_BYTES);
                    if (NARROW) tma_load_5d(dst, &map_a, fb, 0, j0, i0, n0, q);
                    else tma_load_4d(dst, &map_a, fb, q * BK, j0, i0, n0);
                }
                if (++s == kShortStages) { s = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer: A K-major, B MN-major (chunks of 32 columns 4096 B apart, 4-row groups 512 B apart) =====
        // B: MN-major (chunks of 32 columns 4096 B apart, 4-row groups 512 B apart, 8 k rows per MMA = 1024 B), or -
        // read from k directly - K-major like A (128-byte rows, 32 bytes per MMA)
        const bool bk = !NARROW && p.b_direct;
        const uint32_t idesc = make_idesc(0, bk ? 0 : 1, p.bn, BM);
        const uint64_t adesc0 = make_smem_desc(ring, 16u, 1024u, kLayoutSw128);
        const uint64_t bdesc0 = bk ? make_smem_desc(b_res, 16u, 1024u, kLayoutSw128)
                                   : make_smem_desc(b_res, 4096u, 512u, kLayoutSw128Base32);
        const uint32_t b_kstep = bk ? 2u : 64u;
        int s = 0, it = 0, n = 0;
        uint32_t phase = 0;
        bool alive = mbar_wait_warp(b_bar, 0, 1, -1, wait_limit);
        for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x, ++n) {
            const int buf = n & 1;
            // the epilogue has drained this buffer's previous tile (first use: passes at once)
            if (!mbar_wait_warp(acc_empty + 8u * buf, ((uint32_t)(n >> 1) & 1u) ^ 1u, 1, it, wait_limit)) { alive = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int q = 0; q < ksteps; ++q, ++it) {
                if (!mbar_wait_warp(full_bar + 8u * s, phase, 1, it, wait_limit)) { alive = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (elect_one()) {
                    const uint64_t adesc = adesc0 + (uint64_t)((uint32_t)s * (A_STAGE_BYTES >> 4));
                    const uint64_t bdesc = bdesc0 + (uint64_t)((uint32_t)q * (b_bytes >> 4));
#pragma unroll
                    for (int kk = 0; kk < BK / 8; ++kk)
                        tcgen05_mma_tf32(tmem_d + (uint32_t)(buf * p.bn), adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * b_kstep), idesc,
                                         (q > 0 || kk > 0) ? 1u : 0u);
                    tcgen05_commit(empty_bar + 8u * s);
                }
                if (++s == kShortStages) { s = 0; phase ^= 1u; }
            }
            if (elect_one()) tcgen05_commit(acc_full + 8u * buf);   // complete, or abandoned
        }
    } else {
        // ===== epilogue: thread = accumulator row; the two warps of a lane quadrant take alternate 32-column slabs =====
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int tw = row % p.TW, th = (row / p.TW) % p.TH, tn = row / (p.TW * p.TH);
        const EpilogueArgs& e = p.ep;
        const int ncols = p.o_store ? p.o_store : p.O;
        int n = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++n) {
            const int buf = n & 1;
            const int j = (tile % p.tiles_w) * p.TW + tw;
            const int i = ((tile / p.tiles_w) % p.tiles_h) * p.TH + th;
            const int img = (tile / per_image) * p.TN + tn;
            bool ok = mbar_wait(acc_full + 8u * buf, (uint32_t)(n >> 1) & 1u, 2, n, wait_limit);
            ok = __all_sync(0xffffffffu, ok);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool valid = ok && img < p.N && i < p.Ho && j < p.Wo;
            const unsigned long long pix = ((unsigned long long)img * p.Ho + i) * p.Wo + j;
            const int first = (warp - 2) >> 2, nslabs = (p.bn + 31) >> 5;
            for (int sl = first; sl < nslabs; sl += 2) {
                const int c0 = sl * 32;
                uint32_t r[32];
                const uint32_t taddr = tmem_d + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * p.bn + c0);
                const bool full = p.bn - c0 >= 32;
                if (full) tmem_ld_32x32b_x32(taddr, r);
                else tmem_ld_32x32b_x16(taddr, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (sl + 2 >= nslabs) {   // this warp's last read of the buffer: hand it back to the MMA warp
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty + 8u * buf) : "memory");
                }
                if (NARROW) {
                    // 16 columns at a time through this warp's patch: written by rows (lane = row), read back with four
                    // lanes per row, so that a store instruction covers eight 64-byte row pieces
                    float* patch = reinterpret_cast<float*>(smem_raw + (patch_base - smem0)) + (warp - 2) * (kPatchBytes / 4);
                    const long long my_off = valid ? (long long)(pix * (unsigned long long)p.O) : -1;
#pragma unroll
                    for (int hs = 0; hs < 2; ++hs) {
                        if (hs == 1 && !full) break;
                        __syncwarp();
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4)
                            *reinterpret_cast<float4*>(patch + lane * kPatchPitch + 4 * q4) =
                                make_float4(__uint_as_float(r[16 * hs + 4 * q4]), __uint_as_float(r[16 * hs + 4 * q4 + 1]),
                                            __uint_as_float(r[16 * hs + 4 * q4 + 2]), __uint_as_float(r[16 * hs + 4 * q4 + 3]));
                        __syncwarp();
                        float4 acc[4];
                        long long goff[4];
                        int ch[4];
                        const int col = c0 + 16 * hs + 4 * (lane & 3);
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int rl = u * 8 + (lane >> 2);
                            const long long ro = __shfl_sync(0xffffffffu, my_off, rl);
                            acc[u] = *reinterpret_cast<const float4*>(patch + rl * kPatchPitch + 4 * (lane & 3));
                            const bool in = ro >= 0 && col < ncols;
                            goff[u] = in ? ro + col : -1;
                            ch[u] = in ? col : 0;
                        }
                        cf_chain_store4(e, p.out, acc, goff, ch);
                    }
                } else {
#pragma unroll
                    for (int g = 0; g < 2; ++g) {   // four 16-byte column quads at a time; consecutive pixels are consecutive words
                        float4 acc[4];
                        long long goff[4];
                        int ch[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int q4 = g * 4 + u;
                            const int col = c0 + 4 * q4;
                            acc[u] = make_float4(__uint_as_float(r[4 * q4]), __uint_as_float(r[4 * q4 + 1]),
                                                 __uint_as_float(r[4 * q4 + 2]), __uint_as_float(r[4 * q4 + 3]));
                            const bool in = valid && (q4 < 4 || full) && col < ncols;
                            goff[u] = in ? (long long)(pix * 4ull + (unsigned long long)(col >> 2) * p.plane_stride) : -1;
                            ch[u] = in ? col : 0;
                        }
                        cf_chain_store4(e, p.out, acc, goff, ch);
                    }
                }
            }
            if (nslabs <= first) {   // a warp without a slab still has to hand the buffer back
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty + 8u * buf) : "memory");
            }
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
