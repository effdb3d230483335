// conv_tc_kernel<MODE, X3>: the general tcgen05 implicit-GEMM convolution kernel (forward, input gradient by parity
// class, kernel gradient; TF32 and 3xTF32).  Included by conv_tc.cu only.
#pragma once

namespace dcg {
namespace {

// ---- the kernel ---------------------------------------------------------------------------------
template <int MODE, bool X3>
__global__ void __launch_bounds__(kThreads, X3 ? 1 : 2)
conv_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ Params p)
{
    extern __shared__ uint8_t smem_raw[];
    if (threadIdx.x == 64) TC_TRACE(3072);
    TC_CTA_TRACE(0);
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int b_stage_bytes = p.bn * BK * 4;
    const long long wait_limit = p.wait_cycles;
    const uint32_t a_base = smem_base;
    const uint32_t b_base = a_base + (uint32_t)p.stages * A_STAGE_BYTES;
    // 3xTF32: residual tiles (operand minus its TF32 part) of every stage follow the operand tiles
    const uint32_t as_base = b_base + (uint32_t)p.stages * b_stage_bytes;
    const uint32_t bs_base = as_base + (uint32_t)p.stages * A_STAGE_BYTES;
    const uint32_t bar_base = X3 ? bs_base + (uint32_t)p.stages * b_stage_bytes : as_base;
    // barriers: full[stages], empty[stages], tmem_full; then the TMEM base address word
    const uint32_t full_bar = bar_base;
    const uint32_t empty_bar = bar_base + 8u * p.stages;
    const uint32_t resid_bar = bar_base + 16u * p.stages;     // 3xTF32: residual tiles of the stage are written
    const uint32_t tmem_full_bar = bar_base + 24u * p.stages;
    const uint32_t tmem_slot = tmem_full_bar + 8u;
    uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;

    // ---- one-time setup (first: thread 0 and warp 1 are busy with it while everyone decodes) ---------
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(full_bar + 8u * s, 1);
            mbar_init(empty_bar + 8u * s, 1);
            mbar_init(resid_bar + 8u * s, kEpi);
        }
        mbar_init(tmem_full_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    }
    // 3xTF32 keeps the two small cross terms in an accumulator of their own (columns bn .. 2*bn): the
    // tensor core rounds its accumulator toward zero at every step, an error that grows with the
    // number of steps and with the accumulator's size, so the long chain of large terms is kept as
    // short as in the plain TF32 kernel and the small terms round among themselves
    int tmem_cols = 32;
    while (tmem_cols < (X3 ? 2 * p.bn : p.bn)) tmem_cols <<= 1;
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    // ---- decode this CTA's work item -------------------------------------------------------------
    // blockIdx.x = ((group * m_count + m) * n_tiles + n) * splits + split, where group is the parity
    // class (DX), the kernel tap (DK) or absent (FWD), and m a pixel tile (FWD/DX) or channel tile (DK).
    int rem = blockIdx.x;
    const int split = rem % p.splits; rem /= p.splits;
    const int n_tile = rem % p.n_tiles; rem /= p.n_tiles;
    int m_count;
    if (MODE == MODE_DK) m_count = p.m_tiles;
    else m_count = p.tiles_w * p.tiles_h * p.tiles_n;
    const int m_tile = rem % m_count;
    const int group = rem / m_count;

    // pixel-tile origin (FWD/DX)
    int j0 = 0, i0 = 0, n0 = 0;
    if (MODE != MODE_DK) {
        j0 = (m_tile % p.tiles_w) * p.TW;
        i0 = ((m_tile / p.tiles_w) % p.tiles_h) * p.TH;
        n0 = (m_tile / (p.tiles_w * p.tiles_h)) * p.TN;
    }
    // DX: parity class and its taps; DK: the kernel tap
    int ph = 0, pw = 0, rh = 0, rw = 0, eh = 0, ew = 0, taps_h = 1, taps_w = 1, tap_di = 0, tap_dj = 0;
    if (MODE == MODE_DX) {
        ph = group / p.sw; pw = group % p.sw;
        rh = (ph + p.pt) % p.sh; rw = (pw + p.pl) % p.sw;
        eh = (ph + p.pt) / p.sh; ew = (pw + p.pl) / p.sw;
        taps_h = rh < p.KH ? (p.KH - rh + p.sh - 1) / p.sh : 0;
        taps_w = rw < p.KW ? (p.KW - rw + p.sw - 1) / p.sw : 0;
    } else if (MODE == MODE_DK) {
        if (p.narrow) { tap_di = 0; tap_dj = 0; }   // one tile holds every tap: 32 window slots per kernel row
        else { tap_di = group / p.KW; tap_dj = group % p.KW; }
    }
    // K-stage range of this split
    int total_stages;
    if (MODE == MODE_FWD) total_stages = p.narrow ? p.KH : p.KH * p.KW * p.kchunks;
    else if (MODE == MODE_DX) total_stages = taps_h * taps_w * p.kchunks;
    else total_stages = p.tiles_w * p.tiles_h * p.tiles_n;
    const int q0 = (int)((long long)total_stages * split / p.splits);
    const int q1 = (int)((long long)total_stages * (split + 1) / p.splits);
    const int nq = q1 - q0;

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot_ptr;
    // Programmatic dependent launch: everything above (barriers, TMEM, descriptor prefetch) may run
    // while the previous kernel of the stream is still draining; from here on its results are needed.
    // The next kernel's CTAs may in turn be set up as soon as every CTA of this grid has got here.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 64) TC_TRACE(3073);
    TC_CTA_TRACE(1);
#ifdef DCG_TC_TRACING
    if ((p.debug & 8) && threadIdx.x == 64 && blockIdx.x < 1024) {
        unsigned smid;
        asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
        g_tc_cta_trace[blockIdx.x][6] = smid;
    }
#endif

    // ---- epilogue geometry (uniform over the CTA) ---------------------------------------------------
    const int ch0 = n_tile * p.bn;    // channel index of accumulator column 0 (bias axis) unless DK
    int ncols_valid;                  // valid columns in this N tile
    long long col_stride = 1;         // element stride between accumulator columns in the output
    if (MODE == MODE_FWD) ncols_valid = min(p.bn, (p.o_store ? p.o_store : p.O) - ch0);
    else if (MODE == MODE_DX) ncols_valid = min(p.bn, p.C - ch0);
    else if (p.narrow) { ncols_valid = 32 * p.KH; col_stride = p.O; }
    else if (!p.swap) ncols_valid = min(p.bn, p.O - ch0);
    else { ncols_valid = min(p.bn, p.C - ch0); col_stride = p.O; }
    // Row-contiguous outputs whose channel count allows 16-byte stores take the vector path.
    const int ch_total = (MODE == MODE_DX) ? p.C : p.O;
    const bool vec = col_stride == 1 && (ch_total & 3) == 0 && (ncols_valid & 3) == 0;
    float* red = reinterpret_cast<float*>(smem_raw + (a_base - smem_u32(smem_raw)));
    long long* s_rowoff = reinterpret_cast<long long*>(red + kRedFloats(p.bn));

    if (warp == 0) {
        // ===== TMA producer =====
        // One thread issues every load.  All position bookkeeping is incremental: an integer division
        // costs this lone thread ~100 cycles, and the loop has to turn around in well under the 256
        // cycles the tensor core needs per stage.
        {
            const uint32_t tx_bytes = (uint32_t)(A_STAGE_BYTES + b_stage_bytes);
            int s = 0;
            uint32_t phase = 0;
            // counters of stage q0: FWD (chunk, tap, di, dj); DX (chunk, -, th, tw); DK (-, tile_n, tile_h, tile_w)
            int chunk = 0, tap = 0, di = 0, dj = 0;
            if (MODE == MODE_FWD && !p.narrow) {
                tap = q0 / p.kchunks; chunk = q0 % p.kchunks; di = tap / p.KW; dj = tap % p.KW;
            } else if (MODE == MODE_DX) {
                const int t = q0 / p.kchunks;
                chunk = q0 % p.kchunks; di = t / taps_w; dj = t % taps_w;
            } else if (MODE == MODE_DK) {
                dj = q0 % p.tiles_w; di = (q0 / p.tiles_w) % p.tiles_h; tap = q0 / (p.tiles_w * p.tiles_h);
            }
            const int wrap_dj = (MODE == MODE_FWD) ? p.KW : taps_w;
            for (int it = 0; it < nq; ++it) {
                if (!mbar_wait_warp(empty_bar + 8u * s, phase ^ 1u, 0, it, wait_limit)) break;
                const uint32_t fb = full_bar + 8u * s;
                if (it != p.skip_stage && elect_one()) {
                TC_TRACE(it);
                if (TC_DEBUG_BIT(2)) {   // timing experiment: no loads, the stage is declared full at once
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(fb) : "memory");
                } else {
                    mbar_expect_tx(fb, tx_bytes);
                    const uint32_t a_dst = a_base + (uint32_t)s * A_STAGE_BYTES;
                    const uint32_t b_dst = b_base + (uint32_t)s * b_stage_bytes;
                    if (MODE == MODE_FWD && p.narrow) {
                        // stage = kernel row: 128 output pixels x the 32-float window (8 pixels x 4
                        // channels) that starts at padded column s*j of padded row s*i + row
                        const int q = q0 + it;
                        tma_load_5d(a_dst, &map_a, fb, 0, j0, i0, n0, q);
                        tma_load_4d(b_dst, &map_b, fb, 0, 0, q, n_tile * (p.bn / 32));
                    } else if (MODE == MODE_FWD) {
                        if (it < 128) TC_TRACE(256 + it);
                        tma_load_4d(a_dst, &map_a, fb, chunk * BK, p.sw * j0 + dj - p.pl, p.sh * i0 + di - p.pt, n0);
                        if (it < 128) TC_TRACE(512 + it);
                        tma_load_4d(b_dst, &map_b, fb, 0, chunk * BK, tap, n_tile * (p.bn / 32));
                        if (it < 128) TC_TRACE(768 + it);
                    } else if (MODE == MODE_DX) {
                        // (di, dj) count the taps of this parity class: kernel tap (rh + sh*di, rw + sw*dj)
                        tma_load_4d(a_dst, &map_a, fb, chunk * BK, j0 + ew - dj, i0 + eh - di, n0);
                        tma_load_4d(b_dst, &map_b, fb, chunk * BK, n_tile * p.bn, rw + p.sw * dj, rh + p.sh * di);
                    } else {
                        // (tap, di, dj) count the 32-pixel tiles along (n, h, w)
                        const int pj = dj * p.TW, pi = di * p.TH, pn = tap * p.TN;
                        const int xw = p.sw * pj + tap_dj - p.pl, xh = p.sh * pi + tap_di - p.pt;
                        if (p.narrow) {  // A: dy (rows o), B: the KH 32-float windows of 32 output pixels
                            tma_load_5d(a_dst, &map_a, fb, 0, pj, pi, pn, m_tile * (BM / 32));
                            tma_load_5d(b_dst, &map_b, fb, 0, pj, pi, pn, 0);   // box covers all KH kernel rows
                        } else if (!p.swap) {   // A: x (rows c), B: dy (cols o)
                            tma_load_5d(a_dst, &map_a, fb, 0, xw, xh, pn, m_tile * (BM / 32));
                            tma_load_5d(b_dst, &map_b, fb, 0, pj, pi, pn, n_tile * (p.bn / 32));
                        } else {         // A: dy (rows o), B: x (cols c)
                            tma_load_5d(a_dst, &map_a, fb, 0, pj, pi, pn, m_tile * (BM / 32));
                            tma_load_5d(b_dst, &map_b, fb, 0, xw, xh, pn, n_tile * (p.bn / 32));
                        }
                    }
                }
                }
                // advance to the next stage
                if (MODE == MODE_DK) {
                    if (++dj == p.tiles_w) { dj = 0; if (++di == p.tiles_h) { di = 0; ++tap; } }
                } else if (++chunk == p.kchunks) {
                    chunk = 0; ++tap;
                    if (++dj == wrap_dj) { dj = 0; ++di; }
                }
                if (++s == p.stages) { s = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer =====
        {
            const int a_mn = (MODE == MODE_DK) ? 1 : 0;
            const int b_mn = (MODE == MODE_DX) ? 0 : 1;
            const uint32_t idesc = make_idesc(a_mn, b_mn, p.bn, BM);
            // K-major tile: rows of 128 B, 8-row groups 1024 B apart (stride offset); one MMA (K = 8)
            // consumes 32 B of each row.
            // MN-major tile: [32-channel chunk][k row][128 B]: chunks 4096 B apart (leading offset), the
            // 32-byte-chunk swizzle repeats every 4 k rows, so 4-row groups are 512 B apart (stride
            // offset); one MMA consumes 8 k rows = 1024 B.
            const uint32_t a_lbo = a_mn ? 4096u : 16u, b_lbo = b_mn ? 4096u : 16u;
            const uint32_t a_sbo = a_mn ? 512u : 1024u, b_sbo = b_mn ? 512u : 1024u;
            const uint32_t a_lay = a_mn ? kLayoutSw128Base32 : kLayoutSw128;
            const uint32_t b_lay = b_mn ? kLayoutSw128Base32 : kLayoutSw128;
            const uint32_t a_step = a_mn ? 1024u : 32u, b_step = b_mn ? 1024u : 32u;
            // descriptors of stage 0; a stage further on only changes the 14-bit start-address field
            const uint64_t adesc0 = make_smem_desc(a_base, a_lbo, a_sbo, a_lay);
            const uint64_t bdesc0 = make_smem_desc(b_base, b_lbo, b_sbo, b_lay);
            const uint32_t a_stage16 = A_STAGE_BYTES >> 4, b_stage16 = (uint32_t)b_stage_bytes >> 4;
            int s = 0;
            uint32_t phase = 0;
            {
            for (int it = 0; it < nq; ++it) {
                if (!mbar_wait_warp(full_bar + 8u * s, phase, 1, it, wait_limit)) break;
                if (X3 && !mbar_wait_warp(resid_bar + 8u * s, phase, 3, it, wait_limit)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (elect_one()) {
                TC_TRACE(1024 + it);
                if (TC_DEBUG_BIT(1)) {   // timing experiment: no MMA, the stage is released at once
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_bar + 8u * s) : "memory");
                } else {
                    const uint64_t adesc = adesc0 + (uint64_t)(s * a_stage16);
                    const uint64_t bdesc = bdesc0 + (uint64_t)(s * b_stage16);
                    if (X3) {
                        // a*b ~ a_hi*b_lo + a_lo*b_hi + a_hi*b_hi, the small terms first; the tensor core
                        // reads the TF32 part (top 19 bits) of whatever fp32 word it is given
                        const uint64_t ares = adesc + (uint64_t)((as_base - a_base) >> 4);
                        const uint64_t bres = bdesc + (uint64_t)((bs_base - b_base) >> 4);
#pragma unroll
                        for (int kk = 0; kk < BK / 8; ++kk) {
                            const uint64_t ka = (uint64_t)(kk * (a_step >> 4)), kb = (uint64_t)(kk * (b_step >> 4));
                            const uint32_t first = (it > 0 || kk > 0) ? 1u : 0u;
                            tcgen05_mma_tf32(tmem_d + (uint32_t)p.bn, adesc + ka, bres + kb, idesc, first);
                            tcgen05_mma_tf32(tmem_d + (uint32_t)p.bn, ares + ka, bdesc + kb, idesc, 1u);
                            tcgen05_mma_tf32(tmem_d, adesc + ka, bdesc + kb, idesc, first);
                        }
                    } else {
#pragma unroll
                        for (int kk = 0; kk < BK / 8; ++kk)
                            tcgen05_mma_tf32(tmem_d, adesc + (uint64_t)(kk * (a_step >> 4)), bdesc + (uint64_t)(kk * (b_step >> 4)),
                                             idesc, (it > 0 || kk > 0) ? 1u : 0u);
                    }
                    tcgen05_commit(empty_bar + 8u * s);  // frees the stage once these MMAs have read it
                }
                TC_TRACE(2048 + it);
                }
                if (++s == p.stages) { s = 0; phase ^= 1u; }
            }
            if (elect_one()) tcgen05_commit(tmem_full_bar);   // accumulator complete (or abandoned)
            }
        }
    } else {
        // ===== epilogue, part 1 (warps 2..5; TMEM lane quadrant = warp % 4; thread = accumulator row) =====
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        // where does this accumulator row go?  (worked out while the main loop is still running)
        bool row_valid = false;
        unsigned long long row_off = 0;   // element offset of column 0 of this row
        if (MODE == MODE_FWD) {
            const int tw = row % p.TW, th = (row / p.TW) % p.TH, tn = row / (p.TW * p.TH);
            const int n = n0 + tn, i = i0 + th, j = j0 + tw;
            row_valid = n < p.N && i < p.Ho && j < p.Wo;
            row_off = (((unsigned long long)n * p.Ho + i) * p.Wo + j) * p.O + ch0;
            if (p.planes) row_off = (((unsigned long long)n * p.Ho + i) * p.Wo + j) * 4ull;
        } else if (MODE == MODE_DX) {
            const int tw = row % p.TW, th = (row / p.TW) % p.TH, tn = row / (p.TW * p.TH);
            const int n = n0 + tn, h = p.sh * (i0 + th) + ph, w = p.sw * (j0 + tw) + pw;
            row_valid = n < p.N && h < p.H && w < p.W;
            row_off = (((unsigned long long)n * p.H + h) * p.W + w) * p.C + ch0;
        } else {
            const unsigned long long tap_off = (unsigned long long)group * p.C * p.O;
            if (p.narrow) {  // rows o, columns = 32 * kernel row + window slot (kernel column dj = slot / 4, channel = slot % 4)
                const int o = m_tile * BM + row;
                row_valid = o < p.O;
                row_off = o;
            } else if (!p.swap) {   // rows c, columns o
                const int c = m_tile * BM + row;
                row_valid = c < p.C;
                row_off = tap_off + (unsigned long long)c * p.O + ch0;
            } else {         // rows o, columns c
                const int o = m_tile * BM + row;
                row_valid = o < p.O;
                row_off = tap_off + (unsigned long long)ch0 * p.O + o;
            }
        }
        if (X3) {
            // ===== 3xTF32: these four warps turn every landed stage into its residual tiles =====
            // residual = value - (value with the low 13 mantissa bits cleared); element-wise on the raw
            // bytes of the stage, so the swizzled layout carries over unchanged
            const int tid_r = threadIdx.x - 64;
            int s = 0;
            uint32_t phase = 0;
            const int a_q = A_STAGE_BYTES / 16, b_q = b_stage_bytes / 16;   // 16-byte words per tile
            for (int it = 0; it < nq; ++it) {
                if (!mbar_wait(full_bar + 8u * s, phase, 4, it, wait_limit)) break;
                const float4* asrc = reinterpret_cast<const float4*>(smem_raw + (a_base + (uint32_t)s * A_STAGE_BYTES - smem_u32(smem_raw)));
                float4* adst = reinterpret_cast<float4*>(smem_raw + (as_base + (uint32_t)s * A_STAGE_BYTES - smem_u32(smem_raw)));
                const float4* bsrc = reinterpret_cast<const float4*>(smem_raw + (b_base + (uint32_t)s * b_stage_bytes - smem_u32(smem_raw)));
                float4* bdst = reinterpret_cast<float4*>(smem_raw + (bs_base + (uint32_t)s * b_stage_bytes - smem_u32(smem_raw)));
#pragma unroll 4
                for (int i = tid_r; i < a_q; i += kEpi) adst[i] = tf32_residual(asrc[i]);
#pragma unroll 4
                for (int i = tid_r; i < b_q; i += kEpi) bdst[i] = tf32_residual(bsrc[i]);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> tensor core reads
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(resid_bar + 8u * s) : "memory");
                if (++s == p.stages) { s = 0; phase ^= 1u; }
            }
        }
        bool ok = mbar_wait(tmem_full_bar, 0, 2, 0, wait_limit);
        ok = __all_sync(0xffffffffu, ok);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (threadIdx.x == 64) TC_TRACE(3074);
        TC_CTA_TRACE(2);
        if (!ok || nq <= 0) row_valid = false;   // nothing trustworthy to store
        // The pipeline stages are idle from here on (every MMA that read them has completed).
        s_rowoff[row] = row_valid ? (long long)row_off : -1;
    }

    // ===== the K partitions of a tile meet =====
    // The S partitions of one tile form a thread-block cluster, which guarantees that they run at the
    // same time and gives them a hardware barrier.  Each partition writes its partial accumulator
    // to scratch (it stays in L2), the cluster meets, and partition j then finishes a 1/S share of
    // the tile: it adds the S partials in partition order - so the result does not depend on timing -
    // applies the fused chain and writes the final tensor.  (Handing the partials over through
    // distributed shared memory instead was measured at under 10 bytes per clock and SM.)
    // Partials are stored quad-major, [CTA][16-byte column quad][row]: lanes are consecutive rows, so
    // both the partial stores and the loads of the second phase move 512 contiguous bytes per warp.
    // Without partitions the same layout in shared memory (quad pitch QS) is the transposition buffer
    // between "thread = row" (TMEM) and "warp = row segment" (coalesced global stores).
    const int S = p.splits, part = split;
    const bool multi = S > 1;
    const bool finish_here = !p.ext_finish;   // else: partials only, a second kernel adds them
    const int qpr = p.bn >> 2;                // vector path: 16-byte column quads per row,
    const int QPO = (qpr + S - 1) / S;        //   quads per share
    const int QS = BM + 1;                    // shared-memory quad pitch in 16-byte units (odd: lanes = quads hit distinct banks)
    const int CL = (p.bn + S - 1) / S;        // scalar path: columns per share
    float* my_scratch = p.scratch + (size_t)blockIdx.x * BM * p.bn;
    const float* tile_scratch = p.scratch + (size_t)(blockIdx.x - part) * BM * p.bn;
    if (threadIdx.x == 64) TC_TRACE(3000);
    if (warp >= 2) {
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        // the two warps of a lane quadrant (2..5 and 6..9) take alternate 32-column slabs
        for (int c0 = ((warp - 2) >> 2) * 32; c0 < p.bn; c0 += 64) {
            uint32_t r[32];
            const uint32_t taddr = tmem_d + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0;
            const bool full = p.bn - c0 >= 32;   // bn is a multiple of 16: the last slab has 32 or 16 columns
            if (full) tmem_ld_32x32b_x32(taddr, r);
            else tmem_ld_32x32b_x16(taddr, r);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (X3) {   // add the accumulator of the small terms
                uint32_t r2[32];
                if (full) tmem_ld_32x32b_x32(taddr + (uint32_t)p.bn, r2);
                else tmem_ld_32x32b_x16(taddr + (uint32_t)p.bn, r2);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int q = 0; q < 32; ++q)
                    if (q < 16 || full) r[q] = __float_as_uint(__fadd_rn(__uint_as_float(r[q]), __uint_as_float(r2[q])));
            }
            if (vec) {
                if (multi) {
                    float4* d4 = reinterpret_cast<float4*>(my_scratch) + (size_t)(c0 >> 2) * BM + row;
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        if (q < 4 || full)
                            __stcg(d4 + q * BM, make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                            __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3])));
                } else {
                    float4* d4 = reinterpret_cast<float4*>(red) + (c0 >> 2) * QS + row;
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        if (q < 4 || full)
                            d4[q * QS] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                     __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                }
            } else {
                // column-major [column][row], in scratch or in shared memory
                float* d1 = (multi ? my_scratch : red) + (size_t)c0 * BM + row;
#pragma unroll
                for (int q = 0; q < 32; ++q)
                    if (q < 16 || full) d1[q * BM] = __uint_as_float(r[q]);
            }
        }
        // no fence here: every thread's partial stores are ordered before its own arrival at the cluster barrier
        // (barrier.cluster.arrive.release / wait.acquire), and before the finish kernel by the kernel boundary
    }
    if (threadIdx.x == 64) TC_TRACE(3001);
    TC_CTA_TRACE(3);
    __syncwarp();
    if (multi && finish_here) cluster_sync_all();
    else if (warp >= 2) asm volatile("bar.sync 1, %0;" ::"n"(kEpi) : "memory");
    if (threadIdx.x == 64) TC_TRACE(3002);
    TC_CTA_TRACE(4);

    if (warp >= 2 && finish_here) {
        // ===== this partition's share: sum in partition order, fused chain, stores =====
        const int tid_e = threadIdx.x - 64;
        const EpilogueArgs& e = p.ep;
        if (vec) {
            const bool fused = e.raw_out || e.bias || e.pre_act || e.gate || e.act != DCG_ACT_NONE;
            // multi: thread = row, items = the quads of this share.  single: item = (row, quad) with
            // consecutive lanes on consecutive quads, so a warp stores whole 128-byte row segments.
            const int Qm = min(QPO, qpr - part * QPO);
            const bool by_row = multi || p.planes;               // thread = row (else: lanes walk the quads of a row)
            // by_row: the two threads of a row (tid_e and tid_e + 128) take alternate quads
            const int my_row = tid_e & (BM - 1), my_half = tid_e >> 7;
            const int row_quads = multi ? Qm : qpr;              // by_row: quads of this row's share
            const int per_thread = by_row ? (row_quads > my_half ? (row_quads - my_half + 1) / 2 : 0)
                                          : qpr / 2;            // single: 128 * qpr items over 256 threads (qpr is even)
            const int quad0 = ch0 >> 2;                          // planes: global index of this tile's first quad
            const int step_r = kEpi / qpr, step_q = kEpi % qpr;  // single: how (row, quad) moves when the item index grows by kEpi
            int rr = tid_e / qpr, q = tid_e % qpr;
            const long long my_ro = s_rowoff[my_row];
            const float4* red4 = reinterpret_cast<const float4*>(red);
            const float4* ts4 = reinterpret_cast<const float4*>(tile_scratch);
            for (int base = 0; base < per_thread; base += 4) {
                float4 acc[4];
                long long goff[4];
                int cq[4];
                if (by_row) {
                    const float4* src[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const bool in = base + u < per_thread;
                        const int qd = part * QPO + (in ? my_half + 2 * (base + u) : 0);
                        cq[u] = qd << 2;
                        goff[u] = (!in || my_ro < 0 || cq[u] >= ncols_valid) ? -1
                                  : p.planes ? my_ro + (long long)((unsigned long long)(quad0 + qd) * p.plane_stride)
                                             : my_ro + cq[u];
                        src[u] = (multi ? ts4 + (size_t)qd * BM : red4 + qd * QS) + my_row;
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) acc[u] = multi ? __ldcg(src[u]) : *src[u];
#pragma unroll 2
                    for (int sidx = 1; sidx < S; ++sidx) {   // two partitions' loads in flight; the adds keep partition order
                        float4 v[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) v[u] = __ldcg(src[u] + (size_t)sidx * BM * qpr);
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            acc[u].x = __fadd_rn(acc[u].x, v[u].x); acc[u].y = __fadd_rn(acc[u].y, v[u].y);
                            acc[u].z = __fadd_rn(acc[u].z, v[u].z); acc[u].w = __fadd_rn(acc[u].w, v[u].w);
                        }
                    }
                } else {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const bool in = base + u < per_thread;
                        cq[u] = q << 2;
                        const long long ro = in ? s_rowoff[rr] : -1;
                        goff[u] = (ro < 0 || cq[u] >= ncols_valid) ? -1 : ro + cq[u];
                        acc[u] = red4[in ? q * QS + rr : 0];
                        rr += step_r; q += step_q;
                        if (q >= qpr) { q -= qpr; ++rr; }
                    }
                }
                if (fused) {
                    // each optional step of the chain runs over the four items at once, so its
                    // test is paid once and the loads of a step are in flight together
                    if (e.raw_out) {
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            if (goff[u] >= 0) *reinterpret_cast<float4*>(e.raw_out + goff[u]) = acc[u];
                    }
                    if (e.bias) {
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const float4 bv = __ldg(reinterpret_cast<const float4*>(e.bias + ch0 + cq[u]));
                            acc[u].x = __fadd_rn(acc[u].x, bv.x); acc[u].y = __fadd_rn(acc[u].y, bv.y);
                            acc[u].z = __fadd_rn(acc[u].z, bv.z); acc[u].w = __fadd_rn(acc[u].w, bv.w);
                        }
                    }
                    if (e.pre_act) {
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            if (goff[u] >= 0) *reinterpret_cast<float4*>(e.pre_act + goff[u]) = acc[u];
                    }
                    if (e.act != DCG_ACT_NONE) {
                        const int act = e.act;
                        const float alpha = e.alpha;
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            acc[u].x = act_apply(acc[u].x, act, alpha); acc[u].y = act_apply(acc[u].y, act, alpha);
                            acc[u].z = act_apply(acc[u].z, act, alpha); acc[u].w = act_apply(acc[u].w, act, alpha);
                        }
                    }
                    if (e.gate) {
                        float4 gg[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            gg[u] = goff[u] >= 0 ? __ldg(reinterpret_cast<const float4*>(e.gate + goff[u]))
                                                 : make_float4(0.f, 0.f, 0.f, 0.f);
                        const int gact = e.gate_act;
                        const float galpha = e.gate_alpha;
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            acc[u].x = act_grad_apply(gg[u].x, acc[u].x, gact, galpha);
                            acc[u].y = act_grad_apply(gg[u].y, acc[u].y, gact, galpha);
                            acc[u].z = act_grad_apply(gg[u].z, acc[u].z, gact, galpha);
                            acc[u].w = act_grad_apply(gg[u].w, acc[u].w, gact, galpha);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (goff[u] >= 0) *reinterpret_cast<float4*>(p.out + goff[u]) = acc[u];
            }
        } else {
            // thread = row; share = every S-th column.  Used where consecutive ROWS are adjacent in
            // memory (DK with the channel roles swapped, narrow-channel DK) and for channel counts
            // that rule out 16-byte stores.
            const int my_row = tid_e & (BM - 1), my_half = tid_e >> 7;   // the two threads of a row take alternate columns
            const long long ro = s_rowoff[my_row];
            for (int cl0 = 0; 2 * cl0 + my_half < CL; cl0 += 4) {   // four columns at a time: their loads are in flight together
                float acc[4];
                int cols[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int cl = 2 * (cl0 + u) + my_half;
                    const int col = cl * S + part;
                    cols[u] = (cl < CL && col < ncols_valid) ? col : -1;
                    const int cc = cols[u] < 0 ? 0 : cols[u];
                    acc[u] = multi ? __ldcg(tile_scratch + (size_t)cc * BM + my_row) : red[cc * BM + my_row];
                }
                if (multi) {
                    for (int sidx = 1; sidx < S; ++sidx) {
                        float v[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            v[u] = __ldcg(tile_scratch + ((size_t)sidx * p.bn + (cols[u] < 0 ? 0 : cols[u])) * BM + my_row);
#pragma unroll
                        for (int u = 0; u < 4; ++u) acc[u] = __fadd_rn(acc[u], v[u]);
                    }
                }
                if (ro < 0) continue;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int col = cols[u];
                    if (col < 0) continue;
                    unsigned long long id = (unsigned long long)ro + (unsigned long long)col * col_stride;
                    if (MODE == MODE_DK && p.narrow) {
                        const int di = col >> 5, dj = (col & 31) >> 2, c = col & 3;   // slot = 4*dj + channel
                        if (dj >= p.KW || c >= p.C) continue;                          // padding slots
                        id = (unsigned long long)ro + (unsigned long long)((di * p.KW + dj) * p.C + c) * p.O;
                    }
                    // the fused chain only exists for FWD/DX; DK stores raw sums
                    p.out[id] = (MODE == MODE_DK) ? acc[u] : epilogue_apply(e, acc[u], id, ch0 + col);
                }
            }
        }
    }

    if (threadIdx.x == 64) TC_TRACE(3075);
    TC_CTA_TRACE(5);
    // ---- teardown: everyone is done with TMEM before warp 1 releases it --------------------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(tmem_cols) : "memory");
    }
}

}  // namespace
}  // namespace dcg
