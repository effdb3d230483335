// conv_dxf_kernel: input gradient with all parity classes of a pixel tile in one CTA.  Included by conv_tc.cu only.
#pragma once

namespace dcg {
namespace {

// ---- DX with all parity classes of a pixel tile in one CTA -------------------------------------------
// The parity classes of the input gradient (pix mod stride) read the SAME windows of dy, only paired
// with different kernel taps: class (ph, pw), tap (di, dj) reads dy at pixel offset
// ((ph + pad - di) / s, (pw + pad - dj) / s) of the class grid.  For a 5x5 kernel at stride 2 the 25
// (class, tap) pairs share 9 distinct windows.  conv_tc_kernel<DX> runs every class as a tile of its
// own and so fetches a dy tile from L2 once per tap; with a narrow N tile (64 input channels: A 16 KB
// against B 8 KB per stage) that fetch is two thirds of what the SM has to take in, and taking
// operands in is what bounds the main loop.  This kernel gives one CTA the 128 pixels of ALL classes:
// one accumulator per class (classes x bn <= 512 TMEM columns), each window fetched once and
// multiplied against the weight tiles of every pair that reads it - 9 x 16 KB + 25 x 8 KB per 32
// output channels instead of 25 x 24 KB.  A pipeline stage is one window plus the weight tiles of up to
// `pb` pairs that read it (a window with more pairs takes several stages and is fetched again for
// each).  The windows are ordered so that the classes complete one after the other; the epilogue
// of a finished class (through a transposition buffer of its own, not the stage ring) runs under
// the main loop of the rest.  No K partitions: the planner only picks this kernel when the tiles
// alone fill the GPU.
//
// The accumulators of the classes sit side by side in TMEM, and the weight tiles of a stage are stacked
// in shared memory in the same order, so pairs whose classes are neighbours there are ONE MMA with
// N = count x bn columns.  That matters for narrow tiles: an N = 64 MMA takes as long as an N = 128
// one (measured: the MMA-only time of the 64-channel layer is 1.8 x that of its N = 128 forward), so
// the 25 N = 64 products of a channel chunk become 4 of N = 256, 4 of N = 128 and 1 of N = 64.
struct CfWin {
    signed char sy, sx;        // window: dy pixel (i + sy, j + sx) for class pixel (i, j)
    unsigned char n;           // pairs of this stage, in TMEM order
    unsigned char last;        // bit j: pair j is the last contribution to its class (in the last channel chunk)
    unsigned char fresh;       // bit j: pair j is the first contribution to its class (in the first channel chunk)
    unsigned char cls[4], kh[4], kw[4];
    unsigned char slot[4];     // TMEM position of the pair's accumulator (columns slot * bn ...)
    unsigned char glen[4];     // pair j starts an MMA over glen[j] adjacent accumulators (0: it belongs to an earlier one)
};
struct CfTable {
    int nwin, ncls;            // stages per channel chunk, parity classes
    int slot_bytes;            // stage size: A tile + pb weight tiles
    int order[4];              // classes in the order in which they complete
    int slot_of_class[4];      // TMEM position of every class
    CfWin win[32];
};
constexpr int kCfHalf = 64;                // accumulator columns the epilogue moves at a time
__host__ __device__ constexpr int kCfRedBytes() { return kRedFloats(kCfHalf) * 4 + BM * 8; }

// The fused chain over four 16-byte items at once: every optional step is tested once and its loads
// (bias, gate) are in flight together.  goff < 0 marks an item that is not stored.
__device__ __forceinline__ void cf_chain_store4(const EpilogueArgs& e, float* out, float4 (&acc)[4], const long long (&goff)[4],
                                                const int (&ch)[4])
{
    if (e.raw_out) {
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (goff[u] >= 0) *reinterpret_cast<float4*>(e.raw_out + goff[u]) = acc[u];
    }
    if (e.bias) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float4 bv = __ldg(reinterpret_cast<const float4*>(e.bias + ch[u]));
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
        float4 g[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            g[u] = goff[u] >= 0 ? __ldg(reinterpret_cast<const float4*>(e.gate + goff[u])) : make_float4(0.f, 0.f, 0.f, 0.f);
        const int gact = e.gate_act;
        const float galpha = e.gate_alpha;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            acc[u].x = act_grad_apply(g[u].x, acc[u].x, gact, galpha);
            acc[u].y = act_grad_apply(g[u].y, acc[u].y, gact, galpha);
            acc[u].z = act_grad_apply(g[u].z, acc[u].z, gact, galpha);
            acc[u].w = act_grad_apply(g[u].w, acc[u].w, gact, galpha);
        }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
        if (goff[u] >= 0) *reinterpret_cast<float4*>(out + goff[u]) = acc[u];
}

__global__ void __launch_bounds__(kThreads, 1)
conv_dxf_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ Params p, const __grid_constant__ CfTable t)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem0 = smem_u32(smem_raw);
    const uint32_t ring = (smem0 + 1023u) & ~1023u;
    const long long wait_limit = p.wait_cycles;
    const uint32_t slot_bytes = (uint32_t)t.slot_bytes;
    const uint32_t red_base = ring + (uint32_t)p.stages * slot_bytes;
    const uint32_t bar_base = red_base + (uint32_t)kCfRedBytes();
    const uint32_t full_bar = bar_base;
    const uint32_t empty_bar = bar_base + 8u * p.stages;
    const uint32_t cls_bar = bar_base + 16u * p.stages;     // accumulator of class c complete
    const uint32_t tmem_slot = cls_bar + 32u;
    uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem0));
    float* red = reinterpret_cast<float*>(smem_raw + (red_base - smem0));
    long long* s_rowoff = reinterpret_cast<long long*>(red + kRedFloats(kCfHalf));

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const int ncls = t.ncls, nwin = t.nwin;
    const uint32_t b_bytes = (uint32_t)p.bn * BK * 4;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(full_bar + 8u * s, 1);
            mbar_init(empty_bar + 8u * s, 1);
        }
        for (int c = 0; c < 4; ++c) mbar_init(cls_bar + 8u * c, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    }
    int tmem_cols = 32;
    while (tmem_cols < ncls * p.bn) tmem_cols <<= 1;
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // blockIdx.x = pixel tile * n_tiles + channel tile
    const int n_tile = blockIdx.x % p.n_tiles, m_tile = blockIdx.x / p.n_tiles;
    const int j0 = (m_tile % p.tiles_w) * p.TW;
    const int i0 = ((m_tile / p.tiles_w) % p.tiles_h) * p.TH;
    const int n0 = (m_tile / (p.tiles_w * p.tiles_h)) * p.TN;
    const int ch0 = n_tile * p.bn;
    const int ncols_valid = min(p.bn, p.C - ch0);

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot_ptr;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        // ===== TMA producer: for every table entry, for every channel chunk: the window, then its weight tiles =====
        int s = 0, it = 0;
        uint32_t phase = 0;
        bool alive = true;
        for (int w = 0; w < nwin && alive; ++w) {
            const CfWin& wn = t.win[w];
            const int sy = wn.sy, sx = wn.sx, np = wn.n;
            for (int chunk = 0; chunk < p.kchunks; ++chunk, ++it) {
                if (!mbar_wait_warp(empty_bar + 8u * s, phase ^ 1u, 0, it, wait_limit)) { alive = false; break; }
                if (elect_one()) {
                    const uint32_t fb = full_bar + 8u * s;
                    const uint32_t dst = ring + (uint32_t)s * slot_bytes;
                    mbar_expect_tx(fb, (uint32_t)A_STAGE_BYTES + (uint32_t)np * b_bytes);
                    tma_load_4d(dst, &map_a, fb, chunk * BK, j0 + sx, i0 + sy, n0);
                    for (int j = 0; j < np; ++j)
                        tma_load_4d(dst + (uint32_t)A_STAGE_BYTES + (uint32_t)j * b_bytes, &map_b, fb, chunk * BK, ch0,
                                    (int)wn.kw[j], (int)wn.kh[j]);
                }
                if (++s == p.stages) { s = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer =====
        const uint64_t desc0 = make_smem_desc(ring, 16u, 1024u, kLayoutSw128);   // K-major, 128-byte rows, 8-row groups 1024 B apart
        const uint32_t slot16 = slot_bytes >> 4, b16 = b_bytes >> 4;
        int s = 0, it = 0;
        uint32_t phase = 0, done = 0;
        bool alive = true;
        for (int w = 0; w < nwin && alive; ++w) {
            const CfWin& wn = t.win[w];
            const int np = wn.n;
            const uint32_t last = wn.last, fresh = wn.fresh;
            for (int chunk = 0; chunk < p.kchunks; ++chunk, ++it) {
                if (!mbar_wait_warp(full_bar + 8u * s, phase, 1, it, wait_limit)) { alive = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const bool final_chunk = chunk == p.kchunks - 1;
                if (elect_one()) {
                    const uint64_t adesc = desc0 + (uint64_t)((uint32_t)s * slot16);
                    for (int j = 0; j < np; ++j) {
                        const int cnt = wn.glen[j];
                        if (cnt > 0) {   // one MMA per K step over the cnt adjacent accumulators that start here
                            const uint32_t idesc = make_idesc(0, 0, cnt * p.bn, BM);
                            const uint64_t bdesc = adesc + (uint64_t)((uint32_t)(A_STAGE_BYTES >> 4) + (uint32_t)j * b16);
                            const uint32_t acc = tmem_d + (uint32_t)(wn.slot[j] * p.bn);
                            const bool overwrite = chunk == 0 && ((fresh >> j) & 1u);
#pragma unroll
                            for (int kk = 0; kk < BK / 8; ++kk)
                                tcgen05_mma_tf32(acc, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc,
                                                 (overwrite && kk == 0) ? 0u : 1u);
                        }
                    }
                    if (final_chunk)
                        for (int j = 0; j < np; ++j)
                            if ((last >> j) & 1u) tcgen05_commit(cls_bar + 8u * wn.cls[j]);
                    tcgen05_commit(empty_bar + 8u * s);
                }
                if (final_chunk)
                    for (int j = 0; j < np; ++j)
                        if ((last >> j) & 1u) done |= 1u << wn.cls[j];
                if (++s == p.stages) { s = 0; phase ^= 1u; }
            }
        }
        // a pipeline that gave up still releases the epilogue (which stores nothing then)
        if (elect_one())
            for (int c = 0; c < ncls; ++c)
                if (!((done >> c) & 1u)) tcgen05_commit(cls_bar + 8u * c);
    } else {
        // ===== epilogue: classes in completion order, 64 accumulator columns at a time =====
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int tid_e = threadIdx.x - 64;
        const int tw = row % p.TW, th = (row / p.TW) % p.TH, tn = row / (p.TW * p.TH);
        const EpilogueArgs& e = p.ep;
        constexpr int QS = BM + 1;
        // 16-byte stores need whole column quads in every row; else (3 input channels) element by element
        const bool vec = (p.C & 3) == 0 && (ncols_valid & 3) == 0;
        for (int ci = 0; ci < ncls; ++ci) {
            const int cls = t.order[ci];
            const int ph = cls / p.sw, pw = cls % p.sw;
            bool ok = mbar_wait(cls_bar + 8u * cls, 0, 2, cls, wait_limit);
            ok = __all_sync(0xffffffffu, ok);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (warp < 6) {
                const int n = n0 + tn, h = p.sh * (i0 + th) + ph, w = p.sw * (j0 + tw) + pw;
                const bool valid = ok && n < p.N && h < p.H && w < p.W;
                s_rowoff[row] = valid ? (long long)((((unsigned long long)n * p.H + h) * p.W + w) * p.C + ch0) : -1;
            }
            for (int half0 = 0; half0 < p.bn; half0 += kCfHalf) {
                const int hcols = min(kCfHalf, p.bn - half0);
                // TMEM -> transposition buffer: thread = row, the two warps of a lane quadrant take one 32-column slab each
                const int c0 = half0 + ((warp - 2) >> 2) * 32;
                if (c0 < half0 + hcols) {
                    uint32_t r[32];
                    const uint32_t taddr = tmem_d + ((uint32_t)(quad * 32) << 16) + (uint32_t)(t.slot_of_class[cls] * p.bn + c0);
                    const bool full = half0 + hcols - c0 >= 32;
                    if (full) tmem_ld_32x32b_x32(taddr, r);
                    else tmem_ld_32x32b_x16(taddr, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (vec) {
                        float4* d4 = reinterpret_cast<float4*>(red) + ((c0 - half0) >> 2) * QS + row;
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            if (q < 4 || full)
                                d4[q * QS] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                         __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                    } else {   // column-major [column][row]; only the valid columns are ever read back
                        float* d1 = red + (c0 - half0) * BM + row;
                        const int nv = ncols_valid - c0;
#pragma unroll
                        for (int q = 0; q < 32; ++q)
                            if ((q < 16 || full) && q < nv) d1[q * BM] = __uint_as_float(r[q]);
                    }
                }
                asm volatile("bar.sync 1, %0;" ::"n"(kEpi) : "memory");
                // fused chain and stores: consecutive lanes take consecutive 16-byte column quads of a row
                const int hq = hcols >> 2;
                const float4* red4 = reinterpret_cast<const float4*>(red);
                if (!vec) {   // consecutive lanes take the consecutive valid columns of a row
                    const int hv = min(hcols, ncols_valid - half0);
                    for (int idx = tid_e; idx < BM * hv; idx += kEpi) {
                        const int rr = idx / hv, c = idx - rr * hv;
                        const long long ro = s_rowoff[rr];
                        if (ro < 0) continue;
                        const unsigned long long id = (unsigned long long)ro + (unsigned long long)(half0 + c);
                        p.out[id] = epilogue_apply(e, red[c * BM + rr], id, ch0 + half0 + c);
                    }
                }
                const int items = vec ? BM * hq : 0;   // = kEpi * hq / 2: every thread has hq / 2 items, taken four at a time
                for (int base = tid_e; base < items; base += 4 * kEpi) {
                    float4 acc[4];
                    long long goff[4];
                    int ch[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int idx = base + u * kEpi;
                        const bool in = idx < items;
                        const int rr = in ? idx / hq : 0, q = in ? idx - rr * hq : 0;
                        const int col = half0 + (q << 2);
                        const long long ro = in ? s_rowoff[rr] : -1;
                        acc[u] = red4[q * QS + rr];
                        goff[u] = (ro < 0 || col >= ncols_valid) ? -1 : ro + col;
                        ch[u] = ch0 + (col < ncols_valid ? col : 0);
                    }
                    cf_chain_store4(e, p.out, acc, goff, ch);
                }
                asm volatile("bar.sync 1, %0;" ::"n"(kEpi) : "memory");
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
