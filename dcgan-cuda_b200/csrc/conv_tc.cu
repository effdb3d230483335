// tcgen05 implicit-GEMM convolution kernels (TF32 operands, fp32 accumulation in TMEM).
//
// One kernel template covers the three operators; each is a GEMM D[M x N] += A[M x K] B[K x N]
// whose operand tiles are fetched straight from the NHWC / HWIO tensors by TMA - no im2col
// buffer, no zero-inserted gradient, no weight repacking ever exists in memory:
//
//   FWD  y[pix, o]      = sum_{tap, c} x[pix*s + tap - pad, c] * k[tap, c, o]
//        A: x through a 4-D tiled map with traversal stride s, box (32 c, TW, TH, TN) -> 128 output
//           pixels x 32 channels, K-major; taps that fall outside x are zero-filled by TMA, which is
//           the reference's "skip out-of-range taps" (src/cpu/ops.hxx:236-243).
//        B: k as [tap][c][o], o contiguous -> MN-major tile (32 c x BN o).
//   DX   dx[pix, c]     = sum_{tap, o} dy[(pix + pad - tap)/s, o] * k[tap, c, o]
//        split by output parity class (pix mod s): inside a class the taps with matching parity
//        read a dense, stride-1 window of dy, so none of the 4x multiplications by inserted zeros
//        of the reference's formulation (src/gpu/conv2d_gemm.hh:396-412) is ever issued.
//        A: dy, box (32 o, TW, TH, TN), K-major.  B: k rows c, 32 o contiguous, K-major.
//   DK   dk[tap, c, o]  = sum_{pix} x[pix*s + tap - pad, c] * dy[pix, o]
//        reduction over pixels; both operands have the reduction index outermost in memory, so
//        both tiles are MN-major (32 pixels x 128 channels / BN channels), 5-D maps.
//
// CTA = 320 threads: warp 0 issues TMA, warp 1 owns TMEM and issues tcgen05.mma (both walked by the
// whole warp with one elected lane issuing), warps 2-9 - two per TMEM lane quadrant - drain the
// accumulator (tcgen05.ld) through the fused epilogue (raw / bias / pre-activation / activation /
// activation-gradient gate) into HBM; in the 3xTF32 variant they also build the residual tiles of
// every stage.  A ring of smem stages (A 16 KB + B BN*128 B, 128-byte swizzle; 7 deep with one
// CTA per SM) is handed over with mbarriers: TMA complete_tx -> MMA, tcgen05.commit -> TMA.
// The K partitions of one tile form a thread-block cluster: each writes its fp32 partial tile to
// scratch (L2-resident), the cluster meets at a hardware barrier, and every CTA then adds the
// partials of its share of the tile in partition order (deterministic) and finishes it, fused
// epilogue included - one launch per convolution, no reduction kernel.
//
// Every wait is bounded: a barrier that does not complete within ~1 s makes the waiting role
// record an error code in a device status word and leave; TMEM is always released.
//
// Two specialisations of the same machinery live further down in this file: conv_dxf_kernel (input
// gradient with all parity classes of a pixel tile in one CTA, their accumulators merged into wide
// MMAs) and conv_fwd_short_kernel (the two short-K launches of the 3-channel layers as persistent
// CTAs with resident weights and a double-buffered accumulator).
#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "conv.cuh"

namespace dcg {
namespace {

constexpr int BM = 128;                 // accumulator rows (TMEM lanes)
constexpr int BK = 32;                  // K elements per pipeline stage (one 128-byte swizzle row)
constexpr int A_STAGE_BYTES = BM * BK * 4;
constexpr int kEpi = 256;               // epilogue threads: warps 2..9, two per TMEM lane quadrant
constexpr int kThreads = 64 + kEpi;
constexpr int kMaxSmem = 227 * 1024;
constexpr int kMaxCluster = 8;          // portable thread-block cluster size: the cap on K partitions
// Floats of shared memory the epilogue's transposition buffer takes for a 128 x bn tile (quads at a
// pitch of BM + 1 sixteen-byte units); the row-offset table follows it.
__host__ __device__ constexpr int kRedFloats(int bn) { return (bn / 4) * (BM + 1) * 4; }
constexpr long long kWaitCycles = 2000000000LL;  // default wait limit: ~1 s at 2 GHz

enum Mode { MODE_FWD = 0, MODE_DX = 1, MODE_DK = 2 };

// Error word: [0] code (0 = ok), [1] blockIdx, [2] role, [3] stage.  Read by dcg_device_status().
__device__ int g_tc_status[4];

// Tuning aids, compiled in only with -DDCG_TC_TRACING (the default build has none of it): clock
// stamps of CTA 0's pipeline and a per-CTA phase timeline, read back through dcg_debug_trace /
// dcg_debug_cta_trace; Params::debug bit 0 drops the MMAs, bit 1 the loads (results are garbage).
#ifdef DCG_TC_TRACING
// [0..1023] TMA issue of stage i, [1024..2047] stage i seen full by the MMA thread, [2048..3071] MMAs
// of stage i issued, [3072] kernel entry, [3073] setup done, [3074] accumulator ready, [3075] stores done.
__device__ long long g_tc_trace[3080];
#define TC_TRACE(slot)                                                         \
    do {                                                                       \
        if ((p.debug & 4) && blockIdx.x == 0 && (slot) < 3080) g_tc_trace[(slot)] = clock64(); \
    } while (0)
// global-timer stamps (ns) of thread 64 of the first 1024 CTAs at [0] kernel entry, [1] setup done,
// [2] accumulator ready, [3] tile handed over, [4] partitions met, [5] end; [6] = SM id.
__device__ unsigned long long g_tc_cta_trace[1024][8];
__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define TC_CTA_TRACE(slot)                                                                         \
    do {                                                                                           \
        if ((p.debug & 8) && threadIdx.x == 64 && blockIdx.x < 1024) g_tc_cta_trace[blockIdx.x][(slot)] = global_ns(); \
    } while (0)
#define TC_DEBUG_BIT(bit) (p.debug & (bit))
#else
#define TC_TRACE(slot) do { } while (0)
#define TC_CTA_TRACE(slot) do { } while (0)
#define TC_DEBUG_BIT(bit) false
#endif

struct Params {
    int N, H, W, C, KH, KW, O, Ho, Wo, sh, sw, pt, pl;
    int TW, TH, TN;               // pixel-tile extents (FWD/DX: the 128 rows; DK: the 32-pixel K step)
    int tiles_w, tiles_h, tiles_n;  // pixel tiles along each axis
    int m_tiles;                  // DK: 128-row tiles along the M channel axis
    int n_tiles;                  // BN-column tiles along the N channel axis
    int bn;                       // accumulator columns, multiple of 16, <= 256
    int splits;                   // K partitions of a tile = CTAs per cluster (<= 8)
    int skip_stage;               // test hook: the producer leaves this pipeline stage out (-1: never)
    long long wait_cycles;        // SM clocks after which a barrier wait gives up
    int kchunks;                  // 32-wide chunks along the contracted channel axis (FWD: C, DX: O)
    int swap;                     // DK: M axis is o (A from dy, B from x)
    int narrow;                   // FWD/DK with <= 4 input channels: x is read through the window map
    int ext_finish;               // the K partitions only write partials; a second kernel adds them (narrow DK)
    int planes;                   // FWD: 16-byte column quad q of output pixel r goes to out[(q * pixels + r) * 4]
    int o_store;                  // FWD: output columns >= o_store are padding and never stored (0: store all O)
    int b_direct;                 // short-K GEMM: B is read from k itself, K-major (row = 4 * tap + channel, 32 o per row)
    int x3;                       // 3xTF32: every operand tile gets a residual tile, three MMAs per K step
    unsigned long long plane_stride;  // planes: elements between two quads' planes (4 * pixels)
    int debug;                    // DCG_TC_TRACING builds only: 1 = no MMA, 2 = no TMA, 4 / 8 = record timelines
    int stages;                   // pipeline depth
    float* out;                   // the output tensor
    float* scratch;               // splits > 1: partial tiles, [CTA][128 x bn], quad- or column-major
    EpilogueArgs ep;
};

// ---- PTX wrappers ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Bounded wait, slow path.  Returns false (after recording the failure) if the phase never completes.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, int role, int stage, long long limit)
{
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > limit) break;
    }
    if (atomicCAS(&g_tc_status[0], 0, 1) == 0) {
        g_tc_status[1] = blockIdx.x;
        g_tc_status[2] = role;
        g_tc_status[3] = stage;
    }
    return false;
}

// Bounded wait: a non-blocking probe first (the common case in a running pipeline), then the
// suspending, time-limited loop.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int role, int stage, long long limit)
{
    if (mbar_test_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, role, stage, limit);
}

// Warp-uniform form for loops that a whole warp walks in lockstep (one elected lane issues): the
// vote makes the outcome uniform by construction, which keeps the loop state in uniform registers.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, int role, int stage, long long limit)
{
    if (__all_sync(0xffffffffu, mbar_test_wait(bar, parity))) return true;
    return __all_sync(0xffffffffu, mbar_wait_slow(bar, parity, role, stage, limit));
}

__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ---- thread-block cluster barrier -----------------------------------------------------------------
// The barrier is a hardware one (no time limit can be attached); every thread of every CTA of the
// cluster reaches both of its uses on every path, error paths included.
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3, int c4)
{
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}

__device__ __forceinline__ void tcgen05_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tcgen05_mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                                 uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t* r)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t* r)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}

// 3xTF32: what the TF32 part of a value (its top 19 bits, which is what the tensor core reads) leaves over.
// The residual is itself rounded to nearest TF32 here (the tensor core would truncate it, and a
// truncation error always points the same way, so it would add up over a long reduction).
__device__ __forceinline__ float tf32_residual_1(float v)
{
    const float r = __fsub_rn(v, __uint_as_float(__float_as_uint(v) & 0xFFFFE000u));
    return __uint_as_float((__float_as_uint(r) + 0x1000u) & 0xFFFFE000u);
}
__device__ __forceinline__ float4 tf32_residual(float4 v)
{
    return make_float4(tf32_residual_1(v.x), tf32_residual_1(v.y), tf32_residual_1(v.z), tf32_residual_1(v.w));
}

// Shared-memory operand descriptor (tcgen05): start address, leading / stride byte offsets in
// 16-byte units, version 1, swizzle layout.  Layout 2 = 128-byte swizzle of 16-byte chunks (what
// K-major tiles use); layout 1 = 128-byte swizzle of 32-byte chunks, the only swizzled layout the
// tensor core accepts for MN-major 32-bit (TF32) operands.
constexpr uint32_t kLayoutSw128 = 2, kLayoutSw128Base32 = 1;

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t layout)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version
    d |= (uint64_t)layout << 61;
    return d;
}

// Instruction descriptor: fp32 accumulator, TF32 operands, operand majors, N and M.
__device__ __forceinline__ uint32_t make_idesc(int a_mn_major, int b_mn_major, int n, int m)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn_major << 15) |
           ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

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

// ---- host side: tensor maps ---------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

// dims/strides innermost first; strides[i] is the byte stride of dimension i+1.
int encode_map(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, bool mn_major,
               const cuuint64_t* strides, const cuuint32_t* box, const cuuint32_t* estrides)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(DCG_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<void*>(base), dims,
                          strides, box, estrides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return fail(DCG_ERR_CUDA,
                    "cuTensorMapEncodeTiled failed (%d): rank %d dims [%llu,%llu,%llu,%llu,%llu] box [%u,%u,%u,%u,%u]",
                    (int)r, rank, (unsigned long long)dims[0], (unsigned long long)dims[1],
                    (unsigned long long)(rank > 2 ? dims[2] : 0), (unsigned long long)(rank > 3 ? dims[3] : 0),
                    (unsigned long long)(rank > 4 ? dims[4] : 0), box[0], box[1], rank > 2 ? box[2] : 0,
                    rank > 3 ? box[3] : 0, rank > 4 ? box[4] : 0);
    }
    return DCG_OK;
}

// Activation [N, Hh, Ww, Cc] as a 4-D map (c, w, h, n) with a (32, tw, th, tn)-element box and
// traversal strides (1, sw, sh, 1).
int map_act_4d(CUtensorMap* map, const float* base, int N, int Hh, int Ww, int Cc, int tw, int th, int tn,
               int sw, int sh)
{
    const cuuint64_t dims[4] = {(cuuint64_t)Cc, (cuuint64_t)Ww, (cuuint64_t)Hh, (cuuint64_t)N};
    const cuuint64_t strides[3] = {(cuuint64_t)Cc * 4, (cuuint64_t)Ww * Cc * 4, (cuuint64_t)Hh * Ww * Cc * 4};
    const cuuint32_t box[4] = {32, (cuuint32_t)(tw * sw), (cuuint32_t)(th * sh), (cuuint32_t)tn};
    const cuuint32_t es[4] = {1, (cuuint32_t)sw, (cuuint32_t)sh, 1};
    return encode_map(map, base, 4, dims, false, strides, box, es);
}

// Activation [N, Hh, Ww, Cc] as a 5-D map (c%32, w, h, n, c/32): box (32, tw, th, tn, chunks) lands in
// shared memory as [chunk][pixel][32 channels], the MN-major operand layout.
int map_act_5d(CUtensorMap* map, const float* base, int N, int Hh, int Ww, int Cc, int tw, int th, int tn,
               int sw, int sh, int chunks)
{
    const cuuint64_t dims[5] = {32, (cuuint64_t)Ww, (cuuint64_t)Hh, (cuuint64_t)N, (cuuint64_t)(Cc / 32)};
    const cuuint64_t strides[4] = {(cuuint64_t)Cc * 4, (cuuint64_t)Ww * Cc * 4, (cuuint64_t)Hh * Ww * Cc * 4, 128};
    const cuuint32_t box[5] = {32, (cuuint32_t)(tw * sw), (cuuint32_t)(th * sh), (cuuint32_t)tn, (cuuint32_t)chunks};
    const cuuint32_t es[5] = {1, (cuuint32_t)sw, (cuuint32_t)sh, 1, 1};
    return encode_map(map, base, 5, dims, true, strides, box, es);
}

int pow2_ceil(int v)
{
    int r = 1;
    while (r < v) r <<= 1;
    return r;
}

// 128 (or `total`) pixels as a (tw, th, tn) box: w first, then h, then images.
void pixel_tile(int total, int Wd, int Hd, int& tw, int& th, int& tn)
{
    tw = pow2_ceil(Wd); if (tw > total) tw = total;
    th = pow2_ceil(Hd); if (th > total / tw) th = total / tw;
    tn = total / (tw * th);
}

struct Plan {
    Params p;
    int grid;
    size_t smem;
    // scratch layout: [partial tiles of the K partitions][padded 4-channel input xp][repacked weights
    // k4], each part 256-byte aligned; the last two only exist for narrow-channel layers
    size_t partial_bytes = 0, xp_bytes = 0, k4_bytes = 0, ws_bytes = 0;
    int Hp = 0, Wp = 0;   // padded input extent of a narrow-channel layer
    // DX of a narrow-channel layer (GEMM + gather): p describes the 1x1 FWD problem; the transposed
    // weights k2 and the GEMM result ycol follow the partial tiles in the scratch area
    int Jp = 0;
    size_t k2_bytes = 0, ycol_bytes = 0;
    size_t k2_off() const { return align_up(partial_bytes, 256); }
    size_t ycol_off() const { return k2_off() + align_up(k2_bytes, 256); }
    size_t xp_off() const { return align_up(partial_bytes, 256); }
    size_t k4_off() const { return xp_off() + align_up(xp_bytes, 256); }
};

// DCG_TC_SPLITS / DCG_TC_STAGES (environment, read once) pin the K partitioning and the pipeline
// depth for experiments; unset or 0 leaves the heuristics below in charge.
int env_int(const char* name)
{
    const char* v = getenv(name);
    return v ? atoi(v) : 0;
}

// Set by the entry points for the duration of a call: plan for the 3xTF32 variant.
thread_local int t_plan_x3 = 0;
struct PlanX3 {
    int saved;
    explicit PlanX3(bool x3) : saved(t_plan_x3) { t_plan_x3 = x3 ? 1 : 0; }
    ~PlanX3() { t_plan_x3 = saved; }
};

// Accumulator width for a layer with n_ch output columns.  (256-column tiles halve how often an A
// tile is fetched from L2 but leave one CTA per SM with nothing to overlap its set-up and epilogue
// with: measured slower at batch 64, the 256 -> 512 forward layer 38 us against 23 us.)
int tile_width(int n_ch) { return n_ch >= 128 ? 128 : n_ch; }

// K partitions of a tile.  Measured on every DCGAN layer at batch 64 (per-CTA timelines, partition
// counts 1..8 forced): the shortest launch is the one with about ONE CTA per SM - a deeper pipeline
// per CTA and half the partial-tile traffic beat a second resident CTA (e.g. the 256 -> 512 forward
// layer: 18.5 us with 4 partitions = 128 CTAs against 22.3 us with 8 = 256; the 64 -> 128 kernel gradient with
// the channel roles swapped: 25.0 us with 25 taps x 5 = 125 CTAs against 27.0 us with 25 x 8 = 200, 39.8 us
// against 46.7 us over 128 images).
int choose_splits(int tiles, int min_stages_per_tile, int ctas_per_sm = 1)
{
    static const int forced = env_int("DCG_TC_SPLITS");
    if (forced > 0) {
        int f = forced <= min_stages_per_tile ? forced : (min_stages_per_tile > 0 ? min_stages_per_tile : 1);
        return f > kMaxCluster ? kMaxCluster : f;
    }
    const int sms = sm_count();
    if (t_plan_x3) {
        // 3xTF32: as many partitions as the cluster allows - each accumulation chain in the tensor
        // core gets shorter, and the partitions are added in fp32 round-to-nearest
        int s = min_stages_per_tile / 4;
        if (s > kMaxCluster) s = kMaxCluster;
        return s < 1 ? 1 : s;
    }
    if (tiles >= sms) return 1;
    int s = (ctas_per_sm * sms) / tiles;
    const int cap = min_stages_per_tile / 4;         // keep at least 4 K stages per CTA
    if (s > cap) s = cap;
    if (s > kMaxCluster) s = kMaxCluster;
    return s < 1 ? 1 : s;
}

void finish_plan(Plan& pl)
{
    Params& p = pl.p;
    const int b_stage = p.bn * BK * 4;
    const int per_stage = (A_STAGE_BYTES + b_stage) * (p.x3 ? 2 : 1);   // 3xTF32: operand + residual tiles
    // two CTAs per SM when the grid has more CTAs than SMs, else one deep pipeline
    const int budget = (pl.grid > sm_count() && p.bn <= 128 && !p.x3) ? (kMaxSmem / 2 - 2048) : (kMaxSmem - 2048);
    int stages = budget / per_stage;
    if (stages > 8) stages = 8;
    static const int forced_stages = env_int("DCG_TC_STAGES");
    if (forced_stages > 0 && forced_stages < stages) stages = forced_stages;
    if (stages < 2) stages = 2;
    // the epilogue parks the 128 x bn tile (padded rows) and 128 row offsets in the (by then idle) stage ring
    while ((size_t)stages * per_stage < (size_t)kRedFloats(p.bn) * 4 + BM * 8) ++stages;
    p.stages = stages;
#ifdef DCG_TC_TRACING
    static const int debug = env_int("DCG_TC_DEBUG");
    p.debug = debug;
#endif
    pl.smem = (size_t)stages * per_stage + 1024 /*alignment slack*/ + 24 * stages + 32;
    p.skip_stage = -1;
    p.wait_cycles = kWaitCycles;
    pl.partial_bytes = p.splits > 1 ? (size_t)pl.grid * BM * p.bn * sizeof(float) : 0;
    pl.ws_bytes = pl.partial_bytes;
    if (pl.xp_bytes || pl.k4_bytes) pl.ws_bytes = pl.k4_off() + align_up(pl.k4_bytes, 256);
    if (pl.ycol_bytes) pl.ws_bytes = pl.ycol_off() + align_up(pl.ycol_bytes, 256);
}

// Padded-image geometry of a narrow-channel layer: rows s*i + di and columns s*j .. s*j + 7 of xp
// must exist for every output pixel and kernel row.
void narrow_geometry(const dcg_conv_desc& d, Plan& pl)
{
    pl.Hp = d.stride_h * (d.ho - 1) + d.kh;
    pl.Wp = (d.stride_w * (d.wo - 1) + 8 + 3) / 4 * 4;
    if (pl.Hp < d.h + d.pad_top) pl.Hp = d.h + d.pad_top;
    if (pl.Wp < d.w + d.pad_left) pl.Wp = (d.w + d.pad_left + 3) / 4 * 4;
    pl.xp_bytes = (size_t)d.n * pl.Hp * pl.Wp * 16;
}

bool narrow_ok(const dcg_conv_desc& d)
{
    return d.c <= 4 && d.kw <= 8 && d.o % 32 == 0 && d.stride_h <= 8 && d.stride_w <= 8;
}

void base_params(Params& p, const dcg_conv_desc& d)
{
    p = Params{};
    p.x3 = t_plan_x3;
    p.N = d.n; p.H = d.h; p.W = d.w; p.C = d.c; p.KH = d.kh; p.KW = d.kw; p.O = d.o;
    p.Ho = d.ho; p.Wo = d.wo; p.sh = d.stride_h; p.sw = d.stride_w; p.pt = d.pad_top; p.pl = d.pad_left;
    p.m_tiles = 1; p.n_tiles = 1; p.splits = 1; p.kchunks = 1;
}

bool plan_fwd(const dcg_conv_desc& d, Plan& pl)
{
    const bool narrow = narrow_ok(d);
    if (!narrow && (d.c % 4 != 0 || d.o % 32 != 0 || d.stride_h > 8 || d.stride_w > 8)) return false;
    Params& p = pl.p;
    base_params(p, d);
    pixel_tile(BM, d.wo, d.ho, p.TW, p.TH, p.TN);
    if (p.TW * d.stride_w > 256 || p.TH * d.stride_h > 256) return false;
    p.tiles_w = (d.wo + p.TW - 1) / p.TW; p.tiles_h = (d.ho + p.TH - 1) / p.TH; p.tiles_n = (d.n + p.TN - 1) / p.TN;
    p.bn = narrow ? (d.o >= 128 ? 128 : d.o) : tile_width(d.o);
    p.n_tiles = (d.o + p.bn - 1) / p.bn;
    p.kchunks = (d.c + BK - 1) / BK;
    const int tiles = p.tiles_w * p.tiles_h * p.tiles_n * p.n_tiles;
    if (narrow) {
        p.narrow = 1;
        p.kchunks = 1;
        narrow_geometry(d, pl);
        pl.k4_bytes = (size_t)d.kh * 32 * d.o * sizeof(float);
    }
    p.splits = choose_splits(tiles, narrow ? d.kh : d.kh * d.kw * p.kchunks);
    pl.grid = tiles * p.splits;
    finish_plan(pl);
    return true;
}

// The 1x1 FWD problem behind the DX of a narrow-channel layer: dy [n, ho, wo, o] times k2 [o][Jp].
dcg_conv_desc dx_gemm_desc(const dcg_conv_desc& d, int Jp)
{
    dcg_conv_desc g{};
    g.n = d.n; g.h = d.ho; g.w = d.wo; g.c = d.o; g.kh = 1; g.kw = 1; g.o = Jp; g.ho = d.ho; g.wo = d.wo;
    g.stride_h = 1; g.stride_w = 1; g.pad_top = 0; g.pad_left = 0;
    return g;
}

bool plan_fwd(const dcg_conv_desc& d, Plan& pl);

bool plan_dx(const dcg_conv_desc& d, Plan& pl)
{
    if (d.c <= 4 && d.o % 32 == 0 && d.stride_h <= d.kh && d.stride_w <= d.kw) {
        const int Jp = (d.kh * d.kw * 4 + 31) / 32 * 32;   // four columns per tap
        pl.Jp = Jp;
        pl.k2_bytes = (size_t)d.o * Jp * sizeof(float);
        pl.ycol_bytes = (size_t)d.n * d.ho * d.wo * Jp * sizeof(float);
        if (plan_fwd(dx_gemm_desc(d, Jp), pl)) {
            pl.p.planes = 1;
            pl.p.plane_stride = (unsigned long long)d.n * d.ho * d.wo * 4ull;
            pl.p.o_store = d.kh * d.kw * 4;   // the planes beyond the last tap are padding
            return true;
        }
        pl = Plan{};
    }
    if (d.o % 4 != 0 || d.stride_h > 8 || d.stride_w > 8) return false;
    if (d.stride_h > d.kh || d.stride_w > d.kw) return false;   // some parity class would have no tap
    Params& p = pl.p;
    base_params(p, d);
    const int ha = (d.h + d.stride_h - 1) / d.stride_h, wa = (d.w + d.stride_w - 1) / d.stride_w;
    pixel_tile(BM, wa, ha, p.TW, p.TH, p.TN);
    p.tiles_w = (wa + p.TW - 1) / p.TW; p.tiles_h = (ha + p.TH - 1) / p.TH; p.tiles_n = (d.n + p.TN - 1) / p.TN;
    int bn = (d.c + 15) / 16 * 16;
    if (bn > 128) bn = tile_width(bn);
    p.bn = bn;
    p.n_tiles = (d.c + p.bn - 1) / p.bn;
    p.kchunks = (d.o + BK - 1) / BK;
    const int classes = d.stride_h * d.stride_w;
    const int tiles = classes * p.tiles_w * p.tiles_h * p.tiles_n * p.n_tiles;
    const int min_taps = (d.kh / d.stride_h) * (d.kw / d.stride_w);
    p.splits = choose_splits(tiles, (min_taps < 1 ? 1 : min_taps) * p.kchunks);
    pl.grid = tiles * p.splits;
    finish_plan(pl);
    return true;
}

// When the input gradient fuses its parity classes (conv_dxf_kernel): 0 never, 1 where one CTA per tile fills the
// GPU (default), 2 wherever the shape allows.  DCG_TC_DXF sets the default, dcg_debug_set_dx_mode overrides it.
std::atomic<int> g_dxf_mode{-1};
std::atomic<unsigned long long> g_dxf_launches{0};
int dxf_mode()
{
    static const int from_env = [] { const char* v = getenv("DCG_TC_DXF"); return v ? atoi(v) : 1; }();
    const int m = g_dxf_mode.load();
    return m >= 0 ? m : from_env;
}

// The class-fused input gradient (conv_dxf_kernel): windows of dy, the (class, tap) pairs that read each, and
// the order of both.
bool plan_dxf(const dcg_conv_desc& d, Plan& pl, CfTable& t)
{
    const int mode = dxf_mode();
    if (mode == 0 || t_plan_x3) return false;
    if (d.o % 4 != 0) return false;   // rows of dy and of the weights are 16-byte aligned for TMA
    // <= 4 input channels: a tile is 18 short stages and four element-wise epilogues - measured at 46 us against
    // 25 us for GEMM + gather on the 3-channel layer at batch 64 (one CTA per SM has nothing to hide its set-up behind)
    if (d.c <= 4) return false;
    if (d.stride_h > d.kh || d.stride_w > d.kw) return false;
    const int ncls = d.stride_h * d.stride_w;
    if (ncls < 2 || ncls > 4) return false;
    Params& p = pl.p;
    base_params(p, d);
    const int ha = (d.h + d.stride_h - 1) / d.stride_h, wa = (d.w + d.stride_w - 1) / d.stride_w;
    pixel_tile(BM, wa, ha, p.TW, p.TH, p.TN);
    p.tiles_w = (wa + p.TW - 1) / p.TW; p.tiles_h = (ha + p.TH - 1) / p.TH; p.tiles_n = (d.n + p.TN - 1) / p.TN;
    int bn = (d.c + 15) / 16 * 16;
    if (bn > 128) bn = 128;
    if (ncls * bn > 512) return false;
    p.bn = bn;
    p.n_tiles = (d.c + bn - 1) / bn;
    p.kchunks = (d.o + BK - 1) / BK;
    const int tiles = p.tiles_w * p.tiles_h * p.tiles_n * p.n_tiles;
    // one CTA per tile, no K partitions: only where the tiles alone fill (most of) the GPU
    if (mode != 2 && tiles * 4 < sm_count() * 3) return false;
    // every (class, tap) pair with the window it reads
    struct Pair { int sy, sx, cls, kh, kw; };
    std::vector<Pair> pairs;
    for (int ph = 0; ph < d.stride_h; ++ph)
        for (int pw = 0; pw < d.stride_w; ++pw) {
            const int rh = (ph + d.pad_top) % d.stride_h, eh = (ph + d.pad_top) / d.stride_h;
            const int rw = (pw + d.pad_left) % d.stride_w, ew = (pw + d.pad_left) / d.stride_w;
            for (int a = 0; rh + d.stride_h * a < d.kh; ++a)
                for (int b = 0; rw + d.stride_w * b < d.kw; ++b)
                    pairs.push_back({eh - a, ew - b, ph * d.stride_w + pw, rh + d.stride_h * a, rw + d.stride_w * b});
        }
    // classes in the order "fewest windows still to fetch first"; the windows follow that order
    t = CfTable{};
    t.ncls = ncls;
    std::vector<std::pair<int, int>> wins;   // scheduled windows
    auto scheduled = [&](int sy, int sx) {
        for (auto& w : wins) if (w.first == sy && w.second == sx) return true;
        return false;
    };
    bool finished[4] = {false, false, false, false};
    for (int ci = 0; ci < ncls; ++ci) {
        int best = -1, best_need = 1 << 30;
        for (int c = 0; c < ncls; ++c) {
            if (finished[c]) continue;
            std::vector<std::pair<int, int>> need;
            for (auto& q : pairs)
                if (q.cls == c && !scheduled(q.sy, q.sx)) {
                    bool seen = false;
                    for (auto& n : need) seen |= n.first == q.sy && n.second == q.sx;
                    if (!seen) need.push_back({q.sy, q.sx});
                }
            if ((int)need.size() < best_need) { best_need = (int)need.size(); best = c; }
        }
        if (best < 0) return false;
        bool any = false;
        for (auto& q : pairs)
            if (q.cls == best) {
                any = true;
                if (!scheduled(q.sy, q.sx)) wins.push_back({q.sy, q.sx});
            }
        if (!any) return false;   // a class without taps
        finished[best] = true;
        t.order[ci] = best;
    }
    // stages: a window with its pairs, at most pb per stage (the stage ring holds about 48 KB per stage)
    const int b_tile = bn * BK * 4;
    int pb = (48 * 1024 - A_STAGE_BYTES) / b_tile;
    if (pb > 4) pb = 4;
    if (pb < 1) pb = 1;
    // TMEM order of the classes: for 2 x 2 classes the cyclic order (0,0) (0,1) (1,1) (1,0), in which the classes
    // of one row / one column parity are neighbours, so that the pairs of a window merge into wide MMAs
    for (int c = 0; c < ncls; ++c) t.slot_of_class[c] = c;
    if (d.stride_h == 2 && d.stride_w == 2) { t.slot_of_class[2] = 3; t.slot_of_class[3] = 2; }
    int last_stage[4] = {-1, -1, -1, -1}, last_pair[4] = {0, 0, 0, 0};
    bool started[4] = {false, false, false, false};
    int ns = 0;
    for (size_t w = 0; w < wins.size(); ++w) {
        if (wins[w].first < -128 || wins[w].first > 127 || wins[w].second < -128 || wins[w].second > 127) return false;
        // the pairs of this window in TMEM order
        std::vector<Pair> mine;
        for (auto& q : pairs)
            if (q.sy == wins[w].first && q.sx == wins[w].second) mine.push_back(q);
        for (size_t a = 0; a < mine.size(); ++a)
            for (size_t b = a + 1; b < mine.size(); ++b)
                if (t.slot_of_class[mine[b].cls] < t.slot_of_class[mine[a].cls]) std::swap(mine[a], mine[b]);
        for (size_t first = 0; first < mine.size(); first += pb) {
            if (ns == 32) return false;
            CfWin& cw = t.win[ns];
            cw.sy = (signed char)wins[w].first; cw.sx = (signed char)wins[w].second;
            const size_t end = std::min(mine.size(), first + (size_t)pb);
            int group_start = -1;
            for (size_t a = first; a < end; ++a) {
                const Pair& q = mine[a];
                const int j = cw.n;
                const int slot = t.slot_of_class[q.cls];
                const bool fresh = !started[q.cls];
                cw.cls[j] = (unsigned char)q.cls; cw.kh[j] = (unsigned char)q.kh; cw.kw[j] = (unsigned char)q.kw;
                cw.slot[j] = (unsigned char)slot;
                if (fresh) cw.fresh |= (unsigned char)(1u << j);
                // joins the running MMA if its accumulator follows directly, starts the same way and N stays <= 256
                const bool join = group_start >= 0 && cw.slot[j - 1] + 1 == slot &&
                                  (((cw.fresh >> group_start) & 1u) != 0) == fresh &&
                                  (cw.glen[group_start] + 1) * bn <= 256;
                if (join) ++cw.glen[group_start];
                else { group_start = j; cw.glen[j] = 1; }
                last_stage[q.cls] = ns; last_pair[q.cls] = j;
                ++cw.n;
            }
            for (int j = 0; j < cw.n; ++j) started[cw.cls[j]] = true;
            ++ns;
        }
    }
    t.nwin = ns;
    for (int c = 0; c < ncls; ++c) {
        if (last_stage[c] < 0) return false;
        t.win[last_stage[c]].last |= (unsigned char)(1u << last_pair[c]);
    }
    t.slot_bytes = A_STAGE_BYTES + pb * b_tile;
    p.splits = 1;
    pl.grid = tiles;
    int stages = (kMaxSmem - 1024 - kCfRedBytes() - 256) / t.slot_bytes;
    if (stages > 8) stages = 8;
    if (stages < 3) return false;
    p.stages = stages;
    pl.smem = (size_t)stages * t.slot_bytes + 1024 + kCfRedBytes() + 16 * stages + 64;
    p.skip_stage = -1;
    p.wait_cycles = kWaitCycles;
    pl.partial_bytes = 0;
    pl.ws_bytes = 0;
    return true;
}

bool plan_dk(const dcg_conv_desc& d, Plan& pl)
{
    const bool narrow = narrow_ok(d);
    if (!narrow && (d.c % 32 != 0 || d.o % 32 != 0 || d.stride_h > 8 || d.stride_w > 8)) return false;
    Params& p = pl.p;
    base_params(p, d);
    pixel_tile(BK, d.wo, d.ho, p.TW, p.TH, p.TN);   // 32 output pixels per K stage
    if (p.TW * d.stride_w > 256 || p.TH * d.stride_h > 256) return false;
    p.tiles_w = (d.wo + p.TW - 1) / p.TW; p.tiles_h = (d.ho + p.TH - 1) / p.TH; p.tiles_n = (d.n + p.TN - 1) / p.TN;
    if (narrow) {
        // rows = output channels (from dy), columns = 32 window slots per kernel row: one tile holds
        // all of dk, so dy is read exactly once; the parallelism comes from partitioning the pixels
        // over about as many CTAs as there are SMs, whose partial tiles a second kernel adds up
        if (d.kh * 32 > 256) return false;
        p.narrow = 1;
        p.swap = 1;
        p.m_tiles = (d.o + BM - 1) / BM;
        p.bn = 32 * d.kh;
        p.n_tiles = 1;
        narrow_geometry(d, pl);
        const int k_stages = p.tiles_w * p.tiles_h * p.tiles_n;
        int parts = sm_count() / p.m_tiles;
        if (parts > k_stages / 4) parts = k_stages / 4;   // at least 4 K stages per CTA
        if (parts < 1) parts = 1;
        p.splits = parts;
        p.ext_finish = parts > 1 ? 1 : 0;
        pl.grid = p.m_tiles * p.splits;
        finish_plan(pl);
        return true;
    }
    // M (128 accumulator rows) is the input-channel axis - dk rows are then contiguous along the
    // accumulator columns - unless that would leave the M tile part empty and o can fill it
    p.swap = (d.c < BM && d.o > d.c) ? 1 : 0;
    const int m_ch = p.swap ? d.o : d.c, n_ch = p.swap ? d.c : d.o;
    p.m_tiles = (m_ch + BM - 1) / BM;
    p.bn = tile_width(n_ch);
    p.n_tiles = (n_ch + p.bn - 1) / p.bn;
    const int tiles = d.kh * d.kw * p.m_tiles * p.n_tiles;
    p.splits = choose_splits(tiles, p.tiles_w * p.tiles_h * p.tiles_n);
    pl.grid = tiles * p.splits;
    finish_plan(pl);
    return true;
}

bool make_plan(const dcg_conv_desc& d, int kind, Plan& pl)
{
    switch (kind) {
    case kConvFwd: return plan_fwd(d, pl);
    case kConvDx: return plan_dx(d, pl);
    case kConvDk: return plan_dk(d, pl);
    default: return false;
    }
}

// Testing hooks (dcg_debug_set_wait_limit / dcg_debug_skip_stage): the wait limit of every barrier
// wait in SM clocks, and a pipeline stage the producer leaves out so that a wait runs into that limit.
long long default_wait_cycles()
{
    const char* v = getenv("DCG_TC_WAIT_CYCLES");   // experiments: a shorter limit than the ~1 s default
    const long long c = v ? atoll(v) : 0;
    return c > 0 ? c : kWaitCycles;
}
std::atomic<long long> g_wait_cycles{default_wait_cycles()};
std::atomic<int> g_test_skip_stage{-1};

template <int MODE>
int launch_grid(const CUtensorMap& ma, const CUtensorMap& mb, const Params& p, int grid, size_t smem, cudaStream_t stream)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    static const int no_pdl = env_int("DCG_TC_NO_PDL");
    if (!no_pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (p.splits > 1 && !p.ext_finish) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = (unsigned)p.splits;   // blockIdx.x = tile * splits + split: one cluster per tile
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    const cudaError_t err = p.x3 ? cudaLaunchKernelEx(&cfg, conv_tc_kernel<MODE, true>, ma, mb, p)
                                 : cudaLaunchKernelEx(&cfg, conv_tc_kernel<MODE, false>, ma, mb, p);
    if (err != cudaSuccess) return fail(DCG_ERR_CUDA, "conv_tc_kernel launch: %s", cudaGetErrorString(err));
    count_launch();
    return DCG_OK;
}

template <int MODE>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, Plan& pl, float* out, const EpilogueArgs& ep,
           int channels, void* ws, size_t ws_bytes, cudaStream_t stream)
{
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(conv_tc_kernel<MODE, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
        if (attr_err == cudaSuccess)
            attr_err = cudaFuncSetAttribute(conv_tc_kernel<MODE, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
    });
    if (attr_err != cudaSuccess)
        return fail(DCG_ERR_CUDA, "cudaFuncSetAttribute(conv_tc_kernel): %s", cudaGetErrorString(attr_err));
    Params& p = pl.p;
    p.out = out;
    p.ep = ep;
    p.scratch = nullptr;
    p.skip_stage = g_test_skip_stage.load();
    p.wait_cycles = g_wait_cycles.load();
    if (p.splits > 1) {
        if (!ws || ws_bytes < pl.ws_bytes)
            return fail(DCG_ERR_WORKSPACE, "conv (tensor path): workspace %zu < %zu bytes", ws_bytes, pl.ws_bytes);
        p.scratch = static_cast<float*>(ws);
    }
    (void)channels;
    const int st = launch_grid<MODE>(ma, mb, p, pl.grid, pl.smem, stream);
    if (st) return st;
    if (p.ext_finish) {
        const dim3 fgrid((unsigned)p.bn, (unsigned)((p.O + 31) / 32));
        launch_pdl(dk_narrow_finish_kernel, fgrid, 256, 0, stream, p.scratch, out, p.splits, p.bn, p.KH, p.KW, p.C, p.O);
        DCG_LAUNCH_CHECK("dk_narrow_finish_kernel");
    }
    return DCG_OK;
}

struct Prepared;
int launch_dxf(Prepared& pr, float* out, const EpilogueArgs& ep, cudaStream_t stream);
bool short_ok(const Plan& pl);
int launch_short(Prepared& pr, bool narrow, float* out, const EpilogueArgs& ep, cudaStream_t stream);
int launch_dx3(Prepared& pr, float* out, const EpilogueArgs& ep, cudaStream_t stream);

// Narrow-channel layers: builds the padded 4-channel image (and, for FWD, the repacked weights) in
// the caller's scratch and returns their addresses.
int narrow_prepare(const dcg_conv_desc& d, const Plan& pl, const float* x, const float* k, void* ws, size_t ws_bytes,
                   cudaStream_t stream, float** xp_out, float** k4_out)
{
    if (!ws || ws_bytes < pl.ws_bytes)
        return fail(DCG_ERR_WORKSPACE, "conv (tensor path, narrow input): workspace %zu < %zu bytes", ws_bytes, pl.ws_bytes);
    uint8_t* base = static_cast<uint8_t*>(ws);
    float* xp = reinterpret_cast<float*>(base + pl.xp_off());
    const size_t pixels = (size_t)d.n * pl.Hp * pl.Wp;
    size_t blocks = (pixels + 255) / 256;
    const size_t cap = (size_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    *xp_out = xp;
    if (k4_out) {   // forward: image and weights in one launch
        float* k4 = reinterpret_cast<float*>(base + pl.k4_off());
        const int total = d.kh * 32 * d.o;
        const int k4_blocks = (total + 255) / 256;
        launch_pdl(repack_narrow_k4_kernel, (unsigned)(blocks + k4_blocks), 256, 0, stream, x, reinterpret_cast<float4*>(xp),
                   d.n, d.h, d.w, d.c, pl.Hp, pl.Wp, d.pad_top, d.pad_left, k, k4, d.kh, d.kw, d.o, k4_blocks);
        DCG_LAUNCH_CHECK("repack_narrow_k4_kernel");
        *k4_out = k4;
    } else {
        launch_pdl(repack_narrow_kernel, (unsigned)blocks, 256, 0, stream, x, reinterpret_cast<float4*>(xp), d.n, d.h, d.w,
                   d.c, pl.Hp, pl.Wp, d.pad_top, d.pad_left);
        DCG_LAUNCH_CHECK("repack_narrow_kernel");
    }
    return DCG_OK;
}

// The overlapping-window view of xp [n][Hp][Wp][4]: (32 floats, j, i, n, kernel row) where output
// pixel (i, j) and kernel row r address xp[n][s*i + r][s*j][0].  Box (32, tw, th, tn, rows).
int map_window(CUtensorMap* map, const float* xp, const dcg_conv_desc& d, const Plan& pl, int tw, int th, int tn,
               bool mn_major, int rows)
{
    const cuuint64_t row = (cuuint64_t)pl.Wp * 16;
    const cuuint64_t dims[5] = {32, (cuuint64_t)d.wo, (cuuint64_t)d.ho, (cuuint64_t)d.n, (cuuint64_t)d.kh};
    const cuuint64_t strides[4] = {(cuuint64_t)d.stride_w * 16, (cuuint64_t)d.stride_h * row, (cuuint64_t)pl.Hp * row, row};
    const cuuint32_t box[5] = {32, (cuuint32_t)tw, (cuuint32_t)th, (cuuint32_t)tn, (cuuint32_t)rows};
    const cuuint32_t es[5] = {1, 1, 1, 1, 1};
    return encode_map(map, xp, 5, dims, mn_major, strides, box, es);
}

// ---- prepared calls: plan + tensor maps, cached ------------------------------------------------------
// Planning a convolution and encoding its two tensor maps costs the host ~10 us.  A training step
// or the reference's Graph::run issues the same convolutions on the same buffers over and over, so
// the result is kept per (device, operator, shape, operand addresses, scratch address, precision)
// in a small table; a hit leaves only the launch.
struct Prepared {
    Plan pl;
    CUtensorMap ma, mb;
    bool dxf = false;   // input gradient with the parity classes fused (conv_dxf_kernel); cf is its table
    CfTable cf;
    bool dx3 = false;   // input gradient of a <= 4-channel layer as one GEMM + gather kernel (conv_dx3_kernel)
    Dx3Args dx3_args;
};

int launch_dxf(Prepared& pr, float* out, const EpilogueArgs& ep, cudaStream_t stream)
{
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(conv_dxf_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
    });
    if (attr_err != cudaSuccess)
        return fail(DCG_ERR_CUDA, "cudaFuncSetAttribute(conv_dxf_kernel): %s", cudaGetErrorString(attr_err));
    Params& p = pr.pl.p;
    p.out = out;
    p.ep = ep;
    p.scratch = nullptr;
    p.wait_cycles = g_wait_cycles.load();
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)pr.pl.grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = pr.pl.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    int na = 0;
    static const int no_pdl = env_int("DCG_TC_NO_PDL");
    if (!no_pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, conv_dxf_kernel, pr.ma, pr.mb, p, pr.cf);
    if (err != cudaSuccess) return fail(DCG_ERR_CUDA, "conv_dxf_kernel launch: %s", cudaGetErrorString(err));
    count_launch();
    g_dxf_launches.fetch_add(1);
    return DCG_OK;
}

// Whether a forward plan goes to the persistent short-K kernel: a single column tile, no K partitions, weights
// that fit the resident area, more tiles than SMs (else there is nothing to walk).  DCG_TC_SHORT=0 switches it off.
bool short_ok(const Plan& pl)
{
    static const int off = [] { const char* v = getenv("DCG_TC_SHORT"); return v && atoi(v) == 0 ? 1 : 0; }();
    const Params& p = pl.p;
    if (off || p.x3 || p.splits != 1 || p.n_tiles != 1 || p.bn > 128 || p.bn % 32 != 0) return false;
    const int ksteps = p.narrow ? p.KH : p.KH * p.KW * p.kchunks;
    if (!p.narrow && (p.KH != 1 || p.KW != 1 || !p.planes)) return false;   // the GEMM of the 3-channel input gradient
    if (p.narrow && p.planes) return false;
    if (ksteps < 1 || ksteps * p.bn * BK * 4 > kShortMaxB) return false;
    return pl.grid > sm_count();
}

int launch_short(Prepared& pr, bool narrow, float* out, const EpilogueArgs& ep, cudaStream_t stream)
{
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(conv_fwd_short_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem / 2);
        if (attr_err == cudaSuccess)
            attr_err = cudaFuncSetAttribute(conv_fwd_short_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem / 2);
    });
    if (attr_err != cudaSuccess)
        return fail(DCG_ERR_CUDA, "cudaFuncSetAttribute(conv_fwd_short_kernel): %s", cudaGetErrorString(attr_err));
    Params& p = pr.pl.p;
    p.out = out;
    p.ep = ep;
    p.scratch = nullptr;
    p.wait_cycles = g_wait_cycles.load();
    const int tiles = pr.pl.grid;
    const int ksteps = narrow ? p.KH : p.kchunks;
    int grid = 2 * sm_count();
    if (grid > tiles) grid = tiles;
    p.stages = narrow ? 3 : kShortMaxStages;
    const size_t smem = 1024 + (size_t)ksteps * p.bn * BK * 4 + (size_t)p.stages * A_STAGE_BYTES +
                        (narrow ? (size_t)(kEpi / 32) * kPatchBytes : 0) + 16 * kShortMaxStages + 64;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    int na = 0;
    static const int no_pdl = env_int("DCG_TC_NO_PDL");
    if (!no_pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    const cudaError_t err = narrow ? cudaLaunchKernelEx(&cfg, conv_fwd_short_kernel<true>, pr.ma, pr.mb, p, tiles, ksteps)
                                   : cudaLaunchKernelEx(&cfg, conv_fwd_short_kernel<false>, pr.ma, pr.mb, p, tiles, ksteps);
    if (err != cudaSuccess) return fail(DCG_ERR_CUDA, "conv_fwd_short_kernel launch: %s", cudaGetErrorString(err));
    count_launch();
    return DCG_OK;
}

// GEMM + gather in one kernel for the input gradient of a <= 4-channel layer (conv_dx3_kernel): stride 2, at most
// 32 taps, dy rows of at most 32 pixels and at most 64 channels (the resident weights and the products of a tile
// share the CTA's shared memory).  DCG_TC_DX3=0 switches it off.
bool plan_dx3(const dcg_conv_desc& d, Plan& pl, Dx3Args& g)
{
    static const int off = [] { const char* v = getenv("DCG_TC_DX3"); return v && atoi(v) == 0 ? 1 : 0; }();
    if (off || t_plan_x3) return false;
    if (d.c > 4 || d.stride_h != 2 || d.stride_w != 2 || d.kh * d.kw > 32 || d.kh < 2 || d.kw < 2) return false;
    if (d.o % 32 != 0 || d.o > 64 || d.wo > 32 || d.pad_top >= d.kh || d.pad_left >= d.kw) return false;
    // the most output rows (2R) whose contributing dy rows fit the 8 rows of a tile
    int R = 0, lo = 0;
    for (int r = kDx3Rows; r >= 1 && R == 0; --r) {
        int mn = 1 << 30, mx = -(1 << 30);
        for (int hl = 0; hl < 2 * r; ++hl)
            for (int di = (hl + d.pad_top) & 1; di < d.kh; di += 2) {
                const int v = hl + d.pad_top - di;
                const int i = v >= 0 ? v / 2 : -((-v + 1) / 2);   // floor
                if (i < mn) mn = i;
                if (i > mx) mx = i;
            }
        if (mx - mn + 1 <= kDx3Rows) { R = r; lo = mn; }
    }
    if (R == 0) return false;
    Params& p = pl.p;
    base_params(p, d);
    p.kchunks = d.o / BK;
    p.bn = 128;
    p.splits = 1;
    p.skip_stage = -1;
    p.wait_cycles = kWaitCycles;
    g.R = R;
    g.lo = lo;
    g.tiles_per_img = (d.h + 2 * R - 1) / (2 * R);
    g.tiles = d.n * g.tiles_per_img;
    pl.grid = g.tiles < sm_count() ? g.tiles : sm_count();
    pl.smem = 1024 + (size_t)p.kchunks * 128 * BK * 4 + (size_t)kDx3Stages * A_STAGE_BYTES +
              (size_t)d.kh * d.kw * kDx3Rows * 32 * 16 + 16 * kDx3Stages + 64;
    pl.ws_bytes = 0;
    return pl.smem <= (size_t)kMaxSmem;
}

int launch_dx3(Prepared& pr, float* out, const EpilogueArgs& ep, cudaStream_t stream)
{
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(conv_dx3_kernel<5, 5>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
        if (attr_err == cudaSuccess)
            attr_err = cudaFuncSetAttribute(conv_dx3_kernel<0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
    });
    if (attr_err != cudaSuccess)
        return fail(DCG_ERR_CUDA, "cudaFuncSetAttribute(conv_dx3_kernel): %s", cudaGetErrorString(attr_err));
    Params& p = pr.pl.p;
    p.out = out;
    p.ep = ep;
    p.scratch = nullptr;
    p.wait_cycles = g_wait_cycles.load();
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)pr.pl.grid);
    cfg.blockDim = dim3(kDx3Threads);
    cfg.dynamicSmemBytes = pr.pl.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    int na = 0;
    static const int no_pdl = env_int("DCG_TC_NO_PDL");
    if (!no_pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    const cudaError_t err = (p.KH == 5 && p.KW == 5)
                                ? cudaLaunchKernelEx(&cfg, conv_dx3_kernel<5, 5>, pr.ma, pr.mb, p, pr.dx3_args)
                                : cudaLaunchKernelEx(&cfg, conv_dx3_kernel<0, 0>, pr.ma, pr.mb, p, pr.dx3_args);
    if (err != cudaSuccess) return fail(DCG_ERR_CUDA, "conv_dx3_kernel launch: %s", cudaGetErrorString(err));
    count_launch();
    return DCG_OK;
}

struct CacheKey {
    int dev, kind, x3;
    dcg_conv_desc d;
    const void *a, *b, *ws;
    size_t ws_bytes;
};

struct CacheEntry {
    CacheKey key;
    Prepared prep;
};

constexpr size_t kCacheEntries = 512;
std::mutex g_cache_mutex;
std::vector<CacheEntry> g_cache;
size_t g_cache_next = 0;

bool same_key(const CacheKey& u, const CacheKey& v)
{
    return u.dev == v.dev && u.kind == v.kind && u.x3 == v.x3 && u.a == v.a && u.b == v.b &&
           u.ws == v.ws && u.ws_bytes == v.ws_bytes && std::memcmp(&u.d, &v.d, sizeof(dcg_conv_desc)) == 0;
}

// FWD: plan and maps for y = conv(x, k).  xp / k4 of a narrow-channel layer live in the scratch.
int build_fwd(const dcg_conv_desc& d, const float* x, const float* k, void* ws, size_t ws_bytes, Prepared& pr)
{
    Plan& pl = pr.pl;
    if (!plan_fwd(d, pl)) return fail(DCG_ERR_UNSUPPORTED, "conv fwd: shape not supported by the tensor path");
    const Params& p = pl.p;
    int st;
    if (p.narrow) {
        if (!ws || ws_bytes < pl.ws_bytes)
            return fail(DCG_ERR_WORKSPACE, "conv (tensor path, narrow input): workspace %zu < %zu bytes", ws_bytes, pl.ws_bytes);
        uint8_t* base = static_cast<uint8_t*>(ws);
        const float* xp = reinterpret_cast<const float*>(base + pl.xp_off());
        const float* k4 = reinterpret_cast<const float*>(base + pl.k4_off());
        if ((st = map_window(&pr.ma, xp, d, pl, p.TW, p.TH, p.TN, false, 1))) return st;
        // k4 [kh][slot][o] as (o%32, slot, kh, o/32), box (32, 32, 1, bn/32)
        const cuuint64_t dims[4] = {32, 32, (cuuint64_t)d.kh, (cuuint64_t)(d.o / 32)};
        const cuuint64_t strides[3] = {(cuuint64_t)d.o * 4, (cuuint64_t)32 * d.o * 4, 128};
        const cuuint32_t box[4] = {32, 32, 1, (cuuint32_t)(p.bn / 32)};
        const cuuint32_t es[4] = {1, 1, 1, 1};
        return encode_map(&pr.mb, k4, 4, dims, true, strides, box, es);
    }
    if ((st = map_act_4d(&pr.ma, x, d.n, d.h, d.w, d.c, p.TW, p.TH, p.TN, d.stride_w, d.stride_h))) return st;
    // k [tap][c][o] as (o%32, c, tap, o/32), box (32, 32, 1, bn/32)
    const cuuint64_t dims[4] = {32, (cuuint64_t)d.c, (cuuint64_t)(d.kh * d.kw), (cuuint64_t)(d.o / 32)};
    const cuuint64_t strides[3] = {(cuuint64_t)d.o * 4, (cuuint64_t)d.c * d.o * 4, 128};
    const cuuint32_t box[4] = {32, 32, 1, (cuuint32_t)(p.bn / 32)};
    const cuuint32_t es[4] = {1, 1, 1, 1};
    return encode_map(&pr.mb, k, 4, dims, true, strides, box, es);
}

int build_dx(const dcg_conv_desc& d, const float* dy, const float* k, void* ws, size_t ws_bytes, Prepared& pr)
{
    Plan& pl = pr.pl;
    pr.dx3 = plan_dx3(d, pl, pr.dx3_args);
    if (pr.dx3) {
        // dy [n, ho, wo, o] in boxes of (32 o, 32 pixels, 4 rows, 1 image); k [tap][c][o] as (o, c, tap) in boxes of
        // (32 o, 4 c, 32 taps): rows 4 * tap + c, K-major, channel 3 and the taps beyond the last zero-filled
        int st = map_act_4d(&pr.ma, dy, d.n, d.ho, d.wo, d.o, 32, 4, 1, 1, 1);
        if (st) return st;
        const cuuint64_t dims[3] = {(cuuint64_t)d.o, (cuuint64_t)d.c, (cuuint64_t)(d.kh * d.kw)};
        const cuuint64_t strides[2] = {(cuuint64_t)d.o * 4, (cuuint64_t)d.c * d.o * 4};
        const cuuint32_t box[3] = {32, 4, 32};
        const cuuint32_t es[3] = {1, 1, 1};
        return encode_map(&pr.mb, k, 3, dims, false, strides, box, es);
    }
    pl = Plan{};
    pr.dxf = plan_dxf(d, pl, pr.cf);
    if (!pr.dxf) {
        pl = Plan{};
        if (!plan_dx(d, pl)) return fail(DCG_ERR_UNSUPPORTED, "conv dx: shape not supported by the tensor path");
    }
    const Params& p = pl.p;
    int st = map_act_4d(&pr.ma, dy, d.n, d.ho, d.wo, d.o, p.TW, p.TH, p.TN, 1, 1);
    if (st) return st;
    if (pl.ycol_bytes) {   // narrow-channel layer: GEMM over all taps, then gather
        if (!ws || ws_bytes < pl.ws_bytes)
            return fail(DCG_ERR_WORKSPACE, "conv dx (tensor path, narrow input): workspace %zu < %zu bytes", ws_bytes, pl.ws_bytes);
        if (short_ok(pl) && d.c <= 4 && d.kh * d.kw <= 32 && p.bn == 128) {
            // persistent GEMM: B straight from k [tap][c][o] as (o, c, tap) with a (32 o, 4 c, 32 taps) box - rows
            // 4 * tap + c of 32 contiguous o, K-major; channel 3 and the taps beyond the last are zero-filled
            pl.p.b_direct = 1;
            const cuuint64_t dims[3] = {(cuuint64_t)d.o, (cuuint64_t)d.c, (cuuint64_t)(d.kh * d.kw)};
            const cuuint64_t strides[2] = {(cuuint64_t)d.o * 4, (cuuint64_t)d.c * d.o * 4};
            const cuuint32_t box[3] = {32, 4, 32};
            const cuuint32_t es[3] = {1, 1, 1};
            return encode_map(&pr.mb, k, 3, dims, false, strides, box, es);
        }
        const float* k2 = reinterpret_cast<const float*>(static_cast<uint8_t*>(ws) + pl.k2_off());
        const int Jp = pl.Jp;
        // k2 [o][Jp] as (j%32, o, 1, j/32), box (32, 32, 1, bn/32): the FWD kernel's weight view with one tap
        const cuuint64_t dims[4] = {32, (cuuint64_t)d.o, 1, (cuuint64_t)(Jp / 32)};
        const cuuint64_t strides[3] = {(cuuint64_t)Jp * 4, (cuuint64_t)d.o * Jp * 4, 128};
        const cuuint32_t box[4] = {32, 32, 1, (cuuint32_t)(p.bn / 32)};
        const cuuint32_t es[4] = {1, 1, 1, 1};
        return encode_map(&pr.mb, k2, 4, dims, true, strides, box, es);
    }
    // k [kh][kw][c][o] as (o, c, kw, kh), box (32 o, bn c, 1, 1)
    const cuuint64_t dims[4] = {(cuuint64_t)d.o, (cuuint64_t)d.c, (cuuint64_t)d.kw, (cuuint64_t)d.kh};
    const cuuint64_t strides[3] = {(cuuint64_t)d.o * 4, (cuuint64_t)d.c * d.o * 4, (cuuint64_t)d.kw * d.c * d.o * 4};
    const cuuint32_t box[4] = {32, (cuuint32_t)p.bn, 1, 1};
    const cuuint32_t es[4] = {1, 1, 1, 1};
    return encode_map(&pr.mb, k, 4, dims, false, strides, box, es);
}

// DK: ma / mb are the maps of the A / B operand (x and dy, or dy and x when the roles are swapped).
int build_dk(const dcg_conv_desc& d, const float* x, const float* dy, void* ws, size_t ws_bytes, Prepared& pr)
{
    Plan& pl = pr.pl;
    if (!plan_dk(d, pl)) return fail(DCG_ERR_UNSUPPORTED, "conv dk: shape not supported by the tensor path");
    const Params& p = pl.p;
    CUtensorMap mx, mdy;
    int st;
    if (p.narrow) {
        if (!ws || ws_bytes < pl.ws_bytes)
            return fail(DCG_ERR_WORKSPACE, "conv (tensor path, narrow input): workspace %zu < %zu bytes", ws_bytes, pl.ws_bytes);
        const float* xp = reinterpret_cast<const float*>(static_cast<uint8_t*>(ws) + pl.xp_off());
        if ((st = map_window(&mx, xp, d, pl, p.TW, p.TH, p.TN, true, d.kh))) return st;
        if ((st = map_act_5d(&mdy, dy, d.n, d.ho, d.wo, d.o, p.TW, p.TH, p.TN, 1, 1, BM / 32))) return st;
        pr.ma = mdy; pr.mb = mx;
        return DCG_OK;
    }
    const int x_chunks = p.swap ? p.bn / 32 : BM / 32, dy_chunks = p.swap ? BM / 32 : p.bn / 32;
    if ((st = map_act_5d(&mx, x, d.n, d.h, d.w, d.c, p.TW, p.TH, p.TN, d.stride_w, d.stride_h, x_chunks))) return st;
    if ((st = map_act_5d(&mdy, dy, d.n, d.ho, d.wo, d.o, p.TW, p.TH, p.TN, 1, 1, dy_chunks))) return st;
    if (p.swap) { pr.ma = mdy; pr.mb = mx; }
    else { pr.ma = mx; pr.mb = mdy; }
    return DCG_OK;
}

// Looks the call up, building and filing it on a miss.  The entry is copied out under the lock.
int prepared_call(int kind, const dcg_conv_desc& d, const void* a, const void* b, void* ws, size_t ws_bytes, Prepared& out)
{
    CacheKey key;
    std::memset(&key, 0, sizeof(key));
    if (cudaGetDevice(&key.dev) != cudaSuccess) key.dev = -1;
    key.kind = kind; key.x3 = t_plan_x3 | (dxf_mode() << 1);   // the plan depends on both
    key.d = d; key.a = a; key.b = b; key.ws = ws; key.ws_bytes = ws_bytes;
    {
        std::lock_guard<std::mutex> lock(g_cache_mutex);
        for (const CacheEntry& e : g_cache)
            if (same_key(e.key, key)) { out = e.prep; return DCG_OK; }
    }
    int st;
    switch (kind) {
    case kConvFwd: st = build_fwd(d, static_cast<const float*>(a), static_cast<const float*>(b), ws, ws_bytes, out); break;
    case kConvDx: st = build_dx(d, static_cast<const float*>(a), static_cast<const float*>(b), ws, ws_bytes, out); break;
    default: st = build_dk(d, static_cast<const float*>(a), static_cast<const float*>(b), ws, ws_bytes, out); break;
    }
    if (st) return st;
    std::lock_guard<std::mutex> lock(g_cache_mutex);
    if (g_cache.size() < kCacheEntries) {
        g_cache.push_back(CacheEntry{key, out});
    } else {
        g_cache[g_cache_next] = CacheEntry{key, out};
        g_cache_next = (g_cache_next + 1) % kCacheEntries;
    }
    return DCG_OK;
}

}  // namespace

bool conv_tc_supported(const dcg_conv_desc& d, int kind, bool x3)
{
    PlanX3 scope(x3);
    Plan pl;
    return make_plan(d, kind, pl);
}

size_t conv_tc_workspace(const dcg_conv_desc& d, int kind, bool x3)
{
    PlanX3 scope(x3);
    Plan pl;
    if (!make_plan(d, kind, pl)) return 0;
    return pl.ws_bytes;
}

int conv_tc_fwd(const dcg_conv_desc& d, const float* x, const float* k, float* y, const EpilogueArgs& ep,
                void* ws, size_t ws_bytes, cudaStream_t stream, bool x3)
{
    PlanX3 scope(x3);
    Prepared pr;
    int st = prepared_call(kConvFwd, d, x, k, ws, ws_bytes, pr);
    if (st) return st;
    if (pr.pl.p.narrow) {
        float *xp, *k4;
        if ((st = narrow_prepare(d, pr.pl, x, k, ws, ws_bytes, stream, &xp, &k4))) return st;
        if (short_ok(pr.pl)) return launch_short(pr, true, y, ep, stream);
    }
    return launch<MODE_FWD>(pr.ma, pr.mb, pr.pl, y, ep, d.o, ws, ws_bytes, stream);
}

int conv_tc_dx(const dcg_conv_desc& d, const float* dy, const float* k, float* dx, const EpilogueArgs& ep,
               void* ws, size_t ws_bytes, cudaStream_t stream, bool x3)
{
    PlanX3 scope(x3);
    Prepared pr;
    int st = prepared_call(kConvDx, d, dy, k, ws, ws_bytes, pr);
    if (st) return st;
    Plan& pl = pr.pl;
    if (pr.dx3) return launch_dx3(pr, dx, ep, stream);
    if (pl.ycol_bytes) {   // narrow-channel layer: GEMM over all taps, then gather
        uint8_t* base = static_cast<uint8_t*>(ws);
        float* k2 = reinterpret_cast<float*>(base + pl.k2_off());
        float* ycol = reinterpret_cast<float*>(base + pl.ycol_off());
        const int Jp = pl.Jp;
        if (!pl.p.b_direct) {   // the transposed weights k2 [o][Jp]; the persistent GEMM reads k itself
            launch_pdl(repack_k2_kernel, (d.o * Jp + 255) / 256, 256, 0, stream, k, k2, d.kh * d.kw, d.c, Jp, d.o);
            DCG_LAUNCH_CHECK("repack_k2_kernel");
        }
        const EpilogueArgs none{};
        if (short_ok(pl)) st = launch_short(pr, false, ycol, none, stream);
        else st = launch<MODE_FWD>(pr.ma, pr.mb, pl, ycol, none, Jp, ws, ws_bytes, stream);
        if (st) return st;
        const size_t total = (size_t)d.n * d.h * d.w;
        size_t blocks = (total + 255) / 256;
        const size_t cap = (size_t)sm_count() * 16;
        if (blocks > cap) blocks = cap;
        if (d.kh == 5 && d.kw == 5 && d.stride_h == 2 && d.stride_w == 2)
            launch_pdl(col2im_kernel<5, 5, 2>, (unsigned)blocks, 256, 0, stream, reinterpret_cast<const float4*>(ycol), dx, d.n, d.h,
                       d.w, d.c, d.ho, d.wo, d.kh, d.kw, d.stride_h, d.stride_w, d.pad_top, d.pad_left, ep);
        else
            launch_pdl(col2im_kernel<0, 0, 0>, (unsigned)blocks, 256, 0, stream, reinterpret_cast<const float4*>(ycol), dx, d.n, d.h,
                       d.w, d.c, d.ho, d.wo, d.kh, d.kw, d.stride_h, d.stride_w, d.pad_top, d.pad_left, ep);
        DCG_LAUNCH_CHECK("col2im_kernel");
        return DCG_OK;
    }
    if (pr.dxf) return launch_dxf(pr, dx, ep, stream);
    return launch<MODE_DX>(pr.ma, pr.mb, pl, dx, ep, d.c, ws, ws_bytes, stream);
}

int conv_tc_dk(const dcg_conv_desc& d, const float* x, const float* dy, float* dk, void* ws, size_t ws_bytes,
               cudaStream_t stream, bool x3)
{
    PlanX3 scope(x3);
    Prepared pr;
    int st = prepared_call(kConvDk, d, x, dy, ws, ws_bytes, pr);
    if (st) return st;
    if (pr.pl.p.narrow) {
        float* xp;
        if ((st = narrow_prepare(d, pr.pl, x, nullptr, ws, ws_bytes, stream, &xp, nullptr))) return st;
    }
    const EpilogueArgs none{};
    return launch<MODE_DK>(pr.ma, pr.mb, pr.pl, dk, none, d.o, ws, ws_bytes, stream);
}

void conv_tc_set_dx_mode(int mode) { g_dxf_mode.store(mode < 0 || mode > 2 ? -1 : mode); }
unsigned long long conv_tc_fused_dx_launches() { return g_dxf_launches.load(); }

// wait_cycles: > 0 sets the limit, -1 restores the default, 0 leaves it; skip_stage: -2 leaves it.
void conv_tc_set_hooks(long long wait_cycles, int skip_stage)
{
    if (wait_cycles > 0) g_wait_cycles.store(wait_cycles);
    else if (wait_cycles < 0) g_wait_cycles.store(default_wait_cycles());
    if (skip_stage != -2) g_test_skip_stage.store(skip_stage);
}

// Reads (and clears) the device status word of the tensor-path kernels.  Synchronises the device.
int conv_tc_device_status(int* detail /* [4] */)
{
    int h[4] = {0, 0, 0, 0};
    DCG_CUDA(cudaDeviceSynchronize());
    DCG_CUDA(cudaMemcpyFromSymbol(h, g_tc_status, sizeof(h)));
    if (detail) for (int i = 0; i < 4; ++i) detail[i] = h[i];
    if (h[0] != 0) {
        const int zero[4] = {0, 0, 0, 0};
        DCG_CUDA(cudaMemcpyToSymbol(g_tc_status, zero, sizeof(zero)));
        contexts_reset_tickets();   // a launch that gave up may have left column-sum tickets counted up
        return fail(DCG_ERR_DEVICE, "tensor-path kernel gave up waiting: code %d block %d role %d stage %d",
                    h[0], h[1], h[2], h[3]);
    }
    return dp_status_check();
}

}  // namespace dcg

extern "C" int dcg_device_status(void) { return dcg::conv_tc_device_status(nullptr); }

extern "C" void dcg_debug_set_wait_limit(long long sm_clocks)
{
    dcg::conv_tc_set_hooks(sm_clocks > 0 ? sm_clocks : -1, -2);
}

extern "C" void dcg_debug_skip_stage(int stage) { dcg::conv_tc_set_hooks(0, stage < 0 ? -1 : stage); }

extern "C" void dcg_debug_set_dx_mode(int mode) { dcg::conv_tc_set_dx_mode(mode); }
extern "C" uint64_t dcg_debug_fused_dx_launches(void) { return dcg::conv_tc_fused_dx_launches(); }

#ifdef DCG_TC_TRACING
// Tuning aids of -DDCG_TC_TRACING builds, not part of the public header: copy the timelines recorded
// by the last tensor-path launch (DCG_TC_DEBUG bits 4 / 8) to `out`.  Synchronise the device.
extern "C" int dcg_debug_cta_trace(unsigned long long* out /* [1024][8] */)
{
    if (cudaDeviceSynchronize() != cudaSuccess) return DCG_ERR_CUDA;
    return cudaMemcpyFromSymbol(out, dcg::g_tc_cta_trace, sizeof(unsigned long long) * 1024 * 8) == cudaSuccess ? DCG_OK : DCG_ERR_CUDA;
}

extern "C" int dcg_debug_trace(long long* out /* [3080] */)
{
    if (cudaDeviceSynchronize() != cudaSuccess) return DCG_ERR_CUDA;
    return cudaMemcpyFromSymbol(out, dcg::g_tc_trace, sizeof(long long) * 3080) == cudaSuccess ? DCG_OK : DCG_ERR_CUDA;
}
#endif
