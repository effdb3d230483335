// Constants, kernel parameters, PTX wrappers and descriptor helpers shared by the tcgen05 convolution kernels
// (included by conv_tc.cu only: everything lives in that translation unit's anonymous namespace).
#pragma once

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

}  // namespace
}  // namespace dcg
