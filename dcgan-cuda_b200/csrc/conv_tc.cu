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
// This file is the host side (tensor maps, planning, the plan cache, launches, entry points); the
// device code of this translation unit sits in the headers it includes:
//   conv_tc_common.cuh   constants, kernel parameters, PTX wrappers, descriptors
//   conv_tc_kernel.cuh   conv_tc_kernel<MODE, X3>, the general kernel described above
//   conv_tc_dxf.cuh      conv_dxf_kernel: input gradient with all parity classes of a pixel tile in one
//                        CTA, their accumulators merged into wide MMAs
//   conv_tc_short.cuh    conv_fwd_short_kernel: the short-K forward GEMMs of the 3-channel layers as
//                        persistent CTAs with resident weights and a double-buffered accumulator
//   conv_tc_dx3.cuh      conv_dx3_kernel: input gradient of a 3-channel layer, GEMM + gather in one kernel
//   conv_tc_narrow.cuh   repack, partition-finish and gather helpers of the 3-channel layers
#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "conv.cuh"

#include "conv_tc_common.cuh"
#include "conv_tc_kernel.cuh"
#include "conv_tc_dxf.cuh"
#include "conv_tc_short.cuh"
#include "conv_tc_dx3.cuh"
#include "conv_tc_narrow.cuh"

namespace dcg {
namespace {

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
