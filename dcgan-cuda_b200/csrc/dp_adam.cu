// Data-parallel update as ONE kernel over peer memory: gradient sum + Adam + parameter broadcast.
//
// The exchange step of a data-parallel update is "sum this network's gradients over the ranks, then
// every rank applies the same Adam step".  With NCCL that is an all-reduce (each rank ends up holding
// the whole sum) followed by a replicated Adam over all parameters.  Here every rank owns 1/W of the
// parameter range instead: it reads that slice of every rank's gradients straight from the peers'
// memory (NVLink loads, 128 bit), adds them in rank order - every element is summed by exactly one
// rank, so all replicas see the same bits -, applies Adam to its slice (its own first / second
// moments: the moments of a slice only ever live on its owner) and writes the new parameters of the
// slice into every rank's parameter array (NVLink stores).  Bytes over NVLink per rank: (W-1)/W of the
// arena in, the same out - what an all-reduce moves - but the sum never makes a round trip through a
// staging buffer, Adam touches 1/W of the state per rank, and there is one launch instead of two.
//
// Synchronisation: two sets of flags in every rank's arena, written by the peers with system-scope
// stores.  "ready[r] = epoch": rank r's gradients of this update are complete (its earlier kernels
// have finished - the flag is written at the start of its kernel); nobody reads a peer's gradients
// or overwrites a peer's parameters before all W flags are up.  "done[r] = epoch": rank r has written
// its slice of the new parameters into this rank's array; the kernel's last block waits for all of
// them before it exits, so whatever follows in the stream reads complete parameters.  Every wait is
// bounded (SM clock); a rank that gives up records it in a status word (dcg_device_status) and
// leaves without touching anything - its peers then run into their own limits.  The kernels of the
// W ranks run on W different GPUs, one per process: nothing here waits for another launch on the
// same GPU.  No multimem, no TMA, plain peer loads and stores.
#include "adam.cuh"
#include "common.cuh"

namespace dcg {
namespace {

constexpr int kThreads = 256;
constexpr long long kWaitCycles = 2000000000LL;   // ~1 s

// [0] code (0 = ok, 2 = a peer never became ready, 3 = a peer never finished), [1] rank, [2] peer, [3] epoch
__device__ int g_dp_status[4];

struct FusedArgs {
    int rank, world;
    const float* grads[8];      // rank r's gradient arena as seen from this GPU
    float* params[8];           // rank r's parameter arena as seen from this GPU
    float* m;                   // own moments (full-size arrays; only the own slice is ever used)
    float* v;
    unsigned* ready[8];         // rank r's "ready" flags [world] as seen from this GPU
    unsigned* done[8];          // rank r's "done" flags [world]
    unsigned* epoch;            // own: updates completed so far
    unsigned* ticket;           // own: blocks finished in this launch
    unsigned long long n4;      // float4s in the arena
    float a1, b1, a2, b2, eps, scale, lr_t;
    const float* lr_t_dev;
    long long wait_cycles;
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p)
{
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void adam_one(float& p, float g, float& m, float& v, const FusedArgs& c, float lr_t)
{
    m = __fadd_rn(__fmul_rn(c.a1, m), __fmul_rn(c.b1, g));
    v = __fadd_rn(__fmul_rn(c.a2, v), __fmul_rn(__fmul_rn(c.b2, g), g));
    p = __fsub_rn(p, __fdiv_rn(__fmul_rn(lr_t, m), __fadd_rn(__fsqrt_rn(v), c.eps)));
}

// Bounded wait of the first `world` threads of a block on flags[thread] >= epoch.  Returns false (for
// the whole block) if any of them gave up.
__device__ bool wait_flags(const unsigned* flags, unsigned epoch, const FusedArgs& a, int code)
{
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if ((int)threadIdx.x < a.world) {
        const long long t0 = clock64();
        bool ok = true;
        // flags only grow; a difference is compared so that the 32-bit counter may wrap
        while ((int)(ld_acquire_sys(flags + threadIdx.x) - epoch) < 0) {
            if (clock64() - t0 > a.wait_cycles) { ok = false; break; }
            __nanosleep(64);
        }
        if (!ok) {
            s_ok = 0;
            if (atomicCAS(&g_dp_status[0], 0, code) == 0) {
                g_dp_status[1] = a.rank;
                g_dp_status[2] = (int)threadIdx.x;
                g_dp_status[3] = (int)epoch;
            }
        }
    }
    __syncthreads();
    return s_ok != 0;
}

__global__ void __launch_bounds__(kThreads) dp_reduce_adam_kernel(const __grid_constant__ FusedArgs a)
{
    pdl_enter();
    const int W = a.world, R = a.rank;
    // every block reads the epoch before the last block of this launch advances it
    const unsigned epoch = *reinterpret_cast<volatile unsigned*>(a.epoch) + 1u;
    if (blockIdx.x == 0 && (int)threadIdx.x < W) {
        __threadfence_system();
        st_release_sys(a.ready[threadIdx.x] + R, epoch);   // "my gradients are complete", to every rank (self included)
    }
    bool go = wait_flags(a.ready[R], epoch, a, 2);
    if (go) {
        const float lr_t = a.lr_t_dev ? __ldg(a.lr_t_dev) : a.lr_t;
        const unsigned long long chunk = (a.n4 + W - 1) / W;
        const unsigned long long lo = chunk * R, hi = lo + chunk < a.n4 ? lo + chunk : a.n4;
        const unsigned long long stride = (unsigned long long)gridDim.x * kThreads;
        float4* m4 = reinterpret_cast<float4*>(a.m);
        float4* v4 = reinterpret_cast<float4*>(a.v);
        for (unsigned long long i = lo + (unsigned long long)blockIdx.x * kThreads + threadIdx.x; i < hi; i += stride) {
            float4 g[8];
#pragma unroll
            for (int r = 0; r < 8; ++r)
                if (r < W) g[r] = __ldcg(reinterpret_cast<const float4*>(a.grads[r]) + i);   // all ranks' loads in flight
            float4 p = reinterpret_cast<const float4*>(a.params[R])[i];
            float4 m = m4[i], v = v4[i];
            float4 s = g[0];
#pragma unroll
            for (int r = 1; r < 8; ++r)
                if (r < W) {   // rank order: the same bits whichever rank owns the element
                    s.x = __fadd_rn(s.x, g[r].x); s.y = __fadd_rn(s.y, g[r].y);
                    s.z = __fadd_rn(s.z, g[r].z); s.w = __fadd_rn(s.w, g[r].w);
                }
            s.x = __fmul_rn(s.x, a.scale); s.y = __fmul_rn(s.y, a.scale);
            s.z = __fmul_rn(s.z, a.scale); s.w = __fmul_rn(s.w, a.scale);
            adam_one(p.x, s.x, m.x, v.x, a, lr_t);
            adam_one(p.y, s.y, m.y, v.y, a, lr_t);
            adam_one(p.z, s.z, m.z, v.z, a, lr_t);
            adam_one(p.w, s.w, m.w, v.w, a, lr_t);
            m4[i] = m;
            v4[i] = v;
#pragma unroll
            for (int r = 0; r < 8; ++r)
                if (r < W) reinterpret_cast<float4*>(a.params[r])[i] = p;   // the slice's new parameters, to every rank
        }
    }
    // ---- the block that finishes last tells the peers, then waits for theirs ----
    __shared__ unsigned s_last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned t = atomicAdd(a.ticket, 1u);
        s_last = (t == gridDim.x - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence_system();
    if (threadIdx.x == 0) *a.ticket = 0u;
    if (go && (int)threadIdx.x < W) st_release_sys(a.done[threadIdx.x] + R, epoch);
    if (go) wait_flags(a.done[R], epoch, a, 3);
    if (threadIdx.x == 0) *reinterpret_cast<volatile unsigned*>(a.epoch) = epoch;   // also after a failure: the next launch starts a new round
}

}  // namespace

int dp_reduce_adam_launch(int rank, int world, float* const* grads, float* const* params, float* m, float* v,
                          unsigned* const* ready, unsigned* const* done, unsigned* epoch, unsigned* ticket, size_t n_floats,
                          float lr_t, float a1, float b1, float a2, float b2, float eps, float scale, const float* lr_t_dev,
                          cudaStream_t stream)
{
    DCG_CHECK_ARG(world >= 2 && world <= 8 && rank >= 0 && rank < world, "dp_reduce_adam: rank %d of %d", rank, world);
    FusedArgs a{};
    a.rank = rank; a.world = world;
    for (int r = 0; r < world; ++r) {
        DCG_CHECK_ARG(grads[r] && params[r] && ready[r] && done[r], "dp_reduce_adam: rank %d is not mapped", r);
        DCG_CHECK_ARG(((reinterpret_cast<uintptr_t>(grads[r]) | reinterpret_cast<uintptr_t>(params[r])) & 15u) == 0,
                      "dp_reduce_adam: arenas must be 16-byte aligned");
        a.grads[r] = grads[r]; a.params[r] = params[r]; a.ready[r] = ready[r]; a.done[r] = done[r];
    }
    a.m = m; a.v = v; a.epoch = epoch; a.ticket = ticket;
    a.n4 = (n_floats + 3) / 4;
    a.a1 = a1; a.b1 = b1; a.a2 = a2; a.b2 = b2; a.eps = eps; a.scale = scale; a.lr_t = lr_t; a.lr_t_dev = lr_t_dev;
    static const long long limit = [] { const char* e = getenv("DCG_DP_WAIT_CYCLES"); const long long c = e ? atoll(e) : 0; return c > 0 ? c : kWaitCycles; }();
    a.wait_cycles = limit;
    // enough blocks to keep every NVLink busy, few enough that all of them are resident at once next to
    // whatever else runs (they wait on flags): two per SM
    const unsigned long long per_rank = (a.n4 + world - 1) / world;
    unsigned blocks = (unsigned)((per_rank + kThreads - 1) / kThreads);
    const unsigned cap = (unsigned)sm_count() * 2u;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    launch_pdl(dp_reduce_adam_kernel, blocks, kThreads, 0, stream, a);
    DCG_LAUNCH_CHECK("dp_reduce_adam_kernel");
    return DCG_OK;
}

// Reads (and clears) the status word of the fused update.  The caller has synchronised the device.
int dp_status_check()
{
    int h[4] = {0, 0, 0, 0};
    DCG_CUDA(cudaMemcpyFromSymbol(h, g_dp_status, sizeof(h)));
    if (h[0] != 0) {
        const int zero[4] = {0, 0, 0, 0};
        DCG_CUDA(cudaMemcpyToSymbol(g_dp_status, zero, sizeof(zero)));
        return fail(DCG_ERR_DEVICE, "data-parallel update gave up waiting for a peer: code %d (2 = gradients never ready, "
                                    "3 = parameters never written), rank %d, peer %d, update %d", h[0], h[1], h[2], h[3]);
    }
    return DCG_OK;
}

}  // namespace dcg
