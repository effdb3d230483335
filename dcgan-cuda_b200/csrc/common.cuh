// Shared helpers of the dcgan_b200 CUDA library: status/error plumbing, launch
// accounting, small device math used by several translation units.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstddef>
#include <cstdint>
#include <cstdio>

#include "dcgan_b200.h"

namespace dcg {

// ---- error reporting -------------------------------------------------------
// The message of the last failing call on this thread; read by dcg_last_error().
char* last_error_buffer();
int fail(int status, const char* fmt, ...);

// Counts kernels launched by this library (all contexts); read by
// dcg_context_launch_count and by the benchmark's gpu_launches figure.
void count_launch(int n = 1);
uint64_t launches_total();

#define DCG_CHECK_ARG(cond, ...)                                   \
    do {                                                           \
        if (!(cond)) return ::dcg::fail(DCG_ERR_INVALID, __VA_ARGS__); \
    } while (0)

#define DCG_CUDA(call)                                                              \
    do {                                                                            \
        cudaError_t e__ = (call);                                                   \
        if (e__ != cudaSuccess)                                                     \
            return ::dcg::fail(DCG_ERR_CUDA, "%s failed: %s (%s:%d)", #call,        \
                               cudaGetErrorString(e__), __FILE__, __LINE__);        \
    } while (0)

// After a kernel launch: picks up launch-configuration errors without syncing.
#define DCG_LAUNCH_CHECK(name)                                                      \
    do {                                                                            \
        cudaError_t e__ = cudaGetLastError();                                       \
        if (e__ != cudaSuccess)                                                     \
            return ::dcg::fail(DCG_ERR_CUDA, "launch of %s failed: %s", name,       \
                               cudaGetErrorString(e__));                            \
        ::dcg::count_launch();                                                      \
    } while (0)

inline cudaStream_t as_stream(dcg_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// ---- programmatic dependent launch --------------------------------------------------------------
// Every kernel of the library is launched with programmatic stream serialisation and begins with
// pdl_enter(): it waits for the previous kernel of the stream to have completed (its memory
// visible) before touching memory, then lets the next kernel be scheduled.  The data dependencies
// are the ordinary in-order ones; what overlaps is the launch latency and block set-up of kernel
// N+1 with the tail of kernel N.  A kernel launched without the attribute (or first in its stream)
// sees both instructions as no-ops.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_enter()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args&&... args)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);   // errors surface in DCG_LAUNCH_CHECK
}
#endif

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---- column sums: internal launch with caller-owned ticket words (elementwise.cu) ---------------
// kColsumTicketBytes of ZEROED device memory that only stream-ordered launches share; the kernel
// leaves them zero.  colsum_partial_bytes_max: scratch for the partial sums alone (0: none needed).
constexpr size_t kColsumTicketBytes = 4096;
int colsum_launch(const float* a, float* out, size_t rows, size_t cols, void* workspace, size_t workspace_bytes,
                  unsigned* tickets, cudaStream_t stream);
size_t colsum_partial_bytes_max(size_t rows, size_t cols);
// Clears the ticket words of every live context (after a kernel reported an error, a launch may
// have left some of them counted up).  Synchronises the device.
void contexts_reset_tickets();
// Status word of the fused data-parallel update (dp_adam.cu): DCG_OK, or DCG_ERR_DEVICE after a wait for
// a peer ran out.  Reads and clears; the caller has synchronised the device.
int dp_status_check();

// Number of SMs of the current device (cached per device id).
int sm_count();

// ---- device math -----------------------------------------------------------
// Activations written the way the reference's CPU code evaluates them
// (src/cpu/ops.hxx:13-17,345-359): float exp, double around it.
__device__ __forceinline__ float act_apply(float v, int act, float alpha)
{
    switch (act) {
    case DCG_ACT_LEAKY: return v < 0.f ? __fmul_rn(alpha, v) : v;
    case DCG_ACT_RELU: return v < 0.f ? 0.f : v;
    case DCG_ACT_TANH: return (float)((2.0 / (1.0 + (double)expf(-2.f * v))) - 1.0);
    case DCG_ACT_SIGMOID: return (float)(1.0 / (1.0 + (double)expf(-v)));
    default: return v;
    }
}

// d act / d input evaluated from `gate` (pre-activation for LEAKY/RELU, activation
// output for TANH/SIGMOID), multiplied into dout: src/cpu/ops.hxx:423-466,926-931.
__device__ __forceinline__ float act_grad_apply(float gate, float dout, int act, float alpha)
{
    switch (act) {
    case DCG_ACT_LEAKY: return gate < 0.f ? __fmul_rn(alpha, dout) : dout;
    case DCG_ACT_RELU: return gate > 0.f ? dout : 0.f;
    case DCG_ACT_TANH: return (float)((1.0 - (double)gate * (double)gate) * (double)dout);
    case DCG_ACT_SIGMOID: return __fmul_rn(__fmul_rn(gate, __fsub_rn(1.f, gate)), dout);
    default: return dout;
    }
}

// Epilogue parameters as passed to kernels (a copy of dcg_epilogue with NULL
// meaning "absent").
struct EpilogueArgs {
    float* raw_out;
    const float* bias;
    float* pre_act;
    const float* gate;
    int act;
    int gate_act;
    float alpha;
    float gate_alpha;
};

inline EpilogueArgs make_epilogue(const dcg_epilogue* ep)
{
    EpilogueArgs a{};
    if (ep) {
        a.raw_out = ep->raw_out;
        a.bias = ep->bias;
        a.pre_act = ep->pre_act;
        a.gate = ep->gate;
        a.act = ep->act;
        a.gate_act = ep->gate_act;
        a.alpha = ep->alpha;
        a.gate_alpha = ep->gate_alpha;
    }
    return a;
}

// Applies the whole epilogue chain to accumulator `v` destined for linear
// output index `i` with output channel `ch`.
__device__ __forceinline__ float epilogue_apply(const EpilogueArgs& ep, float v, size_t i, int ch)
{
    if (ep.raw_out) ep.raw_out[i] = v;
    if (ep.bias) v = __fadd_rn(v, __ldg(ep.bias + ch));
    if (ep.pre_act) ep.pre_act[i] = v;
    v = act_apply(v, ep.act, ep.alpha);
    if (ep.gate) v = act_grad_apply(__ldg(ep.gate + i), v, ep.gate_act, ep.gate_alpha);
    return v;
}

}  // namespace dcg
