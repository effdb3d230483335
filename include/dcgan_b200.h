/*
 * dcgan_b200 - C ABI of the B200 (sm_100a) convolution / Adam hot path that
 * replaces the GPU backend (src/gpu) of obs145628/dcgan-cuda.
 *
 * Conventions
 *   - every pointer named x, k, y, dy, dx, dk, bias, ... is a DEVICE pointer to
 *     fp32 data unless the comment says "host";
 *   - activations are NHWC, conv2d kernels HWIO [kh][kw][Cin][Cout],
 *     conv2d_transpose kernels [kh][kw][Cout][Cin] (the layouts of the
 *     reference's ops, src/ops/conv2d.cu, src/ops/conv2d-transpose.cu);
 *   - every entry point returns a dcg_status (0 = ok, negative = error), is
 *     asynchronous on the given stream, never synchronises the device and
 *     never allocates: scratch memory is passed in as (workspace, bytes);
 *   - dcg_last_error() returns a human-readable message for the last non-zero
 *     status returned on the calling thread.
 *
 * File:line citations name the reference interface each entry point replaces.
 */
#ifndef DCGAN_B200_H
#define DCGAN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* dcg_stream_t; /* a cudaStream_t; NULL = the default stream */

enum dcg_status {
    DCG_OK = 0,
    DCG_ERR_INVALID = -1,     /* bad argument (null pointer, non-positive size, unknown enum) */
    DCG_ERR_CUDA = -2,        /* a CUDA runtime/driver call failed */
    DCG_ERR_WORKSPACE = -3,   /* workspace too small / missing */
    DCG_ERR_UNSUPPORTED = -4, /* shape outside what the requested path supports */
    DCG_ERR_DEVICE = -5       /* a kernel reported an error through its status word */
};

enum dcg_act {
    DCG_ACT_NONE = 0,
    DCG_ACT_LEAKY = 1,   /* x<0 ? alpha*x : x        (src/gpu/relu.cu:26-37)   */
    DCG_ACT_RELU = 2,    /* x<0 ? 0 : x              (src/gpu/relu.cu:39-48)   */
    DCG_ACT_TANH = 3,    /* 2/(1+exp(-2x)) - 1       (src/gpu/sigmoid.cu:113)  */
    DCG_ACT_SIGMOID = 4  /* 1/(1+exp(-x))            (src/gpu/sigmoid.cu:21)   */
};

enum dcg_precision {
    DCG_PREC_TF32 = 0,   /* tcgen05 kind::tf32, fp32 accumulate in TMEM; falls back to
                            DCG_PREC_FP32 kernels for shapes the tensor path cannot take */
    DCG_PREC_3XTF32 = 1, /* opt-in: operand = TF32 part + residual, three tensor-core products per
                            K step; <= 1e-5 * max|ref|, about three times the TF32 cost */
    DCG_PREC_FP32 = 2    /* CUDA-core fp32 with the reference CPU's summation order,
                            unfused multiply/add: bit-comparable with src/cpu/ops.hxx */
};

/* Geometry of one strided convolution y = conv2d(x, k).  The same descriptor
 * drives the forward, input-gradient and kernel-gradient entry points; the
 * transposed convolution and its gradients reuse them with roles swapped,
 * exactly as src/gpu/conv2d.cu:167-307 does. */
typedef struct dcg_conv_desc {
    int n, h, w, c;         /* x  [n, h, w, c]             */
    int kh, kw, o;          /* k  [kh, kw, c, o]           */
    int ho, wo;             /* y  [n, ho, wo, o]           */
    int stride_h, stride_w;
    int pad_top, pad_left;  /* taps outside x contribute nothing (src/cpu/ops.hxx:236-243) */
} dcg_conv_desc;

/* Work fused behind the accumulator of dcg_conv2d_fwd / dcg_conv2d_dx, applied
 * per output element v with output-channel index ch, in this order:
 *   raw_out[i] = v           if raw_out   (the bare convolution result)
 *   v += bias[ch]            if bias      (mvrow_add,   src/gpu/matmul.cu:27-38)
 *   pre_act[i] = v           if pre_act   (the z tensor backward needs)
 *   v = act(v)               if act       (src/gpu/relu.cu, sigmoid.cu)
 *   v *= act'(gate[i])       if gate      (leaky/relu grad take the pre-activation,
 *                                          tanh grad takes the tanh OUTPUT:
 *                                          src/gpu/relu.cu:50-66, sigmoid.cu:42-50)
 *   out[i] = v
 * A NULL dcg_epilogue* means "store the accumulator". */
typedef struct dcg_epilogue {
    float* raw_out;
    const float* bias;
    float* pre_act;
    int act;          /* dcg_act */
    float alpha;      /* leaky slope for act */
    const float* gate;
    int gate_act;     /* dcg_act whose derivative gates the result */
    float gate_alpha; /* leaky slope for gate_act */
} dcg_epilogue;

/* ---- convolutions -------------------------------------------------------- */

/* Scratch bytes the three conv entry points need for `desc` at `precision`
 * (kind: 0 = fwd, 1 = dx, 2 = dk).  0 when none is needed. */
size_t dcg_conv_workspace_bytes(const dcg_conv_desc* desc, int kind, int precision);

/* y = conv2d(x, k) [+ epilogue].
 * Replaces gpu::kernel_conv2d (src/gpu/conv2d.cu:13-62) and, with dy as x,
 * gpu::kernel_conv2d_transpose_input_grad (src/gpu/conv2d.cu:214-259). */
int dcg_conv2d_fwd(const dcg_conv_desc* desc, const float* x, const float* k, float* y,
                   const dcg_epilogue* ep, int precision,
                   void* workspace, size_t workspace_bytes, dcg_stream_t stream);

/* dx = d conv2d / d x given dy [+ epilogue]; dx has desc's x shape.
 * Replaces gpu::kernel_conv2d_input_grad (src/gpu/conv2d.cu:70-117) and, with
 * the layer input as dy, gpu::kernel_conv2d_transpose (src/gpu/conv2d.cu:167-212). */
int dcg_conv2d_dx(const dcg_conv_desc* desc, const float* dy, const float* k, float* dx,
                  const dcg_epilogue* ep, int precision,
                  void* workspace, size_t workspace_bytes, dcg_stream_t stream);

/* dk = d conv2d / d k given x and dy; dk has desc's k shape.
 * Replaces gpu::kernel_conv2d_kernel_grad (src/gpu/conv2d.cu:119-165) and, with
 * (dy, x) swapped, gpu::kernel_conv2d_transpose_kernel_grad (src/gpu/conv2d.cu:264-307). */
int dcg_conv2d_dk(const dcg_conv_desc* desc, const float* x, const float* dy, float* dk,
                  int precision, void* workspace, size_t workspace_bytes, dcg_stream_t stream);

/* ---- memory-bound operators ---------------------------------------------- */

/* z = a + bias[col] and/or act(z) over a row-major [rows, cols] matrix: either
 * output pointer may be NULL.  Replaces gpu::kernel_mat_rvect_add
 * (src/gpu/matmul.cu:106-119) chained with an activation node. */
int dcg_bias_act(const float* a, const float* bias, float* z_out, float* act_out,
                 size_t rows, size_t cols, int act, float alpha, dcg_stream_t stream);

/* out = act(a).  Replaces gpu::kernel_relu / relu_leaky / tanh / sigmoid
 * (src/gpu/relu.cu:88-109, src/gpu/sigmoid.cu:124-165). */
int dcg_act_fwd(const float* a, float* out, size_t n, int act, float alpha, dcg_stream_t stream);

/* out = dout * act'(gate).  gate is the pre-activation for LEAKY/RELU and the
 * activation OUTPUT for TANH/SIGMOID.  Replaces gpu::kernel_leaky_relu_grad,
 * relu_grad, tanh_grad, sigmoid_grad (src/gpu/relu.cu:50-66, sigmoid.cu:31-50). */
int dcg_act_grad(const float* gate, const float* dout, float* out, size_t n,
                 int act, float alpha, dcg_stream_t stream);

/* out[c] = sum_r a[r, c]: the conv/dense bias gradient.
 * Replaces gpu::kernel_mat_sum_cols (src/gpu/sum.cu:111-151,238-243).
 * workspace: dcg_colsum_workspace_bytes(rows, cols) bytes (may be 0). */
size_t dcg_colsum_workspace_bytes(size_t rows, size_t cols);
int dcg_colsum(const float* a, float* out, size_t rows, size_t cols,
               void* workspace, size_t workspace_bytes, dcg_stream_t stream);

/* The same column sum for callers that cannot allocate device memory and have none to spare for
 * scratch - for instance a backend plugged in behind a handler that is given operand pointers only
 * and runs under a memory budget fixed at start-up, or inside a loop that must stay out of the
 * driver's allocator.  This entry point has no counterpart in the reference.
 * The scratch is a 256 KiB array built into the library image (dcg_colsum_noalloc_max_bytes()); every
 * GPU the library is loaded on holds it until the process exits.  A shape whose partial sums do not
 * fit (dcg_colsum_workspace_bytes(rows, cols) larger than that) is refused with DCG_ERR_WORKSPACE.
 * No cudaMalloc, cudaFree or other allocating call is made.  The first call on a device looks up
 * the array's device address (one cudaGetSymbolAddress); make that first call before any stream
 * capture.  All calls on a device share the one array: two calls whose kernels can overlap on the
 * GPU (different streams, no ordering between them) race on it and corrupt each other's result. */
size_t dcg_colsum_noalloc_max_bytes(void);
int dcg_colsum_noalloc(const float* a, float* out, size_t rows, size_t cols, dcg_stream_t stream);

/* out[r] = sum_c a[r, c].  Replaces gpu::kernel_mat_sum_rows (src/gpu/sum.cu:66-109). */
int dcg_rowsum(const float* a, float* out, size_t rows, size_t cols, dcg_stream_t stream);

/* out = a + b.  Replaces gpu::kernel_add (src/gpu/sum.cu:206-214,251-257). */
int dcg_add(const float* a, const float* b, float* out, size_t n, dcg_stream_t stream);

/* Image decode on the device: out[i] = (float)((double)in[i] / 127.5 - 1.), the scaling of pixel
 * bytes to [-1, 1] that celeba::load does on the host for every batch (src/datasets/celeba.cu:16-34),
 * bit for bit.  Both buffers 16-byte aligned. */
int dcg_u8_to_unit(const unsigned char* in, float* out, size_t n, dcg_stream_t stream);

/* out += coeff[0] * dv, coeff a DEVICE scalar.
 * Replaces gpu::kernel_update (src/gpu/update.cu:13-21,58-63). */
int dcg_update(const float* dv, float* out, const float* coeff, size_t n, dcg_stream_t stream);

/* Dense layers on row-major matrices (src/gpu/matmul.cu:11-86):
 *   dcg_matmul   out[m,p] = a[m,n] b[n,p] (+ bias[p] if bias)   mat_mat_mul / mat_mul_add
 *   dcg_matmul_tn out[m,p] = a[n,m]^T b[n,p]                    tmat_mat_mul  (dW = x^T dy)
 *   dcg_matmul_nt out[m,p] = a[m,n] b[p,n]^T                    mat_tmat_mul  (dx = dy W^T) */
int dcg_matmul(const float* a, const float* b, const float* bias, float* out,
               size_t m, size_t n, size_t p, dcg_stream_t stream);
int dcg_matmul_tn(const float* a, const float* b, float* out,
                  size_t m, size_t n, size_t p, dcg_stream_t stream);
int dcg_matmul_nt(const float* a, const float* b, float* out,
                  size_t m, size_t n, size_t p, dcg_stream_t stream);

/* out[0] = mean_i( max(x,0) - x*y + log(1+exp(-|x|)) ).
 * Replaces gpu::kernel_sigmoid_cross_entropy (src/gpu/sigmoid.cu:52-100,167-172). */
int dcg_sigmoid_xent(const float* y, const float* logits, float* out, size_t n, dcg_stream_t stream);
/* out = (sigmoid(logits) - y) / n.  Replaces src/gpu/sigmoid.cu:102-111,174-181. */
int dcg_sigmoid_xent_grad(const float* y, const float* logits, float* out, size_t n,
                          dcg_stream_t stream);

/* Operators the MNIST example needs to keep working (src/gpu/sum.cu, softmax.cu). */
int dcg_mse(const float* y, const float* y_hat, float* out, size_t rows, size_t cols,
            dcg_stream_t stream);
int dcg_mse_grad(const float* y, const float* y_hat, float* out, size_t n, dcg_stream_t stream);
int dcg_softmax(const float* a, float* out, size_t rows, size_t cols, dcg_stream_t stream);
int dcg_log_softmax(const float* a, float* out, size_t rows, size_t cols, dcg_stream_t stream);
int dcg_softmax_xent(const float* y, const float* logits, float* out, size_t rows, size_t cols,
                     dcg_stream_t stream);
int dcg_softmax_xent_grad(const float* y, const float* logits, float* out, size_t rows,
                          size_t cols, dcg_stream_t stream);
/* out[0] = number of rows whose first arg-max agrees (bit-exact integer count).
 * Replaces gpu::kernel_argmax_acc (src/gpu/sum.cu:153-204). */
int dcg_argmax_acc(const float* y, const float* y_hat, float* out, size_t rows, size_t cols,
                   dcg_stream_t stream);

/* ---- Adam ---------------------------------------------------------------- */

/* One variable of a fused multi-tensor Adam step. */
typedef struct dcg_adam_tensor {
    float* p;        /* parameter, updated in place */
    const float* g;  /* gradient */
    const float* g2; /* optional second gradient path, added to g (NULL if none) */
    float* m;        /* first moment, updated in place */
    float* v;        /* second moment, updated in place */
    size_t n;        /* element count */
} dcg_adam_tensor;

/* The reference's step size: t += 1; lr*sqrt(1-beta2^t)/(1-beta1^t)
 * (src/gpu/update.cu:80-96).  `t` is a HOST float, as rt::Node::out2 of the
 * adam_update node is (src/ops/adam-update.cu:45-48). */
float dcg_adam_lr_t(float* t_host, float lr, float beta1, float beta2);

/* For every tensor:  g' = grad_scale*(g [+ g2]);  m = b1*m + (1-b1)*g';
 * v = b2*v + (1-b2)*g'*g';  p = p - lr_t*m/(sqrt(v)+eps).
 * One launch replaces the moment_update / moment_update2 / adam_update triple
 * of every variable (src/gpu/update.cu:23-54,65-96).  `tensors` is a HOST array. */
int dcg_adam_multi(const dcg_adam_tensor* tensors, int count,
                   float lr_t, float beta1, float beta2, float eps, float grad_scale,
                   dcg_stream_t stream);

/* ---- node-level backend: the drop-in boundary ---------------------------- */

/* The operand record of one runtime instruction: field for field what the
 * reference's kernels read from rt::Node (src/runtime/node.hh:215-243).  `type`
 * uses the rt::Node::OP_* numbering (src/runtime/node.hh:16-54). */
typedef struct dcg_node {
    int type;
    const float* in1;
    const float* in2;
    const float* in3;
    float* out1;
    float* out2; /* adam_update: HOST pointer to the step counter t */
    float cons1, cons2, cons3, cons4;
    size_t len1, len2, len3;
    int intconst[2];
    int intconst2[2];
    int sizes1[4];
    int sizes2[4];
    int sizes3[4];
    int int_cons1, int_cons2;
    float alpha_leaky;
    unsigned flags; /* DCG_NODE_* bits; 0 when translated from an rt::Node */
} dcg_node;

#define DCG_NODE_OUT_DEAD 1u /* out1 is read by nobody but the next fusable node: a fused
                                kernel may skip storing it */
#define DCG_NODE_SIDE 2u     /* nothing later in the list reads this node's outputs or overwrites its
                                inputs (a weight or bias gradient): dcg_run_nodes may run it on a
                                second stream, concurrently with the nodes that follow, and joins it
                                before returning.  Honoured only by contexts that own their scratch. */

#define DCG_OP_MAT_MAT_MUL 0
#define DCG_OP_MAT_RVECT_ADD 1
#define DCG_OP_SIGMOID 2
#define DCG_OP_MSE 3
#define DCG_OP_SOFTMAX 4
#define DCG_OP_LOG_SOFTMAX 5
#define DCG_OP_SOFTMAX_CROSS_ENTROPY 6
#define DCG_OP_CONV2D 7
#define DCG_OP_RELU 8
#define DCG_OP_RELU_LEAKY 9
#define DCG_OP_TANH 10
#define DCG_OP_MSE_GRAD 11
#define DCG_OP_SIGMOID_GRAD 12
#define DCG_OP_MAT_MUL_ADD 13
#define DCG_OP_TMAT_MAT_MUL 14
#define DCG_OP_MAT_TMAT_MUL 15
#define DCG_OP_MAT_SUM_ROWS 16
#define DCG_OP_MAT_SUM_COLS 17
#define DCG_OP_SOFTMAX_CROSS_ENTROPY_GRAD 18
#define DCG_OP_RELU_GRAD 19
#define DCG_OP_CONV2D_BIAS_ADD 20
#define DCG_OP_UPDATE 21
#define DCG_OP_SIGMOID_CROSS_ENTROPY 22
#define DCG_OP_SIGMOID_CROSS_ENTROPY_GRAD 23
#define DCG_OP_CONV2D_INPUT_GRAD 24
#define DCG_OP_CONV2D_KERNEL_GRAD 25
#define DCG_OP_ARGMAX_ACC 26
#define DCG_OP_MOMENT_UPDATE 27
#define DCG_OP_MOMENT_UPDATE2 28
#define DCG_OP_ADAM_UPDATE 29
#define DCG_OP_LEAKY_RELU_GRAD 30
#define DCG_OP_CONV2D_BIAS_ADD_GRAD 31
#define DCG_OP_TANH_GRAD 32
#define DCG_OP_CONV2D_TRANSPOSE 33
#define DCG_OP_CONV2D_TRANSPOSE_INPUT_GRAD 34
#define DCG_OP_CONV2D_TRANSPOSE_KERNEL_GRAD 35
#define DCG_OP_ADD 36
#define DCG_OP_COUNT 37

/* Execution context of the node-level backend: stream, precision, scratch. */
typedef struct dcg_context dcg_context;

/* workspace may be NULL with workspace_bytes 0: the context then owns a scratch
 * buffer it grows on demand with cudaMalloc (what src/gpu/conv2d_gemm.hh does on
 * every call); a caller-provided buffer is never reallocated. */
int dcg_context_create(dcg_context** out, int precision, void* workspace, size_t workspace_bytes,
                       dcg_stream_t stream);
void dcg_context_destroy(dcg_context* ctx);
int dcg_context_set_precision(dcg_context* ctx, int precision);
/* Number of kernels launched through this context so far. */
uint64_t dcg_context_launch_count(const dcg_context* ctx);

/* Profiling mode: the counterpart of the reference's Graph::debug_set timing printout
 * (src/ops/graph.cu:153-221), per launch group instead of per run.  Between begin and end every
 * group the context launches (a fused convolution, a single node, a multi-tensor Adam) is
 * bracketed by CUDA events on the context's stream.  end synchronises the stream and returns one
 * row per distinct group name: calls, summed device milliseconds, summed algorithmic FLOPs
 * (2*B*Ho*Wo*KH*KW*Cin*Cout for the convolutions, 0 for the memory-bound groups). */
typedef struct dcg_profile_row {
    char name[96];
    uint64_t calls;
    double ms;
    double flops;
} dcg_profile_row;
int dcg_context_profile_begin(dcg_context* ctx);
int dcg_context_profile_end(dcg_context* ctx, dcg_profile_row* rows, int max_rows, int* n_rows);

/* Executes one node: the function gpu::kernels_list[node->type] stands for
 * (src/gpu/kernels.cu:20-64).  Asynchronous on the context's stream. */
int dcg_run_node(dcg_context* ctx, const dcg_node* node);

/* Executes nodes in order, the body of gpu::run (src/gpu/runner.cu:10-18)
 * without its per-node device synchronisation.  With fuse != 0 adjacent nodes
 * are combined: conv -> bias add -> activation into the conv epilogue,
 * input-gradient -> activation-gradient likewise, and every
 * moment_update / moment_update2 / adam_update triple of the list into one
 * multi-tensor launch.  Results are identical to unfused execution except for
 * buffers flagged DCG_NODE_OUT_DEAD. */
int dcg_run_nodes(dcg_context* ctx, const dcg_node* nodes, int count, int fuse);

/* ---- data parallelism ------------------------------------------------------
 * The path shards over the batch: one process per GPU, every rank trains its own images with a
 * full replica of the 20 variables; the one exchange of an update is a sum of that network's
 * contiguous gradient arena over the ranks (ncclAllReduce over NVLink / NVSwitch), then the replicated
 * Adam step divides by the world size.  The reference has no multi-GPU code (its training loop is
 * dcgan/main.cu:378-391 on one device); these entry points have no counterpart in it.
 * NCCL is looked up at run time (libnccl.so.2), so the library loads without it.
 *   dcg_dp_unique_id  rank 0 makes the 128-byte id; the caller hands it to every rank (any transport);
 *   dcg_dp_init       collective: every rank calls it with its rank, on its own current device;
 *   dcg_dp_allreduce  in-place sum over the ranks, enqueued on `stream` (no synchronisation);
 *   dcg_dp_info       rank, world and the version of the NCCL library that was loaded. */
#define DCG_DP_ID_BYTES 128
typedef struct dcg_dp dcg_dp;
int dcg_dp_unique_id(void* id_out);
int dcg_dp_init(dcg_dp** out, int rank, int world, const void* unique_id);
int dcg_dp_allreduce(dcg_dp* dp, float* buf, size_t count, dcg_stream_t stream);
int dcg_dp_info(const dcg_dp* dp, int* rank, int* world, int* nccl_version);
void dcg_dp_finalize(dcg_dp* dp);

/* ---- DCGAN training step: the caller of the hot path ----------------------
 * Host-side counterpart of dcgan/main.cu:271-410: the generator / discriminator
 * of that file lowered to node lists (forward, autodiff gradients) and executed
 * through dcg_run_nodes, followed by the fused Adam update.  One training
 * iteration is one discriminator update and two generator updates, each
 * recomputing its forward passes, as dcgan/main.cu:378-391 does. */
typedef struct dcg_trainer dcg_trainer;

typedef struct dcg_trainer_config {
    int batch;           /* images per step on this GPU (dcgan/main.cu:33: 64) */
    int world;           /* data-parallel ranks; > 1 makes d_backward sum the two gradient paths
                            so one all-reduce of "d_grads" averages the final gradients */
    int precision;       /* dcg_precision of the convolutions */
    int fuse;            /* node fusion on/off (dcg_run_nodes) */
    int g_leaky;         /* generator activation: 0 = relu (dcgan/main.cu:69,97), 1 = leaky-relu(0.2) */
    float lr, beta1, beta2, eps; /* Adam (dcgan/main.cu:35-36, src/api/adam-optimizer.hh:11-14) */
    uint64_t seed;       /* weights ~ N(0, 0.02) from the xorshift generator, biases 0 */
    int share_g_forward; /* dcg_trainer_step only, single GPU: 1 = the first G run of an iteration re-uses the generator
                            forward pass of the D run (same generator parameters, so the same numbers) instead of
                            recomputing it as dcgan/main.cu:378-391 does; 0 = recompute (the benchmarked workload) */
} dcg_trainer_config;

/* Allocates one device arena (parameters, Adam state, gradients, activations) and builds the
 * node lists.  The only allocating entry point besides dcg_context_create. */
int dcg_trainer_create(dcg_trainer** out, const dcg_trainer_config* cfg, dcg_stream_t stream);
/* The same for data-parallel training with the communicator behind the C ABI (cfg->world ranks; `dp`
 * stays the caller's and must outlive the trainer): the arena comes from NCCL's own allocator where
 * that exists (its in-switch reduction needs memory it mapped itself), the gradient arenas are
 * registered with the communicator, and dcg_trainer_step runs the whole data-parallel iteration -
 * node lists, the three gradient sums, the three Adam steps - as one CUDA graph. */
int dcg_trainer_create_dp(dcg_trainer** out, const dcg_trainer_config* cfg, dcg_stream_t stream, dcg_dp* dp);
void dcg_trainer_destroy(dcg_trainer* t);
/* Device tensors by name: "x" [B,64,64,3] real images and "z" [B,100] noise (inputs the caller
 * fills), "g_out", "d_loss", "g_loss", "logits_fake", "logits_real", the contiguous per-network
 * arenas "d_params", "g_params", "d_grads", "g_grads", and single variables "d_param0".."d_param9",
 * "g_param0".., "d_grad0".., "d_gradb0".. (second path), "g_grad0".., "d_m0", "d_v0", "g_m0", "g_v0"..
 * Variable order: (kernel, bias) of conv layers 0..3, then dense weight, dense bias.
 * With DCG_PREC_FP32 the D run is the reference's two discriminator passes: "d_grad*" holds the
 * gradients of the fake pass, "d_gradb*" those of the real pass, and Adam adds them
 * (src/ops/graph.cu:302-309).  On the tensor path the two passes run as ONE pass over the batch
 * [g_out | x] of 2*batch images (same math per image, half the launches): "d_grad*" then holds
 * the sum of both paths and "d_gradb*" stays zero. */
int dcg_trainer_tensor(dcg_trainer* t, const char* name, float** ptr, size_t* count);
/* Generator forward only (z -> g_out): dcgan/main.cu:252-269. */
int dcg_trainer_generate(dcg_trainer* t);
/* Discriminator forward + backward on the real images "x" alone against labels of all ones: sigmoid
 * cross-entropy, then the kernel, bias and input gradient of every layer (the image gradient lands
 * in the generator-output gradient buffer).  Weight gradients go to "d_gradb0..9".  A measurement and
 * test entry; it leaves parameters untouched. */
int dcg_trainer_d_fwd_bwd(dcg_trainer* t);
/* graph.run({d_opti, d_loss}) minus the update: G forward, D on fake and real, d_loss, D gradients. */
int dcg_trainer_d_backward(dcg_trainer* t);
/* Adam on the discriminator with gradients scaled by grad_scale (1/world after an all-reduce). */
int dcg_trainer_d_apply(dcg_trainer* t, float grad_scale);
/* graph.run({g_opti, g_loss}) minus the update: G forward, D on fake, g_loss, G gradients. */
int dcg_trainer_g_backward(dcg_trainer* t);
/* The same in two parts, for callers that overlap something with the first: part 0 is the generator's
 * forward pass (reads z and the generator's parameters only - in data-parallel training it can run
 * while the discriminator's gradients are still being all-reduced), part 1 everything after it. */
int dcg_trainer_g_backward_part(dcg_trainer* t, int part);
int dcg_trainer_g_apply(dcg_trainer* t, float grad_scale);
/* One whole iteration: d_backward, d_apply, then twice g_backward, g_apply; with a communicator
 * (dcg_trainer_create_dp) each *_apply is preceded by the sum of that network's gradients over the
 * ranks and scales by 1/world.  The third call onwards replays the iteration as one CUDA graph. */
int dcg_trainer_step(dcg_trainer* t);
/* Checkpoint / resume, the counterpart of ops::Graph::save_vars / load_vars (src/ops/graph.cu:326-361).
 * dcg_trainer_save enqueues a device -> pinned-host snapshot behind the updates enqueued so far and
 * returns; a host thread writes the file once the copy has landed, so training continues meanwhile
 * (dcg_trainer_save_wait joins it and returns its status; the next save, a load and destroy wait too).
 * File: raw tensor archive ("DCGT", u32 1, u32 count, per tensor u32 rank, extents, fp32 values) holding the
 * generator's 10 variables, the discriminator's 10, Adam's first and second moments of both (which the
 * reference does not save, src/api/adam-optimizer.cu:39-45) and the step counters [g_t, d_t].
 * dcg_trainer_load also accepts an archive of the 20 variables alone. */
int dcg_trainer_save(dcg_trainer* t, const char* path);
int dcg_trainer_save_wait(dcg_trainer* t);
int dcg_trainer_load(dcg_trainer* t, const char* path);
/* The trainer's execution context (for dcg_context_profile_begin / _end around its phases). */
dcg_context* dcg_trainer_context(dcg_trainer* t);
/* How a data-parallel trainer exchanges gradients: 0 = no communicator, 1 = NCCL all-reduce + replicated Adam,
 * 2 = the fused kernel over peer memory (every rank sums its 1/W slice of all ranks' gradients over NVLink,
 * applies Adam to it and writes the new parameters of the slice to every rank; the default where the ranks
 * can map each other's memory, DCG_DP_FUSED=0 selects 1). */
int dcg_trainer_dp_mode(const dcg_trainer* t);
/* How dcg_trainer_step runs: 2 = the whole iteration replays as one CUDA graph, 1 = still warming up
 * (eager / per-list graphs), 0 = capturing the iteration failed and it stays eager. */
int dcg_trainer_step_mode(const dcg_trainer* t);
/* Kernels launched by the last dcg_trainer_step. */
uint64_t dcg_trainer_step_launches(const dcg_trainer* t);
size_t dcg_trainer_arena_bytes(const dcg_trainer* t);

/* ---- diagnostics --------------------------------------------------------- */
/* Synchronises the device, then reads and clears the status word the tensor-path
 * kernels write when one of their bounded waits (mbarrier, ~1 s) runs out.
 * Returns DCG_OK or DCG_ERR_DEVICE (dcg_last_error() names block, role, stage). */
int dcg_device_status(void);
const char* dcg_last_error(void);
/* Testing hooks of the tensor-path convolution kernels (no counterpart in the reference; process-wide,
 * they affect launches enqueued after the call):
 *  dcg_debug_set_wait_limit  limit of every bounded barrier wait in SM clocks (<= 0 restores ~1 s);
 *  dcg_debug_skip_stage      the TMA producer leaves pipeline stage `stage` of every tile out (< 0: never), so
 *                            that a consumer's wait runs into the limit: the kernel then records the failure,
 *                            still terminates, and dcg_device_status() returns DCG_ERR_DEVICE;
 *  dcg_debug_set_dx_mode     which input-gradient kernel the tensor path plans: 0 = one tile per parity class,
 *                            1 = the parity classes of a tile fused in one CTA where one CTA per tile fills the
 *                            GPU (default), 2 = fused wherever the shape allows, < 0 = back to the default;
 *  dcg_debug_fused_dx_launches  how often the fused kernel has been launched (tests check which kernel ran). */
void dcg_debug_set_wait_limit(long long sm_clocks);
void dcg_debug_skip_stage(int stage);
void dcg_debug_set_dx_mode(int mode);
uint64_t dcg_debug_fused_dx_launches(void);   /* launches of the class-fused input-gradient kernel so far */
/* Library version and the architecture the kernels were built for ("sm_100a"). */
const char* dcg_build_info(void);
/* Kernels launched by this library since it was loaded (all contexts, all threads). */
uint64_t dcg_launches_total(void);

#ifdef __cplusplus
}
#endif
#endif /* DCGAN_B200_H */
