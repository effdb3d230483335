// Node-level backend: the drop-in boundary of the reference's GPU runtime.
//
// The reference dispatches every runtime instruction through
// gpu::kernels_list[node->type](node) (src/gpu/kernels.cu:20-64) from the serial
// loop gpu::run (src/gpu/runner.cu:10-18).  dcg_run_node is that table,
// dcg_run_nodes that loop - minus the per-node device synchronisation, plus
// optional fusion of adjacent nodes.  Operand decoding follows the reference
// handlers field for field, including which size array each handler reads.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <set>
#include <string>
#include <utility>
#include <vector>

#include "adam.cuh"
#include "backend.cuh"
#include "common.cuh"
#include "conv.cuh"

// One timed launch group of a profiled run: CUDA events on the context's stream around it.
struct ProfRec {
    std::string name;
    double flops;
    cudaEvent_t e0, e1;
    int repeat = 1;   // launches between the two events; the elapsed time is divided by it
};

struct dcg_context {
    cudaStream_t stream = nullptr;
    int precision = DCG_PREC_TF32;
    void* ws = nullptr;
    size_t ws_bytes = 0;          // usable by the operators; an owned allocation has the ticket words behind it
    unsigned* tickets = nullptr;  // kColsumTicketBytes of zeroed ticket words of the column sums (owned scratch only)
    bool owns_ws = false;
    // Bumped whenever something a captured CUDA graph bakes in changes: a scratch buffer (main or
    // side) moved, or the precision (which selects kernels and plans) was switched.
    uint64_t generation = 0;
    // Second stream with scratch of its own for nodes flagged DCG_NODE_SIDE (created on first use,
    // only when the context owns its scratch): they fork off the main stream, run concurrently with
    // the nodes that follow, and are joined at the end of the list.
    // Two of them: kernel gradients (convolutions) on one, the small reductions and dense weight
    // gradients on the other, so that a 10 us column sum does not queue behind a 20 us convolution.
    cudaStream_t side[2] = {nullptr, nullptr};
    void* side_ws[2] = {nullptr, nullptr};
    size_t side_ws_bytes[2] = {0, 0};
    unsigned* side_tickets[2] = {nullptr, nullptr};
    cudaEvent_t ev_fork = nullptr, ev_join[2] = {nullptr, nullptr};
    bool side_busy[2] = {false, false}, side_failed = false;
    uint64_t launches_base = 0;
    bool profiling = false;
    std::vector<ProfRec> recs;
};

namespace dcg {

bool context_is_profiling(const dcg_context* ctx) { return ctx && ctx->profiling; }
uint64_t context_generation(const dcg_context* ctx) { return ctx ? ctx->generation : 0; }

namespace {
std::mutex g_registry_mutex;
std::set<dcg_context*> g_registry;
}  // namespace

void contexts_reset_tickets()
{
    std::lock_guard<std::mutex> lock(g_registry_mutex);
    cudaDeviceSynchronize();
    for (dcg_context* c : g_registry) {
        if (c->tickets) cudaMemset(c->tickets, 0, kColsumTicketBytes);
        for (int i = 0; i < 2; ++i)
            if (c->side_tickets[i]) cudaMemset(c->side_tickets[i], 0, kColsumTicketBytes);
    }
    cudaGetLastError();
}

// Times everything enqueued on the context's stream during its lifetime when profiling is on.
ProfScope::ProfScope(dcg_context* c, const char* name, double flops) : ctx(c), active(c && c->profiling)
{
    if (!active) return;
    ProfRec r;
    r.name = name;
    r.flops = flops;
    if (cudaEventCreate(&r.e0) != cudaSuccess || cudaEventCreate(&r.e1) != cudaSuccess) { active = false; return; }
    cudaEventRecord(r.e0, ctx->stream);
    ctx->recs.push_back(r);
}

ProfScope::~ProfScope()
{
    if (active) cudaEventRecord(ctx->recs.back().e1, ctx->stream);
}

namespace {

const char* node_type_name(int type)
{
    static const char* names[DCG_OP_COUNT] = {
        "mat_mat_mul", "mat_rvect_add", "sigmoid", "mse", "softmax", "log_softmax", "softmax_cross_entropy",
        "conv2d", "relu", "relu_leaky", "tanh", "mse_grad", "sigmoid_grad", "mat_mul_add", "tmat_mat_mul",
        "mat_tmat_mul", "mat_sum_rows", "mat_sum_cols", "softmax_cross_entropy_grad", "relu_grad",
        "conv2d_bias_add", "update", "sigmoid_cross_entropy", "sigmoid_cross_entropy_grad",
        "conv2d_input_grad", "conv2d_kernel_grad", "argmax_acc", "moment_update", "moment_update2",
        "adam_update", "leaky_relu_grad", "conv2d_bias_add_grad", "tanh_grad", "conv2d_transpose",
        "conv2d_transpose_input_grad", "conv2d_transpose_kernel_grad", "add"};
    return (type >= 0 && type < DCG_OP_COUNT) ? names[type] : "unknown";
}


// Makes sure the context has `bytes` of scratch.  A context that owns its
// scratch grows it (cudaFree synchronises, so kernels still reading the old
// buffer finish first); a caller-provided buffer is only checked.
int ensure_workspace(dcg_context* ctx, size_t bytes)
{
    if (bytes <= ctx->ws_bytes) return DCG_OK;
    if (!ctx->owns_ws && ctx->ws)
        return fail(DCG_ERR_WORKSPACE, "context workspace %zu < %zu bytes needed", ctx->ws_bytes, bytes);
    if (ctx->ws) DCG_CUDA(cudaFree(ctx->ws));
    ctx->ws = nullptr;
    ctx->ws_bytes = 0;
    ctx->tickets = nullptr;
    ++ctx->generation;   // graphs captured with the old address are stale
    const size_t want = align_up(bytes + bytes / 4, (size_t)1 << 20);
    DCG_CUDA(cudaMalloc(&ctx->ws, want + kColsumTicketBytes));
    // the ticket words of the column sums sit behind the usable part and start out zero
    ctx->tickets = reinterpret_cast<unsigned*>(static_cast<unsigned char*>(ctx->ws) + want);
    DCG_CUDA(cudaMemset(ctx->tickets, 0, kColsumTicketBytes));
    ctx->ws_bytes = want;
    ctx->owns_ws = true;
    return DCG_OK;
}

// Column sum on the context's scratch.  Owned scratch carries its own zeroed ticket words; a
// caller-provided buffer goes through the public entry point, which clears them per call.
int context_colsum(dcg_context* ctx, const float* a, float* out, size_t rows, size_t cols)
{
    DCG_CHECK_ARG(a && out && rows > 0 && cols > 0 && cols <= 0x7fffffffu, "column sum node: bad operands");
    if (ctx->ws && !ctx->owns_ws) {
        const size_t need = dcg_colsum_workspace_bytes(rows, cols);
        if (need > ctx->ws_bytes)
            return fail(DCG_ERR_WORKSPACE, "context workspace %zu < %zu bytes needed", ctx->ws_bytes, need);
        return dcg_colsum(a, out, rows, cols, ctx->ws, ctx->ws_bytes, ctx->stream);
    }
    const size_t need = colsum_partial_bytes_max(rows, cols);
    int st = ensure_workspace(ctx, need > 0 ? need : 1);
    if (st) return st;
    return colsum_launch(a, out, rows, cols, ctx->ws, ctx->ws_bytes, ctx->tickets, ctx->stream);
}

struct ConvCall {
    dcg_conv_desc d;
    int kind;           // ConvKind
    const float* a;     // fwd: x, dx: dy, dk: x
    const float* b;     // fwd: k, dx: k,  dk: dy
    float* out;
    int out_channels;   // channel count of the tensor `out` (epilogue broadcast axis)
    size_t out_elems;
};

inline void fill_same(dcg_conv_desc& d, int n, int h, int w, int c, int kh, int kw, int o, int ho,
                      int wo, int sh, int sw, int pad_h, int pad_w)
{
    d.n = n; d.h = h; d.w = w; d.c = c; d.kh = kh; d.kw = kw; d.o = o; d.ho = ho; d.wo = wo;
    d.stride_h = sh; d.stride_w = sw; d.pad_top = pad_h / 2; d.pad_left = pad_w / 2;
}

// Decodes the six convolution node types into a ConvCall.
int decode_conv(const dcg_node* nd, ConvCall& cc)
{
    dcg_conv_desc& d = cc.d;
    switch (nd->type) {
    case DCG_OP_CONV2D: {  // src/gpu/conv2d.cu:13-62
        const int n = nd->sizes1[0], h = nd->sizes1[1], w = nd->sizes1[2], c = nd->sizes1[3];
        const int kh = nd->sizes2[0], kw = nd->sizes2[1], o = nd->sizes2[3];
        const int sh = nd->intconst[0], sw = nd->intconst[1];
        DCG_CHECK_ARG(sh > 0 && sw > 0, "conv2d node: bad strides");
        const int ho = (h + nd->int_cons1 - kh) / sh + 1, wo = (w + nd->int_cons2 - kw) / sw + 1;
        fill_same(d, n, h, w, c, kh, kw, o, ho, wo, sh, sw, nd->int_cons1, nd->int_cons2);
        cc.kind = kConvFwd; cc.a = nd->in1; cc.b = nd->in2; cc.out = nd->out1;
        cc.out_channels = o; cc.out_elems = (size_t)n * ho * wo * o;
        return DCG_OK;
    }
    case DCG_OP_CONV2D_INPUT_GRAD: {  // src/gpu/conv2d.cu:70-117 (both strides = intconst[0])
        const int kh = nd->sizes2[0], kw = nd->sizes2[1], c = nd->sizes2[2], o = nd->sizes2[3];
        const int n = nd->sizes1[0], ho = nd->sizes1[1], wo = nd->sizes1[2];
        const int s = nd->intconst[0];
        const int h = nd->intconst2[0], w = nd->intconst2[1];
        fill_same(d, n, h, w, c, kh, kw, o, ho, wo, s, s, (ho - 1) * s - h + kh, (wo - 1) * s - w + kw);
        cc.kind = kConvDx; cc.a = nd->in1; cc.b = nd->in2; cc.out = nd->out1;
        cc.out_channels = c; cc.out_elems = (size_t)n * h * w * c;
        return DCG_OK;
    }
    case DCG_OP_CONV2D_KERNEL_GRAD: {  // src/gpu/conv2d.cu:119-165
        const int n = nd->sizes2[0], h = nd->sizes2[1], w = nd->sizes2[2], c = nd->sizes2[3];
        const int ho = nd->sizes1[1], wo = nd->sizes1[2], o = nd->sizes1[3];
        const int sh = nd->intconst[0], sw = nd->intconst[1];
        const int pad_h = nd->intconst2[0], pad_w = nd->intconst2[1];
        const int kh = h + pad_h - sh * (ho - 1), kw = w + pad_w - sw * (wo - 1);
        fill_same(d, n, h, w, c, kh, kw, o, ho, wo, sh, sw, pad_h, pad_w);
        cc.kind = kConvDk; cc.a = nd->in2; cc.b = nd->in1; cc.out = nd->out1;
        cc.out_channels = o; cc.out_elems = (size_t)kh * kw * c * o;
        return DCG_OK;
    }
    case DCG_OP_CONV2D_TRANSPOSE: {  // src/gpu/conv2d.cu:167-212: the dx of a conv whose y is the input
        const int n = nd->sizes2[0], ho = nd->sizes2[1], wo = nd->sizes2[2], o = nd->sizes2[3];
        const int kh = nd->sizes3[0], kw = nd->sizes3[1], c = nd->sizes3[2];
        const int sh = nd->intconst[0], sw = nd->intconst[1];
        const int h = nd->sizes1[1], w = nd->sizes1[2];
        fill_same(d, n, h, w, c, kh, kw, o, ho, wo, sh, sw, (ho - 1) * sh - h + kh, (wo - 1) * sw - w + kw);
        cc.kind = kConvDx; cc.a = nd->in1; cc.b = nd->in2; cc.out = nd->out1;
        cc.out_channels = c; cc.out_elems = (size_t)n * h * w * c;
        return DCG_OK;
    }
    case DCG_OP_CONV2D_TRANSPOSE_INPUT_GRAD: {  // src/gpu/conv2d.cu:214-259: a forward conv of dy
        const int kh = nd->sizes2[0], kw = nd->sizes2[1], c = nd->sizes2[2], o = nd->sizes2[3];
        const int n = nd->sizes1[0], h = nd->sizes1[1], w = nd->sizes1[2];
        const int s = nd->intconst[0];
        const int ho = nd->intconst2[0], wo = nd->intconst2[1];
        fill_same(d, n, h, w, c, kh, kw, o, ho, wo, s, s, (ho - 1) * s + kh - h, (wo - 1) * s + kw - w);
        cc.kind = kConvFwd; cc.a = nd->in1; cc.b = nd->in2; cc.out = nd->out1;
        cc.out_channels = o; cc.out_elems = (size_t)n * ho * wo * o;
        return DCG_OK;
    }
    case DCG_OP_CONV2D_TRANSPOSE_KERNEL_GRAD: {  // src/gpu/conv2d.cu:264-307: dk with (dy, x) swapped
        // in1 = dy [n,h,w,c] plays the conv input, in2 = x [n,ho,wo,o] the conv output gradient
        const int n = nd->sizes2[0], ho = nd->sizes2[1], wo = nd->sizes2[2], o = nd->sizes2[3];
        const int h = nd->sizes1[1], w = nd->sizes1[2], c = nd->sizes1[3];
        const int sh = nd->intconst[0], sw = nd->intconst[1];
        const int kh = nd->sizes3[0], kw = nd->sizes3[1];
        fill_same(d, n, h, w, c, kh, kw, o, ho, wo, sh, sw, (ho - 1) * sh + kh - h, (wo - 1) * sw + kw - w);
        cc.kind = kConvDk; cc.a = nd->in1; cc.b = nd->in2; cc.out = nd->out1;
        cc.out_channels = o; cc.out_elems = (size_t)kh * kw * c * o;
        return DCG_OK;
    }
    default:
        return fail(DCG_ERR_INVALID, "node type %d is not a convolution", nd->type);
    }
}

int run_conv(dcg_context* ctx, const ConvCall& cc, const dcg_epilogue* ep)
{
    const size_t need = dcg_conv_workspace_bytes(&cc.d, cc.kind, ctx->precision);
    int st = ensure_workspace(ctx, need);
    if (st) return st;
    char name[96];
    if (ctx->profiling) {
        static const char* kinds[3] = {"conv_fwd", "conv_dx", "conv_dk"};
        snprintf(name, sizeof(name), "%s x[%d,%d,%d,%d] k[%d,%d,%d,%d]", kinds[cc.kind], cc.d.n, cc.d.h, cc.d.w,
                 cc.d.c, cc.d.kh, cc.d.kw, cc.d.c, cc.d.o);
    }
    // algorithmic work of any of the three operators: 2 * B*Ho*Wo * KH*KW * Cin * Cout
    ProfScope scope(ctx, name, 2.0 * cc.d.n * cc.d.ho * cc.d.wo * cc.d.kh * cc.d.kw * (double)cc.d.c * cc.d.o);
    // Profiling may launch the convolution several times back to back between its two events
    // (DCG_PROFILE_REPEAT): a convolution only reads its operands and writes its outputs, so the
    // repeats leave the same results, and the event pair then measures device time per launch
    // rather than one launch plus the gap to the previous kernel.
    int repeat = 1;
    if (ctx->profiling && !ctx->recs.empty()) {
        static const int env_repeat = [] { const char* v = getenv("DCG_PROFILE_REPEAT"); return v ? atoi(v) : 1; }();
        repeat = env_repeat > 1 ? env_repeat : 1;
        ctx->recs.back().repeat = repeat;
    }
    int rc = DCG_OK;
    for (int r = 0; r < repeat && rc == DCG_OK; ++r) {
        switch (cc.kind) {
        case kConvFwd:
            rc = dcg_conv2d_fwd(&cc.d, cc.a, cc.b, cc.out, ep, ctx->precision, ctx->ws, ctx->ws_bytes, ctx->stream);
            break;
        case kConvDx:
            rc = dcg_conv2d_dx(&cc.d, cc.a, cc.b, cc.out, ep, ctx->precision, ctx->ws, ctx->ws_bytes, ctx->stream);
            break;
        default:
            rc = dcg_conv2d_dk(&cc.d, cc.a, cc.b, cc.out, ctx->precision, ctx->ws, ctx->ws_bytes, ctx->stream);
            break;
        }
    }
    return rc;
}

inline bool is_conv_with_epilogue(int type)
{
    return type == DCG_OP_CONV2D || type == DCG_OP_CONV2D_INPUT_GRAD ||
           type == DCG_OP_CONV2D_TRANSPOSE || type == DCG_OP_CONV2D_TRANSPOSE_INPUT_GRAD;
}

inline int act_of_node(int type)
{
    switch (type) {
    case DCG_OP_RELU: return DCG_ACT_RELU;
    case DCG_OP_RELU_LEAKY: return DCG_ACT_LEAKY;
    case DCG_OP_TANH: return DCG_ACT_TANH;
    case DCG_OP_SIGMOID: return DCG_ACT_SIGMOID;
    default: return -1;
    }
}

inline int grad_act_of_node(int type)
{
    switch (type) {
    case DCG_OP_RELU_GRAD: return DCG_ACT_RELU;
    case DCG_OP_LEAKY_RELU_GRAD: return DCG_ACT_LEAKY;
    case DCG_OP_TANH_GRAD: return DCG_ACT_TANH;
    case DCG_OP_SIGMOID_GRAD: return DCG_ACT_SIGMOID;
    default: return -1;
    }
}

// Tries to run nodes[i..] as one fused convolution; returns the number of nodes
// consumed (>= 1) or a negative status.
int run_fused_conv(dcg_context* ctx, const dcg_node* nodes, int i, int count)
{
    ConvCall cc;
    int st = decode_conv(&nodes[i], cc);
    if (st) return st;
    dcg_epilogue ep{};
    int used = 1;
    const float* cur = cc.out;       // tensor produced so far
    float* final_out = cc.out;
    bool raw_dead = (nodes[i].flags & DCG_NODE_OUT_DEAD) != 0;
    bool need_raw = false;

    // bias add directly after
    if (i + used < count) {
        const dcg_node& b = nodes[i + used];
        if (b.type == DCG_OP_MAT_RVECT_ADD && b.in1 == cur && b.len2 == (size_t)cc.out_channels &&
            b.len1 * b.len2 == cc.out_elems && b.out1 != cur) {
            ep.bias = b.in2;
            need_raw = !raw_dead;
            cur = b.out1;
            final_out = b.out1;
            ++used;
        }
    }
    // activation, or activation gradient, directly after
    if (i + used < count) {
        const dcg_node& a = nodes[i + used];
        const int act = act_of_node(a.type), gact = grad_act_of_node(a.type);
        if (act >= 0 && a.in1 == cur && a.len1 == cc.out_elems && a.out1 != cur) {
            const bool prev_dead = (nodes[i + used - 1].flags & DCG_NODE_OUT_DEAD) != 0;
            if (ep.bias) {
                if (!prev_dead) ep.pre_act = const_cast<float*>(cur);
            } else {
                need_raw = !raw_dead;
            }
            ep.act = act;
            ep.alpha = a.type == DCG_OP_RELU_LEAKY ? a.alpha_leaky : 0.f;
            final_out = a.out1;
            ++used;
        } else if (gact >= 0 && !ep.bias && a.in2 == cur && a.len1 == cc.out_elems &&
                   a.out1 != cur && a.in1 != cur) {
            need_raw = !raw_dead;
            ep.gate = a.in1;
            ep.gate_act = gact;
            ep.gate_alpha = a.type == DCG_OP_LEAKY_RELU_GRAD ? a.cons1 : 0.f;
            final_out = a.out1;
            ++used;
        }
    }
    if (used == 1) {
        st = run_conv(ctx, cc, nullptr);
        return st ? st : 1;
    }
    if (need_raw) ep.raw_out = cc.out;
    cc.out = final_out;
    st = run_conv(ctx, cc, &ep);
    return st ? st : used;
}

struct AdamTriple {
    dcg_adam_tensor t;
    float a1, b1, a2, b2, lr, beta1, beta2, eps;
    float* t_host;
};

// Recognises moment_update + moment_update2 (either order) + adam_update on one variable.
bool match_adam_triple(const dcg_node* n, int i, int count, AdamTriple& out)
{
    if (i + 2 >= count) return false;
    const dcg_node *m1 = nullptr, *m2 = nullptr;
    for (int k = 0; k < 2; ++k) {
        if (n[i + k].type == DCG_OP_MOMENT_UPDATE) m1 = &n[i + k];
        else if (n[i + k].type == DCG_OP_MOMENT_UPDATE2) m2 = &n[i + k];
    }
    const dcg_node& ad = n[i + 2];
    if (!m1 || !m2 || ad.type != DCG_OP_ADAM_UPDATE) return false;
    if (m1->in1 != m2->in1 || m1->len1 != m2->len1 || ad.len1 != m1->len1) return false;
    if (ad.in1 != m1->out1 || ad.in2 != m2->out1 || !ad.out2) return false;
    out.t.p = ad.out1; out.t.g = m1->in1; out.t.g2 = nullptr;
    out.t.m = m1->out1; out.t.v = m2->out1; out.t.n = ad.len1;
    out.a1 = m1->cons1; out.b1 = m1->cons2; out.a2 = m2->cons1; out.b2 = m2->cons2;
    out.lr = ad.cons1; out.beta1 = ad.cons2; out.beta2 = ad.cons3; out.eps = ad.cons4;
    out.t_host = ad.out2;
    return true;
}

}  // namespace
}  // namespace dcg

using namespace dcg;

extern "C" int dcg_context_create(dcg_context** out, int precision, void* workspace,
                                  size_t workspace_bytes, dcg_stream_t stream)
{
    DCG_CHECK_ARG(out, "dcg_context_create: null output pointer");
    DCG_CHECK_ARG(precision == DCG_PREC_TF32 || precision == DCG_PREC_FP32 || precision == DCG_PREC_3XTF32,
                  "dcg_context_create: unknown precision %d", precision);
    DCG_CHECK_ARG((workspace == nullptr) == (workspace_bytes == 0),
                  "dcg_context_create: workspace pointer and size disagree");
    dcg_context* ctx = new dcg_context();
    ctx->stream = as_stream(stream);
    ctx->precision = precision;
    ctx->ws = workspace;
    ctx->ws_bytes = workspace_bytes;
    ctx->owns_ws = false;
    ctx->launches_base = launches_total();
    {
        std::lock_guard<std::mutex> lock(g_registry_mutex);
        g_registry.insert(ctx);
    }
    *out = ctx;
    return DCG_OK;
}

extern "C" void dcg_context_destroy(dcg_context* ctx)
{
    if (!ctx) return;
    {
        std::lock_guard<std::mutex> lock(g_registry_mutex);
        g_registry.erase(ctx);
    }
    if (ctx->owns_ws && ctx->ws) cudaFree(ctx->ws);
    for (int i = 0; i < 2; ++i) {
        if (ctx->side_ws[i]) cudaFree(ctx->side_ws[i]);
        if (ctx->ev_join[i]) cudaEventDestroy(ctx->ev_join[i]);
        if (ctx->side[i]) cudaStreamDestroy(ctx->side[i]);
    }
    if (ctx->ev_fork) cudaEventDestroy(ctx->ev_fork);
    delete ctx;
}

extern "C" int dcg_context_set_precision(dcg_context* ctx, int precision)
{
    DCG_CHECK_ARG(ctx, "dcg_context_set_precision: null context");
    DCG_CHECK_ARG(precision == DCG_PREC_TF32 || precision == DCG_PREC_FP32 || precision == DCG_PREC_3XTF32,
                  "dcg_context_set_precision: unknown precision %d", precision);
    if (ctx->precision != precision) ++ctx->generation;   // captured graphs hold the old precision's kernels
    ctx->precision = precision;
    return DCG_OK;
}

extern "C" uint64_t dcg_context_launch_count(const dcg_context* ctx)
{
    return ctx ? launches_total() - ctx->launches_base : 0;
}

namespace {
// On the tensor path a wide dense layer (the generator's 100 -> 8192 projection) is a 1x1 convolution over
// a 1x1 image: x [m,1,1,n], k [1,1,n,p], bias in the epilogue; K that is not a multiple of 32 is zero-filled by
// TMA.  With act_out the activation node that follows is part of the same launch (nd->out1 still receives the
// pre-activation).  Returns 1 if the shape or the precision keeps the node off the tensor path.
int run_dense_on_tensor_path(dcg_context* ctx, const dcg_node* nd, int act, float alpha, float* act_out)
{
    const size_t m = nd->len1, n = nd->len2, pp = nd->len3;
    if (!(ctx->precision != DCG_PREC_FP32 && pp >= 1024 && pp % 32 == 0 && n % 4 == 0 && n >= 32 && m >= 32 &&
          m <= 65536 && n <= 65536 && pp <= 65536 &&
          ((reinterpret_cast<uintptr_t>(nd->in1) | reinterpret_cast<uintptr_t>(nd->in2) |
            reinterpret_cast<uintptr_t>(nd->in3) | reinterpret_cast<uintptr_t>(nd->out1) |
            reinterpret_cast<uintptr_t>(act_out)) & 15u) == 0))
        return 1;
    dcg_conv_desc d{};
    d.n = (int)m; d.h = 1; d.w = 1; d.c = (int)n; d.kh = 1; d.kw = 1; d.o = (int)pp; d.ho = 1; d.wo = 1;
    d.stride_h = 1; d.stride_w = 1; d.pad_top = 0; d.pad_left = 0;
    const bool x3 = ctx->precision == DCG_PREC_3XTF32;
    if (!conv_tc_supported(d, kConvFwd, x3)) return 1;
    int st = ensure_workspace(ctx, conv_tc_workspace(d, kConvFwd, x3));
    if (st) return st;
    dcg_epilogue ep{};
    ep.bias = nd->in3;
    ep.act = DCG_ACT_NONE;
    float* out = nd->out1;
    if (act_out) {
        ep.act = act;
        ep.alpha = alpha;
        ep.pre_act = nd->out1;
        out = act_out;
    }
    ProfScope scope(act_out ? ctx : nullptr, "mat_mul_add", 0.0);   // the fused form does not pass through dcg_run_node
    return dcg_conv2d_fwd(&d, nd->in1, nd->in2, out, &ep, ctx->precision, ctx->ws, ctx->ws_bytes, ctx->stream);
}
}  // namespace

extern "C" int dcg_run_node(dcg_context* ctx, const dcg_node* nd)
{
    DCG_CHECK_ARG(ctx && nd, "dcg_run_node: null argument");
    dcg_stream_t s = ctx->stream;
    const bool is_conv = is_conv_with_epilogue(nd->type) || nd->type == DCG_OP_CONV2D_KERNEL_GRAD ||
                         nd->type == DCG_OP_CONV2D_TRANSPOSE_KERNEL_GRAD;
    ProfScope scope(is_conv ? nullptr : ctx, node_type_name(nd->type), 0.0);  // convolutions time themselves
    switch (nd->type) {
    case DCG_OP_MAT_MAT_MUL:  // src/gpu/matmul.cu:90-104
        return dcg_matmul(nd->in1, nd->in2, nullptr, nd->out1, nd->len1, nd->len2, nd->len3, s);
    case DCG_OP_MAT_RVECT_ADD:  // src/gpu/matmul.cu:106-119
        return dcg_bias_act(nd->in1, nd->in2, nd->out1, nullptr, nd->len1, nd->len2, DCG_ACT_NONE, 0.f, s);
    case DCG_OP_SIGMOID:  // src/gpu/sigmoid.cu:129-136
        return dcg_act_fwd(nd->in1, nd->out1, nd->len1, DCG_ACT_SIGMOID, 0.f, s);
    case DCG_OP_MSE:  // src/gpu/sum.cu:218-222
        return dcg_mse(nd->in1, nd->in2, nd->out1, nd->len1, nd->len2, s);
    case DCG_OP_SOFTMAX:  // src/gpu/softmax.cu:322-327
        return dcg_softmax(nd->in1, nd->out1, nd->len1, nd->len2, s);
    case DCG_OP_LOG_SOFTMAX:  // src/gpu/softmax.cu:329-334
        return dcg_log_softmax(nd->in1, nd->out1, nd->len1, nd->len2, s);
    case DCG_OP_SOFTMAX_CROSS_ENTROPY:  // src/gpu/softmax.cu:336-350
        return dcg_softmax_xent(nd->in1, nd->in2, nd->out1, nd->len1, nd->len2, s);
    case DCG_OP_RELU:  // src/gpu/relu.cu:70-77
        return dcg_act_fwd(nd->in1, nd->out1, nd->len1, DCG_ACT_RELU, 0.f, s);
    case DCG_OP_RELU_LEAKY:  // src/gpu/relu.cu:88-97
        return dcg_act_fwd(nd->in1, nd->out1, nd->len1, DCG_ACT_LEAKY, nd->alpha_leaky, s);
    case DCG_OP_TANH:  // src/gpu/sigmoid.cu:148-155
        return dcg_act_fwd(nd->in1, nd->out1, nd->len1, DCG_ACT_TANH, 0.f, s);
    case DCG_OP_MSE_GRAD:  // src/gpu/sum.cu:224-229
        return dcg_mse_grad(nd->in1, nd->in2, nd->out1, nd->len1, s);
    case DCG_OP_SIGMOID_GRAD:  // src/gpu/sigmoid.cu:138-146
        return dcg_act_grad(nd->in1, nd->in2, nd->out1, nd->len1, DCG_ACT_SIGMOID, 0.f, s);
    case DCG_OP_MAT_MUL_ADD: {  // src/gpu/matmul.cu:121-137
        const int st = run_dense_on_tensor_path(ctx, nd, DCG_ACT_NONE, 0.f, nullptr);
        if (st != 1) return st;
        return dcg_matmul(nd->in1, nd->in2, nd->in3, nd->out1, nd->len1, nd->len2, nd->len3, s);
    }
    case DCG_OP_TMAT_MAT_MUL:  // src/gpu/matmul.cu:139-153
        return dcg_matmul_tn(nd->in1, nd->in2, nd->out1, nd->len1, nd->len2, nd->len3, s);
    case DCG_OP_MAT_TMAT_MUL:  // src/gpu/matmul.cu:155-169
        return dcg_matmul_nt(nd->in1, nd->in2, nd->out1, nd->len1, nd->len2, nd->len3, s);
    case DCG_OP_MAT_SUM_ROWS:  // src/gpu/sum.cu:231-236
        return dcg_rowsum(nd->in1, nd->out1, nd->len1, nd->len2, s);
    case DCG_OP_MAT_SUM_COLS:  // src/gpu/sum.cu:238-243
        return context_colsum(ctx, nd->in1, nd->out1, nd->len1, nd->len2);
    case DCG_OP_SOFTMAX_CROSS_ENTROPY_GRAD:  // src/gpu/softmax.cu:352-359
        return dcg_softmax_xent_grad(nd->in1, nd->in2, nd->out1, nd->len1, nd->len2, s);
    case DCG_OP_RELU_GRAD:  // src/gpu/relu.cu:79-86
        return dcg_act_grad(nd->in1, nd->in2, nd->out1, nd->len1, DCG_ACT_RELU, 0.f, s);
    case DCG_OP_CONV2D_BIAS_ADD: {  // slot left empty by the reference (src/gpu/kernels.cu:44)
        const size_t cols = (size_t)nd->sizes1[3];
        const size_t rows = (size_t)nd->sizes1[0] * nd->sizes1[1] * nd->sizes1[2];
        return dcg_bias_act(nd->in1, nd->in2, nd->out1, nullptr, rows, cols, DCG_ACT_NONE, 0.f, s);
    }
    case DCG_OP_UPDATE:  // src/gpu/update.cu:58-63
        return dcg_update(nd->in1, nd->out1, nd->in2, nd->len1, s);
    case DCG_OP_SIGMOID_CROSS_ENTROPY:  // src/gpu/sigmoid.cu:167-171
        return dcg_sigmoid_xent(nd->in1, nd->in2, nd->out1, nd->len1, s);
    case DCG_OP_SIGMOID_CROSS_ENTROPY_GRAD:  // src/gpu/sigmoid.cu:173-181
        return dcg_sigmoid_xent_grad(nd->in1, nd->in2, nd->out1, nd->len1, s);
    case DCG_OP_ARGMAX_ACC:  // src/gpu/sum.cu:245-249
        return dcg_argmax_acc(nd->in1, nd->in2, nd->out1, nd->len1, nd->len2, s);
    case DCG_OP_MOMENT_UPDATE:  // src/gpu/update.cu:65-71
        return moment_update_launch(nd->in1, nd->out1, nd->cons1, nd->cons2, nd->len1, false, ctx->stream);
    case DCG_OP_MOMENT_UPDATE2:  // src/gpu/update.cu:73-79
        return moment_update_launch(nd->in1, nd->out1, nd->cons1, nd->cons2, nd->len1, true, ctx->stream);
    case DCG_OP_ADAM_UPDATE: {  // src/gpu/update.cu:81-96
        DCG_CHECK_ARG(nd->out2, "adam_update node: null step counter");
        const float lr_t = dcg_adam_lr_t(nd->out2, nd->cons1, nd->cons2, nd->cons3);
        return adam_apply_launch(nd->in1, nd->in2, nd->out1, lr_t, nd->cons4, nd->len1, ctx->stream);
    }
    case DCG_OP_LEAKY_RELU_GRAD:  // src/gpu/relu.cu:99-109
        return dcg_act_grad(nd->in1, nd->in2, nd->out1, nd->len1, DCG_ACT_LEAKY, nd->cons1, s);
    case DCG_OP_CONV2D_BIAS_ADD_GRAD: {  // slot left empty by the reference (src/gpu/kernels.cu:55)
        const size_t cols = (size_t)nd->sizes1[3];
        const size_t rows = (size_t)nd->sizes1[0] * nd->sizes1[1] * nd->sizes1[2];
        return context_colsum(ctx, nd->in1, nd->out1, rows, cols);
    }
    case DCG_OP_TANH_GRAD:  // src/gpu/sigmoid.cu:157-165
        return dcg_act_grad(nd->in1, nd->in2, nd->out1, nd->len1, DCG_ACT_TANH, 0.f, s);
    case DCG_OP_ADD:  // src/gpu/sum.cu:251-257
        return dcg_add(nd->in1, nd->in2, nd->out1, nd->len1, s);
    case DCG_OP_CONV2D:
    case DCG_OP_CONV2D_INPUT_GRAD:
    case DCG_OP_CONV2D_KERNEL_GRAD:
    case DCG_OP_CONV2D_TRANSPOSE:
    case DCG_OP_CONV2D_TRANSPOSE_INPUT_GRAD:
    case DCG_OP_CONV2D_TRANSPOSE_KERNEL_GRAD: {
        ConvCall cc;
        int st = decode_conv(nd, cc);
        if (st) return st;
        return run_conv(ctx, cc, nullptr);
    }
    default:
        return fail(DCG_ERR_INVALID, "dcg_run_node: unknown node type %d", nd->type);
    }
}

namespace dcg {
int sigmoid_xent_with_grad(const float* y, const float* logits, float* loss, float* grad, size_t n, cudaStream_t stream);
int matmul_nt_gated(const float* a, const float* b, float* out, size_t m, size_t n, size_t p, const float* gate,
                    float* gated_out, int gate_act, float gate_alpha, cudaStream_t stream);
}  // namespace dcg

namespace {

// Whether DCG_NODE_SIDE nodes can leave the main stream: the context must be free to allocate a
// second scratch buffer, and not be profiling (whose event pairs sit on the main stream).
bool side_usable(dcg_context* ctx)
{
    if (ctx->side_failed || ctx->profiling || (ctx->ws && !ctx->owns_ws)) return false;
    if (ctx->side[0]) return true;
    static const bool off = [] { const char* v = getenv("DCG_NO_SIDE_STREAM"); return v && atoi(v) != 0; }();
    bool ok = !off && cudaEventCreateWithFlags(&ctx->ev_fork, cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; i < 2 && ok; ++i)
        ok = cudaStreamCreateWithFlags(&ctx->side[i], cudaStreamNonBlocking) == cudaSuccess &&
             cudaEventCreateWithFlags(&ctx->ev_join[i], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        ctx->side_failed = true;
        ctx->side[0] = nullptr;
        return false;
    }
    return true;
}

// Runs one node on the side stream, after everything enqueued on the main stream so far.
int run_side_node(dcg_context* ctx, const dcg_node* nd)
{
    const int i = (nd->type == DCG_OP_CONV2D_KERNEL_GRAD || nd->type == DCG_OP_CONV2D_TRANSPOSE_KERNEL_GRAD) ? 0 : 1;
    DCG_CUDA(cudaEventRecord(ctx->ev_fork, ctx->stream));
    DCG_CUDA(cudaStreamWaitEvent(ctx->side[i], ctx->ev_fork, 0));
    std::swap(ctx->stream, ctx->side[i]);
    std::swap(ctx->ws, ctx->side_ws[i]);
    std::swap(ctx->ws_bytes, ctx->side_ws_bytes[i]);
    std::swap(ctx->tickets, ctx->side_tickets[i]);
    const bool owns = ctx->owns_ws;
    ctx->owns_ws = true;
    const int st = dcg_run_node(ctx, nd);
    ctx->owns_ws = owns;
    std::swap(ctx->stream, ctx->side[i]);
    std::swap(ctx->ws, ctx->side_ws[i]);
    std::swap(ctx->ws_bytes, ctx->side_ws_bytes[i]);
    std::swap(ctx->tickets, ctx->side_tickets[i]);
    ctx->side_busy[i] = true;
    return st;
}

// The main stream waits for whatever the side stream still has to do.
int join_side(dcg_context* ctx)
{
    for (int i = 0; i < 2; ++i) {
        if (!ctx->side_busy[i]) continue;
        ctx->side_busy[i] = false;
        DCG_CUDA(cudaEventRecord(ctx->ev_join[i], ctx->side[i]));
        DCG_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->ev_join[i], 0));
    }
    return DCG_OK;
}

int run_nodes_impl(dcg_context* ctx, const dcg_node* nodes, int count, int fuse);

}  // namespace

extern "C" int dcg_run_nodes(dcg_context* ctx, const dcg_node* nodes, int count, int fuse)
{
    DCG_CHECK_ARG(ctx && (nodes || count == 0) && count >= 0, "dcg_run_nodes: bad arguments");
    const int st = run_nodes_impl(ctx, nodes, count, fuse);
    const int js = join_side(ctx);   // on every path: a capture must never end with the side stream forked
    return st ? st : js;
}

namespace {
int run_nodes_impl(dcg_context* ctx, const dcg_node* nodes, int count, int fuse)
{
    int i = 0;
    while (i < count) {
        if ((nodes[i].flags & DCG_NODE_SIDE) && side_usable(ctx)) {
            int st = run_side_node(ctx, &nodes[i]);
            if (st) return st;
            ++i;
            continue;
        }
        if (!fuse) {
            int st = dcg_run_node(ctx, &nodes[i]);
            if (st) return st;
            ++i;
            continue;
        }
        if (is_conv_with_epilogue(nodes[i].type)) {
            int used = run_fused_conv(ctx, nodes, i, count);
            if (used < 0) return used;
            i += used;
            continue;
        }
        if (i + 1 < count && !(nodes[i + 1].flags & DCG_NODE_SIDE)) {
            const dcg_node& a = nodes[i];
            const dcg_node& b = nodes[i + 1];
            // dense layer + activation (tensor path only)
            const int act = act_of_node(b.type);
            if (a.type == DCG_OP_MAT_MUL_ADD && act >= 0 && b.in1 == a.out1 && b.len1 == a.len1 * a.len3 && b.out1 != a.out1) {
                const int st = run_dense_on_tensor_path(ctx, &a, act, b.type == DCG_OP_RELU_LEAKY ? b.alpha_leaky : 0.f, b.out1);
                if (st < 0) return st;
                if (st == 0) { i += 2; continue; }
            }
            // loss + its gradient on the same labels and logits
            if (a.type == DCG_OP_SIGMOID_CROSS_ENTROPY && b.type == DCG_OP_SIGMOID_CROSS_ENTROPY_GRAD && a.in1 == b.in1 &&
                a.in2 == b.in2 && a.len1 == b.len1 && a.len1 <= 65536 && a.out1 != b.out1) {
                ProfScope scope(ctx, "sigmoid_xent_with_grad", 0.0);
                const int st = dcg::sigmoid_xent_with_grad(a.in1, a.in2, a.out1, b.out1, a.len1, ctx->stream);
                if (st) return st;
                i += 2;
                continue;
            }
            // x W^T + the activation gradient that gates it (the discriminator head's input gradient)
            const int gact = grad_act_of_node(b.type);
            if (a.type == DCG_OP_MAT_TMAT_MUL && gact >= 0 && b.in2 == a.out1 && b.in1 != a.out1 && b.out1 != a.out1 &&
                b.len1 == a.len1 * a.len3) {
                ProfScope scope(ctx, "mat_tmat_mul_gated", 0.0);
                const int st = dcg::matmul_nt_gated(a.in1, a.in2, a.out1, a.len1, a.len2, a.len3, b.in1, b.out1, gact,
                                                    b.type == DCG_OP_LEAKY_RELU_GRAD ? b.cons1 : 0.f, ctx->stream);
                if (st) return st;
                i += 2;
                continue;
            }
        }
        AdamTriple first;
        if (match_adam_triple(nodes, i, count, first)) {
            // gather the run of adjacent triples that share coefficients and step count
            std::vector<dcg_adam_tensor> batch;
            std::vector<float*> counters;
            int j = i;
            AdamTriple cur = first;
            while (true) {
                batch.push_back(cur.t);
                counters.push_back(cur.t_host);
                j += 3;
                if (!match_adam_triple(nodes, j, count, cur)) break;
                if (cur.a1 != first.a1 || cur.b1 != first.b1 || cur.a2 != first.a2 ||
                    cur.b2 != first.b2 || cur.lr != first.lr || cur.beta1 != first.beta1 ||
                    cur.beta2 != first.beta2 || cur.eps != first.eps ||
                    *cur.t_host != *first.t_host)
                    break;
            }
            float lr_t = 0.f;
            for (size_t q = 0; q < counters.size(); ++q) {
                bool seen = false;  // two variables may share one counter
                for (size_t r = 0; r < q; ++r) seen |= counters[r] == counters[q];
                if (!seen) lr_t = dcg_adam_lr_t(counters[q], first.lr, first.beta1, first.beta2);
            }
            int st;
            {
                ProfScope scope(ctx, "adam_multi", 0.0);
                st = adam_multi_launch(batch.data(), (int)batch.size(), lr_t, first.a1, first.b1,
                                       first.a2, first.b2, first.eps, 1.f, ctx->stream);
            }
            if (st) return st;
            i = j;
            continue;
        }
        int st = dcg_run_node(ctx, &nodes[i]);
        if (st) return st;
        ++i;
    }
    return DCG_OK;
}
}  // namespace

// ---- profiling mode ---------------------------------------------------------------------------
extern "C" int dcg_context_profile_begin(dcg_context* ctx)
{
    DCG_CHECK_ARG(ctx, "dcg_context_profile_begin: null context");
    for (ProfRec& r : ctx->recs) { cudaEventDestroy(r.e0); cudaEventDestroy(r.e1); }
    ctx->recs.clear();
    ctx->profiling = true;
    return DCG_OK;
}

extern "C" int dcg_context_profile_end(dcg_context* ctx, dcg_profile_row* rows, int max_rows, int* n_rows)
{
    DCG_CHECK_ARG(ctx && n_rows && (rows || max_rows == 0), "dcg_context_profile_end: bad arguments");
    ctx->profiling = false;
    DCG_CUDA(cudaStreamSynchronize(ctx->stream));
    std::vector<dcg_profile_row> agg;
    for (ProfRec& r : ctx->recs) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, r.e0, r.e1);
        ms /= (float)(r.repeat > 0 ? r.repeat : 1);
        cudaEventDestroy(r.e0);
        cudaEventDestroy(r.e1);
        size_t k = 0;
        for (; k < agg.size(); ++k)
            if (r.name == agg[k].name) break;
        if (k == agg.size()) {
            dcg_profile_row row;
            std::memset(&row, 0, sizeof(row));
            snprintf(row.name, sizeof(row.name), "%s", r.name.c_str());
            agg.push_back(row);
        }
        agg[k].calls += 1;
        agg[k].ms += ms;
        agg[k].flops += r.flops;
    }
    ctx->recs.clear();
    *n_rows = (int)agg.size();
    for (int i = 0; i < (int)agg.size() && i < max_rows; ++i) rows[i] = agg[i];
    return DCG_OK;
}
