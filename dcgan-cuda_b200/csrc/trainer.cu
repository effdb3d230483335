// DCGAN training step as node lists: the host-side counterpart of dcgan/main.cu.
//
// The reference builds the generator / discriminator with its ops graph, lets autodiff add the
// gradient ops and AdamOptimizer::minimize the update ops (dcgan/main.cu:271-332), then every
// iteration runs graph.run({d_opti, d_loss}) once and graph.run({g_opti, g_loss}) twice
// (dcgan/main.cu:378-391).  Each run lowers to a flat list of rt::Node instructions.  This file
// writes those lists down directly for the fixed DCGAN topology - same instructions, same
// operands, same recomputation of the forward passes in every run - and executes them through the
// node backend (dcg_run_nodes) with fusion on.  All device memory comes from one arena allocated
// at creation; parameters and gradients of each network are contiguous so a data-parallel caller
// can average a network's gradients with a single all-reduce between *_backward and *_apply.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "adam.cuh"
#include "backend.cuh"
#include "common.cuh"

namespace dcg {
// data-parallel plumbing (dp.cu)
void* dp_mem_alloc(size_t bytes);
void dp_mem_free(void* p);
void dp_register(dcg_dp* dp, void* buf, size_t bytes);
int dp_world(const dcg_dp* dp);
int dp_rank(const dcg_dp* dp);
int dp_map_peers(dcg_dp* dp, void* local_base, void** bases);
void dp_unmap_peers(dcg_dp* dp, void** bases);
// dp_adam.cu: gradient sum over the ranks + Adam + parameter broadcast as one kernel over peer memory
int dp_reduce_adam_launch(int rank, int world, float* const* grads, float* const* params, float* m, float* v,
                          unsigned* const* ready, unsigned* const* done, unsigned* epoch, unsigned* ticket, size_t n_floats,
                          float lr_t, float a1, float b1, float a2, float b2, float eps, float scale, const float* lr_t_dev,
                          cudaStream_t stream);
int dp_allreduce_group(dcg_dp* dp, float* const* bufs, const size_t* counts, int n, cudaStream_t stream);
}  // namespace dcg

namespace {

constexpr int kZ = 100;       // dcgan/main.cu:34
constexpr int kImg = 64;
constexpr int kLayers = 4;
const int kGChan[kLayers + 1] = {512, 256, 128, 64, 3};   // generator feature maps 4x4 -> 64x64
const int kDChan[kLayers + 1] = {3, 64, 128, 256, 512};   // discriminator feature maps 64x64 -> 4x4

struct Tensor {
    float* p = nullptr;
    size_t n = 0;
};

// xorshift generator of the reference (src/utils/xorshift.cu:11-34) with Box-Muller on top: a
// seeded stand-in for the reference's clock-seeded std::normal_distribution initialiser
// (src/api/normal-initializer.cu:6-9).
struct Rng {
    uint64_t s[4];
    explicit Rng(uint64_t x) { s[0] = 1000 * x; s[1] = 2000 * x; s[2] = 3000 * x; s[3] = 4000 * x; }
    uint64_t next_u64()
    {
        uint64_t t = s[0] ^ (s[0] << 11);
        s[0] = s[1]; s[1] = s[2]; s[2] = s[3];
        s[3] = s[3] ^ (s[3] >> 19) ^ t ^ (t >> 8);
        return s[3];
    }
    float next_f32() { return (float)next_u64() / (float)0xFFFFFFFFFFFFFFFFull; }
    float normal(float sd)
    {
        float u1 = next_f32(), u2 = next_f32();
        if (u1 < 1e-12f) u1 = 1e-12f;
        return sd * std::sqrt(-2.f * std::log(u1)) * std::cos(6.28318530718f * u2);
    }
};

}  // namespace

struct dcg_trainer {
    dcg_trainer_config cfg;
    cudaStream_t stream = nullptr;
    dcg_context* ctx = nullptr;
    uint8_t* arena = nullptr;
    size_t arena_bytes = 0, arena_used = 0;
    bool arena_from_nccl = false;   // allocated by ncclMemAlloc (NCCL can then reduce it in the switch)
    // Data parallelism: the communicator (not owned), and a stream for the discriminator's gradient
    // sum, which runs while the main stream computes the generator's forward pass of the next update.
    dcg_dp* dp = nullptr;
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t ev_grads = nullptr, ev_summed = nullptr;
    // Fused update (dp_adam.cu): every rank's arena mapped into this process, and per network the
    // flag words the peers write (in the arena, so that they are mapped along with it).
    bool fused_update = false;
    void* peer_arena[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    Tensor sync_words[2];   // [0] discriminator, [1] generator: ready[8] | done[8] | epoch | ticket

    // parameters / gradients / Adam moments: index 0..9 = (k0,b0,...,k3,b3,dense w,dense b)
    Tensor g_param[10], g_grad[10], g_m[10], g_v[10];
    Tensor d_param[10], d_grad[10], d_grad2[10], d_m[10], d_v[10];
    Tensor g_params_all, g_grads_all, d_params_all, d_grads_all;
    float g_t = 0.f, d_t = 0.f;   // Adam step counters (host, as rt::Node::out2 of adam_update)
    // Tensor path: the discriminator's fake and real passes of the D run are one pass over
    // [g_out | x] with batch 2B (half the launches, twice the work per launch); d_grad then holds the
    // sum of both gradient paths and d_grad2 stays zero.  The fp32 path keeps the reference's two
    // passes and its summation order.
    bool batched_d = false;

    // inputs, constants, losses
    Tensor x, z, ones, zeros, d_loss, d1_loss, d2_loss, g_loss;
    // generator activations
    Tensor g0z, g0a, gc[kLayers], gz[kLayers], ga[kLayers], g_out;
    // discriminator activations for the fake (0) and real (1) pass
    Tensor dc[2][kLayers], dz[2][kLayers], da[2][kLayers], logits[2];
    // backward scratch
    Tensor dlogits[2], dda[kLayers + 1], ddz[kLayers], dg_out, dgz[kLayers], dga[kLayers], dg0a, dg0z;

    std::vector<dcg_node> d_nodes, g_nodes, gen_nodes, dfb_nodes;
    uint64_t last_step_launches = 0;

    // A node list is launched eagerly twice (scratch grows to its final size, one-time attributes
    // get set), then captured from the stream into a CUDA graph and replayed: the list, its operand
    // addresses and its launch shapes never change, and a replay costs the host one call and the
    // GPU less inter-kernel latency than ~100 dependent launches.
    struct ListGraph {
        cudaGraphExec_t exec = nullptr;
        int eager_runs = 0;
        uint64_t launches = 0;     // kernels in the graph (the library's launch counter advances by this per replay)
        uint64_t generation = 0;   // the context's generation the graph was captured under
        bool failed = false;
    };
    ListGraph d_graph, g_graph, gen_graph, dfb_graph, g_part_graph[2];
    // Single-GPU iteration as ONE graph: D list, Adam, G list, Adam, G list, Adam.  The three Adam
    // step sizes change every iteration, so the captured launches read them from `lr_dev`, which the
    // host rewrites (one 12-byte copy) before each replay.
    ListGraph step_graph;
    Tensor lr_dev;
    size_t g_forward_nodes = 0;   // the G run's leading nodes that only compute the generator's forward pass
    int step_warm_runs = 0;       // eager whole iterations so far
    bool use_graphs = true;

    // Checkpoint writer: a pinned snapshot buffer the device copies into (stream-ordered), and the
    // host thread that waits for that copy and writes the file while training goes on.
    float* snap = nullptr;
    size_t snap_floats = 0;
    cudaEvent_t ev_snap = nullptr;
    std::thread writer;
    int writer_status = DCG_OK;
    std::string writer_error;
};

namespace {

using dcg::fail;

// Bump allocator over the arena, 256-byte aligned.  A dry pass only measures.
struct Alloc {
    dcg_trainer* t;
    bool dry;
    size_t off = 0;
    Tensor get(size_t n)
    {
        Tensor r;
        r.n = n;
        off = dcg::align_up(off, 256);
        if (!dry) r.p = reinterpret_cast<float*>(t->arena + off);
        off += n * sizeof(float);
        return r;
    }
};

// Lays every tensor out in the arena.  Called twice: dry (sizes only) and for real.
void layout(dcg_trainer* t, Alloc& a)
{
    const int B = t->cfg.batch;
    auto pack = [&](Tensor* dst, const size_t* sizes, Tensor& all) {
        const size_t start = dcg::align_up(a.off, 256);
        for (int i = 0; i < 10; ++i) dst[i] = a.get(sizes[i]);
        all.n = (a.off - start) / sizeof(float);
        all.p = a.dry ? nullptr : reinterpret_cast<float*>(t->arena + start);
    };
    size_t gs[10], ds[10];
    for (int i = 0; i < kLayers; ++i) {
        gs[2 * i] = (size_t)25 * kGChan[i + 1] * kGChan[i];  // [5,5,Cout,Cin]
        gs[2 * i + 1] = kGChan[i + 1];
        ds[2 * i] = (size_t)25 * kDChan[i] * kDChan[i + 1];  // [5,5,Cin,Cout]
        ds[2 * i + 1] = kDChan[i + 1];
    }
    gs[8] = (size_t)kZ * 8192; gs[9] = 8192;
    ds[8] = 8192; ds[9] = 1;
    Tensor dummy;
    pack(t->g_param, gs, t->g_params_all);
    pack(t->g_grad, gs, t->g_grads_all);
    pack(t->g_m, gs, dummy);
    pack(t->g_v, gs, dummy);
    pack(t->d_param, ds, t->d_params_all);
    pack(t->d_grad, ds, t->d_grads_all);
    pack(t->d_grad2, ds, dummy);
    pack(t->d_m, ds, dummy);
    pack(t->d_v, ds, dummy);

    // [g_out | x] are one buffer so that the batched discriminator pass reads both as one batch
    const size_t img_n = (size_t)B * kImg * kImg * 3;
    Tensor img2 = a.get(2 * img_n);
    t->g_out = img2; t->g_out.n = img_n;
    t->x = img2; t->x.n = img_n;
    if (!a.dry) t->x.p = img2.p + img_n;
    t->z = a.get((size_t)B * kZ);
    t->ones = a.get(B); t->zeros = a.get(B);
    t->lr_dev = a.get(4);
    t->sync_words[0] = a.get(32);
    t->sync_words[1] = a.get(32);
    t->d_loss = a.get(1); t->d1_loss = a.get(1); t->d2_loss = a.get(1); t->g_loss = a.get(1);
    t->g0z = a.get((size_t)B * 8192); t->g0a = a.get((size_t)B * 8192);
    for (int i = 0; i < kLayers; ++i) {
        const int hw = 8 << i;
        const size_t n = (size_t)B * hw * hw * kGChan[i + 1];
        t->gc[i] = a.get(n); t->gz[i] = a.get(n);
        if (i < kLayers - 1) t->ga[i] = a.get(n);
        t->dgz[i] = a.get(n); t->dga[i] = a.get(n);
    }
    t->dg_out = a.get((size_t)B * kImg * kImg * 3);
    t->dg0a = a.get((size_t)B * 8192); t->dg0z = a.get((size_t)B * 8192);
    // pass 0 (fake) and pass 1 (real) of every discriminator tensor are adjacent: [fake | real]
    auto pair = [&](Tensor& t0, Tensor& t1, size_t n) {
        Tensor both = a.get(2 * n);
        t0 = both; t0.n = n;
        t1 = both; t1.n = n;
        if (!a.dry) t1.p = both.p + n;
    };
    for (int i = 0; i < kLayers; ++i) {
        const int hw = 32 >> i;
        const size_t n = (size_t)B * hw * hw * kDChan[i + 1];
        pair(t->dc[0][i], t->dc[1][i], n);
        pair(t->dz[0][i], t->dz[1][i], n);
        pair(t->da[0][i], t->da[1][i], n);
    }
    pair(t->logits[0], t->logits[1], B);
    pair(t->dlogits[0], t->dlogits[1], B);
    for (int i = 0; i < kLayers; ++i) {   // backward scratch, sized for the batched pass
        const int hw = 32 >> i;
        t->ddz[i] = a.get((size_t)2 * B * hw * hw * kDChan[i + 1]);
        t->dda[i + 1] = a.get((size_t)2 * B * hw * hw * kDChan[i + 1]);
    }
}

// ---- node construction: field packing as in src/runtime/node.cu ----------------------------------
dcg_node node(int type)
{
    dcg_node n;
    std::memset(&n, 0, sizeof(n));
    n.type = type;
    return n;
}

void set4(int* dst, int a, int b, int c, int d) { dst[0] = a; dst[1] = b; dst[2] = c; dst[3] = d; }

dcg_node n_mat_mul_add(const float* x, const float* w, const float* b, float* out, size_t m, size_t n, size_t p)
{
    dcg_node nd = node(DCG_OP_MAT_MUL_ADD);
    nd.in1 = x; nd.in2 = w; nd.in3 = b; nd.out1 = out; nd.len1 = m; nd.len2 = n; nd.len3 = p;
    return nd;
}

dcg_node n_unary(int type, const float* in, float* out, size_t len, float alpha = 0.f)
{
    dcg_node nd = node(type);
    nd.in1 = in; nd.out1 = out; nd.len1 = len; nd.alpha_leaky = alpha;
    return nd;
}

dcg_node n_binary(int type, const float* a, const float* b, float* out, size_t len, float cons1 = 0.f)
{
    dcg_node nd = node(type);
    nd.in1 = a; nd.in2 = b; nd.out1 = out; nd.len1 = len; nd.cons1 = cons1;
    return nd;
}

dcg_node n_rows_cols(int type, const float* a, const float* b, float* out, size_t rows, size_t cols)
{
    dcg_node nd = node(type);
    nd.in1 = a; nd.in2 = b; nd.out1 = out; nd.len1 = rows; nd.len2 = cols;
    return nd;
}

dcg_node n_mat3(int type, const float* a, const float* b, float* out, size_t l1, size_t l2, size_t l3)
{
    dcg_node nd = node(type);
    nd.in1 = a; nd.in2 = b; nd.out1 = out; nd.len1 = l1; nd.len2 = l2; nd.len3 = l3;
    return nd;
}

// conv2d [B,h,h,c] -> [B,h/2,h/2,o], 5x5, stride 2, SAME (total pad 3): src/ops/conv2d.cu:44-77
dcg_node n_conv2d(const float* x, const float* k, float* y, int B, int h, int c, int o)
{
    dcg_node nd = node(DCG_OP_CONV2D);
    nd.in1 = x; nd.in2 = k; nd.out1 = y;
    nd.intconst[0] = nd.intconst[1] = 2;
    nd.int_cons1 = nd.int_cons2 = 3;
    set4(nd.sizes1, B, h, h, c);
    set4(nd.sizes2, 5, 5, c, o);
    return nd;
}

dcg_node n_conv2d_input_grad(const float* dy, const float* k, float* dx, int B, int h, int c, int o)
{
    dcg_node nd = node(DCG_OP_CONV2D_INPUT_GRAD);
    nd.in1 = dy; nd.in2 = k; nd.out1 = dx;
    nd.intconst[0] = nd.intconst[1] = 2;
    nd.intconst2[0] = nd.intconst2[1] = h;
    set4(nd.sizes1, B, h / 2, h / 2, o);
    set4(nd.sizes2, 5, 5, c, o);
    return nd;
}

dcg_node n_conv2d_kernel_grad(const float* dy, const float* x, float* dk, int B, int h, int c, int o)
{
    dcg_node nd = node(DCG_OP_CONV2D_KERNEL_GRAD);
    nd.in1 = dy; nd.in2 = x; nd.out1 = dk;
    nd.intconst[0] = nd.intconst[1] = 2;
    nd.intconst2[0] = nd.intconst2[1] = 3;
    set4(nd.sizes1, B, h / 2, h / 2, o);
    set4(nd.sizes2, B, h, h, c);
    return nd;
}

// conv2d_transpose [B,h,h,cin] -> [B,2h,2h,cout], kernel [5,5,cout,cin]: src/ops/conv2d-transpose.cu:31-52
dcg_node n_conv2d_transpose(const float* x, const float* k, float* y, int B, int h, int cin, int cout)
{
    dcg_node nd = node(DCG_OP_CONV2D_TRANSPOSE);
    nd.in1 = x; nd.in2 = k; nd.out1 = y;
    nd.intconst[0] = nd.intconst[1] = 2;
    set4(nd.sizes1, B, 2 * h, 2 * h, cout);
    set4(nd.sizes2, B, h, h, cin);
    set4(nd.sizes3, 5, 5, cout, cin);
    return nd;
}

dcg_node n_conv2d_transpose_input_grad(const float* dy, const float* k, float* dx, int B, int h, int cin, int cout)
{
    dcg_node nd = node(DCG_OP_CONV2D_TRANSPOSE_INPUT_GRAD);
    nd.in1 = dy; nd.in2 = k; nd.out1 = dx;
    nd.intconst[0] = nd.intconst[1] = 2;
    nd.intconst2[0] = nd.intconst2[1] = h;
    set4(nd.sizes1, B, 2 * h, 2 * h, cout);
    set4(nd.sizes2, 5, 5, cout, cin);
    return nd;
}

dcg_node n_conv2d_transpose_kernel_grad(const float* dy, const float* x, float* dk, int B, int h, int cin, int cout)
{
    dcg_node nd = node(DCG_OP_CONV2D_TRANSPOSE_KERNEL_GRAD);
    nd.in1 = dy; nd.in2 = x; nd.out1 = dk;
    nd.intconst[0] = nd.intconst[1] = 2;
    set4(nd.sizes1, B, 2 * h, 2 * h, cout);
    set4(nd.sizes2, B, h, h, cin);
    set4(nd.sizes3, 5, 5, cout, cin);
    return nd;
}

dcg_node dead(dcg_node n)
{
    n.flags |= DCG_NODE_OUT_DEAD;
    return n;
}

// Weight and bias gradients are read by nobody before Adam: they may leave the main stream.
dcg_node side(dcg_node n)
{
    n.flags |= DCG_NODE_SIDE;
    return n;
}

// Generator forward: dcgan/main.cu:89-120 and :288 (tanh on the last layer's pre-activation).
void build_generator(dcg_trainer* t, std::vector<dcg_node>& L)
{
    const int B = t->cfg.batch;
    const int act = t->cfg.g_leaky ? DCG_OP_RELU_LEAKY : DCG_OP_RELU;
    L.push_back(n_mat_mul_add(t->z.p, t->g_param[8].p, t->g_param[9].p, t->g0z.p, B, kZ, 8192));
    L.push_back(n_unary(act, t->g0z.p, t->g0a.p, (size_t)B * 8192, 0.2f));
    const float* in = t->g0a.p;   // reshape to [B,4,4,512] is an alias (src/ops/reshape.cu:20-44)
    for (int i = 0; i < kLayers; ++i) {
        const int h = 4 << i, hw = 2 * h;
        const size_t rows = (size_t)B * hw * hw;
        L.push_back(dead(n_conv2d_transpose(in, t->g_param[2 * i].p, t->gc[i].p, B, h, kGChan[i], kGChan[i + 1])));
        L.push_back(n_rows_cols(DCG_OP_MAT_RVECT_ADD, t->gc[i].p, t->g_param[2 * i + 1].p, t->gz[i].p, rows, kGChan[i + 1]));
        if (i < kLayers - 1) {
            L.push_back(n_unary(act, t->gz[i].p, t->ga[i].p, rows * kGChan[i + 1], 0.2f));
            in = t->ga[i].p;
        } else {
            L.push_back(n_unary(DCG_OP_TANH, t->gz[i].p, t->g_out.p, rows * 3));
        }
    }
}

// Discriminator forward on `img` into pass `ps` buffers: dcgan/main.cu:123-249.
void build_discriminator(dcg_trainer* t, std::vector<dcg_node>& L, const float* img, int ps, int B)
{
    const float* in = img;
    for (int i = 0; i < kLayers; ++i) {
        const int h = 64 >> i, ho = h / 2;
        const size_t rows = (size_t)B * ho * ho;
        L.push_back(dead(n_conv2d(in, t->d_param[2 * i].p, t->dc[ps][i].p, B, h, kDChan[i], kDChan[i + 1])));
        L.push_back(n_rows_cols(DCG_OP_MAT_RVECT_ADD, t->dc[ps][i].p, t->d_param[2 * i + 1].p, t->dz[ps][i].p, rows, kDChan[i + 1]));
        L.push_back(n_unary(DCG_OP_RELU_LEAKY, t->dz[ps][i].p, t->da[ps][i].p, rows * kDChan[i + 1], 0.2f));
        in = t->da[ps][i].p;
    }
    L.push_back(n_mat_mul_add(in, t->d_param[8].p, t->d_param[9].p, t->logits[ps].p, B, 8192, 1));
}

// Backward through the discriminator for pass `ps`, starting from dlogits[ps].
// grads != nullptr: weight gradients into grads[0..9]; to_image: also the gradient w.r.t. the input.
void build_discriminator_backward(dcg_trainer* t, std::vector<dcg_node>& L, const float* img, int ps,
                                  Tensor* grads, bool to_image, int B)
{
    // The two-pass (fp32) D run sends both passes through the same backward scratch, so there a
    // gradient node must finish before the next pass overwrites what it reads: main stream only.
    auto grad_node = [&](dcg_node n) { return t->batched_d ? side(n) : n; };
    if (grads) {
        L.push_back(grad_node(n_mat3(DCG_OP_TMAT_MAT_MUL, t->da[ps][3].p, t->dlogits[ps].p, grads[8].p, 8192, B, 1)));
        L.push_back(grad_node(n_rows_cols(DCG_OP_MAT_SUM_COLS, t->dlogits[ps].p, nullptr, grads[9].p, B, 1)));
    }
    L.push_back(n_mat3(DCG_OP_MAT_TMAT_MUL, t->dlogits[ps].p, t->d_param[8].p, t->dda[4].p, B, 1, 8192));
    for (int i = kLayers - 1; i >= 0; --i) {
        const int h = 64 >> i, ho = h / 2;
        const size_t rows = (size_t)B * ho * ho;
        const float* in = i == 0 ? img : t->da[ps][i - 1].p;
        // dda[i+1] is produced by the layer above; its leaky gradient is this layer's dz
        L.push_back(n_binary(DCG_OP_LEAKY_RELU_GRAD, t->dz[ps][i].p, t->dda[i + 1].p, t->ddz[i].p, rows * kDChan[i + 1], 0.2f));
        if (grads) {
            L.push_back(grad_node(n_rows_cols(DCG_OP_MAT_SUM_COLS, t->ddz[i].p, nullptr, grads[2 * i + 1].p, rows, kDChan[i + 1])));
            L.push_back(grad_node(n_conv2d_kernel_grad(t->ddz[i].p, in, grads[2 * i].p, B, h, kDChan[i], kDChan[i + 1])));
        }
        // the input gradient is only ever read by the activation gradient that follows it
        if (i > 0)
            L.push_back(dead(n_conv2d_input_grad(t->ddz[i].p, t->d_param[2 * i].p, t->dda[i].p, B, h, kDChan[i], kDChan[i + 1])));
        else if (to_image)
            L.push_back(dead(n_conv2d_input_grad(t->ddz[i].p, t->d_param[2 * i].p, t->dg_out.p, B, h, kDChan[i], kDChan[i + 1])));
    }
}

void build_lists(dcg_trainer* t)
{
    const int B = t->cfg.batch;
    // ---- generate: G forward only ----
    build_generator(t, t->gen_nodes);

    // ---- discriminator forward + backward on the real images alone (labels all ones): every layer's
    // kernel, bias and input gradient, the image gradient included.  Pass-1 buffers, gradients into
    // the second gradient set, so the training lists are not disturbed.
    std::vector<dcg_node>& F = t->dfb_nodes;
    build_discriminator(t, F, t->x.p, 1, B);
    F.push_back(n_binary(DCG_OP_SIGMOID_CROSS_ENTROPY, t->ones.p, t->logits[1].p, t->d2_loss.p, B));
    F.push_back(n_binary(DCG_OP_SIGMOID_CROSS_ENTROPY_GRAD, t->ones.p, t->logits[1].p, t->dlogits[1].p, B));
    build_discriminator_backward(t, F, t->x.p, 1, t->d_grad2, true, B);

    // ---- D run: graph.run({d_opti, d_loss}) ----
    std::vector<dcg_node>& D = t->d_nodes;
    build_generator(t, D);
    if (t->batched_d) {
        build_discriminator(t, D, t->g_out.p, 0, 2 * B);   // [g_out | x] through pass-0 buffers of 2B
    } else {
        build_discriminator(t, D, t->g_out.p, 0, B);
        build_discriminator(t, D, t->x.p, 1, B);
    }
    // each loss next to its gradient: the pair is one launch when the list runs fused
    D.push_back(n_binary(DCG_OP_SIGMOID_CROSS_ENTROPY, t->zeros.p, t->logits[0].p, t->d1_loss.p, B));
    D.push_back(n_binary(DCG_OP_SIGMOID_CROSS_ENTROPY_GRAD, t->zeros.p, t->logits[0].p, t->dlogits[0].p, B));
    D.push_back(n_binary(DCG_OP_SIGMOID_CROSS_ENTROPY, t->ones.p, t->logits[1].p, t->d2_loss.p, B));
    D.push_back(n_binary(DCG_OP_SIGMOID_CROSS_ENTROPY_GRAD, t->ones.p, t->logits[1].p, t->dlogits[1].p, B));
    D.push_back(n_binary(DCG_OP_ADD, t->d1_loss.p, t->d2_loss.p, t->d_loss.p, 1));
    if (t->batched_d) {
        // dlogits = [fake | real], each half already divided by its own B: the 2B-row backward pass
        // sums both gradient paths (the Add of src/ops/graph.cu:302-309) inside its reductions
        build_discriminator_backward(t, D, t->g_out.p, 0, t->d_grad, false, 2 * B);
    } else {
        build_discriminator_backward(t, D, t->g_out.p, 0, t->d_grad, false, B);
        build_discriminator_backward(t, D, t->x.p, 1, t->d_grad2, false, B);
    }

    // ---- G run: graph.run({g_opti, g_loss}) ----
    std::vector<dcg_node>& G = t->g_nodes;
    build_generator(t, G);
    t->g_forward_nodes = G.size();
    build_discriminator(t, G, t->g_out.p, 0, B);
    G.push_back(n_binary(DCG_OP_SIGMOID_CROSS_ENTROPY, t->ones.p, t->logits[0].p, t->g_loss.p, B));
    G.push_back(n_binary(DCG_OP_SIGMOID_CROSS_ENTROPY_GRAD, t->ones.p, t->logits[0].p, t->dlogits[0].p, B));
    build_discriminator_backward(t, G, t->g_out.p, 0, nullptr, true, B);
    // through tanh and the generator (src/ops/vect-tanh.cu:41: the gradient takes the tanh OUTPUT)
    G.push_back(n_binary(DCG_OP_TANH_GRAD, t->g_out.p, t->dg_out.p, t->dgz[3].p, (size_t)B * 64 * 64 * 3));
    const int gact_grad = t->cfg.g_leaky ? DCG_OP_LEAKY_RELU_GRAD : DCG_OP_RELU_GRAD;
    for (int i = kLayers - 1; i >= 0; --i) {
        const int h = 4 << i, hw = 2 * h;
        const size_t rows = (size_t)B * hw * hw;
        const float* in = i == 0 ? t->g0a.p : t->ga[i - 1].p;
        G.push_back(side(n_rows_cols(DCG_OP_MAT_SUM_COLS, t->dgz[i].p, nullptr, t->g_grad[2 * i + 1].p, rows, kGChan[i + 1])));
        G.push_back(side(n_conv2d_transpose_kernel_grad(t->dgz[i].p, in, t->g_grad[2 * i].p, B, h, kGChan[i], kGChan[i + 1])));
        float* dprev_a = i == 0 ? t->dg0a.p : t->dga[i - 1].p;
        G.push_back(dead(n_conv2d_transpose_input_grad(t->dgz[i].p, t->g_param[2 * i].p, dprev_a, B, h, kGChan[i], kGChan[i + 1])));
        const float* zprev = i == 0 ? t->g0z.p : t->gz[i - 1].p;
        float* dprev_z = i == 0 ? t->dg0z.p : t->dgz[i - 1].p;
        const size_t nprev = i == 0 ? (size_t)B * 8192 : (size_t)B * h * h * kGChan[i];
        G.push_back(n_binary(gact_grad, zprev, dprev_a, dprev_z, nprev, 0.2f));
    }
    G.push_back(side(n_mat3(DCG_OP_TMAT_MAT_MUL, t->z.p, t->dg0z.p, t->g_grad[8].p, kZ, B, 8192)));
    G.push_back(side(n_rows_cols(DCG_OP_MAT_SUM_COLS, t->dg0z.p, nullptr, t->g_grad[9].p, B, 8192)));
}

int run_list(dcg_trainer* t, const std::vector<dcg_node>& all, dcg_trainer::ListGraph& g, size_t begin = 0,
             size_t end = (size_t)-1)
{
    if (end > all.size()) end = all.size();
    const std::vector<dcg_node> L(all.begin() + begin, all.begin() + end);   // ~100 small records
    const bool eager = !t->use_graphs || g.failed || dcg::context_is_profiling(t->ctx);
    if (eager || g.eager_runs < 2) {
        if (!eager) ++g.eager_runs;
        return dcg_run_nodes(t->ctx, L.data(), (int)L.size(), t->cfg.fuse);
    }
    if (g.exec && g.generation != dcg::context_generation(t->ctx)) {   // scratch moved or precision switched: stale
        cudaGraphExecDestroy(g.exec);
        g.exec = nullptr;
    }
    if (!g.exec) {
        const uint64_t before = dcg_launches_total();
        cudaGraph_t graph = nullptr;
        if (cudaStreamBeginCapture(t->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
            if (getenv("DCG_TRAINER_VERBOSE"))
                fprintf(stderr, "dcg_trainer: cudaStreamBeginCapture failed: %s\n", cudaGetErrorString(cudaGetLastError()));
            cudaGetLastError();
            g.failed = true;
            return dcg_run_nodes(t->ctx, L.data(), (int)L.size(), t->cfg.fuse);
        }
        const int st = dcg_run_nodes(t->ctx, L.data(), (int)L.size(), t->cfg.fuse);
        const cudaError_t ce = cudaStreamEndCapture(t->stream, &graph);
        cudaError_t ie = cudaSuccess;
        if (st != DCG_OK || ce != cudaSuccess || !graph ||
            (ie = cudaGraphInstantiate(&g.exec, graph, 0)) != cudaSuccess) {
            if (getenv("DCG_TRAINER_VERBOSE"))
                fprintf(stderr, "dcg_trainer: graph capture failed (list status %d, end capture: %s, instantiate: %s); "
                                "staying eager\n", st, cudaGetErrorString(ce), cudaGetErrorString(ie));
            cudaGetLastError();
            if (graph) cudaGraphDestroy(graph);
            g.exec = nullptr;
            g.failed = true;   // stay eager from here on
            return dcg_run_nodes(t->ctx, L.data(), (int)L.size(), t->cfg.fuse);
        }
        cudaGraphDestroy(graph);
        g.launches = dcg_launches_total() - before;
        g.generation = dcg::context_generation(t->ctx);
        dcg::count_launch(-(int)g.launches);   // the capture launched nothing; the replay below counts
    }
    if (cudaGraphLaunch(g.exec, t->stream) != cudaSuccess)
        return fail(DCG_ERR_CUDA, "cudaGraphLaunch: %s", cudaGetErrorString(cudaGetLastError()));
    dcg::count_launch((int)g.launches);
    return DCG_OK;
}

// step != nullptr: advances the host step counter and passes the step size by value.
// lr_dev != nullptr: the launch reads the step size from that device scalar (whole-step graph).
int apply_adam(dcg_trainer* t, Tensor* param, Tensor* grad, Tensor* grad2, Tensor* m, Tensor* v, float* step,
               float grad_scale, const float* lr_dev = nullptr)
{
    dcg_adam_tensor ts[10];
    for (int i = 0; i < 10; ++i) {
        ts[i].p = param[i].p; ts[i].g = grad[i].p; ts[i].g2 = grad2 ? grad2[i].p : nullptr;
        ts[i].m = m[i].p; ts[i].v = v[i].p; ts[i].n = param[i].n;
    }
    const float lr_t = lr_dev ? 0.f : dcg_adam_lr_t(step, t->cfg.lr, t->cfg.beta1, t->cfg.beta2);
    dcg::ProfScope scope(t->ctx, "adam_multi", 0.0);
    return dcg::adam_multi_launch(ts, 10, lr_t, t->cfg.beta1, 1.f - t->cfg.beta1, t->cfg.beta2, 1.f - t->cfg.beta2,
                                  t->cfg.eps, grad_scale, t->stream, lr_dev);
}

int sum_over_ranks(dcg_trainer* t, Tensor& grads, cudaStream_t stream)
{
    float* bufs[1] = {grads.p};
    const size_t counts[1] = {grads.n};
    return dcg::dp_allreduce_group(t->dp, bufs, counts, 1, stream);
}

// One network's data-parallel update as a single kernel: sum of the ranks' gradients + Adam on this rank's
// slice + broadcast of the slice's new parameters (dp_adam.cu).  net: 0 discriminator, 1 generator.
int fused_update(dcg_trainer* t, int net, float* step, float scale, const float* lr_dev, cudaStream_t stream)
{
    const int W = t->cfg.world, R = dcg::dp_rank(t->dp);
    Tensor& params = net == 0 ? t->d_params_all : t->g_params_all;
    Tensor& grads = net == 0 ? t->d_grads_all : t->g_grads_all;
    Tensor* m = net == 0 ? t->d_m : t->g_m;
    Tensor* v = net == 0 ? t->d_v : t->g_v;
    float *g_ptr[8], *p_ptr[8];
    unsigned *ready[8], *done[8];
    for (int r = 0; r < W; ++r) {   // same layout on every rank: a peer's tensor sits at the same offset in its arena
        uint8_t* base = static_cast<uint8_t*>(t->peer_arena[r]);
        g_ptr[r] = reinterpret_cast<float*>(base + (reinterpret_cast<uint8_t*>(grads.p) - t->arena));
        p_ptr[r] = reinterpret_cast<float*>(base + (reinterpret_cast<uint8_t*>(params.p) - t->arena));
        unsigned* words = reinterpret_cast<unsigned*>(base + (reinterpret_cast<uint8_t*>(t->sync_words[net].p) - t->arena));
        ready[r] = words;
        done[r] = words + 8;
    }
    unsigned* mine = reinterpret_cast<unsigned*>(t->sync_words[net].p);
    const float lr_t = lr_dev ? 0.f : dcg_adam_lr_t(step, t->cfg.lr, t->cfg.beta1, t->cfg.beta2);
    dcg::ProfScope scope(t->ctx, "dp_reduce_adam", 0.0);
    // m / v of a network are contiguous like its parameters: the arrays start at m[0] / v[0]
    return dcg::dp_reduce_adam_launch(R, W, g_ptr, p_ptr, m[0].p, v[0].p, ready, done, mine + 16, mine + 17, params.n, lr_t,
                                      t->cfg.beta1, 1.f - t->cfg.beta1, t->cfg.beta2, 1.f - t->cfg.beta2, t->cfg.eps, scale,
                                      lr_dev, stream);
}

// The data-parallel iteration (world > 1, communicator attached): the same three runs, each followed
// by ONE sum of that network's gradient arena over the ranks and the replicated Adam step, which
// divides by the world size.  The discriminator's sum runs on the communication stream under the
// generator's forward pass of the first G update (which reads neither the discriminator's
// gradients nor its parameters).  Everything is stream-ordered, so the whole iteration - collectives
// included - can be captured into one CUDA graph.
int enqueue_step_dp(dcg_trainer* t, const float* lr_dev)
{
    int st;
    const float scale = 1.f / (float)t->cfg.world;
    const int fwd = (int)t->g_forward_nodes, all = (int)t->g_nodes.size();
    if ((st = dcg_run_nodes(t->ctx, t->d_nodes.data(), (int)t->d_nodes.size(), t->cfg.fuse))) return st;
    if (!t->batched_d)   // the two gradient paths are summed first (the Add of src/ops/graph.cu:302-309)
        for (int i = 0; i < 10; ++i)
            if ((st = dcg_add(t->d_grad[i].p, t->d_grad2[i].p, t->d_grad[i].p, t->d_grad[i].n, t->stream))) return st;
    DCG_CUDA(cudaEventRecord(t->ev_grads, t->stream));
    DCG_CUDA(cudaStreamWaitEvent(t->comm_stream, t->ev_grads, 0));
    if (t->fused_update) {   // sum + Adam + broadcast in one kernel, under the generator's forward pass
        if ((st = fused_update(t, 0, &t->d_t, scale, lr_dev, t->comm_stream))) return st;
    } else if ((st = sum_over_ranks(t, t->d_grads_all, t->comm_stream))) {
        return st;
    }
    DCG_CUDA(cudaEventRecord(t->ev_summed, t->comm_stream));
    if ((st = dcg_run_nodes(t->ctx, t->g_nodes.data(), fwd, t->cfg.fuse))) return st;
    DCG_CUDA(cudaStreamWaitEvent(t->stream, t->ev_summed, 0));
    if (!t->fused_update &&
        (st = apply_adam(t, t->d_param, t->d_grad, nullptr, t->d_m, t->d_v, &t->d_t, scale, lr_dev)))
        return st;
    if ((st = dcg_run_nodes(t->ctx, t->g_nodes.data() + fwd, all - fwd, t->cfg.fuse))) return st;
    for (int rep = 0; rep < 2; ++rep) {
        if (rep == 1 && (st = dcg_run_nodes(t->ctx, t->g_nodes.data(), all, t->cfg.fuse))) return st;
        const float* lr = lr_dev ? lr_dev + 1 + rep : nullptr;
        if (t->fused_update) {
            if ((st = fused_update(t, 1, &t->g_t, scale, lr, t->stream))) return st;
        } else {
            if ((st = sum_over_ranks(t, t->g_grads_all, t->stream))) return st;
            if ((st = apply_adam(t, t->g_param, t->g_grad, nullptr, t->g_m, t->g_v, &t->g_t, scale, lr))) return st;
        }
    }
    return DCG_OK;
}

// The whole single-GPU iteration, enqueued node list by node list (used eagerly and under capture).
int enqueue_step(dcg_trainer* t, const float* lr_dev)
{
    if (t->cfg.world > 1 && t->dp) return enqueue_step_dp(t, lr_dev);
    int st;
    Tensor* d_second = (t->cfg.world > 1 || t->batched_d) ? nullptr : t->d_grad2;
    if ((st = dcg_run_nodes(t->ctx, t->d_nodes.data(), (int)t->d_nodes.size(), t->cfg.fuse))) return st;
    if ((st = apply_adam(t, t->d_param, t->d_grad, d_second, t->d_m, t->d_v, &t->d_t, 1.f, lr_dev))) return st;
    for (int rep = 0; rep < 2; ++rep) {
        // share_g_forward: the first G run re-uses the generator activations the D run just computed
        // (the generator's parameters have not changed in between) instead of recomputing them
        const int first = (rep == 0 && t->cfg.share_g_forward) ? (int)t->g_forward_nodes : 0;
        if ((st = dcg_run_nodes(t->ctx, t->g_nodes.data() + first, (int)t->g_nodes.size() - first, t->cfg.fuse))) return st;
        if ((st = apply_adam(t, t->g_param, t->g_grad, nullptr, t->g_m, t->g_v, &t->g_t, 1.f,
                             lr_dev ? lr_dev + 1 + rep : nullptr)))
            return st;
    }
    return DCG_OK;
}

// Replays (capturing first if need be) the whole-iteration graph.  Returns 1 if it did, 0 if the
// caller should run the phases instead, a negative status on error.
int step_as_one_graph(dcg_trainer* t)
{
    dcg_trainer::ListGraph& g = t->step_graph;
    if (!t->use_graphs || g.failed || (t->cfg.world > 1 && !t->dp) || dcg::context_is_profiling(t->ctx)) return 0;
    if (t->step_warm_runs < 2) return 0;   // every list has to run eagerly twice first (scratch sizes, one-time attributes)
    if (g.exec && g.generation != dcg::context_generation(t->ctx)) {
        cudaGraphExecDestroy(g.exec);
        g.exec = nullptr;
    }
    // this iteration's three step sizes; the copy is from pageable memory, which the runtime stages
    // before the call returns, so the array may go out of scope
    float lr[3];
    lr[0] = dcg_adam_lr_t(&t->d_t, t->cfg.lr, t->cfg.beta1, t->cfg.beta2);
    lr[1] = dcg_adam_lr_t(&t->g_t, t->cfg.lr, t->cfg.beta1, t->cfg.beta2);
    lr[2] = dcg_adam_lr_t(&t->g_t, t->cfg.lr, t->cfg.beta1, t->cfg.beta2);
    if (cudaMemcpyAsync(t->lr_dev.p, lr, sizeof(lr), cudaMemcpyHostToDevice, t->stream) != cudaSuccess)
        return fail(DCG_ERR_CUDA, "dcg_trainer_step: copy of the Adam step sizes failed");
    if (!g.exec) {
        const uint64_t before = dcg_launches_total();
        cudaGraph_t graph = nullptr;
        bool ok = cudaStreamBeginCapture(t->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
        int st = DCG_OK;
        if (ok) {
            st = enqueue_step(t, t->lr_dev.p);
            ok = cudaStreamEndCapture(t->stream, &graph) == cudaSuccess && st == DCG_OK && graph &&
                 cudaGraphInstantiate(&g.exec, graph, 0) == cudaSuccess;
        }
        if (graph) cudaGraphDestroy(graph);
        const uint64_t captured = dcg_launches_total() - before;
        dcg::count_launch(-(int)captured);   // a capture launches nothing
        if (!ok) {
            cudaGetLastError();
            g.exec = nullptr;
            g.failed = true;
            if (getenv("DCG_TRAINER_VERBOSE"))
                fprintf(stderr, "dcg_trainer: whole-step graph capture failed (list status %d: %s); running %s\n", st,
                        st ? dcg_last_error() : "capture / instantiate", t->dp ? "eagerly" : "per-list graphs");
            // the step counters already advanced: finish this iteration eagerly with the same step sizes
            return (st = enqueue_step(t, t->lr_dev.p)) ? st : 1;
        }
        g.launches = captured;
        g.generation = dcg::context_generation(t->ctx);
    }
    if (cudaGraphLaunch(g.exec, t->stream) != cudaSuccess)
        return fail(DCG_ERR_CUDA, "cudaGraphLaunch: %s", cudaGetErrorString(cudaGetLastError()));
    dcg::count_launch((int)g.launches);
    return 1;
}

}  // namespace

extern "C" int dcg_trainer_create(dcg_trainer** out, const dcg_trainer_config* cfg, dcg_stream_t stream)
{
    return dcg_trainer_create_dp(out, cfg, stream, nullptr);
}

extern "C" int dcg_trainer_create_dp(dcg_trainer** out, const dcg_trainer_config* cfg, dcg_stream_t stream, dcg_dp* dp)
{
    DCG_CHECK_ARG(out && cfg, "dcg_trainer_create: null argument");
    DCG_CHECK_ARG(cfg->batch > 0 && cfg->batch <= 4096, "dcg_trainer_create: bad batch %d", cfg->batch);
    DCG_CHECK_ARG(!dp || dcg::dp_world(dp) == cfg->world, "dcg_trainer_create_dp: the communicator has %d ranks, the configuration %d",
                  dcg::dp_world(dp), cfg->world);
    dcg_trainer* t = new dcg_trainer();
    t->cfg = *cfg;
    t->dp = (dp && cfg->world > 1) ? dp : nullptr;
    t->stream = dcg::as_stream(stream);
    {
        const char* off = getenv("DCG_TRAINER_TWO_PASSES");   // experiments: keep the two passes on the tensor path too
        t->batched_d = cfg->precision != DCG_PREC_FP32 && !(off && atoi(off) != 0);
        const char* eager = getenv("DCG_TRAINER_EAGER");       // experiments: no CUDA graphs
        t->use_graphs = !(eager && atoi(eager) != 0);
    }
    Alloc dry{t, true};
    layout(t, dry);
    t->arena_bytes = dcg::align_up(dry.off, 256) + 256;
    // Data parallel: by default the update is the fused kernel over peer memory (dp_adam.cu), which
    // needs a cudaMalloc'ed arena (CUDA IPC); DCG_DP_FUSED=0 keeps NCCL all-reduce + replicated Adam,
    // with the arena from NCCL's own allocator (eligible for its in-switch reduction of user buffers).
    bool want_fused = false;
    if (t->dp) {
        const char* f = getenv("DCG_DP_FUSED");
        want_fused = !(f && atoi(f) == 0) && cfg->world <= 8;
    }
    if (t->dp && !want_fused) {
        t->arena = static_cast<uint8_t*>(dcg::dp_mem_alloc(t->arena_bytes));
        t->arena_from_nccl = t->arena != nullptr;
    }
    if (!t->arena && cudaMalloc(&t->arena, t->arena_bytes) != cudaSuccess) {
        const size_t want = t->arena_bytes;
        delete t;
        return fail(DCG_ERR_CUDA, "dcg_trainer_create: cudaMalloc of %zu bytes failed", want);
    }
    if (t->dp) {
        bool ok = cudaStreamCreateWithFlags(&t->comm_stream, cudaStreamNonBlocking) == cudaSuccess &&
                  cudaEventCreateWithFlags(&t->ev_grads, cudaEventDisableTiming) == cudaSuccess &&
                  cudaEventCreateWithFlags(&t->ev_summed, cudaEventDisableTiming) == cudaSuccess;
        if (!ok) {
            dcg_trainer_destroy(t);
            return fail(DCG_ERR_CUDA, "dcg_trainer_create_dp: could not create the communication stream");
        }
    }
    cudaMemsetAsync(t->arena, 0, t->arena_bytes, t->stream);
    Alloc real{t, false};
    layout(t, real);
    t->arena_used = real.off;
    int st = dcg_context_create(&t->ctx, cfg->precision, nullptr, 0, stream);
    if (st) { dcg_trainer_destroy(t); return st; }

    // weights ~ N(0, 0.02), biases 0 (dcgan/main.cu:60-63, 148-151); labels
    Rng rng(cfg->seed ? cfg->seed : 234);
    auto fill_normal = [&](Tensor& w) {
        std::vector<float> h(w.n);
        for (size_t i = 0; i < w.n; ++i) h[i] = rng.normal(0.02f);
        cudaMemcpyAsync(w.p, h.data(), w.n * sizeof(float), cudaMemcpyHostToDevice, t->stream);
        cudaStreamSynchronize(t->stream);
    };
    for (int i = 0; i < 10; i += 2) { fill_normal(t->g_param[i]); fill_normal(t->d_param[i]); }
    std::vector<float> one(cfg->batch, 1.f);
    cudaMemcpyAsync(t->ones.p, one.data(), one.size() * sizeof(float), cudaMemcpyHostToDevice, t->stream);
    cudaStreamSynchronize(t->stream);
    build_lists(t);
    if (t->dp && want_fused) {
        // collective: every rank maps every other rank's arena; all ranks agree on the outcome
        cudaStreamSynchronize(t->stream);   // the arena (flag words included) is zeroed before anyone may write to it
        t->fused_update = dcg::dp_map_peers(t->dp, t->arena, t->peer_arena) == DCG_OK;
    }
    if (t->dp && !t->fused_update) {   // the two buffers the communicator reduces every iteration
        dcg::dp_register(t->dp, t->d_grads_all.p, t->d_grads_all.n * sizeof(float));
        dcg::dp_register(t->dp, t->g_grads_all.p, t->g_grads_all.n * sizeof(float));
    }
    if (cudaGetLastError() != cudaSuccess) {
        dcg_trainer_destroy(t);
        return fail(DCG_ERR_CUDA, "dcg_trainer_create: initialisation copies failed");
    }
    *out = t;
    return DCG_OK;
}

extern "C" void dcg_trainer_destroy(dcg_trainer* t)
{
    if (!t) return;
    for (dcg_trainer::ListGraph* g : {&t->d_graph, &t->g_graph, &t->gen_graph, &t->dfb_graph, &t->g_part_graph[0], &t->g_part_graph[1],
                                      &t->step_graph})
        if (g->exec) cudaGraphExecDestroy(g->exec);
    if (t->ctx) dcg_context_destroy(t->ctx);
    if (t->fused_update) {
        // COLLECTIVE: an exported arena must not be freed while a peer still has it mapped, so every rank
        // closes its mappings, then the ranks meet (a one-float all-reduce), then the arenas go
        cudaDeviceSynchronize();
        dcg::dp_unmap_peers(t->dp, t->peer_arena);
        float* token[1] = {t->lr_dev.p + 3};
        const size_t one[1] = {1};
        if (dcg::dp_allreduce_group(t->dp, token, one, 1, t->stream) == DCG_OK) cudaStreamSynchronize(t->stream);
        cudaGetLastError();
    }
    if (t->arena) {
        if (t->arena_from_nccl) dcg::dp_mem_free(t->arena);
        else cudaFree(t->arena);
    }
    if (t->writer.joinable()) t->writer.join();
    if (t->snap) cudaFreeHost(t->snap);
    if (t->ev_snap) cudaEventDestroy(t->ev_snap);
    if (t->ev_grads) cudaEventDestroy(t->ev_grads);
    if (t->ev_summed) cudaEventDestroy(t->ev_summed);
    if (t->comm_stream) cudaStreamDestroy(t->comm_stream);
    delete t;
}

extern "C" int dcg_trainer_generate(dcg_trainer* t)
{
    DCG_CHECK_ARG(t, "dcg_trainer_generate: null trainer");
    return run_list(t, t->gen_nodes, t->gen_graph);
}

extern "C" int dcg_trainer_d_fwd_bwd(dcg_trainer* t)
{
    DCG_CHECK_ARG(t, "dcg_trainer_d_fwd_bwd: null trainer");
    return run_list(t, t->dfb_nodes, t->dfb_graph);
}

extern "C" int dcg_trainer_d_backward(dcg_trainer* t)
{
    DCG_CHECK_ARG(t, "dcg_trainer_d_backward: null trainer");
    int st = run_list(t, t->d_nodes, t->d_graph);
    if (st) return st;
    if (t->cfg.world > 1 && !t->batched_d) {
        // sum the two gradient paths now (the Add op of src/ops/graph.cu:302-309) so that one
        // all-reduce of the gradient arena averages the final gradients
        for (int i = 0; i < 10; ++i)
            if ((st = dcg_add(t->d_grad[i].p, t->d_grad2[i].p, t->d_grad[i].p, t->d_grad[i].n, t->stream))) return st;
    }
    return DCG_OK;
}

extern "C" int dcg_trainer_d_apply(dcg_trainer* t, float grad_scale)
{
    DCG_CHECK_ARG(t, "dcg_trainer_d_apply: null trainer");
    return apply_adam(t, t->d_param, t->d_grad, (t->cfg.world > 1 || t->batched_d) ? nullptr : t->d_grad2, t->d_m,
                      t->d_v, &t->d_t, grad_scale);
}

extern "C" int dcg_trainer_g_backward(dcg_trainer* t)
{
    DCG_CHECK_ARG(t, "dcg_trainer_g_backward: null trainer");
    return run_list(t, t->g_nodes, t->g_graph);
}

extern "C" int dcg_trainer_g_backward_part(dcg_trainer* t, int part)
{
    DCG_CHECK_ARG(t && (part == 0 || part == 1), "dcg_trainer_g_backward_part: bad arguments");
    if (part == 0) return run_list(t, t->g_nodes, t->g_part_graph[0], 0, t->g_forward_nodes);
    return run_list(t, t->g_nodes, t->g_part_graph[1], t->g_forward_nodes);
}

extern "C" int dcg_trainer_g_apply(dcg_trainer* t, float grad_scale)
{
    DCG_CHECK_ARG(t, "dcg_trainer_g_apply: null trainer");
    return apply_adam(t, t->g_param, t->g_grad, nullptr, t->g_m, t->g_v, &t->g_t, grad_scale);
}

extern "C" int dcg_trainer_step(dcg_trainer* t)
{
    DCG_CHECK_ARG(t, "dcg_trainer_step: null trainer");
    DCG_CHECK_ARG(t->cfg.world <= 1 || t->dp,
                  "dcg_trainer_step: a data-parallel trainer without a communicator (dcg_trainer_create_dp) is driven phase by phase");
    const uint64_t before = dcg_launches_total();
    int st = step_as_one_graph(t);   // 1: replayed; 0: not (yet) available
    if (st < 0) return st;
    if (st == 0) {
        if (t->dp) {
            st = enqueue_step(t, nullptr);   // eager, collectives included
            if (st) return st;
        } else if (t->cfg.share_g_forward) {
            if ((st = enqueue_step(t, nullptr))) return st;   // eager; the per-list graphs have no shared form
        } else {
            if ((st = dcg_trainer_d_backward(t))) return st;
            if ((st = dcg_trainer_d_apply(t, 1.f))) return st;
            for (int rep = 0; rep < 2; ++rep) {
                if ((st = dcg_trainer_g_backward(t))) return st;
                if ((st = dcg_trainer_g_apply(t, 1.f))) return st;
            }
        }
        if (!dcg::context_is_profiling(t->ctx)) ++t->step_warm_runs;
    }
    t->last_step_launches = dcg_launches_total() - before;
    return DCG_OK;
}

// ---- checkpoints -----------------------------------------------------------------------------------
// Counterpart of ops::Graph::save_vars / load_vars (src/ops/graph.cu:326-361), which write every
// trainable variable as an fp32 tensor with its dims through the tensor-archive library.  The file
// here is the raw archive of this repository's stand-in for that library (shim/tocha/tensor.hh):
// "DCGT", u32 version 1, u32 count, then per tensor u32 rank, rank x u32 extents, fp32 values.
// Tensors: the generator's 10 variables (k0,b0,..,k3,b3,dense w,dense b), the discriminator's 10,
// then - which the reference drops (src/api/adam-optimizer.cu:39-45), so its restarts lose the
// optimiser state - Adam's first and second moments of both networks in the same order, and the two
// step counters [g_t, d_t].  A loader that only wants the variables reads the first 20 tensors.
namespace {

struct CkptTensor {
    Tensor t;
    int rank;
    unsigned dims[4];
};

std::vector<CkptTensor> checkpoint_layout(dcg_trainer* t)
{
    std::vector<CkptTensor> v;
    auto add_net = [&](Tensor* arr, bool gen) {
        for (int i = 0; i < 10; ++i) {
            CkptTensor c{};
            c.t = arr[i];
            if (i < 8 && i % 2 == 0) {
                const int l = i / 2;
                c.rank = 4; c.dims[0] = 5; c.dims[1] = 5;
                c.dims[2] = gen ? kGChan[l + 1] : kDChan[l];
                c.dims[3] = gen ? kGChan[l] : kDChan[l + 1];
            } else if (i == 8) {
                c.rank = 2; c.dims[0] = gen ? kZ : 8192; c.dims[1] = gen ? 8192 : 1;
            } else {
                c.rank = 1; c.dims[0] = (unsigned)arr[i].n;
            }
            v.push_back(c);
        }
    };
    add_net(t->g_param, true); add_net(t->d_param, false);
    add_net(t->g_m, true); add_net(t->g_v, true);
    add_net(t->d_m, false); add_net(t->d_v, false);
    return v;
}

int write_checkpoint(const std::string& path, const std::vector<CkptTensor>& lay, const float* host, float g_t, float d_t,
                     std::string& err)
{
    std::FILE* f = std::fopen(path.c_str(), "wb");
    if (!f) { err = "cannot write " + path; return DCG_ERR_INVALID; }
    const unsigned head[2] = {1u, (unsigned)lay.size() + 1u};
    bool ok = std::fwrite("DCGT", 1, 4, f) == 4 && std::fwrite(head, 4, 2, f) == 2;
    size_t off = 0;
    for (const CkptTensor& c : lay) {
        const unsigned rank = (unsigned)c.rank;
        ok = ok && std::fwrite(&rank, 4, 1, f) == 1 && std::fwrite(c.dims, 4, rank, f) == rank &&
             std::fwrite(host + off, sizeof(float), c.t.n, f) == c.t.n;
        off += c.t.n;
    }
    const unsigned tail[2] = {1u, 2u};
    const float counters[2] = {g_t, d_t};
    ok = ok && std::fwrite(tail, 4, 2, f) == 2 && std::fwrite(counters, sizeof(float), 2, f) == 2;
    if (std::fclose(f) != 0 || !ok) { err = "write failed: " + path; return DCG_ERR_INVALID; }
    return DCG_OK;
}

}  // namespace

extern "C" int dcg_trainer_save_wait(dcg_trainer* t)
{
    DCG_CHECK_ARG(t, "dcg_trainer_save_wait: null trainer");
    if (t->writer.joinable()) t->writer.join();
    const int st = t->writer_status;
    t->writer_status = DCG_OK;
    if (st) return fail(st, "checkpoint: %s", t->writer_error.c_str());
    return DCG_OK;
}

extern "C" int dcg_trainer_save(dcg_trainer* t, const char* path)
{
    DCG_CHECK_ARG(t && path, "dcg_trainer_save: null argument");
    int st = dcg_trainer_save_wait(t);   // one checkpoint in flight at a time
    if (st) return st;
    const std::vector<CkptTensor> lay = checkpoint_layout(t);
    size_t total = 0;
    for (const CkptTensor& c : lay) total += c.t.n;
    if (!t->snap) {
        DCG_CUDA(cudaMallocHost(&t->snap, total * sizeof(float)));
        t->snap_floats = total;
        DCG_CUDA(cudaEventCreateWithFlags(&t->ev_snap, cudaEventDisableTiming));
    }
    if (t->fused_update) {
        // The moments of a parameter slice only live on the rank that owns it.  COLLECTIVE in this mode:
        // every rank calls save after the same iteration; between two barriers each rank copies the
        // other owners' slices of m and v out of their arenas, so that the file holds complete state.
        const int W = t->cfg.world, R = dcg::dp_rank(t->dp);
        float* token[1] = {t->lr_dev.p + 3};
        const size_t one[1] = {1};
        if ((st = dcg::dp_allreduce_group(t->dp, token, one, 1, t->stream))) return st;   // everybody's updates are done
        for (int net = 0; net < 2; ++net) {
            const Tensor& params = net == 0 ? t->d_params_all : t->g_params_all;
            Tensor* mv[2] = {net == 0 ? t->d_m : t->g_m, net == 0 ? t->d_v : t->g_v};
            const size_t n4 = (params.n + 3) / 4, chunk = (n4 + W - 1) / W;
            for (int r = 0; r < W; ++r) {
                if (r == R) continue;
                const size_t lo = chunk * r, hi = lo + chunk < n4 ? lo + chunk : n4;
                if (hi <= lo) continue;
                for (int q = 0; q < 2; ++q) {
                    uint8_t* mine = reinterpret_cast<uint8_t*>(mv[q][0].p) + lo * 16;
                    const uint8_t* theirs = static_cast<uint8_t*>(t->peer_arena[r]) + (mine - t->arena);
                    DCG_CUDA(cudaMemcpyAsync(mine, theirs, (hi - lo) * 16, cudaMemcpyDefault, t->stream));
                }
            }
        }
        if ((st = dcg::dp_allreduce_group(t->dp, token, one, 1, t->stream))) return st;   // nobody moves on while a peer still reads
    }
    size_t off = 0;
    for (const CkptTensor& c : lay) {   // stream-ordered behind the updates enqueued so far
        DCG_CUDA(cudaMemcpyAsync(t->snap + off, c.t.p, c.t.n * sizeof(float), cudaMemcpyDeviceToHost, t->stream));
        off += c.t.n;
    }
    DCG_CUDA(cudaEventRecord(t->ev_snap, t->stream));
    const float g_t = t->g_t, d_t = t->d_t;
    const std::string file(path);
    int dev = 0;
    DCG_CUDA(cudaGetDevice(&dev));
    t->writer = std::thread([t, lay, file, g_t, d_t, dev] {
        cudaSetDevice(dev);
        if (cudaEventSynchronize(t->ev_snap) != cudaSuccess) {
            t->writer_status = DCG_ERR_CUDA;
            t->writer_error = "the snapshot copy failed";
            return;
        }
        t->writer_status = write_checkpoint(file, lay, t->snap, g_t, d_t, t->writer_error);
    });
    return DCG_OK;
}

extern "C" int dcg_trainer_load(dcg_trainer* t, const char* path)
{
    DCG_CHECK_ARG(t && path, "dcg_trainer_load: null argument");
    int st = dcg_trainer_save_wait(t);
    if (st) return st;
    std::FILE* f = std::fopen(path, "rb");
    if (!f) return fail(DCG_ERR_INVALID, "dcg_trainer_load: cannot read %s", path);
    const std::vector<CkptTensor> lay = checkpoint_layout(t);
    char magic[4];
    unsigned head[2] = {0, 0};
    bool ok = std::fread(magic, 1, 4, f) == 4 && std::memcmp(magic, "DCGT", 4) == 0 && std::fread(head, 4, 2, f) == 2 &&
              head[0] == 1u;
    // the variables alone (20 tensors, e.g. written by the reference's save_vars through the stand-in
    // archive) or a full checkpoint (60 tensors + the counters)
    const size_t have = head[1];
    ok = ok && (have == 20 || have == lay.size() + 1);
    std::vector<float> host;
    for (size_t i = 0; ok && i < lay.size() && i < have; ++i) {
        const CkptTensor& c = lay[i];
        unsigned rank = 0, dims[8] = {0};
        ok = std::fread(&rank, 4, 1, f) == 1 && rank >= 1 && rank <= 4 && std::fread(dims, 4, rank, f) == rank;
        size_t n = 1;
        for (unsigned r = 0; ok && r < rank; ++r) n *= dims[r];
        ok = ok && n == c.t.n;
        if (!ok) break;
        host.resize(n);
        ok = std::fread(host.data(), sizeof(float), n, f) == n;
        if (ok && cudaMemcpyAsync(c.t.p, host.data(), n * sizeof(float), cudaMemcpyHostToDevice, t->stream) != cudaSuccess) ok = false;
        if (ok && cudaStreamSynchronize(t->stream) != cudaSuccess) ok = false;   // `host` is reused
    }
    if (ok && have == lay.size() + 1) {
        unsigned tail[2] = {0, 0};
        float counters[2] = {0.f, 0.f};
        ok = std::fread(tail, 4, 2, f) == 2 && tail[0] == 1u && tail[1] == 2u && std::fread(counters, sizeof(float), 2, f) == 2;
        if (ok) { t->g_t = counters[0]; t->d_t = counters[1]; }
    }
    std::fclose(f);
    if (!ok) return fail(DCG_ERR_INVALID, "dcg_trainer_load: %s is not a checkpoint of this model", path);
    return DCG_OK;
}

extern "C" int dcg_trainer_tensor(dcg_trainer* t, const char* name, float** ptr, size_t* count)
{
    DCG_CHECK_ARG(t && name && ptr && count, "dcg_trainer_tensor: null argument");
    const std::string s(name);
    Tensor r;
    auto indexed = [&](const char* prefix, Tensor* arr, int n) -> bool {
        const size_t len = std::strlen(prefix);
        if (s.compare(0, len, prefix) != 0 || s.size() != len + 1) return false;
        const int i = s[len] - '0';
        if (i < 0 || i >= n) return false;
        r = arr[i];
        return true;
    };
    if (s == "x") r = t->x;
    else if (s == "z") r = t->z;
    else if (s == "g_out") r = t->g_out;
    else if (s == "d_loss") r = t->d_loss;
    else if (s == "g_loss") r = t->g_loss;
    else if (s == "d_params") r = t->d_params_all;
    else if (s == "g_params") r = t->g_params_all;
    else if (s == "d_grads") r = t->d_grads_all;
    else if (s == "g_grads") r = t->g_grads_all;
    else if (s == "logits_fake") r = t->logits[0];
    else if (s == "logits_real") r = t->logits[1];
    else if (indexed("d_param", t->d_param, 10) || indexed("g_param", t->g_param, 10) ||
             indexed("d_grad", t->d_grad, 10) || indexed("g_grad", t->g_grad, 10) ||
             indexed("d_gradb", t->d_grad2, 10) || indexed("d_m", t->d_m, 10) || indexed("d_v", t->d_v, 10) ||
             indexed("g_m", t->g_m, 10) || indexed("g_v", t->g_v, 10)) {
    } else {
        return fail(DCG_ERR_INVALID, "dcg_trainer_tensor: unknown tensor '%s'", name);
    }
    *ptr = r.p;
    *count = r.n;
    return DCG_OK;
}

extern "C" dcg_context* dcg_trainer_context(dcg_trainer* t) { return t ? t->ctx : nullptr; }

extern "C" uint64_t dcg_trainer_step_launches(const dcg_trainer* t) { return t ? t->last_step_launches : 0; }

extern "C" int dcg_trainer_dp_mode(const dcg_trainer* t)
{
    if (!t || !t->dp) return 0;
    return t->fused_update ? 2 : 1;
}

extern "C" int dcg_trainer_step_mode(const dcg_trainer* t)
{
    if (!t) return -1;
    if (t->step_graph.exec) return 2;
    return t->step_graph.failed ? 0 : 1;
}

extern "C" size_t dcg_trainer_arena_bytes(const dcg_trainer* t) { return t ? t->arena_bytes : 0; }
