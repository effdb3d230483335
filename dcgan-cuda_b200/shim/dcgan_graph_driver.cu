// A user program of the reference project: builds the DCGAN of dcgan/main.cu:43-332 with the
// reference's own public API (ops::OpsBuilder, ops::Graph, AdamOptimizer, the src/api layers) and
// runs it through ops::Graph::run - the caller of the convolution / Adam path.  Unlike dcgan/main.cu
// the batch size is a run-time argument, the weights are seeded (xorshift + Box-Muller instead of a
// clock-seeded std::normal_distribution, src/api/normal-initializer.cu:6-9) and the inputs are
// synthetic (images and z ~ U(-1,1); no JPEG directory is read), so that the same program gives the
// same numbers under RT_MODE=CPU, MCPU and GPU and can be timed in each.
//
//   dcgan_graph_driver gen   BATCH ITERS OUT [leaky|relu] [SEED]   generator forward only
//   dcgan_graph_driver train BATCH ITERS OUT [leaky|relu] [SEED]   ITERS x (1 D update + 2 G updates)
//
// OUT receives a tensor archive: gen -> [g_out]; train -> [d_loss per iteration, g_loss of the
// second G run per iteration, the 10 generator variables (k0,b0,..,k3,b3,dense w,dense b), the 10
// discriminator variables, g_loss of the first G run per iteration].  One JSON line with the wall-clock milliseconds of every Graph::run group goes to stdout.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "api/activ.hh"
#include "api/adam-optimizer.hh"
#include "api/copy-initializer.hh"
#include "api/layers.hh"
#include "memory/alloc.hh"
#include "memory/copy.hh"
#include "ops/add.hh"
#include "ops/conv2d-bias-add.hh"
#include "ops/conv2d-transpose.hh"
#include "ops/conv2d.hh"
#include "ops/graph.hh"
#include "ops/input.hh"
#include "ops/mat-mul-add.hh"
#include "ops/ops-builder.hh"
#include "ops/reshape.hh"
#include "ops/sigmoid-cross-entropy.hh"
#include "ops/variable.hh"
#include "ops/vect-relu-leaky.hh"
#include "ops/vect-relu.hh"
#include "ops/vect-tanh.hh"
#include "utils/xorshift.hh"

#include <tocha/tensor.hh>

namespace
{

    constexpr int kZ = 100;
    int g_strides[] = {2, 2};

    float normal(float sd)
    {
        float u1 = xorshift::next_f32(), u2 = xorshift::next_f32();
        if (u1 < 1e-12f) u1 = 1e-12f;
        return sd * std::sqrt(-2.f * std::log(u1)) * std::cos(6.28318530718f * u2);
    }

    struct Layer
    {
        ops::Variable* w = nullptr;
        ops::Variable* b = nullptr;
    };

    ops::Variable* make_var(const ops::Shape& shape, const char* name)
    {
        auto v = ops::OpsBuilder::instance().variable(shape, true);
        v->extend_name(name);
        std::vector<dbl_t> zero(shape.total(), 0.f);
        tensor_write(v->data_begin(), v->data_end(), zero.data());
        return v;
    }

    void fill_normal(ops::Variable* v)
    {
        std::vector<dbl_t> h(v->data_end() - v->data_begin());
        for (auto& e : h) e = normal(0.02f);
        tensor_write(v->data_begin(), v->data_end(), h.data());
    }

    ops::Op* activation(ops::Op* z, bool leaky)
    {
        auto& builder = ops::OpsBuilder::instance();
        return leaky ? static_cast<ops::Op*>(builder.vect_relu_leaky(z, 0.2)) : static_cast<ops::Op*>(builder.vect_relu(z));
    }

    // generator: dcgan/main.cu:43-120
    ops::Op* generator(ops::Op* z, int B, bool leaky, Layer* layers /* [5]: 4 conv layers, then dense */)
    {
        auto& builder = ops::OpsBuilder::instance();
        const int ch[5] = {512, 256, 128, 64, 3};
        layers[4].w = make_var(ops::Shape({kZ, 8192}), "dense_w");
        layers[4].b = make_var(ops::Shape({8192}), "dense_b");
        ops::Op* cur = activation(builder.mat_mul_add(z, layers[4].w, layers[4].b), leaky);
        cur = builder.reshape(cur, ops::Shape({B, 4, 4, 512}));
        for (int i = 0; i < 4; ++i) {
            const int hw = 8 << i;
            layers[i].w = make_var(ops::Shape({5, 5, ch[i + 1], ch[i]}), "conv2d_transpose_w");
            layers[i].b = make_var(ops::Shape({ch[i + 1]}), "conv2d_transpose_b");
            // the op keeps the POINTER to its output extents (src/ops/conv2d-transpose.cu:20): static storage
            static int out_sizes[4][4];
            int* out_size = out_sizes[i];
            out_size[0] = B; out_size[1] = hw; out_size[2] = hw; out_size[3] = ch[i + 1];
            ops::Op* conv = builder.conv2d_transpose(cur, layers[i].w, out_size, g_strides);
            cur = builder.conv2d_bias_add(conv, layers[i].b);
            if (i < 3) cur = activation(cur, leaky);
        }
        return cur;   // logits; the caller applies tanh (dcgan/main.cu:288)
    }

    // discriminator: dcgan/main.cu:123-249
    ops::Op* discriminator(ops::Op* x, int B, Layer* layers /* [5] */, bool reuse)
    {
        auto& builder = ops::OpsBuilder::instance();
        const int ch[5] = {3, 64, 128, 256, 512};
        ops::Op* cur = x;
        for (int i = 0; i < 4; ++i) {
            if (!reuse) {
                layers[i].w = make_var(ops::Shape({5, 5, ch[i], ch[i + 1]}), "conv2d_w");
                layers[i].b = make_var(ops::Shape({ch[i + 1]}), "conv2d_b");
            }
            ops::Op* conv = builder.conv2d(cur, layers[i].w, g_strides);
            cur = builder.vect_relu_leaky(builder.conv2d_bias_add(conv, layers[i].b), 0.2);
        }
        cur = builder.reshape(cur, ops::Shape({B, 8192}));
        if (!reuse) {
            layers[4].w = make_var(ops::Shape({8192, 1}), "dense_w");
            layers[4].b = make_var(ops::Shape({1}), "dense_b");
        }
        return builder.mat_mul_add(cur, layers[4].w, layers[4].b);
    }

    double now_ms()
    {
        using namespace std::chrono;
        return duration<double, std::milli>(steady_clock::now().time_since_epoch()).count();
    }

    void add_var(tocha::Tensors& out, ops::Variable* v)
    {
        const auto& d = v->shape_get().dims();
        tocha::Tensor t = tocha::Tensor::make(d, nullptr);
        tensor_read(v->data_begin(), v->data_end(), reinterpret_cast<dbl_t*>(t.data));
        out.add(t);
    }

}

int main(int argc, char** argv)
{
    if (argc < 5) {
        std::fprintf(stderr, "usage: %s gen|train BATCH ITERS OUT [leaky|relu] [SEED]\n", argv[0]);
        return 2;
    }
    const std::string mode = argv[1];
    const int B = std::atoi(argv[2]), iters = std::atoi(argv[3]);
    const std::string out_path = argv[4];
    const bool leaky = argc > 5 ? std::strcmp(argv[5], "leaky") == 0 : mode == "gen";
    const unsigned long long seed = argc > 6 ? std::strtoull(argv[6], nullptr, 10) : 234ull;
    if ((mode != "gen" && mode != "train") || B <= 0 || iters <= 0) {
        std::fprintf(stderr, "bad arguments\n");
        return 2;
    }

    auto& graph = ops::Graph::instance();
    auto& builder = ops::OpsBuilder::instance();
    auto z = builder.input(ops::Shape({B, kZ}));
    auto x = builder.input(ops::Shape({B, 64, 64, 3}));

    Layer g[5], d[5];
    ops::Op* g_out = builder.vect_tanh(generator(z, B, leaky, g));
    ops::Op* d1_logits = discriminator(g_out, B, d, false);
    ops::Op* d2_logits = discriminator(x, B, d, true);

    // weights ~ N(0, 0.02) in the order (g k0, d k0, g k1, d k1, ..., g dense, d dense); biases 0
    xorshift::seed(seed);
    for (int i = 0; i < 5; ++i) {
        fill_normal(g[i].w);
        fill_normal(d[i].w);
    }
    std::vector<dbl_t> x_h((std::size_t)B * 64 * 64 * 3), z_h((std::size_t)B * kZ), zeros(B, 0.f), ones(B, 1.f);
    for (auto& e : x_h) e = 2.f * xorshift::next_f32() - 1.f;
    for (auto& e : z_h) e = 2.f * xorshift::next_f32() - 1.f;

    std::vector<double> ms;
    tocha::Tensors out;
    if (mode == "gen") {
        tocha::Tensor img = tocha::Tensor::f32(B, 64, 64, 3);
        for (int it = 0; it < iters; ++it) {
            const double t0 = now_ms();
            graph.run({g_out}, {{z, {z_h.data(), ops::Shape({B, kZ})}}}, {reinterpret_cast<dbl_t*>(img.data)});
            ms.push_back(now_ms() - t0);
        }
        out.add(img);
    } else {
        auto logits0 = builder.input(ops::Shape({B, 1}));
        auto logits1 = builder.input(ops::Shape({B, 1}));
        auto g_loss = builder.sigmoid_cross_entropy(logits1, d1_logits);
        auto d1_loss = builder.sigmoid_cross_entropy(logits0, d1_logits);
        auto d2_loss = builder.sigmoid_cross_entropy(logits1, d2_logits);
        auto d_loss = builder.add(d1_loss, d2_loss);
        std::vector<ops::Variable*> g_vars, d_vars;
        for (int i = 0; i < 5; ++i) {
            g_vars.push_back(g[i].w); g_vars.push_back(g[i].b);
            d_vars.push_back(d[i].w); d_vars.push_back(d[i].b);
        }
        AdamOptimizer g_adam(0.0002, 0.5), d_adam(0.0002, 0.5);
        auto g_opti = g_adam.minimize(g_loss, g_vars);
        auto d_opti = d_adam.minimize(d_loss, d_vars);
        tocha::Tensor dl = tocha::Tensor::f32(iters), gl = tocha::Tensor::f32(iters), gl_first = tocha::Tensor::f32(iters);
        for (int it = 0; it < iters; ++it) {
            dbl_t d_loss_val = 0, g_loss_val = 0;
            const double t0 = now_ms();
            // one iteration exactly as dcgan/main.cu:378-391
            graph.run({d_opti, d_loss},
                      {{logits0, {zeros.data(), ops::Shape({B, 1})}},
                       {logits1, {ones.data(), ops::Shape({B, 1})}},
                       {z, {z_h.data(), ops::Shape({B, kZ})}},
                       {x, {x_h.data(), ops::Shape({B, 64, 64, 3})}}},
                      {nullptr, &d_loss_val});
            for (int k = 0; k < 2; ++k) {
                graph.run({g_opti, g_loss},
                          {{logits1, {ones.data(), ops::Shape({B, 1})}}, {z, {z_h.data(), ops::Shape({B, kZ})}}},
                          {nullptr, &g_loss_val});
                if (k == 0) reinterpret_cast<dbl_t*>(gl_first.data)[it] = g_loss_val;
            }
            ms.push_back(now_ms() - t0);
            reinterpret_cast<dbl_t*>(dl.data)[it] = d_loss_val;
            reinterpret_cast<dbl_t*>(gl.data)[it] = g_loss_val;
        }
        out.add(dl);
        out.add(gl);
        for (auto v : g_vars) add_var(out, v);
        for (auto v : d_vars) add_var(out, v);
        out.add(gl_first);
    }
    out.save(out_path);

    std::printf("{\"mode\": \"%s\", \"batch\": %d, \"leaky\": %s, \"ms\": [", mode.c_str(), B, leaky ? "true" : "false");
    for (std::size_t i = 0; i < ms.size(); ++i) std::printf("%s%.3f", i ? ", " : "", ms[i]);
    std::printf("]}\n");
    graph.exit_graph();
    return 0;
}
