// Reference-side binding: the replacement for the reference's src/gpu/*.cu.
//
// The reference reaches its GPU backend through two symbols, gpu::kernels_list[512] (indexed by
// rt::Node::type, src/gpu/kernels.cu:20-64) and gpu::run(rt::NodesList&) (src/gpu/runner.cu:10-18,
// called by ops::Graph::run, src/ops/graph.cu:194-200).  This file defines both on top of the C ABI
// of libdcgan_b200.so; it is compiled against the reference's own headers (src/gpu/kernels.hh,
// src/gpu/runner.hh, src/runtime/node.hh, src/runtime/nodes-list.hh) and linked with the reference's
// unmodified src/{api,ops,runtime,memory,utils,cpu} objects in place of its src/gpu objects.
// RT_MODE=GPU then runs every runtime instruction on the B200 path.
//
// Environment: DCG_SHIM_PRECISION = tf32 (default) | fp32 | 3xtf32, DCG_SHIM_FUSE = 1 (default) | 0.
#include "gpu/kernels.hh"
#include "gpu/runner.hh"
#include "runtime/node.hh"
#include "runtime/nodes-list.hh"

#include <dcgan_b200.h>

#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace gpu
{

    namespace
    {

        int env_precision()
        {
            const char* v = std::getenv("DCG_SHIM_PRECISION");
            if (!v || !std::strcmp(v, "tf32")) return DCG_PREC_TF32;
            if (!std::strcmp(v, "fp32")) return DCG_PREC_FP32;
            if (!std::strcmp(v, "3xtf32")) return DCG_PREC_3XTF32;
            throw std::runtime_error(std::string("DCG_SHIM_PRECISION: unknown value ") + v);
        }

        int env_fuse()
        {
            const char* v = std::getenv("DCG_SHIM_FUSE");
            return (v && std::atoi(v) == 0) ? 0 : 1;
        }

        // One context per process, on the legacy default stream: the reference's tensor_write /
        // tensor_read are blocking cudaMemcpy calls on that stream (src/memory/copy.hxx:29-46), so
        // uploads, these launches and the read-back are ordered without any extra synchronisation.
        dcg_context* context()
        {
            static dcg_context* ctx = nullptr;
            if (!ctx && dcg_context_create(&ctx, env_precision(), nullptr, 0, nullptr) != DCG_OK)
                throw std::runtime_error(std::string("dcgan_b200: ") + dcg_last_error());
            return ctx;
        }

        // rt::Node -> dcg_node, field for field (src/runtime/node.hh:215-243).
        dcg_node translate(const rt::Node* n)
        {
            dcg_node d;
            std::memset(&d, 0, sizeof(d));
            d.type = n->type;
            d.in1 = n->in1; d.in2 = n->in2; d.in3 = n->in3;
            d.out1 = n->out1; d.out2 = n->out2;
            d.cons1 = n->cons1; d.cons2 = n->cons2; d.cons3 = n->cons3; d.cons4 = n->cons4;
            d.len1 = n->len1; d.len2 = n->len2; d.len3 = n->len3;
            for (int i = 0; i < 2; ++i) {
                d.intconst[i] = n->intconst[i];
                d.intconst2[i] = n->intconst2[i];
            }
            for (int i = 0; i < 4; ++i) {
                d.sizes1[i] = n->sizes1[i];
                d.sizes2[i] = n->sizes2[i];
                d.sizes3[i] = n->sizes3[i];
            }
            d.int_cons1 = n->int_cons1;
            d.int_cons2 = n->int_cons2;
            d.alpha_leaky = n->alpha_leaky;
            d.flags = 0;   // every node output stays observable, nothing leaves the main stream
            return d;
        }

        void check(int status)
        {
            if (status != DCG_OK) throw std::runtime_error(std::string("dcgan_b200: ") + dcg_last_error());
        }

        // One handler serves every slot of the table (the reference leaves slots 20 and 31 empty,
        // src/gpu/kernels.cu:44,55; the library implements those two as well).
        void dispatch(rt::Node* n)
        {
            const dcg_node d = translate(n);
            check(dcg_run_node(context(), &d));
        }

        struct FillTable
        {
            FillTable();
        };

    }

    kernel_f kernels_list[512];

    namespace
    {
        FillTable::FillTable()
        {
            for (int i = 0; i < 512; ++i) kernels_list[i] = nullptr;
            for (int i = 0; i < DCG_OP_COUNT; ++i) kernels_list[i] = dispatch;
            // The reference frees its device tensors from the destructor of a function-local static
            // (ops::Graph::instance(), src/ops/graph.cu:20-39, tensor_free throws on error,
            // src/memory/alloc.cu:28-37).  Its own GPU objects register device code before main, which
            // brings the CUDA runtime up - and queues its shutdown - before that static exists; without
            // them the runtime would start at the first cudaMalloc, shut down BEFORE the graph's
            // destructor, and every program would end in "driver shutting down".  Same order here:
            const char* mode = std::getenv("RT_MODE");
            if (mode && !std::strcmp(mode, "GPU")) cudaFree(nullptr);
        }
        FillTable fill_table;
    }

    // src/gpu/runner.cu:10-18 without the device synchronisation after every node: the list is
    // enqueued in order on one stream (adjacent conv / bias / activation nodes and Adam triples are
    // fused unless DCG_SHIM_FUSE=0), then the device is synchronised once and the tensor-path status
    // word is read, so a kernel that gave up on a bounded wait surfaces here as an exception.
    void run(rt::NodesList& tasks)
    {
        std::vector<dcg_node> list;
        list.reserve(tasks.nodes().size());
        for (auto n : tasks.nodes()) list.push_back(translate(n));
        static const int fuse = env_fuse();
        check(dcg_run_nodes(context(), list.data(), (int)list.size(), fuse));
        check(dcg_device_status());
    }

}
