// Internal interface of the node backend's profiling mode (see backend.cu).
#pragma once
#include "dcgan_b200.h"

namespace dcg {

// RAII timer: when the context is profiling, records a CUDA event on the context's stream at
// construction and another at destruction, and files the pair under `name` with `flops` of
// algorithmic work.  A no-op otherwise.
struct ProfScope {
    ProfScope(dcg_context* ctx, const char* name, double flops);
    ~ProfScope();
    ProfScope(const ProfScope&) = delete;
    ProfScope& operator=(const ProfScope&) = delete;
    dcg_context* ctx;
    bool active;
};

}  // namespace dcg

namespace dcg {
// For the trainer: whether the context is in profiling mode, and a counter that advances whenever
// something a captured CUDA graph bakes in has changed (a scratch buffer of the main or a side
// stream was reallocated, the precision was switched): a graph captured under another value is stale.
bool context_is_profiling(const dcg_context* ctx);
uint64_t context_generation(const dcg_context* ctx);
}  // namespace dcg
