// Internal interfaces between the convolution translation units.
#pragma once
#include <cuda_runtime.h>

#include "common.cuh"

namespace dcg {

enum ConvKind { kConvFwd = 0, kConvDx = 1, kConvDk = 2 };

// CUDA-core fp32 kernels, any shape (conv_generic.cu).
int conv_fwd_generic(const dcg_conv_desc& d, const float* x, const float* k, float* y,
                     const EpilogueArgs& ep, cudaStream_t stream);
int conv_dx_generic(const dcg_conv_desc& d, const float* dy, const float* k, float* dx,
                    const EpilogueArgs& ep, cudaStream_t stream);
int conv_dk_generic(const dcg_conv_desc& d, const float* x, const float* dy, float* dk,
                    cudaStream_t stream);

// tcgen05 TF32 implicit-GEMM kernels (conv_tc.cu); x3 selects the 3xTF32 variant (operand = TF32 part +
// residual, three MMAs per K step).  *_supported tells whether the
// tensor path takes the shape; *_workspace its scratch need in bytes.
bool conv_tc_supported(const dcg_conv_desc& d, int kind, bool x3 = false);
size_t conv_tc_workspace(const dcg_conv_desc& d, int kind, bool x3 = false);
int conv_tc_fwd(const dcg_conv_desc& d, const float* x, const float* k, float* y,
                const EpilogueArgs& ep, void* ws, size_t ws_bytes, cudaStream_t stream, bool x3 = false);
int conv_tc_dx(const dcg_conv_desc& d, const float* dy, const float* k, float* dx,
               const EpilogueArgs& ep, void* ws, size_t ws_bytes, cudaStream_t stream, bool x3 = false);
int conv_tc_dk(const dcg_conv_desc& d, const float* x, const float* dy, float* dk,
               void* ws, size_t ws_bytes, cudaStream_t stream, bool x3 = false);

// Testing hooks of the tensor path.  wait_cycles: > 0 sets the limit of every barrier wait (SM clocks),
// -1 restores the default, 0 leaves it; skip_stage: pipeline stage the producer leaves out (-1: none,
// -2: leave as is).
void conv_tc_set_hooks(long long wait_cycles, int skip_stage);
// Input gradient with the parity classes of a tile in one CTA: 0 never, 1 where it pays (default), 2 wherever
// the shape allows, anything else: back to the default.
void conv_tc_set_dx_mode(int mode);
unsigned long long conv_tc_fused_dx_launches();   // launches of the class-fused kernel so far

// Shape validation shared by the entry points: 0 or a negative dcg_status.
int conv_check_desc(const dcg_conv_desc* d, const char* who);

}  // namespace dcg
