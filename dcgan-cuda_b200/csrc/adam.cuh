// Internal entry of the fused multi-tensor Adam launch (see adam.cu).
#pragma once
#include <cuda_runtime.h>

#include "dcgan_b200.h"

namespace dcg {
// m = a1*m + b1*g';  v = a2*v + b2*g'*g';  p -= lr_t*m/(sqrt(v)+eps), g' = scale*(g [+ g2]).
// The (a, b) pairs are passed separately because the node-level backend gets
// them as the cons1/cons2 fields of the two moment nodes.
// lr_t_dev != nullptr: the kernel reads the step size from that device scalar instead of lr_t.
int adam_multi_launch(const dcg_adam_tensor* tensors, int count, float lr_t, float a1, float b1,
                      float a2, float b2, float eps, float grad_scale, cudaStream_t stream,
                      const float* lr_t_dev = nullptr);
// out = a*out + b*dv (squared: b*dv*dv) and out -= lr_t*m/(sqrt(v)+eps): the reference's
// three separate node kernels.
int moment_update_launch(const float* dv, float* out, float a, float b, size_t n, bool squared,
                         cudaStream_t stream);
int adam_apply_launch(const float* m, const float* v, float* out, float lr_t, float eps, size_t n,
                      cudaStream_t stream);
}  // namespace dcg
