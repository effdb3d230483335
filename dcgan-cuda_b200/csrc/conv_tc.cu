// placeholder until the tcgen05 kernels land
#include "common.cuh"
#include "conv.cuh"
namespace dcg {
bool conv_tc_supported(const dcg_conv_desc&, int) { return false; }
size_t conv_tc_workspace(const dcg_conv_desc&, int) { return 0; }
int conv_tc_fwd(const dcg_conv_desc&, const float*, const float*, float*, const EpilogueArgs&, void*, size_t, cudaStream_t) { return fail(DCG_ERR_UNSUPPORTED, "tensor path not built"); }
int conv_tc_dx(const dcg_conv_desc&, const float*, const float*, float*, const EpilogueArgs&, void*, size_t, cudaStream_t) { return fail(DCG_ERR_UNSUPPORTED, "tensor path not built"); }
int conv_tc_dk(const dcg_conv_desc&, const float*, const float*, float*, void*, size_t, cudaStream_t) { return fail(DCG_ERR_UNSUPPORTED, "tensor path not built"); }
}
