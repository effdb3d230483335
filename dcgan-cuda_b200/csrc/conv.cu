// C-ABI entry points of the three convolution operators and the choice between
// the tcgen05 tensor path and the CUDA-core fp32 path.
#include "common.cuh"
#include "conv.cuh"

namespace dcg {

int conv_check_desc(const dcg_conv_desc* d, const char* who)
{
    DCG_CHECK_ARG(d, "%s: null descriptor", who);
    DCG_CHECK_ARG(d->n > 0 && d->h > 0 && d->w > 0 && d->c > 0, "%s: bad input shape [%d,%d,%d,%d]",
                  who, d->n, d->h, d->w, d->c);
    DCG_CHECK_ARG(d->kh > 0 && d->kw > 0 && d->o > 0, "%s: bad kernel shape [%d,%d,%d,%d]", who,
                  d->kh, d->kw, d->c, d->o);
    DCG_CHECK_ARG(d->ho > 0 && d->wo > 0, "%s: bad output shape [%d,%d]", who, d->ho, d->wo);
    DCG_CHECK_ARG(d->stride_h > 0 && d->stride_w > 0, "%s: bad strides", who);
    DCG_CHECK_ARG(d->pad_top >= 0 && d->pad_left >= 0 && d->pad_top < d->kh && d->pad_left < d->kw,
                  "%s: pad (%d,%d) outside the kernel", who, d->pad_top, d->pad_left);
    // the last output row/column must start inside the padded input
    DCG_CHECK_ARG((d->ho - 1) * d->stride_h - d->pad_top < d->h &&
                      (d->wo - 1) * d->stride_w - d->pad_left < d->w,
                  "%s: output [%d,%d] does not fit input [%d,%d]", who, d->ho, d->wo, d->h, d->w);
    return DCG_OK;
}

// The tensor path moves tiles with TMA and 128-bit epilogue accesses: every tensor it touches
// must start on a 16-byte boundary.
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static bool epilogue_aligned(const EpilogueArgs& e)
{
    return aligned16(e.raw_out) && aligned16(e.bias) && aligned16(e.pre_act) && aligned16(e.gate);
}

static int check_precision(int precision, const char* who)
{
    DCG_CHECK_ARG(precision == DCG_PREC_TF32 || precision == DCG_PREC_3XTF32 ||
                      precision == DCG_PREC_FP32,
                  "%s: unknown precision %d", who, precision);
    return DCG_OK;
}

}  // namespace dcg

using namespace dcg;

extern "C" size_t dcg_conv_workspace_bytes(const dcg_conv_desc* desc, int kind, int precision)
{
    if (!desc || precision == DCG_PREC_FP32) return 0;
    if (kind < kConvFwd || kind > kConvDk) return 0;
    const bool x3 = precision == DCG_PREC_3XTF32;
    if (!conv_tc_supported(*desc, kind, x3)) return 0;
    return conv_tc_workspace(*desc, kind, x3);
}

extern "C" int dcg_conv2d_fwd(const dcg_conv_desc* desc, const float* x, const float* k, float* y,
                              const dcg_epilogue* ep, int precision, void* workspace,
                              size_t workspace_bytes, dcg_stream_t stream)
{
    int st = conv_check_desc(desc, "dcg_conv2d_fwd");
    if (st) return st;
    if ((st = check_precision(precision, "dcg_conv2d_fwd"))) return st;
    DCG_CHECK_ARG(x && k && y, "dcg_conv2d_fwd: null tensor pointer");
    const EpilogueArgs e = make_epilogue(ep);
    const bool x3 = precision == DCG_PREC_3XTF32;
    if (precision != DCG_PREC_FP32 && conv_tc_supported(*desc, kConvFwd, x3) && aligned16(x) && aligned16(k) &&
        aligned16(y) && epilogue_aligned(e))
        return conv_tc_fwd(*desc, x, k, y, e, workspace, workspace_bytes, as_stream(stream), x3);
    return conv_fwd_generic(*desc, x, k, y, e, as_stream(stream));
}

extern "C" int dcg_conv2d_dx(const dcg_conv_desc* desc, const float* dy, const float* k, float* dx,
                             const dcg_epilogue* ep, int precision, void* workspace,
                             size_t workspace_bytes, dcg_stream_t stream)
{
    int st = conv_check_desc(desc, "dcg_conv2d_dx");
    if (st) return st;
    if ((st = check_precision(precision, "dcg_conv2d_dx"))) return st;
    DCG_CHECK_ARG(dy && k && dx, "dcg_conv2d_dx: null tensor pointer");
    const EpilogueArgs e = make_epilogue(ep);
    const bool x3 = precision == DCG_PREC_3XTF32;
    if (precision != DCG_PREC_FP32 && conv_tc_supported(*desc, kConvDx, x3) && aligned16(dy) && aligned16(k) &&
        aligned16(dx) && epilogue_aligned(e))
        return conv_tc_dx(*desc, dy, k, dx, e, workspace, workspace_bytes, as_stream(stream), x3);
    return conv_dx_generic(*desc, dy, k, dx, e, as_stream(stream));
}

extern "C" int dcg_conv2d_dk(const dcg_conv_desc* desc, const float* x, const float* dy, float* dk,
                             int precision, void* workspace, size_t workspace_bytes,
                             dcg_stream_t stream)
{
    int st = conv_check_desc(desc, "dcg_conv2d_dk");
    if (st) return st;
    if ((st = check_precision(precision, "dcg_conv2d_dk"))) return st;
    DCG_CHECK_ARG(x && dy && dk, "dcg_conv2d_dk: null tensor pointer");
    const bool x3 = precision == DCG_PREC_3XTF32;
    if (precision != DCG_PREC_FP32 && conv_tc_supported(*desc, kConvDk, x3) && aligned16(x) && aligned16(dy) &&
        aligned16(dk))
        return conv_tc_dk(*desc, x, dy, dk, workspace, workspace_bytes, as_stream(stream), x3);
    return conv_dk_generic(*desc, x, dy, dk, as_stream(stream));
}
