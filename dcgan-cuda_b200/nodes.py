"""Runtime-instruction records and their execution context.

The factories below mirror the reference's rt::Node::op_* factories
(src/runtime/node.cu:52-560): same names, same argument order, same field
packing, so a test can lower an operator exactly as the reference's
Op::compile() does (e.g. src/ops/conv2d.cu:44-77) and hand the record to the
backend.  Tensor arguments are torch CUDA tensors (fp32, contiguous); only their
device pointers enter the record.
"""
import ctypes

from . import _lib
from ._lib import Node, check, lib

OP = {
    "mat_mat_mul": 0, "mat_rvect_add": 1, "sigmoid": 2, "mse": 3, "softmax": 4, "log_softmax": 5,
    "softmax_cross_entropy": 6, "conv2d": 7, "relu": 8, "relu_leaky": 9, "tanh": 10, "mse_grad": 11,
    "sigmoid_grad": 12, "mat_mul_add": 13, "tmat_mat_mul": 14, "mat_tmat_mul": 15,
    "mat_sum_rows": 16, "mat_sum_cols": 17, "softmax_cross_entropy_grad": 18, "relu_grad": 19,
    "conv2d_bias_add": 20, "update": 21, "sigmoid_cross_entropy": 22,
    "sigmoid_cross_entropy_grad": 23, "conv2d_input_grad": 24, "conv2d_kernel_grad": 25,
    "argmax_acc": 26, "moment_update": 27, "moment_update2": 28, "adam_update": 29,
    "leaky_relu_grad": 30, "conv2d_bias_add_grad": 31, "tanh_grad": 32, "conv2d_transpose": 33,
    "conv2d_transpose_input_grad": 34, "conv2d_transpose_kernel_grad": 35, "add": 36,
}


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, int):
        return t
    assert t.is_cuda and t.is_contiguous() and str(t.dtype) == "torch.float32", \
        "node operands are contiguous fp32 CUDA tensors"
    return t.data_ptr()


def _node(kind, **kw):
    n = Node()
    n.type = OP[kind]
    for k, v in kw.items():
        if k in ("intconst", "intconst2", "sizes1", "sizes2", "sizes3"):
            arr = getattr(n, k)
            for i, x in enumerate(v):
                arr[i] = int(x)
        elif k in ("in1", "in2", "in3", "out1"):
            setattr(n, k, _ptr(v))
        else:
            setattr(n, k, v)
    return n


# ---- convolutions (src/runtime/node.cu:112-291) ------------------------------
def op_conv2d(input, kernel, strides, pad_top, pad_left, output, input_size, kernel_size):
    """pad_top / pad_left carry the TOTAL pad along height / width, as
    ops::Conv2D::compile passes them (src/ops/conv2d.cu:73-76)."""
    return _node("conv2d", in1=input, in2=kernel, out1=output, intconst=strides,
                 int_cons1=pad_top, int_cons2=pad_left, sizes1=input_size, sizes2=kernel_size)


def op_conv2d_bias_add(z, bias, output, input_size):
    return _node("conv2d_bias_add", in1=z, in2=bias, out1=output, sizes1=input_size)


def op_conv2d_bias_add_grad(z, size, output):
    return _node("conv2d_bias_add_grad", in1=z, out1=output, sizes1=size)


def op_conv2d_input_grad(y, kernel, strides, output, y_size, kernel_size, input_size):
    return _node("conv2d_input_grad", in1=y, in2=kernel, out1=output, intconst=strides,
                 intconst2=(input_size[1], input_size[2]), sizes1=y_size, sizes2=kernel_size)


def op_conv2d_kernel_grad(y, input, strides, output, y_size, input_size, padded_size):
    return _node("conv2d_kernel_grad", in1=y, in2=input, out1=output, intconst=strides,
                 intconst2=padded_size, sizes1=y_size, sizes2=input_size)


def op_conv2d_transpose(input, kernel, out_size, strides, output, input_size, kernel_size):
    return _node("conv2d_transpose", in1=input, in2=kernel, out1=output, sizes1=out_size,
                 intconst=strides, sizes2=input_size, sizes3=kernel_size)


def op_conv2d_transpose_input_grad(y, kernel, strides, output, y_size, kernel_size, input_size):
    return _node("conv2d_transpose_input_grad", in1=y, in2=kernel, out1=output, intconst=strides,
                 intconst2=(input_size[1], input_size[2]), sizes1=y_size, sizes2=kernel_size)


def op_conv2d_transpose_kernel_grad(y, input, strides, output, y_size, input_size, kernel_size):
    return _node("conv2d_transpose_kernel_grad", in1=y, in2=input, out1=output, intconst=strides,
                 sizes1=y_size, sizes2=input_size, sizes3=kernel_size)


# ---- matrices ----------------------------------------------------------------
def op_mat_mat_mul(left, right, output, rowsl, colsl, colsr):
    return _node("mat_mat_mul", in1=left, in2=right, out1=output, len1=rowsl, len2=colsl, len3=colsr)


def op_mat_rvect_add(left, right, output, rows, cols):
    return _node("mat_rvect_add", in1=left, in2=right, out1=output, len1=rows, len2=cols)


def op_mat_mul_add(x, w, b, output, rowsx, colsx, colsw):
    return _node("mat_mul_add", in1=x, in2=w, in3=b, out1=output, len1=rowsx, len2=colsx, len3=colsw)


def op_tmat_mat_mul(left, right, output, rowsl, colsl, colsr):
    return _node("tmat_mat_mul", in1=left, in2=right, out1=output, len1=rowsl, len2=colsl, len3=colsr)


def op_mat_tmat_mul(left, right, output, rowsl, colsl, colsr):
    return _node("mat_tmat_mul", in1=left, in2=right, out1=output, len1=rowsl, len2=colsl, len3=colsr)


def op_mat_sum_rows(arg, out, rows, cols):
    return _node("mat_sum_rows", in1=arg, out1=out, len1=rows, len2=cols)


def op_mat_sum_cols(arg, out, rows, cols):
    return _node("mat_sum_cols", in1=arg, out1=out, len1=rows, len2=cols)


# ---- activations and their gradients -----------------------------------------
def op_relu(args, out, len):
    return _node("relu", in1=args, out1=out, len1=len)


def op_relu_leaky(args, out, len, alpha):
    return _node("relu_leaky", in1=args, out1=out, len1=len, alpha_leaky=alpha)


def op_sigmoid(args, out, len):
    return _node("sigmoid", in1=args, out1=out, len1=len)


def op_tanh(args, out, len):
    return _node("tanh", in1=args, out1=out, len1=len)


def op_relu_grad(z, dout, out, len):
    return _node("relu_grad", in1=z, in2=dout, out1=out, len1=len)


def op_leaky_relu_grad(z, dout, out, alpha, len):
    return _node("leaky_relu_grad", in1=z, in2=dout, out1=out, cons1=alpha, len1=len)


def op_tanh_grad(tanh_out, dout, out, len):
    return _node("tanh_grad", in1=tanh_out, in2=dout, out1=out, len1=len)


def op_sigmoid_grad(sig_out, dout, out, len):
    return _node("sigmoid_grad", in1=sig_out, in2=dout, out1=out, len1=len)


# ---- losses --------------------------------------------------------------------
def op_mse(y, y_hat, out, rows, cols):
    return _node("mse", in1=y, in2=y_hat, out1=out, len1=rows, len2=cols)


def op_mse_grad(y, y_hat, out, len):
    return _node("mse_grad", in1=y, in2=y_hat, out1=out, len1=len)


def op_softmax(args, out, rows, cols):
    return _node("softmax", in1=args, out1=out, len1=rows, len2=cols)


def op_log_softmax(args, out, rows, cols):
    return _node("log_softmax", in1=args, out1=out, len1=rows, len2=cols)


def op_softmax_cross_entropy(y, logits, out, rows, cols):
    return _node("softmax_cross_entropy", in1=y, in2=logits, out1=out, len1=rows, len2=cols)


def op_softmax_cross_entropy_grad(y, logits, out, rows, cols):
    return _node("softmax_cross_entropy_grad", in1=y, in2=logits, out1=out, len1=rows, len2=cols)


def op_sigmoid_cross_entropy(y, logits, out, len):
    return _node("sigmoid_cross_entropy", in1=y, in2=logits, out1=out, len1=len)


def op_sigmoid_cross_entropy_grad(y, logits, out, len):
    return _node("sigmoid_cross_entropy_grad", in1=y, in2=logits, out1=out, len1=len)


def op_argmax_acc(y, y_hat, out, rows, cols):
    return _node("argmax_acc", in1=y, in2=y_hat, out1=out, len1=rows, len2=cols)


# ---- updates -------------------------------------------------------------------
def op_update(var, dt, coeff, len):
    return _node("update", in1=dt, in2=coeff, out1=var, len1=len)


def op_moment_update(var, dt, coeff1, coeff2, len):
    return _node("moment_update", in1=dt, out1=var, cons1=coeff1, cons2=coeff2, len1=len)


def op_moment_update2(var, dt, coeff1, coeff2, len):
    return _node("moment_update2", in1=dt, out1=var, cons1=coeff1, cons2=coeff2, len1=len)


def op_adam_update(var, t, m, v, lr, beta1, beta2, eps, len):
    """`t` is a ctypes.c_float living on the host: the per-variable step counter
    the reference keeps in the AdamUpdate op (src/ops/adam-update.hh:32)."""
    n = _node("adam_update", in1=m, in2=v, out1=var, cons1=lr, cons2=beta1, cons3=beta2,
              cons4=eps, len1=len)
    n.out2 = ctypes.cast(ctypes.pointer(t), ctypes.c_void_p)
    n._keepalive = t
    return n


def op_add(a, b, out, len):
    return _node("add", in1=a, in2=b, out1=out, len1=len)


class Context:
    """Execution context of the node backend (dcg_context): a stream, a
    precision and scratch memory the backend owns and grows on demand."""

    def __init__(self, precision=_lib.PREC_TF32, stream=None):
        self._h = ctypes.c_void_p()
        check(lib.dcg_context_create(ctypes.byref(self._h), precision, None, 0, stream))

    def set_precision(self, precision):
        check(lib.dcg_context_set_precision(self._h, precision))

    def launch_count(self):
        return int(lib.dcg_context_launch_count(self._h))

    def run_node(self, node):
        check(lib.dcg_run_node(self._h, ctypes.byref(node)))

    def run(self, nodes, fuse=False):
        """gpu::run over a list of nodes (src/gpu/runner.cu:10-18)."""
        arr = (Node * len(nodes))(*nodes)
        check(lib.dcg_run_nodes(self._h, arr, len(nodes), 1 if fuse else 0))

    def close(self):
        if self._h:
            lib.dcg_context_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
