"""numpy front-end of the CPU oracle (test infrastructure only).

Two back-ends with one Python interface:

* ``port()``      - oracle/dcgan_oracle.c, the plain-C restatement.
* ``reference()`` - the reference's own CPU code (src/cpu/ops.hxx) compiled
  from its sources into oracle/_ref/; ``None`` when that library was never
  built on this machine.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may
import this package.  The product library never does.

All arrays are C-contiguous float32; activations NHWC, conv2d kernels HWIO,
conv2d_transpose kernels [kh, kw, Cout, Cin].
"""
import ctypes
import os

import numpy as np

from . import build_oracle

_f32p = ctypes.POINTER(ctypes.c_float)
_i32p = ctypes.POINTER(ctypes.c_int)


def _fp(a):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"], (a.dtype, a.flags)
    return a.ctypes.data_as(_f32p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _ints(*v):
    return (ctypes.c_int * len(v))(*[int(x) for x in v])


def same_pad(in_size, k_size, stride):
    """Total SAME pad along one axis, as ops::Conv2D computes it
    (src/ops/conv2d.cu:33-41)."""
    if in_size % stride == 0:
        return max(k_size - stride, 0)
    return max(k_size - (in_size % stride), 0)


class _Base:
    prefix = None

    def __init__(self, path):
        self.path = path
        self.lib = ctypes.CDLL(path)
        L, p = self.lib, self.prefix
        getattr(L, p + "sigmoid_cross_entropy").restype = ctypes.c_float
        getattr(L, p + "mse").restype = ctypes.c_float
        getattr(L, p + "argmax_acc").restype = ctypes.c_float
        getattr(L, p + "adam_lr_t").restype = ctypes.c_float
        getattr(L, p + "xorshift_next_f32").restype = ctypes.c_float
        getattr(L, p + "xorshift_next_u64").restype = ctypes.c_uint64

    def _f(self, name):
        return getattr(self.lib, self.prefix + name)

    # ---- seeded generator (src/utils/xorshift.cu) -------------------------
    def xorshift_seed(self, s):
        self._f("xorshift_seed")(ctypes.c_uint64(s))

    def xorshift_next_u64(self):
        return int(self._f("xorshift_next_u64")())

    def xorshift_next_f32(self):
        return float(self._f("xorshift_next_f32")())

    def xorshift_fill(self, shape):
        out = np.empty(shape, dtype=np.float32)
        self._f("xorshift_fill")(_fp(out), ctypes.c_size_t(out.size))
        return out

    # ---- matrices ---------------------------------------------------------
    def _mat3(self, name, a, b, m, n, p):
        a, b = _f32(a), _f32(b)
        out = np.empty((m, p), dtype=np.float32)
        self._f(name)(_fp(a), _fp(b), _fp(out), ctypes.c_size_t(m),
                      ctypes.c_size_t(n), ctypes.c_size_t(p))
        return out

    def mm_mul(self, a, b):
        return self._mat3("mm_mul", a, b, a.shape[0], a.shape[1], b.shape[1])

    def tmm_mul(self, a, b):
        """a^T b with a [n, m], b [n, p]."""
        return self._mat3("tmm_mul", a, b, a.shape[1], a.shape[0], b.shape[1])

    def mtm_mul(self, a, b):
        """a b^T with a [m, n], b [p, n]."""
        return self._mat3("mtm_mul", a, b, a.shape[0], a.shape[1], b.shape[0])

    def mat_mul_add(self, x, w, b):
        x, w, b = _f32(x), _f32(w), _f32(b)
        m, n = x.shape
        p = w.shape[1]
        out = np.empty((m, p), dtype=np.float32)
        self._f("mat_mul_add")(_fp(x), _fp(w), _fp(b), _fp(out), ctypes.c_size_t(m),
                               ctypes.c_size_t(n), ctypes.c_size_t(p))
        return out

    def mvrow_add(self, a, b):
        a, b = _f32(a), _f32(b)
        n = a.shape[-1]
        m = a.size // n
        out = np.empty_like(a)
        self._f("mvrow_add")(_fp(a), _fp(b), _fp(out), ctypes.c_size_t(m), ctypes.c_size_t(n))
        return out

    def mat_sum_cols(self, a):
        a = _f32(a)
        n = a.shape[-1]
        m = a.size // n
        out = np.empty((n,), dtype=np.float32)
        self._f("mat_sum_cols")(_fp(a), _fp(out), ctypes.c_size_t(m), ctypes.c_size_t(n))
        return out

    def mat_sum_rows(self, a):
        a = _f32(a)
        m, n = a.shape
        out = np.empty((m,), dtype=np.float32)
        self._f("mat_sum_rows")(_fp(a), _fp(out), ctypes.c_size_t(m), ctypes.c_size_t(n))
        return out

    # ---- elementwise ------------------------------------------------------
    def _unary(self, name, a, *extra):
        a = _f32(a)
        out = np.empty_like(a)
        self._f(name)(_fp(a), _fp(out), ctypes.c_size_t(a.size), *extra)
        return out

    def vect_sigmoid(self, a):
        return self._unary("vect_sigmoid", a)

    def vect_relu(self, a):
        return self._unary("vect_relu", a)

    def vect_relu_leaky(self, a, alpha=0.2):
        return self._unary("vect_relu_leaky", a, ctypes.c_float(alpha))

    def vect_tanh(self, a):
        return self._unary("vect_tanh", a)

    def _binary(self, name, a, b, *mid):
        a, b = _f32(a), _f32(b)
        out = np.empty_like(a)
        self._f(name)(_fp(a), _fp(b), _fp(out), *mid, ctypes.c_size_t(a.size))
        return out

    def relu_grad(self, z, dout):
        return self._binary("relu_grad", z, dout)

    def leaky_relu_grad(self, z, dout, alpha=0.2):
        return self._binary("leaky_relu_grad", z, dout, ctypes.c_float(alpha))

    def tanh_grad(self, tanh_out, dout):
        return self._binary("tanh_grad", tanh_out, dout)

    def sigmoid_grad(self, sig_out, dout):
        return self._binary("sigmoid_grad", sig_out, dout)

    def vect_add(self, a, b):
        return self._binary("vect_add", a, b)

    def vect_update(self, dv, out, coeff):
        dv = _f32(dv)
        out = _f32(out).copy()
        self._f("vect_update")(_fp(dv), _fp(out), ctypes.c_float(coeff), ctypes.c_size_t(dv.size))
        return out

    # ---- losses -----------------------------------------------------------
    def sigmoid_cross_entropy(self, y, logits):
        y, logits = _f32(y), _f32(logits)
        return np.float32(self._f("sigmoid_cross_entropy")(_fp(y), _fp(logits),
                                                           ctypes.c_size_t(y.size)))

    def sigmoid_cross_entropy_grad(self, y, logits):
        return self._binary("sigmoid_cross_entropy_grad", y, logits)

    def mse(self, y, y_hat):
        y, y_hat = _f32(y), _f32(y_hat)
        m, n = y.shape
        return np.float32(self._f("mse")(_fp(y), _fp(y_hat), ctypes.c_size_t(m), ctypes.c_size_t(n)))

    def mse_grad(self, y, y_hat):
        return self._binary("mse_grad", y, y_hat)

    def argmax_acc(self, y, y_hat):
        y, y_hat = _f32(y), _f32(y_hat)
        m, n = y.shape
        return np.float32(self._f("argmax_acc")(_fp(y), _fp(y_hat), ctypes.c_size_t(m),
                                                ctypes.c_size_t(n)))

    # ---- Adam (src/cpu/kernels.cu:183-206) --------------------------------
    def adam_step(self, p, g, m, v, t, lr, beta1, beta2, eps):
        """One reference Adam update of one variable: the moment_update,
        moment_update2 and adam_update nodes in graph order.  Returns new
        (p, m, v, t, lr_t)."""
        p, g = _f32(p).copy(), _f32(g)
        m, v = _f32(m).copy(), _f32(v).copy()
        n = ctypes.c_size_t(p.size)
        self._f("moment_update")(_fp(g), _fp(m), ctypes.c_float(beta1),
                                 ctypes.c_float(np.float32(1) - np.float32(beta1)), n)
        self._f("moment_update2")(_fp(g), _fp(v), ctypes.c_float(beta2),
                                  ctypes.c_float(np.float32(1) - np.float32(beta2)), n)
        tt = ctypes.c_float(t)
        lrt = self._f("adam_lr_t")(ctypes.byref(tt), ctypes.c_float(lr), ctypes.c_float(beta1),
                                   ctypes.c_float(beta2))
        self._f("adam_update")(_fp(m), _fp(v), _fp(p), ctypes.c_float(lrt), ctypes.c_float(eps), n)
        return p, m, v, tt.value, np.float32(lrt)


class Port(_Base):
    """oracle/dcgan_oracle.c"""
    prefix = "orc_"

    def conv2d_out_size(self, H, W, KH, KW, sh, sw, pad_h, pad_w, valid):
        ho, wo = ctypes.c_int(), ctypes.c_int()
        self.lib.orc_conv2d_out_size(H, W, KH, KW, sh, sw, pad_h, pad_w, int(valid),
                                     ctypes.byref(ho), ctypes.byref(wo))
        return ho.value, wo.value

    def conv2d(self, x, k, strides=(2, 2), pad=None, valid=False):
        x, k = _f32(x), _f32(k)
        N, H, W, C = x.shape
        KH, KW, C2, O = k.shape
        assert C == C2
        if pad is None:
            pad = (same_pad(H, KH, strides[0]), same_pad(W, KW, strides[1]))
        Ho, Wo = self.conv2d_out_size(H, W, KH, KW, strides[0], strides[1], pad[0], pad[1], valid)
        y = np.empty((N, Ho, Wo, O), dtype=np.float32)
        self.lib.orc_conv2d(_fp(x), _fp(k), _fp(y), N, H, W, C, KH, KW, O,
                            strides[0], strides[1], pad[0], pad[1], int(valid))
        return y

    def conv2d_input_grad(self, dy, k, stride, in_hw):
        dy, k = _f32(dy), _f32(k)
        in_hw = (int(in_hw[0]), int(in_hw[1]))
        N, Ho, Wo, O = dy.shape
        KH, KW, C, O2 = k.shape
        assert O == O2
        dx = np.empty((N, in_hw[0], in_hw[1], C), dtype=np.float32)
        self.lib.orc_conv2d_input_grad(_fp(dy), _fp(k), stride, N, Ho, Wo, O, KH, KW, C,
                                       _fp(dx), in_hw[0], in_hw[1])
        return dx

    def conv2d_kernel_grad(self, dy, x, stride, pad_hw):
        dy, x = _f32(dy), _f32(x)
        pad_hw = (int(pad_hw[0]), int(pad_hw[1]))
        N, Ho, Wo, O = dy.shape
        N2, H, W, C = x.shape
        assert N == N2
        kh, kw = ctypes.c_int(), ctypes.c_int()
        self.lib.orc_conv2d_kernel_grad_size(H, W, Ho, Wo, stride, pad_hw[0], pad_hw[1],
                                             ctypes.byref(kh), ctypes.byref(kw))
        dk = np.empty((kh.value, kw.value, C, O), dtype=np.float32)
        self.lib.orc_conv2d_kernel_grad(_fp(dy), _fp(x), stride, N, Ho, Wo, O, H, W, C,
                                        _fp(dk), pad_hw[0], pad_hw[1])
        return dk

    def conv2d_transpose(self, x, k, out_size, stride):
        x, k = _f32(x), _f32(k)
        N, Hx, Wx, Cx = x.shape
        KH, KW, Cy, Cx2 = k.shape
        assert Cx == Cx2 and out_size[3] == Cy and out_size[0] == N
        y = np.empty(tuple(out_size), dtype=np.float32)
        self.lib.orc_conv2d_transpose(_fp(x), _fp(k), stride, N, Hx, Wx, Cx, KH, KW, Cy,
                                      _fp(y), out_size[1], out_size[2])
        return y

    def conv2d_transpose_input_grad(self, dy, k, stride, in_hw):
        dy, k = _f32(dy), _f32(k)
        N, Hy, Wy, Cy = dy.shape
        KH, KW, Cy2, Cx = k.shape
        assert Cy == Cy2
        dx = np.empty((N, in_hw[0], in_hw[1], Cx), dtype=np.float32)
        self.lib.orc_conv2d_transpose_input_grad(_fp(dy), _fp(k), stride, N, Hy, Wy, Cy,
                                                 KH, KW, Cx, _fp(dx), in_hw[0], in_hw[1])
        return dx

    def conv2d_transpose_kernel_grad(self, dy, x, stride, k_hw):
        dy, x = _f32(dy), _f32(x)
        N, Hy, Wy, Cy = dy.shape
        N2, Hx, Wx, Cx = x.shape
        assert N == N2
        dk = np.empty((k_hw[0], k_hw[1], Cy, Cx), dtype=np.float32)
        self.lib.orc_conv2d_transpose_kernel_grad(_fp(dy), _fp(x), stride, N, Hy, Wy, Cy,
                                                  Hx, Wx, Cx, _fp(dk), k_hw[0], k_hw[1])
        return dk


class Reference(_Base):
    """The reference's own CPU math, compiled from its sources (oracle/_ref/).

    conv2d_transpose_input_grad / conv2d_transpose_kernel_grad follow
    src/cpu/ops.hxx:808-902, which run with zero padding: they are only the
    adjoint of conv2d_transpose when (Hx-1)*stride + KH == Hy, and the callers
    here assert exactly that."""
    prefix = "ref_"

    def conv2d(self, x, k, strides=(2, 2), pad=None, valid=False):
        x, k = _f32(x), _f32(k)
        N, H, W, C = x.shape
        KH, KW, C2, O = k.shape
        assert C == C2
        if pad is None:
            pad = (same_pad(H, KH, strides[0]), same_pad(W, KW, strides[1]))
        if valid:
            Ho = (H + pad[0] - KH) // strides[0] + 1
            Wo = (W + pad[1] - KW) // strides[1] + 1
        else:
            Ho = -(-H // strides[0])
            Wo = -(-W // strides[1])
        y = np.empty((N, Ho, Wo, O), dtype=np.float32)
        self.lib.ref_conv2d(_fp(x), _fp(k), _fp(y), _ints(*strides), pad[0], pad[1],
                            _ints(*x.shape), _ints(*k.shape), int(valid))
        return y

    def conv2d_input_grad(self, dy, k, stride, in_hw):
        dy, k = _f32(dy), _f32(k)
        dx = np.empty((dy.shape[0], in_hw[0], in_hw[1], k.shape[2]), dtype=np.float32)
        self.lib.ref_conv2d_input_grad(_fp(dy), _fp(k), stride, _ints(*dy.shape),
                                       _ints(*k.shape), _fp(dx), _ints(*in_hw))
        return dx

    def conv2d_kernel_grad(self, dy, x, stride, pad_hw):
        dy, x = _f32(dy), _f32(x)
        sH = stride * (dy.shape[1] - 1) + 1
        sW = stride * (dy.shape[2] - 1) + 1
        KH = x.shape[1] + pad_hw[0] - sH + 1
        KW = x.shape[2] + pad_hw[1] - sW + 1
        dk = np.empty((KH, KW, x.shape[3], dy.shape[3]), dtype=np.float32)
        self.lib.ref_conv2d_kernel_grad(_fp(dy), _fp(x), stride, _ints(*dy.shape),
                                        _ints(*x.shape), _fp(dk), _ints(*pad_hw))
        return dk

    def conv2d_transpose(self, x, k, out_size, stride):
        x, k = _f32(x), _f32(k)
        y = np.empty(tuple(out_size), dtype=np.float32)
        self.lib.ref_conv2d_transpose(_fp(x), _fp(k), _ints(*out_size), stride, _fp(y),
                                      _ints(*x.shape), _ints(*k.shape))
        return y

    def conv2d_transpose_input_grad(self, dy, k, stride, in_hw):
        dy, k = _f32(dy), _f32(k)
        assert (in_hw[0] - 1) * stride + k.shape[0] == dy.shape[1], "reference CPU path is zero-pad only"
        assert (in_hw[1] - 1) * stride + k.shape[1] == dy.shape[2], "reference CPU path is zero-pad only"
        dx = np.empty((dy.shape[0], in_hw[0], in_hw[1], k.shape[3]), dtype=np.float32)
        self.lib.ref_conv2d_transpose_input_grad(_fp(dy), _fp(k), stride, _ints(*dy.shape),
                                                 _ints(*k.shape), _fp(dx), _ints(*in_hw))
        return dx

    def conv2d_transpose_kernel_grad(self, dy, x, stride, k_hw):
        dy, x = _f32(dy), _f32(x)
        assert (x.shape[1] - 1) * stride + k_hw[0] == dy.shape[1], "reference CPU path is zero-pad only"
        assert (x.shape[2] - 1) * stride + k_hw[1] == dy.shape[2], "reference CPU path is zero-pad only"
        dk = np.empty((k_hw[0], k_hw[1], dy.shape[3], x.shape[3]), dtype=np.float32)
        self.lib.ref_conv2d_transpose_kernel_grad(_fp(dy), _fp(x), stride, _ints(*dy.shape),
                                                  _ints(*x.shape), _fp(dk))
        return dk


_port = None
_ref = None
_ref_tried = False


def port():
    global _port
    if _port is None:
        _port = Port(build_oracle.build_port())
    return _port


def reference():
    """The reference-compiled back-end, or None when it is not available."""
    global _ref, _ref_tried
    if not _ref_tried:
        _ref_tried = True
        path = build_oracle.build_ref()
        if path is not None and os.path.exists(path):
            _ref = Reference(path)
    return _ref
