"""Direct calls into the C-ABI operators on torch CUDA tensors.

torch is used for device memory and streams only; all arithmetic happens in
libdcgan_b200.so.  Shapes follow the reference: activations NHWC, conv2d kernels
HWIO, conv2d_transpose kernels [kh, kw, Cout, Cin].
"""
import ctypes

import torch

from . import _lib
from ._lib import AdamTensor, ConvDesc, Epilogue, check, lib


def same_pad(in_size, k_size, stride):
    """Total SAME pad along one axis (src/ops/conv2d.cu:33-41)."""
    if in_size % stride == 0:
        return max(k_size - stride, 0)
    return max(k_size - (in_size % stride), 0)


def _p(t):
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous() and t.dtype == torch.float32
    return t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def conv_desc(x_shape, k_shape, strides=(2, 2), pad=None, out_hw=None):
    """Descriptor of y = conv2d(x, k).  `pad` is the TOTAL (height, width) pad,
    SAME by default; out_hw defaults to (in + pad - k)//stride + 1."""
    n, h, w, c = x_shape
    kh, kw, c2, o = k_shape
    assert c == c2, "kernel input channels %d != activation channels %d" % (c2, c)
    if pad is None:
        pad = (same_pad(h, kh, strides[0]), same_pad(w, kw, strides[1]))
    if out_hw is None:
        out_hw = ((h + pad[0] - kh) // strides[0] + 1, (w + pad[1] - kw) // strides[1] + 1)
    return ConvDesc(n, h, w, c, kh, kw, o, out_hw[0], out_hw[1], strides[0], strides[1],
                    pad[0] // 2, pad[1] // 2)


def make_epilogue(bias=None, act=_lib.ACT_NONE, alpha=0.2, pre_act=None, raw_out=None, gate=None,
                  gate_act=_lib.ACT_NONE, gate_alpha=0.2):
    return Epilogue(_p(raw_out), _p(bias), _p(pre_act), act, alpha, _p(gate), gate_act, gate_alpha)


class Workspace:
    """A grow-only scratch buffer handed to the conv entry points."""

    def __init__(self, device="cuda"):
        self.device = device
        self.buf = None

    def get(self, nbytes):
        if nbytes == 0:
            return None, 0
        if self.buf is None or self.buf.numel() < nbytes:
            self.buf = torch.empty(int(nbytes * 1.25) + 256, dtype=torch.uint8, device=self.device)
        return self.buf.data_ptr(), self.buf.numel()


_ws = {}


def _workspace(dev):
    if dev not in _ws:
        _ws[dev] = Workspace(dev)
    return _ws[dev]


def conv2d_fwd(x, k, strides=(2, 2), pad=None, out_hw=None, epilogue=None, precision=_lib.PREC_TF32,
               out=None):
    d = conv_desc(x.shape, k.shape, strides, pad, out_hw)
    if out is None:
        out = torch.empty((d.n, d.ho, d.wo, d.o), dtype=torch.float32, device=x.device)
    ws, nb = _workspace(x.device).get(lib.dcg_conv_workspace_bytes(ctypes.byref(d), _lib.KIND_FWD, precision))
    check(lib.dcg_conv2d_fwd(ctypes.byref(d), _p(x), _p(k), _p(out),
                             ctypes.byref(epilogue) if epilogue is not None else None, precision,
                             ws, nb, _stream()))
    return out


def conv2d_dx(dy, k, in_hw, strides=(2, 2), pad=None, epilogue=None, precision=_lib.PREC_TF32, out=None):
    """Input gradient of conv2d: dy [n, ho, wo, o], k [kh, kw, c, o] -> dx [n, h, w, c]."""
    n, ho, wo, o = dy.shape
    kh, kw, c, o2 = k.shape
    assert o == o2
    d = conv_desc((n, in_hw[0], in_hw[1], c), k.shape, strides, pad, (ho, wo))
    if out is None:
        out = torch.empty((n, in_hw[0], in_hw[1], c), dtype=torch.float32, device=dy.device)
    ws, nb = _workspace(dy.device).get(lib.dcg_conv_workspace_bytes(ctypes.byref(d), _lib.KIND_DX, precision))
    check(lib.dcg_conv2d_dx(ctypes.byref(d), _p(dy), _p(k), _p(out),
                            ctypes.byref(epilogue) if epilogue is not None else None, precision,
                            ws, nb, _stream()))
    return out


def conv2d_dk(x, dy, k_hw, strides=(2, 2), pad=None, precision=_lib.PREC_TF32, out=None):
    """Kernel gradient of conv2d: x [n, h, w, c], dy [n, ho, wo, o] -> dk [kh, kw, c, o]."""
    n, h, w, c = x.shape
    n2, ho, wo, o = dy.shape
    assert n == n2
    d = conv_desc(x.shape, (k_hw[0], k_hw[1], c, o), strides, pad, (ho, wo))
    if out is None:
        out = torch.empty((k_hw[0], k_hw[1], c, o), dtype=torch.float32, device=x.device)
    ws, nb = _workspace(x.device).get(lib.dcg_conv_workspace_bytes(ctypes.byref(d), _lib.KIND_DK, precision))
    check(lib.dcg_conv2d_dk(ctypes.byref(d), _p(x), _p(dy), _p(out), precision, ws, nb, _stream()))
    return out


def adam_multi(params, grads, ms, vs, lr_t, beta1, beta2, eps, grad_scale=1.0, grads2=None):
    """One fused launch over a list of variables (tensors updated in place)."""
    cnt = len(params)
    arr = (AdamTensor * cnt)()
    for i in range(cnt):
        arr[i] = AdamTensor(_p(params[i]), _p(grads[i]), _p(grads2[i]) if grads2 else None,
                            _p(ms[i]), _p(vs[i]), params[i].numel())
    check(lib.dcg_adam_multi(arr, cnt, lr_t, beta1, beta2, eps, grad_scale, _stream()))


def adam_lr_t(t, lr, beta1, beta2):
    """Advances the host step counter `t` (ctypes.c_float) and returns the
    reference's step size for it."""
    return float(lib.dcg_adam_lr_t(ctypes.byref(t), lr, beta1, beta2))


def colsum(a, out=None):
    cols = a.shape[-1]
    rows = a.numel() // cols
    if out is None:
        out = torch.empty((cols,), dtype=torch.float32, device=a.device)
    ws, nb = _workspace(a.device).get(lib.dcg_colsum_workspace_bytes(rows, cols))
    check(lib.dcg_colsum(_p(a), _p(out), rows, cols, ws, nb, _stream()))
    return out
