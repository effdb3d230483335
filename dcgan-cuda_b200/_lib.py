"""ctypes binding of libdcgan_b200.so (declared in include/dcgan_b200.h).

The library must exist: there is no Python or CPU fallback.  Importing this
module when the shared object is missing raises ImportError with the build
command.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libdcgan_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        "dcgan_b200: %s is missing - build it with `python dcgan-cuda_b200/build.py` "
        "(or __graft_entry__.build()); there is no fallback path" % LIB_PATH)

lib = ctypes.CDLL(LIB_PATH)

c_float_p = ctypes.POINTER(ctypes.c_float)
c_void_p = ctypes.c_void_p
c_size_t = ctypes.c_size_t
c_int = ctypes.c_int
c_float = ctypes.c_float

# status codes
OK, ERR_INVALID, ERR_CUDA, ERR_WORKSPACE, ERR_UNSUPPORTED, ERR_DEVICE = 0, -1, -2, -3, -4, -5
# activations
ACT_NONE, ACT_LEAKY, ACT_RELU, ACT_TANH, ACT_SIGMOID = 0, 1, 2, 3, 4
# precisions
PREC_TF32, PREC_3XTF32, PREC_FP32 = 0, 1, 2
# conv kinds for workspace queries
KIND_FWD, KIND_DX, KIND_DK = 0, 1, 2

NODE_OUT_DEAD = 1


class ConvDesc(ctypes.Structure):
    _fields_ = [(n, c_int) for n in ("n", "h", "w", "c", "kh", "kw", "o", "ho", "wo",
                                     "stride_h", "stride_w", "pad_top", "pad_left")]


class Epilogue(ctypes.Structure):
    _fields_ = [("raw_out", c_void_p), ("bias", c_void_p), ("pre_act", c_void_p),
                ("act", c_int), ("alpha", c_float), ("gate", c_void_p),
                ("gate_act", c_int), ("gate_alpha", c_float)]


class AdamTensor(ctypes.Structure):
    _fields_ = [("p", c_void_p), ("g", c_void_p), ("g2", c_void_p), ("m", c_void_p),
                ("v", c_void_p), ("n", c_size_t)]


class Node(ctypes.Structure):
    _fields_ = [("type", c_int), ("in1", c_void_p), ("in2", c_void_p), ("in3", c_void_p),
                ("out1", c_void_p), ("out2", c_void_p),
                ("cons1", c_float), ("cons2", c_float), ("cons3", c_float), ("cons4", c_float),
                ("len1", c_size_t), ("len2", c_size_t), ("len3", c_size_t),
                ("intconst", c_int * 2), ("intconst2", c_int * 2),
                ("sizes1", c_int * 4), ("sizes2", c_int * 4), ("sizes3", c_int * 4),
                ("int_cons1", c_int), ("int_cons2", c_int), ("alpha_leaky", c_float),
                ("flags", ctypes.c_uint)]


class ProfileRow(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char * 96), ("calls", ctypes.c_uint64), ("ms", ctypes.c_double),
                ("flops", ctypes.c_double)]


class TrainerConfig(ctypes.Structure):
    _fields_ = [("batch", c_int), ("world", c_int), ("precision", c_int), ("fuse", c_int),
                ("g_leaky", c_int), ("lr", c_float), ("beta1", c_float), ("beta2", c_float),
                ("eps", c_float), ("seed", ctypes.c_uint64), ("share_g_forward", c_int)]


DP_ID_BYTES = 128   # DCG_DP_ID_BYTES

# Every exported symbol of include/dcgan_b200.h: name -> (restype, argtypes)
_P = c_void_p
SIGNATURES = {
    "dcg_conv_workspace_bytes": (c_size_t, [ctypes.POINTER(ConvDesc), c_int, c_int]),
    "dcg_conv2d_fwd": (c_int, [ctypes.POINTER(ConvDesc), _P, _P, _P, ctypes.POINTER(Epilogue), c_int, _P, c_size_t, _P]),
    "dcg_conv2d_dx": (c_int, [ctypes.POINTER(ConvDesc), _P, _P, _P, ctypes.POINTER(Epilogue), c_int, _P, c_size_t, _P]),
    "dcg_conv2d_dk": (c_int, [ctypes.POINTER(ConvDesc), _P, _P, _P, c_int, _P, c_size_t, _P]),
    "dcg_bias_act": (c_int, [_P, _P, _P, _P, c_size_t, c_size_t, c_int, c_float, _P]),
    "dcg_act_fwd": (c_int, [_P, _P, c_size_t, c_int, c_float, _P]),
    "dcg_act_grad": (c_int, [_P, _P, _P, c_size_t, c_int, c_float, _P]),
    "dcg_colsum_workspace_bytes": (c_size_t, [c_size_t, c_size_t]),
    "dcg_colsum": (c_int, [_P, _P, c_size_t, c_size_t, _P, c_size_t, _P]),
    "dcg_colsum_noalloc_max_bytes": (c_size_t, []),
    "dcg_colsum_noalloc": (c_int, [_P, _P, c_size_t, c_size_t, _P]),
    "dcg_rowsum": (c_int, [_P, _P, c_size_t, c_size_t, _P]),
    "dcg_add": (c_int, [_P, _P, _P, c_size_t, _P]),
    "dcg_u8_to_unit": (c_int, [_P, _P, c_size_t, _P]),
    "dcg_update": (c_int, [_P, _P, _P, c_size_t, _P]),
    "dcg_matmul": (c_int, [_P, _P, _P, _P, c_size_t, c_size_t, c_size_t, _P]),
    "dcg_matmul_tn": (c_int, [_P, _P, _P, c_size_t, c_size_t, c_size_t, _P]),
    "dcg_matmul_nt": (c_int, [_P, _P, _P, c_size_t, c_size_t, c_size_t, _P]),
    "dcg_sigmoid_xent": (c_int, [_P, _P, _P, c_size_t, _P]),
    "dcg_sigmoid_xent_grad": (c_int, [_P, _P, _P, c_size_t, _P]),
    "dcg_mse": (c_int, [_P, _P, _P, c_size_t, c_size_t, _P]),
    "dcg_mse_grad": (c_int, [_P, _P, _P, c_size_t, _P]),
    "dcg_softmax": (c_int, [_P, _P, c_size_t, c_size_t, _P]),
    "dcg_log_softmax": (c_int, [_P, _P, c_size_t, c_size_t, _P]),
    "dcg_softmax_xent": (c_int, [_P, _P, _P, c_size_t, c_size_t, _P]),
    "dcg_softmax_xent_grad": (c_int, [_P, _P, _P, c_size_t, c_size_t, _P]),
    "dcg_argmax_acc": (c_int, [_P, _P, _P, c_size_t, c_size_t, _P]),
    "dcg_adam_lr_t": (c_float, [c_float_p, c_float, c_float, c_float]),
    "dcg_adam_multi": (c_int, [ctypes.POINTER(AdamTensor), c_int, c_float, c_float, c_float, c_float, c_float, _P]),
    "dcg_context_create": (c_int, [ctypes.POINTER(_P), c_int, _P, c_size_t, _P]),
    "dcg_context_destroy": (None, [_P]),
    "dcg_context_set_precision": (c_int, [_P, c_int]),
    "dcg_context_launch_count": (ctypes.c_uint64, [_P]),
    "dcg_run_node": (c_int, [_P, ctypes.POINTER(Node)]),
    "dcg_run_nodes": (c_int, [_P, ctypes.POINTER(Node), c_int, c_int]),
    "dcg_dp_unique_id": (c_int, [_P]),
    "dcg_dp_init": (c_int, [ctypes.POINTER(_P), c_int, c_int, _P]),
    "dcg_dp_allreduce": (c_int, [_P, _P, c_size_t, _P]),
    "dcg_dp_info": (c_int, [_P, ctypes.POINTER(c_int), ctypes.POINTER(c_int), ctypes.POINTER(c_int)]),
    "dcg_dp_finalize": (None, [_P]),
    "dcg_trainer_create": (c_int, [ctypes.POINTER(_P), ctypes.POINTER(TrainerConfig), _P]),
    "dcg_trainer_create_dp": (c_int, [ctypes.POINTER(_P), ctypes.POINTER(TrainerConfig), _P, _P]),
    "dcg_trainer_destroy": (None, [_P]),
    "dcg_trainer_tensor": (c_int, [_P, ctypes.c_char_p, ctypes.POINTER(_P), ctypes.POINTER(c_size_t)]),
    "dcg_trainer_generate": (c_int, [_P]),
    "dcg_trainer_d_fwd_bwd": (c_int, [_P]),
    "dcg_trainer_d_backward": (c_int, [_P]),
    "dcg_trainer_d_apply": (c_int, [_P, c_float]),
    "dcg_trainer_g_backward": (c_int, [_P]),
    "dcg_trainer_g_backward_part": (c_int, [_P, c_int]),
    "dcg_trainer_g_apply": (c_int, [_P, c_float]),
    "dcg_trainer_step": (c_int, [_P]),
    "dcg_trainer_save": (c_int, [_P, ctypes.c_char_p]),
    "dcg_trainer_save_wait": (c_int, [_P]),
    "dcg_trainer_load": (c_int, [_P, ctypes.c_char_p]),
    "dcg_trainer_context": (_P, [_P]),
    "dcg_context_profile_begin": (c_int, [_P]),
    "dcg_context_profile_end": (c_int, [_P, ctypes.POINTER(ProfileRow), c_int, ctypes.POINTER(c_int)]),
    "dcg_trainer_dp_mode": (c_int, [_P]),
    "dcg_trainer_step_mode": (c_int, [_P]),
    "dcg_trainer_step_launches": (ctypes.c_uint64, [_P]),
    "dcg_trainer_arena_bytes": (c_size_t, [_P]),
    "dcg_device_status": (c_int, []),
    "dcg_last_error": (ctypes.c_char_p, []),
    "dcg_debug_set_wait_limit": (None, [ctypes.c_longlong]),
    "dcg_debug_skip_stage": (None, [c_int]),
    "dcg_debug_set_dx_mode": (None, [c_int]),
    "dcg_debug_fused_dx_launches": (ctypes.c_uint64, []),
    "dcg_build_info": (ctypes.c_char_p, []),
    "dcg_launches_total": (ctypes.c_uint64, []),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)  # AttributeError here = header and library disagree
    _fn.restype = _res
    _fn.argtypes = _args


class DcgError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("dcgan_b200 status %d: %s" % (status, message))
        self.status = status


def check(status):
    """Raises DcgError for a non-zero dcg_status."""
    if status != 0:
        raise DcgError(status, lib.dcg_last_error().decode("utf-8", "replace"))


def last_error():
    return lib.dcg_last_error().decode("utf-8", "replace")
