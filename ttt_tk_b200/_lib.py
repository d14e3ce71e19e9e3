"""ctypes binding of libttt_mlp_b200.so (declarations: include/ttt_mlp_b200.h).

There is no fallback: if the library is missing the import fails.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libttt_mlp_b200.so")

c_void_p, c_int32, c_uint32 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_uint32

FWD_FIELDS = ["XQ", "XK", "XV", "last_eta", "ttt_norm_weight", "ttt_norm_bias", "W1", "b1", "W2", "b2",
              "W1_checkpoints", "b1_checkpoints", "W2_checkpoints", "b2_checkpoints", "Out"]
FWD_TAIL = ["W1_final", "b1_final", "W2_final", "b2_final"]
BWD_FIELDS = ["XQ", "XK", "XV", "last_eta", "ttt_norm_weight", "ttt_norm_bias",
              "W1_checkpoints", "b1_checkpoints", "W2_checkpoints", "b2_checkpoints", "Out",
              "W1_init_group", "b1_init_group", "W2_init_group", "b2_init_group",
              "x_hat_ln_group", "std_ln_group", "X2_group", "Z1_group", "Z1_bar_group", "X2_bar_group",
              "grad_l_wrt_Z2_group", "grad_l_wrt_Z1_group", "x_hat_fused_group", "grad_x_hat_fused_group",
              "grad_output_fused_group", "std_fused_group",
              "grad_L_W1_last", "grad_L_b1_last", "grad_L_W2_last", "grad_L_b2_last", "grad_L_XQW_mini_batch",
              "grad_L_ttt_norm_weight", "grad_L_ttt_norm_bias", "grad_L_W1_init", "grad_L_b1_init",
              "grad_L_W2_init", "grad_L_b2_init", "grad_L_last_eta", "grad_L_XQ", "grad_L_XK", "grad_L_XV"]
_DIMS = [("B", c_int32), ("H", c_int32), ("NC", c_int32), ("checkpoint_group_size", c_int32),
         ("num_checkpoints", c_int32), ("flags", c_uint32)]


class FwdArgs(ctypes.Structure):
    _fields_ = [(n, c_void_p) for n in FWD_FIELDS] + _DIMS + [(n, c_void_p) for n in FWD_TAIL]


# ttt_b200_linear_forward: the forward's tensors without W2 / b2 and their checkpoints
LINEAR_FWD_FIELDS = ["XQ", "XK", "XV", "last_eta", "ttt_norm_weight", "ttt_norm_bias", "W1", "b1",
                     "W1_checkpoints", "b1_checkpoints", "Out"]
LINEAR_FWD_TAIL = ["W1_final", "b1_final"]


class LinearFwdArgs(ctypes.Structure):
    _fields_ = [(n, c_void_p) for n in LINEAR_FWD_FIELDS] + _DIMS + [(n, c_void_p) for n in LINEAR_FWD_TAIL]


LINEAR_BWD_FIELDS = ["XQ", "XK", "XV", "last_eta", "ttt_norm_weight", "ttt_norm_bias", "W1_checkpoints", "b1_checkpoints",
                     "grad_L_W1_last", "grad_L_b1_last", "grad_L_XQW_mini_batch", "scratch", "grad_L_ttt_norm_weight",
                     "grad_L_ttt_norm_bias", "grad_L_W1_init", "grad_L_b1_init", "grad_L_last_eta", "grad_L_XQ",
                     "grad_L_XK", "grad_L_XV"]


class LinearBwdArgs(ctypes.Structure):
    _fields_ = [(n, c_void_p) for n in LINEAR_BWD_FIELDS] + _DIMS + [("scratch_bytes", ctypes.c_uint64)]


class BwdArgs(ctypes.Structure):
    _fields_ = [(n, c_void_p) for n in BWD_FIELDS] + _DIMS


# ttt_b200_backward_noalloc: the backward's tensors without `Out` and the sixteen scratch tensors
BWD_NOALLOC_FIELDS = BWD_FIELDS[:10] + BWD_FIELDS[27:]
NOALLOC_MAX_SLOTS = 128


class BwdNoAllocArgs(ctypes.Structure):
    _fields_ = [(n, c_void_p) for n in BWD_NOALLOC_FIELDS] + _DIMS


EXPORTS = ["ttt_b200_forward", "ttt_b200_linear_forward", "ttt_b200_linear_backward", "ttt_b200_linear_backward_scratch_bytes", "ttt_b200_backward", "ttt_b200_backward_noalloc", "ttt_b200_last_error", "ttt_b200_take_status",
           "ttt_b200_version", "ttt_b200_pick_cluster", "ttt_b200_cluster_capacity", "ttt_b200_umma_selftest", "ttt_b200_wait_selftest", "ttt_b200_pack_tokens",
           "ttt_b200_unpack_tokens", "ttt_b200_eta_gate", "ttt_b200_eta_gate_backward", "ttt_b200_unpack_layernorm",
           "ttt_b200_pack_layernorm_backward"]

FLAG_SYNC = 1
FLAG_TEST_LOST_LOAD = 2


def load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m ttt_tk_b200.build` (needs nvcc); "
            "this package has no CPU or PyTorch fallback")
    lib = ctypes.CDLL(LIB_PATH)
    lib.ttt_b200_forward.argtypes = [ctypes.POINTER(FwdArgs), c_void_p]
    lib.ttt_b200_forward.restype = ctypes.c_int
    lib.ttt_b200_linear_forward.argtypes = [ctypes.POINTER(LinearFwdArgs), c_void_p]
    lib.ttt_b200_linear_forward.restype = ctypes.c_int
    lib.ttt_b200_linear_backward.argtypes = [ctypes.POINTER(LinearBwdArgs), c_void_p]
    lib.ttt_b200_linear_backward.restype = ctypes.c_int
    lib.ttt_b200_linear_backward_scratch_bytes.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int]
    lib.ttt_b200_linear_backward_scratch_bytes.restype = ctypes.c_uint64
    lib.ttt_b200_backward.argtypes = [ctypes.POINTER(BwdArgs), c_void_p]
    lib.ttt_b200_backward.restype = ctypes.c_int
    lib.ttt_b200_backward_noalloc.argtypes = [ctypes.POINTER(BwdNoAllocArgs), c_void_p]
    lib.ttt_b200_backward_noalloc.restype = ctypes.c_int
    lib.ttt_b200_last_error.argtypes = []
    lib.ttt_b200_last_error.restype = ctypes.c_char_p
    lib.ttt_b200_take_status.argtypes = []
    lib.ttt_b200_take_status.restype = ctypes.c_int
    lib.ttt_b200_version.argtypes = []
    lib.ttt_b200_version.restype = ctypes.c_int
    lib.ttt_b200_pick_cluster.argtypes = [ctypes.c_int, ctypes.c_int]
    lib.ttt_b200_pick_cluster.restype = ctypes.c_int
    lib.ttt_b200_cluster_capacity.argtypes = [ctypes.c_int, ctypes.c_int]
    lib.ttt_b200_cluster_capacity.restype = ctypes.c_int
    lib.ttt_b200_umma_selftest.argtypes = [c_void_p, c_void_p, c_void_p] + [ctypes.c_int] * 7 + [c_void_p]
    lib.ttt_b200_umma_selftest.restype = ctypes.c_int
    lib.ttt_b200_wait_selftest.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_ulonglong), c_void_p]
    lib.ttt_b200_wait_selftest.restype = ctypes.c_int
    for name in ("ttt_b200_pack_tokens", "ttt_b200_unpack_tokens"):
        fn = getattr(lib, name)
        fn.argtypes = [ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p)] + [ctypes.c_int] * 4 + [c_void_p]
        fn.restype = ctypes.c_int
    lib.ttt_b200_eta_gate.argtypes = [c_void_p, c_void_p, ctypes.c_float] + [ctypes.c_int] * 3 + [c_void_p]
    lib.ttt_b200_eta_gate.restype = ctypes.c_int
    lib.ttt_b200_eta_gate_backward.argtypes = [c_void_p, c_void_p, c_void_p, ctypes.c_float] + [ctypes.c_int] * 3 + [c_void_p]
    lib.ttt_b200_eta_gate_backward.restype = ctypes.c_int
    lib.ttt_b200_unpack_layernorm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_float] + \
        [ctypes.c_int] * 3 + [c_void_p]
    lib.ttt_b200_unpack_layernorm.restype = ctypes.c_int
    lib.ttt_b200_pack_layernorm_backward.argtypes = [c_void_p] * 7 + [ctypes.c_int] * 3 + [c_void_p]
    lib.ttt_b200_pack_layernorm_backward.restype = ctypes.c_int
    return lib


_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        _LIB = load()
    return _LIB
