"""ctypes binding of libpipedream_b200.so (the C-ABI declared in include/pipedream_b200.h).

There is no fallback: if the library is missing or the device is not sm_100 the
first call raises.
"""
import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_uint64, c_void_p, POINTER

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "lib", "libpipedream_b200.so")

PD_F32 = 0
PD_BF16 = 1
PD_U8 = 2

_lib = None

P = c_void_p
I = c_int
L = c_int64
F = c_float
U64 = c_uint64

# name -> (restype, argtypes)
SIGNATURES = {
    "pd_last_error": (c_char_p, []),
    "pd_abi_version": (I, []),
    "pd_device_ok": (I, []),
    "pd_sm_count": (I, []),
    "pd_opt_sgd_multi_tensor": (I, [P, L, I, I, I, P, P, P, L, F, F, F, F, I, I, F, P]),
    "pd_opt_adam_multi_tensor": (I, [P, L, I, I, I, P, P, P, P, L, F, F, F, F, F, L, F, P]),
    "pd_scale": (I, [P, L, I, F, P]),
    "pd_convert": (I, [P, I, P, I, L, P]),
    "pd_pack_pnhwc": (I, [P, I, L, L, L, L, I, I, I, I, P, I, P]),
    "pd_unpack_pnhwc": (I, [P, I, I, I, I, I, P, I, P]),
    "pd_im2col3x3": (I, [P, I, L, L, L, L, I, I, I, I, I, P, I, P]),
    "pd_relu_fwd": (I, [P, P, L, I, P]),
    "pd_relu_bwd": (I, [P, P, P, L, I, P]),
    "pd_colsum_workspace_bytes": (L, [I]),
    "pd_relu_bwd_colsum": (I, [P, P, P, L, I, I, P, I, P, L, P]),
    "pd_maxpool2_fwd": (I, [P, I, I, I, I, P, I, I, P]),
    "pd_maxpool2_bwd": (I, [P, P, I, I, I, I, P, I, I, I, P]),
    "pd_maxpool2_bwd_colsum": (I, [P, P, I, I, I, I, P, I, I, P, L, P, P]),
    "pd_colsum_finish": (I, [P, I, I, P, I, P]),
    "pd_dropout_fwd": (I, [P, P, P, L, F, U64, U64, I, P]),
    "pd_dropout_bwd": (I, [P, P, P, L, F, I, P]),
    "pd_add": (I, [P, P, P, L, I, P]),
    "pd_layernorm_workspace_bytes": (L, [L, I]),
    "pd_layernorm_fwd": (I, [I, P, L, I, P, P, F, P, P, P, P]),
    "pd_layernorm_bwd": (I, [I, P, P, P, P, P, L, I, P, P, P, I, P, L, P]),
    "pd_sdpa_causal_fwd": (I, [I, P, I, I, I, I, F, P, P, P]),
    "pd_sdpa_causal_bwd": (I, [I, P, P, P, I, I, I, I, F, P, P, P]),
    "pd_gelu_fwd": (I, [I, P, P, L, I, P]),
    "pd_gelu_bwd": (I, [I, P, P, P, L, I, P]),
    "pd_bn_workspace_bytes": (L, [I]),
    "pd_bn_fwd": (I, [I, P, P, I, I, I, I, P, P, F, F, I, P, P, P, P, P, P, L, P]),
    "pd_bn_apply": (I, [I, P, P, I, I, I, I, P, P, P, P, I, P, P]),
    "pd_bn_bwd": (I, [I, P, P, P, I, I, I, I, P, P, P, P, P, I, P, P, P, P, L, P]),
    "pd_im2col": (I, [P, I, L, L, L, L, I, I, I, I, I, I, I, I, I, I, I, P, I, P]),
    "pd_col2im_pnhwc": (I, [P, I, I, I, I, I, I, I, I, I, I, I, P, I, P]),
    "pd_maxpool3s2_fwd": (I, [P, I, I, I, I, P, P, I, P]),
    "pd_maxpool3s2_bwd": (I, [P, P, I, I, I, I, P, I, P]),
    "pd_avgpool_fwd": (I, [P, I, I, I, I, P, I, P]),
    "pd_avgpool_bwd": (I, [P, I, I, I, I, P, I, P]),
    "pd_softmax_ce_fwd": (I, [P, I, P, L, I, F, L, F, P, P, P, P]),
    "pd_softmax_ce_bwd": (I, [P, I, P, P, L, I, F, L, P, F, P, P]),
    "pd_softmax_ce_fwd_static": (I, [P, I, P, L, I, F, L, F, P, P, P]),
    "pd_softmax_ce_static_max_rows": (L, []),
    "pd_revert_varlen": (I, [P, P, P, I, I, L, P]),
    "pd_length_mask": (I, [P, I, I, P, I, P]),
    "pd_mul_rows": (I, [P, P, P, L, I, I, P]),
    "pd_embedding_fwd": (I, [P, P, L, I, L, P, I, P]),
    "pd_embedding_bwd": (I, [P, P, L, I, L, L, P, I, P]),
    "pd_gemm_nt": (I, [I, P, L, P, L, P, I, L, I, I, I, P, I, I, I, I, P]),
    "pd_gemm_nt_splitk_workspace_bytes": (L, [I, I]),
    "pd_gemm_nt_splitk": (I, [I, P, L, P, L, P, I, L, I, I, I, P, I, I, P, L, P]),
    "pd_gemm_nn": (I, [I, P, L, P, L, P, I, L, I, I, I, P, L, P]),
    "pd_gemm_tn": (I, [I, P, L, P, L, P, L, I, I, I, I, I, P]),
    "pd_conv2d_fwd": (I, [I, P, I, I, I, I, P, L, I, P, I, I, P, P]),
    "pd_conv2d_dgrad": (I, [I, P, I, I, I, I, P, L, I, P, P, P]),
    "pd_conv2d_wgrad": (I, [I, P, P, I, I, I, I, I, P, L, I, I, P]),
    "pd_lstm_fwd": (I, [I, P, P, P, I, I, I, P, P, P, P, P]),
    "pd_lstm_bwd": (I, [I, P, P, P, P, I, I, I, P, P, P, P]),
    "pd_lstm_fwd_rows": (I, [I, P, P, P, I, I, I, I, I, P, P, P, P, P]),
    "pd_lstm_bwd_rows": (I, [I, P, P, P, P, I, I, I, I, I, P, P, P, P]),
    "pd_attn_bahdanau_fwd": (I, [I, P, P, P, L, L, P, P, P, I, I, I, I, I, P, P, L, L, P]),
    "pd_attn_bahdanau_bwd": (I, [I, P, P, P, L, L, P, P, P, P, L, L, I, I, I, I, I, P, P, P, L, L, P, P, P, P]),
    "pd_gemm_poll_error": (I, [POINTER(c_int)]),
    "pd_gemm_set_pair_mode": (I, [I]),
    "pd_gemm_set_stall_counters": (I, [P]),
    "pd_chan_create": (I, [L, I, I, POINTER(c_void_p)]),
    "pd_chan_export_handle": (I, [P, P]),
    "pd_chan_open": (I, [P, I, POINTER(c_void_p)]),
    "pd_chan_open_local": (I, [P, I, POINTER(c_void_p)]),
    "pd_chan_push": (I, [P, P, L, I, POINTER(c_int64), P]),
    "pd_chan_wait": (I, [P, P, L, P]),
    "pd_chan_peek_header": (I, [P, POINTER(c_int64), P]),
    "pd_chan_status": (I, [P, P]),
    "pd_chan_poll": (I, [P]),
    "pd_chan_close": (I, [P]),
}


class PipedreamB200Error(RuntimeError):
    pass


def lib_path():
    return _LIB_PATH


def load():
    """Load the shared library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise PipedreamB200Error(
            "%s not found: build it with `python -m pipedream_b200.build` "
            "(there is no non-CUDA fallback)" % _LIB_PATH)
    lib = ctypes.CDLL(_LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error():
    msg = load().pd_last_error()
    return msg.decode() if msg else ""


# kernels launched per call of each entry point (for launch accounting in benchmarks)
LAUNCHES = {"pd_relu_bwd_colsum": 2, "pd_softmax_ce_fwd": 2, "pd_gemm_nt_splitk": 2, "pd_sdpa_causal_fwd": 3,
            "pd_sdpa_causal_bwd": 5}
COUNTERS = None          # dict name -> calls, when a benchmark switches counting on


def count_calls(enable=True):
    """Start (or stop) counting entry-point calls; returns the previous counters."""
    global COUNTERS
    old = COUNTERS
    COUNTERS = {} if enable else None
    return old


def launches_counted():
    if not COUNTERS:
        return 0
    return sum(n * LAUNCHES.get(name, 1) for name, n in COUNTERS.items())


def call_or_decline(name, *args):
    """Like `call`, for entry points that may answer 1 = "not applicable, nothing enqueued": returns False then."""
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc == 1:
        return False
    if rc != 0:
        raise PipedreamB200Error("%s failed (status %d): %s" % (name, rc, last_error()))
    if COUNTERS is not None:
        COUNTERS[name] = COUNTERS.get(name, 0) + 1
    return True


def call(name, *args):
    """Call an int-status entry point and raise on a non-zero status."""
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise PipedreamB200Error("%s failed (status %d): %s" % (name, rc, last_error()))
    if COUNTERS is not None:
        COUNTERS[name] = COUNTERS.get(name, 0) + 1
    return rc
