"""ctypes binding of liblwb200.so (the C ABI declared in include/lwb200.h).

The library is the product: there is no Python or CPU stand-in for it.  If it has not been built, importing a
function from here raises with the command that builds it.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("LWB200_LIB") or os.path.join(_HERE, "liblwb200.so")

LW_OK, LW_ERR, LW_ERR_ARG, LW_ERR_FORMAT, LW_ERR_CUDA, LW_ERR_TOO_LARGE, LW_ERR_NO_DEVICE = 0, -1, -2, -3, -4, -5, -6
FMT = {"none": 0, "Q4_K": 1, "Q5_K": 2, "Q6_K": 3, "IQ4_XS": 4}
FMT_NAME = {v: k for k, v in FMT.items()}

_u8p = C.POINTER(C.c_uint8)
_SIGNATURES = {
    # name: (restype, argtypes)
    "rt_open": (C.c_void_p, [C.c_char_p, C.c_int, C.c_int, C.c_longlong, C.c_int, C.c_int]),
    "rt_close": (None, [C.c_void_p]),
    "rt_test_matmul": (C.c_int, [C.c_void_p, C.c_char_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int]),
    "rt_test_decode": (C.c_int, [C.c_void_p, C.c_char_p, C.c_void_p]),
    "rt_test_cpu_decode": (C.c_int, [C.c_void_p, C.c_char_p, C.c_int, C.c_void_p]),
    "rt_gpu_decode_all": (C.c_double, [C.c_void_p, C.c_int]),
    "rt_cpu_decode_all": (C.c_double, [C.c_void_p, C.c_int, C.POINTER(C.c_longlong)]),
    "rt_stat": (C.c_double, [C.c_void_p, C.c_char_p]),
    "rt_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int]),
    "rt_reset": (None, [C.c_void_p]),
    "rt_set_window": (None, [C.c_void_p, C.c_int]),
    "rt_set_pos": (None, [C.c_void_p, C.c_int]),
    "rt_pos": (C.c_int, [C.c_void_p]),
    "rt_vocab": (C.c_int, [C.c_void_p]),
    "lw_tp_unique_id": (C.c_int, [C.c_void_p]),
    "rt_tp_init": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "rt_tp_peer_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "rt_tp_peer_open": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int]),
    "rt_tp_error": (C.c_int, [C.c_void_p]),
    "rt_decode_greedy": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "rt_tp_set_timeout": (C.c_int, [C.c_void_p, C.c_int]),
    "lw_debug_stream_stall": (C.c_int, [C.c_void_p, C.c_int]),
    "lw_matrix_id": (C.c_int, [C.c_void_p, C.c_char_p]),
    "lw_host_layout": (C.c_longlong, [C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_longlong,
                                      C.POINTER(C.c_int), C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong,
                                      C.c_void_p, C.c_longlong]),
    "lw_host_layout_table": (C.c_int, [C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_longlong, C.c_void_p]),
    "lw_matrix_plan": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_double)]),
    "lw_matrix_info": (C.c_int, [C.c_void_p, C.c_int] + [C.POINTER(C.c_int)] * 3 + [C.POINTER(C.c_longlong)] * 3),
    "lw_linear": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "lw_linear_batch": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "lw_linear_static": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "lw_matrix_make_twin": (C.c_int, [C.c_void_p, C.c_int]),
    "lw_matrix_drop_twin": (C.c_int, [C.c_void_p, C.c_int]),
    "lw_matrix_twin_bytes": (C.c_longlong, [C.c_void_p, C.c_int]),
    "lw_matrix_pair_bytes": (C.c_longlong, [C.c_void_p, C.c_int]),
    "lw_host_pairs": (C.c_longlong, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_longlong, C.POINTER(C.c_int),
                                     C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong]),
    "lw_linear_twin": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "lw_decode_weights": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "lw_decode_codes": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "lw_matrix_create": (C.c_void_p, [C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_longlong]),
    "lw_encode_huf8": (C.c_longlong, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_longlong, C.POINTER(C.c_longlong)]),
    "lw_validate_blob": (C.c_int, [C.c_void_p, C.c_longlong, C.c_int, C.c_int]),
    "lw_cpu_decode": (C.c_int, [C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "lw_validate_bundle": (C.c_int, [C.c_char_p]),
    "lw_block_bytes": (C.c_int, [C.c_int]),
    "lw_split_blocks": (C.c_int, [C.c_int, C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p]),
    "lw_join_blocks": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p]),
    "lw_ngram_create": (C.c_void_p, []),
    "lw_ngram_destroy": (None, [C.c_void_p]),
    "lw_ngram_push": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int]),
    "lw_ngram_draft": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int]),
    "lw_debug_set": (C.c_int, [C.c_char_p, C.c_longlong]),
    "lw_debug_wait_probe": (C.c_int, [C.c_longlong]),
    "lw_last_error": (C.c_char_p, []),
    "lw_last_status": (C.c_int, []),
    "lw_kernel_error": (C.c_int, []),
    "lw_launch_count": (C.c_longlong, []),
}

_lib = None


class LwError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("liblwb200 status %d: %s" % (status, message))
        self.status = status


def lib():
    """The loaded library with argument and return types set."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("liblwb200.so is not built (%s): run `python -m lazyweights_b200.build`; "
                              "there is no fallback implementation" % LIB_PATH)
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def exported_names():
    return sorted(_SIGNATURES)


def last_error():
    return (lib().lw_last_error() or b"").decode("utf-8", "replace")


def check(status):
    if status is None or (isinstance(status, int) and status < 0):
        raise LwError(-1 if status is None else status, last_error())
    return status
