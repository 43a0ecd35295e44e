"""ctypes binding of the C ABI declared in include/ntb_gemm.h.

Loading fails loudly when the CUDA library has not been built: there is no CPU path and
no fallback implementation behind these names.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libntb_gemm.so")

X_INT, X_INT8, X_FLOAT, X_FLOAT16, X_DOUBLE = 0, 1, 2, 3, 4
X_TRANS, X_NOTRANS = 0, 1
COUNT_REPACK = 7
ROUTE_NONE, ROUTE_TC_F16, ROUTE_TC_3XTF32, ROUTE_SIMT, ROUTE_TC_F16_PAIR, ROUTE_TC_F16X2 = 0, 1, 2, 3, 4, 5
OK, ERR_ARG, ERR_SHAPE, ERR_DTYPE, ERR_CUDA, ERR_DEVICE_WAIT, ERR_LIMIT = range(7)
MAX_PEERS = 8
PLAN_PAIR_256X256, PLAN_PAIR_512X256, PLAN_SPLIT_K2, PLAN_SPLIT_K4, PLAN_PAIR_256X128, PLAN_PAIR_512X128 = 0, -1, -2, -4, -8, -9
PLAN_PAIRSPLIT_K2, PLAN_PAIRSPLIT_K4 = -18, -20
NOALLOC_MAX_BYTES = 16 << 20
ACT_NONE, ACT_RECTIFY = 0, 1
SHARD_COLUMNS, SHARD_BATCH = 0, 1

_vp = ctypes.c_void_p
_i = ctypes.c_int
_ll = ctypes.c_longlong
_f = ctypes.c_float

#: every symbol include/ntb_gemm.h declares, with its argument types
PROTOTYPES = {
    "ntb_gemm": (_i, [_i, _vp, _vp, _i, _vp, _i, _vp, _i, _i] + [_i] * 6 + [_ll] * 3 + [_f, _f]),
    "ntb_gemm_bias_act": (_i, [_i, _vp, _vp, _i, _vp, _i, _vp, _vp, _i, _i] + [_i] * 6 + [_ll] * 3 + [_f, _f, _i]),
    "ntb_attention": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _ll, _f]),
    "ntb_attention_dropout": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _ll, _f, _f]),
    "ntb_row_stats": (_i, [_i, _vp, _vp, _i, _i, _i, _ll, _vp, _vp]),
    "ntb_logsoftmax_apply": (_i, [_i, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _vp, _vp]),
    "ntb_gemm_grad": (_i, [_i, _vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f]),
    "ntb_gemm_strided_batched": (_i, [_i, _vp, _vp, _i, _vp, _i, _vp, _i, _i] + [_i] * 6 + [_ll] * 6 + [_i, _f, _f]),
    "ntb_gemm_broadcast": (_i, [_i, _vp, _vp, _i, _vp, _i, _vp, _i, _i] + [_i] * 6 + [_i, _i, _f, _f]),
    "ntb_gemm_peers": (_i, [_i, _vp, _vp, _i, _vp, _i, _vp, ctypes.POINTER(_vp), _i, _i, _i] + [_i] * 6 + [_ll] * 3 + [_f, _f]),
    "ntb_gemm_multicast": (_i, [_i, _vp, _vp, _i, _vp, _i, _vp, _vp, _i, _i] + [_i] * 6 + [_ll] * 3 + [_f, _f]),
    "ntb_gemm_list": (_i, [_i, _vp, ctypes.POINTER(_vp), _i, ctypes.POINTER(_vp), _i, ctypes.POINTER(_vp),
                           _i, _i, _i] + [_i] * 6 + [_f, _f]),
    "ntb_gemm_sharded": (_i, [ctypes.POINTER(_i), _i, ctypes.POINTER(_vp), ctypes.POINTER(_vp), _i, ctypes.POINTER(_vp), _i,
                              ctypes.POINTER(_vp), _i, _i] + [_i] * 6 + [_i, _i, _i, _f, _f]),
    "ntb_shard_range": (None, [_i, _i, _i, _i, ctypes.POINTER(_i), ctypes.POINTER(_i)]),
    "ntb_unshard_columns": (_i, [_i, _vp, _vp, _vp, _i, _ll, _i, _i, _ll]),
    "ntb_gemm_grouped": (_i, [_i, _vp, _i, ctypes.POINTER(_vp), _i, ctypes.POINTER(_vp), _i, ctypes.POINTER(_vp), _i, _i] +
                         [ctypes.POINTER(_i)] * 6 + [_f, _f]),
    "ntb_gemm_host": (_i, [_i, _vp, _vp, _i, _vp, _i, _vp, _i, _i] + [_i] * 6 + [_ll] * 3 + [_i, _f, _f]),
    "ntb_gemm_host_resident_a": (_i, [_i, _vp, _vp, _i, _vp, _i, _vp, _i, _i] + [_i] * 6 + [_ll] * 3 + [_i, _f, _f]),
    "ntb_gemm_host_noalloc": (_i, [_i, _vp, _vp, _i, _vp, _i, _vp, _i, _i] + [_i] * 6 + [_f, _f]),
    "ntb_last_route": (_i, []),
    "ntb_set_route": (_i, [_i]),
    "ntb_device_status": (_i, [_i]),
    "ntb_plan": (_i, [_i] * 6),
    "ntb_debug_inject": (_i, [_i, _i, _i]),
    "ntb_route_count": (_ll, [_i]),
    "ntb_launch_count": (_ll, []),
    "ntb_release": (None, []),
    "ntb_strerror": (ctypes.c_char_p, [_i]),
}

_lib = None


class NtbError(RuntimeError):
    def __init__(self, code, what):
        self.code = code
        RuntimeError.__init__(self, "%s failed: %s (code %d)" % (what, strerror(code), code))


def lib():
    """The loaded shared library; raises if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "niutensor_b200: %s is missing -- build it with `python -m niutensor_b200.build`; "
                "there is no fallback implementation" % LIB_PATH)
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def strerror(code):
    return lib().ntb_strerror(int(code)).decode()


def check(code, what):
    if code != OK:
        raise NtbError(code, what)
