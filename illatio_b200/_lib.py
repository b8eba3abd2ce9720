"""ctypes binding of libillatio_b200.so -- the same C ABI a Lisp host binds.

There is no fallback: if the library is missing or a call fails, an exception
is raised.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libillatio_b200.so")

_c = ctypes
_P = _c.c_uint64   # ill_dptr
_S = _c.c_void_p   # ill_stream
_I = _c.c_int
_L = _c.c_int64
_F = _c.c_float

class DecodeOp(_c.Structure):
    """ill_decode_op of include/illatio_b200.h."""
    _fields_ = [("w", _P), ("w2", _P), ("x", _P), ("norm_w", _P), ("y", _P), ("bias", _P),
                ("fmt", _c.c_int32), ("kind", _c.c_int32), ("rows", _c.c_int32), ("cols", _c.c_int32),
                ("acc", _c.c_int32), ("after", _c.c_int32), ("f16_scale", _c.c_int32), ("eps", _c.c_float)]


SIGNATURES = {
    "ill_decode_plan_bytes": (_L, [_I]),
    "ill_decode_plan": (_I, [_c.POINTER(DecodeOp), _I, _P, _L, _c.POINTER(_c.c_int32), _S]),
    "ill_decode_run": (_I, [_P, _c.POINTER(_c.c_int32), _S]),
    "ill_b200_version": (_I, []),
    "ill_error_string": (_c.c_char_p, [_I]),
    "ill_last_cuda_error": (_I, []),
    "ill_block_bytes": (_I, [_I]),
    "ill_block_weights": (_I, [_I]),
    "ill_test_wait_timeout": (_I, [_L, _P, _S]),
    "ill_device_status": (_I, [_c.POINTER(_c.c_uint), _S]),
    "ill_quant_q8_0": (_I, [_P, _P, _P, _P, _L, _I, _S]),
    "ill_quant_q8_k": (_I, [_P, _P, _P, _P, _L, _S]),
    "ill_rmsnorm_q8": (_I, [_I, _P, _P, _P, _P, _P, _P, _I, _F, _L, _I, _S]),
    "ill_dequant_rows": (_I, [_I, _P, _I, _P, _L, _I, _P, _S]),
    "ill_mv": (_I, [_I, _P, _I, _I, _P, _P, _P, _P, _P, _I, _I, _S]),
    "ill_mv_3": (_I, [_I, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _S]),
    "ill_mv_glu": (_I, [_I, _P, _P, _I, _I, _P, _P, _P, _P, _S]),
    "ill_moe_mv": (_I, [_I, _I, _I, _L, _P, _I, _P, _P, _P, _I, _P, _L, _S]),
    "ill_moe_glu": (_I, [_I, _I, _I, _L, _L, _P, _I, _P, _P, _P, _I, _F, _P, _P, _L, _S]),
    "ill_swiglu_w": (_I, [_L, _I, _F, _P, _P, _P, _P, _S]),
    "ill_moe_sum": (_I, [_I, _I, _L, _P, _P, _P, _P, _S]),
    "ill_swiglu_q8k_f16": (_I, [_L, _I, _F, _P, _P, _P, _P, _P, _P, _P, _S]),
    "ill_mv_dense": (_I, [_I, _P, _I, _I, _P, _P, _I, _L, _S]),
    "ill_moe_route": (_I, [_I, _I, _I, _F, _L, _P, _P, _P, _P, _S]),
    "ill_moe_group_scratch_bytes": (_L, [_L, _I]),
    "ill_moe_group": (_I, [_L, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _S]),
    "ill_moe_group_static": (_I, [_L, _I, _I, _P, _P, _P, _P, _P, _P, _P, _S]),
    "ill_moe_row_ptrs": (_I, [_I, _P, _P, _P, _L, _P, _S]),
    "ill_gather_rows": (_I, [_L, _L, _P, _P, _P, _S]),
    "ill_act_f16": (_I, [_L, _I, _P, _P, _P, _P, _P, _S]),
    "ill_moe_mm_id": (_I, [_I, _I, _I, _L, _P, _P, _P, _I, _L, _P, _P, _P, _P, _P, _P, _L, _S]),
    "ill_ep_plan_rows": (_I, [_I, _P, _P, _P, _P, _P, _S]),
    "ill_ep_row_bytes": (_L, [_I]),
    "ill_ep_pack": (_I, [_L, _I, _P, _P, _P, _P, _P, _P, _S]),
    "ill_ep_pack_cap": (_I, [_L, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _P, _P, _P, _I, _S]),
    "ill_ep_put_counts": (_I, [_I, _I, _I, _P, _P, _P, _S]),
    "ill_ep_plan_dev": (_I, [_I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _S]),
    "ill_moe_mm_id2": (_I, [_I, _I, _I, _L, _L, _P, _P, _P, _I, _L, _P, _P, _P, _P, _P, _P, _L, _S]),
    "ill_moe_mm_id_peers": (_I, [_I, _I, _I, _L, _P, _P, _P, _I, _L, _P, _P, _P, _P, _P, _P, _L, _S]),
    "ill_ep_ipc_export": (_I, [_P, _c.c_char_p, _c.POINTER(_c.c_int64)]),
    "ill_ep_ipc_open": (_I, [_c.c_char_p, _L, _c.POINTER(_c.c_uint64)]),
    "ill_ep_ipc_close": (_I, [_P, _L]),
    "ill_ep_flags_bytes": (_L, []),
    "ill_ep_barrier": (_I, [_P, _P, _I, _I, _I, _c.c_uint32, _L, _S]),
    "ill_quant_q8_k_f16": (_I, [_P, _P, _P, _P, _P, _P, _L, _S]),
    "ill_rmsnorm_q8k_f16": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _c.c_float, _L, _S]),
    "ill_mm_chunk": (_I, [_I, _P, _I, _I, _P, _P, _P, _L, _P, _I, _S]),
    "ill_mm_chunk2": (_I, [_I, _P, _P, _I, _I, _P, _P, _P, _L, _P, _P, _S]),
    "ill_mv_peers": (_I, [_I, _P, _I, _I, _P, _P, _P, _P, _L, _P, _P, _P, _I, _I, _I, _c.c_uint32, _L, _S]),
    "ill_peer_put": (_I, [_P, _L, _P, _L, _P, _P, _I, _I, _I, _c.c_uint32, _L, _S]),
    "ill_ep_plan_dev_sync": (_I, [_I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _c.c_uint32, _L, _S]),
    "ill_moe_sum_sync": (_I, [_I, _I, _L, _P, _P, _P, _P, _P, _P, _P, _I, _I, _c.c_uint32, _L, _P, _P, _S]),
    "ill_ep_dispatch": (_I, [_L, _I, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _P, _c.c_uint32, _S]),
    "ill_ep_unpack": (_I, [_L, _I, _P, _P, _P, _P, _P, _P, _P, _S]),
}


class IllatioError(RuntimeError):
    def __init__(self, fn, code, text, cuda=0):
        super().__init__("%s failed: %s (status %d%s)" % (fn, text, code, ", cudaError %d" % cuda if cuda else ""))
        self.code = code
        self.cuda = cuda


_lib = None


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "libillatio_b200.so is not built (run `python -m illatio_b200.build`); there is no fallback path")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            if not hasattr(L, name):
                continue
            f = getattr(L, name)
            f.restype = res
            f.argtypes = args
        _lib = L
    return _lib


def register(name, res, args):
    """Add the signature of an entry point declared after this module was written."""
    SIGNATURES[name] = (res, args)
    if _lib is not None and hasattr(_lib, name):
        f = getattr(_lib, name)
        f.restype = res
        f.argtypes = args


def call(name, *args):
    """Call entry point NAME; a non-zero status becomes an IllatioError."""
    L = lib()
    rc = getattr(L, name)(*args)
    if rc != 0:
        raise IllatioError(name, rc, L.ill_error_string(rc).decode(), L.ill_last_cuda_error() if rc == 4 else 0)
    return rc


def status(name, *args):
    """Call entry point NAME and return its status code without raising."""
    return getattr(lib(), name)(*args)
