"""TEST INFRASTRUCTURE: ctypes binding of oracle/_ref/libref_kernels.so, the reference's own CUDA kernels compiled for
sm_100a behind the C ABI of oracle/ref_kernels_shim.cu (`make -C oracle -j8 refgpu REF=<reference tree>`).  Pointers are
device addresses (torch tensor.data_ptr()).  Only the GPU tests use this module."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
PATH = os.path.join(_HERE, "_ref", "libref_kernels.so")
_lib = None
_p, _i, _f, _z = C.c_void_p, C.c_int, C.c_float, C.c_size_t
_SIGS = {
    "ref_quantize_q8_1": [_p, _p, _i, _i, _p],
    "ref_router_route": [_p, _p, _p, _i, _p, _p, _p, _p, _p, _p],
    "ref_moe_gate_up_q4k": [_p, _z, _i, _i, _p, _p, _i, _p, _p, _p],
    "ref_q8s_gemv": [_p, _p, _i, _i, _p, _p, _i, _i, _p],
    "ref_gdn_core": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _p, _i, _f, _p, _p],
    "ref_attn_part_lanes": [_p, _p, _p, _z, _i, _p, _p, _i, _p, _i, _p],
    "ref_argmax": [_p, _i, _i, _i, _p, _p, _p, _p, _p],
    "ref_top_tokens": [_p, _i, _i, _i, _p, _p, _p, _i, _p, _p, _p, _p, _p],
}
NAMES = ("N", "NEXP", "TOPK", "FF", "NKH", "NVH", "HS", "NQH", "NKVH", "HD", "NROT", "MAXT", "NCARD", "ATT_ROWS")


def available():
    return os.path.exists(PATH)


def load():
    global _lib
    if _lib is None:
        lib = C.CDLL(PATH)
        for name, args in _SIGS.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, _i
        lib.ref_last_error.restype = C.c_char_p
        lib.ref_gdn_scratch_floats.restype, lib.ref_gdn_scratch_floats.argtypes = _z, [_i]
        lib.ref_attn_scratch_floats.restype = _z
        lib.ref_attn_mz_offset.restype = _z
        _lib = lib
    return _lib


def shapes():
    out = (C.c_int * 14)()
    load().ref_shapes(out)
    return dict(zip(NAMES, out))


def call(name, *args):
    lib = load()
    if getattr(lib, name)(*args) != 0:
        raise RuntimeError("reference %s: %s" % (name, lib.ref_last_error().decode()))
