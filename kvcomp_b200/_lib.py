"""ctypes binding of libkvcomp_b200.so (the C ABI declared in include/kvcomp_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
import ctypes as C
import os

from . import build as _build

KVC_OK = 0
FLAGS = {
    0x001: "ZERO_SCALE", 0x002: "MIN_OVERFLOW", 0x004: "CODE_OVERFLOW", 0x008: "SYMBOL_MISSING",
    0x010: "VECTOR_LONG", 0x020: "BLOCK_LONG", 0x040: "STREAM_FULL", 0x080: "BAD_STREAM",
    0x100: "CODE_TOO_LONG", 0x200: "NO_SYMBOLS", 0x400: "WAIT_TIMEOUT",
}
FLAG_ZERO_SCALE, FLAG_MIN_OVERFLOW, FLAG_CODE_OVERFLOW, FLAG_SYMBOL_MISSING = 0x1, 0x2, 0x4, 0x8
FLAG_VECTOR_LONG, FLAG_BLOCK_LONG, FLAG_STREAM_FULL, FLAG_BAD_STREAM = 0x10, 0x20, 0x40, 0x80
FLAG_CODE_TOO_LONG, FLAG_NO_SYMBOLS, FLAG_WAIT_TIMEOUT = 0x100, 0x200, 0x400
# conditions under which the produced data cannot be trusted (the rest are informational)
FATAL_FLAGS = FLAG_CODE_OVERFLOW | FLAG_SYMBOL_MISSING | FLAG_BLOCK_LONG | FLAG_STREAM_FULL | \
    FLAG_BAD_STREAM | FLAG_CODE_TOO_LONG | FLAG_NO_SYMBOLS | FLAG_WAIT_TIMEOUT

MODE_BLOCK, MODE_CHANNEL, MODE_TOKEN, MODE_VECTOR = 0, 1, 2, 3

LUT_BITS = 12
BOOK_OFF_ENC = 64
BOOK_OFF_REFTREE = BOOK_OFF_ENC + 2048
BOOK_OFF_TREE = BOOK_OFF_REFTREE + 1536
BOOK_OFF_LUT = BOOK_OFF_TREE + 2048
BOOK_BYTES = BOOK_OFF_LUT + 4 * (1 << LUT_BITS)


class QMeta(C.Structure):
    _fields_ = [("min_int", C.c_void_p), ("scale", C.c_void_p), ("min_bytes", C.c_int32),
                ("tok_div", C.c_int32), ("sj", C.c_int64), ("sb", C.c_int64), ("sh", C.c_int64),
                ("sc", C.c_int64)]


class Cache(C.Structure):
    _fields_ = [("encoded", C.c_void_p), ("encoded_bytes", C.c_int64), ("block_info", C.c_void_p),
                ("thread_info", C.c_void_p), ("book", C.c_void_p), ("q", QMeta),
                ("max_block_bytes", C.c_int32), ("reserved", C.c_int32)]


class KvcError(RuntimeError):
    pass


_lib = None

_i64, _i32, _vp, _f32, _u32 = C.c_int64, C.c_int, C.c_void_p, C.c_float, C.c_uint32

_SIGNATURES = {
    "kvc_last_error": (C.c_char_p, []),
    "kvc_version": (_i32, []),
    "kvc_buffer_sizes": (_i32, [_i64, _i64, _i32, C.POINTER(_i64)]),
    "kvc_qmeta_make": (_i32, [_i32, _i32, _i64, _i64, _i64, _i64, _i64, C.POINTER(QMeta), C.POINTER(_i64)]),
    "kvc_quantize_workspace": (_i64, [_i32, _i32, _i64, _i64, _i64]),
    "kvc_quantize": (_i32, [_vp, _i64, _i64, _i64, _i64, _i32, _i32, _i64, _f32, _vp, _vp, _i32, _vp, _vp,
                            _vp, _i64, _vp, _vp]),
    "kvc_quant_minmax": (_i32, [_vp, _i64, _i64, _i64, _i64, _i32, _i32, _i64, _vp, _vp, _vp, _i64, _vp]),
    "kvc_quantize_ranged": (_i32, [_vp, _i64, _i64, _i64, _i64, _i32, _i32, _i64, _f32, _vp, _vp, _vp, _vp, _i32, _vp,
                                   _vp, _vp, _i64, _vp, _vp]),
    "kvc_rope_store": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp]),
    "kvc_kv_store": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp]),
    "kvc_dequant": (_i32, [_vp, C.POINTER(QMeta), _i64, _i64, _i64, _i64, _vp, _vp]),
    "kvc_histogram": (_i32, [_vp, _i64, _vp, _vp]),
    "kvc_build_codebook": (_i32, [_vp, _vp, _vp]),
    "kvc_book_from_tree": (_i32, [_vp, _i64, _vp, _vp]),
    "kvc_encode_workspace": (_i64, [_i64, _i64, _i32]),
    "kvc_encode_debug": (None, [_i32, _i32]),
    "kvc_encode": (_i32, [_vp, _i64, _i64, _i32, _vp, _i32, _u32, _vp, _vp, _vp, _i64, _vp, _vp, _i64, _vp, _vp]),
    "kvc_decode": (_i32, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _i32, _vp, _vp, _vp]),
    "kvc_decode_bounded": (_i32, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _i32, _u32, _vp, _vp, _vp]),
    "kvc_fused_qk": (_i32, [C.POINTER(Cache), _i64, _i64, _i64, _i64, _vp, _vp, _i32, _vp, _vp]),
    "kvc_fused_pv": (_i32, [C.POINTER(Cache), _i64, _i64, _i64, _i64, _vp, _vp, _vp, _vp]),
    "kvc_attn_workspace": (_i64, [_i64, _i64, _i32]),
    "kvc_attn_splits": (_i32, [_i64, _i64, _i64, _i32]),
    "kvc_attn_decode": (_i32, [C.POINTER(Cache), C.POINTER(Cache), _i64, _i64, _i64, _i64, _vp, _f32, _vp, _vp,
                               _i64, _vp, _i32, _vp, _i64, _vp, _vp]),
    "kvc_attn_debug": (None, [_i32, _i32]),
    "kvc_attn_static_capacity": (_i64, []),
    "kvc_attn_decode_static": (_i32, [C.POINTER(Cache), C.POINTER(Cache), _i64, _i64, _i64, _i64, _vp, _f32, _vp, _vp,
                                      _i64, _vp, _i32, _vp, _vp]),
    "kvc_k_matvec": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp]),
}

EXPORTS = tuple(_SIGNATURES)


def lib_path():
    return _build.LIB


def load():
    """Load (building first when the sources are newer) the CUDA library.  Raises if it cannot."""
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("KVCOMP_B200_LIB")          # an alternative build of the same library
    if not path:
        path = _build.LIB
        if _build.is_stale():
            path = _build.build()
    if not os.path.exists(path):
        raise KvcError("libkvcomp_b200.so is missing and could not be built; there is no CPU fallback")
    lib = C.CDLL(path)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)      # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc, what):
    if rc != KVC_OK:
        msg = load().kvc_last_error()
        raise KvcError("%s failed (code %d): %s" % (what, rc, msg.decode() if msg else ""))


def flag_names(status):
    return [n for bit, n in FLAGS.items() if status & bit]
