"""ctypes view of include/b200const.h: descriptor structs, constants and the loader of
libb200const.so.  The library is the only implementation: if it is missing or cannot be
loaded, importing a compute entry point raises -- there is no CPU path behind it."""
import ctypes as C
import os

MAX_RANK = 8

CLS_FLOAT, CLS_BFLOAT, CLS_INT, CLS_SINT, CLS_UINT = 1, 2, 3, 4, 5


def DTYPE(cls, bits):
    return (cls << 8) | bits


def dtype_bits(dt):
    return dt & 0xFF


def dtype_class(dt):
    return (dt >> 8) & 0xFF


F64, F32, F16 = DTYPE(CLS_FLOAT, 64), DTYPE(CLS_FLOAT, 32), DTYPE(CLS_FLOAT, 16)
BF16 = DTYPE(CLS_BFLOAT, 16)
I1, UI1 = DTYPE(CLS_INT, 1), DTYPE(CLS_UINT, 1)
I4, SI4, UI4 = DTYPE(CLS_INT, 4), DTYPE(CLS_SINT, 4), DTYPE(CLS_UINT, 4)
I8, SI8, UI8 = DTYPE(CLS_INT, 8), DTYPE(CLS_SINT, 8), DTYPE(CLS_UINT, 8)
I16, SI16, UI16 = DTYPE(CLS_INT, 16), DTYPE(CLS_SINT, 16), DTYPE(CLS_UINT, 16)
I32, SI32, UI32 = DTYPE(CLS_INT, 32), DTYPE(CLS_SINT, 32), DTYPE(CLS_UINT, 32)
I64, SI64, UI64 = DTYPE(CLS_INT, 64), DTYPE(CLS_SINT, 64), DTYPE(CLS_UINT, 64)

Q_NONE, Q_PER_TENSOR, Q_PER_AXIS = 0, 1, 2

X_CONVERT_ELEM_TYPE = 1
X_QUANT_CAST = 2
X_DEQUANTIZE = 3
X_RESCALE = 4
X_ADD = 5
X_REORDER = 6
X_SUBVIEW = 7
X_PAD_WITH_ZERO = 8
X_BIT_PACK = 9
X_GET_SPARSITY_MAP = 10
X_SPARSIFY = 11
X_SWIZZLE_CONSTANT = 12
X_RESHAPE = 13
X_CHANGE_SHAPE_AND_ELEM_TYPE = 14
X_BROADCAST = 15
X_TRANSPOSE = 16
X_REVERSE = 17
X_EXPAND_DILATED = 18
X_RELOCATE_WEIGHTS_TABLE = 19
X_QUANTIZE_SYNTH = 100

QSYNTH_SYM_I8, QSYNTH_ASYM_U4 = 0, 1

OK, NOT_SMALLER = 0, 1
ERR_INVALID, ERR_THROW, ERR_CUDA, ERR_NOMEM, ERR_CAPACITY, ERR_UNSUPPORTED = -1, -2, -3, -4, -5, -6

FOLD_ASYNC = 1
NOALLOC_MAX_INPUT = 16 << 20


class b200c_type(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32),
        ("rank", C.c_int32),
        ("shape", C.c_int64 * MAX_RANK),
        ("order", C.c_uint8 * MAX_RANK),
        ("qkind", C.c_int32),
        ("qaxis", C.c_int32),
        ("qexpressed", C.c_int32),
        ("_pad", C.c_int32),
        ("qmin", C.c_int64),
        ("qmax", C.c_int64),
        ("nq", C.c_int64),
        ("scales", C.POINTER(C.c_double)),
        ("zps", C.POINTER(C.c_int64)),
    ]


class b200c_xform(C.Structure):
    _fields_ = [
        ("kind", C.c_int32),
        ("n", C.c_int32),
        ("a", C.c_int64 * MAX_RANK),
        ("b", C.c_int64 * MAX_RANK),
        ("f", C.c_double),
        ("i0", C.c_int64),
        ("i1", C.c_int64),
        ("type", b200c_type),
        ("aux", C.POINTER(C.c_int64)),
        ("naux", C.c_int64),
        ("side0", C.c_void_p),
        ("side1", C.c_void_p),
    ]


class b200c_fold_item(C.Structure):
    _fields_ = [
        ("base", C.POINTER(b200c_type)),
        ("data", C.c_void_p),
        ("nbytes", C.c_size_t),
        ("is_splat", C.c_int32),
        ("n", C.c_int32),
        ("chain", C.POINTER(b200c_xform)),
        ("out", C.c_void_p),
        ("out_cap", C.c_size_t),
        ("out_bytes", C.c_size_t),
    ]


# the caller's device allocator (b200c_set_allocator)
ALLOC_FN = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_size_t)
FREE_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p)


class b200c_ipc_handle(C.Structure):
    _fields_ = [("handle", C.c_ubyte * 64), ("offset", C.c_uint64), ("size", C.c_uint64)]


class b200c_copy_seg(C.Structure):
    _fields_ = [("src", C.c_void_p), ("dst", C.c_void_p), ("n", C.c_size_t)]


# name -> (restype, argtypes) of every symbol include/b200const.h declares
_P = C.POINTER
SYMBOLS = {
    "b200c_create": (C.c_int, [C.c_int, _P(C.c_void_p)]),
    "b200c_destroy": (None, [C.c_void_p]),
    "b200c_set_allocator": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200c_set_stream": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200c_get_stream": (C.c_void_p, [C.c_void_p]),
    "b200c_synchronize": (C.c_int, [C.c_void_p]),
    "b200c_launch_count": (C.c_int64, [C.c_void_p]),
    "b200c_last_error": (C.c_char_p, []),
    "b200c_version": (C.c_char_p, []),
    "b200c_infer_type": (C.c_int, [_P(b200c_type), _P(b200c_xform), C.c_int, _P(b200c_type)]),
    "b200c_insert_position": (C.c_int, [_P(C.c_int32), C.c_int, C.c_int32, _P(C.c_int)]),
    "b200c_total_alloc_size": (C.c_int64, [_P(b200c_type)]),
    "b200c_fold": (C.c_int, [C.c_void_p, _P(b200c_type), C.c_void_p, C.c_size_t, C.c_int, C.c_int, _P(b200c_xform),
                             C.c_int, C.c_void_p, C.c_size_t, C.c_int, _P(C.c_size_t), _P(b200c_type), C.c_int]),
    "b200c_fold_batch": (C.c_int, [C.c_void_p, C.POINTER(b200c_fold_item), C.c_int, C.c_int, C.c_int, C.c_int]),
    "b200c_count_nonsparse_per_oc": (C.c_int, [C.c_void_p, _P(b200c_type), C.c_void_p, C.c_size_t, C.c_int, C.c_int,
                                               _P(b200c_xform), C.c_int, _P(C.c_int64), C.c_int64]),
    "b200c_btc_bound": (C.c_int, [C.c_size_t, _P(C.c_size_t)]),
    "b200c_btc_compress": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p, C.c_size_t, C.c_int,
                                     _P(C.c_size_t)]),
    "b200c_btc_compress_noalloc": (C.c_int, [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p,
                                             _P(C.c_size_t)]),
    "b200c_btc_decompress": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p, C.c_size_t, C.c_int,
                                       _P(C.c_size_t)]),
    "b200c_btc_compress_batch": (C.c_int, [C.c_void_p, C.c_int, _P(C.c_void_p), _P(C.c_size_t), C.c_void_p,
                                           C.c_size_t, _P(C.c_size_t), _P(C.c_size_t), _P(C.c_int32)]),
    "b200c_btc_compress_inplace_batch": (C.c_int, [C.c_void_p, C.c_int, _P(C.c_void_p), _P(C.c_size_t), _P(C.c_size_t),
                                                   _P(C.c_int32)]),
    "b200c_btc_compress_inplace_begin": (C.c_int, [C.c_void_p, C.c_int, _P(C.c_void_p), _P(C.c_size_t), _P(C.c_int)]),
    "b200c_btc_compress_inplace_end": (C.c_int, [C.c_void_p, C.c_int, _P(C.c_size_t), _P(C.c_int32)]),
    "b200c_synth_fill": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_double, C.c_double,
                                   C.c_uint64, C.c_uint64]),
    "b200c_detect_splat": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, _P(C.c_int)]),
    "b200c_digest64_batch": (C.c_int, [C.c_void_p, C.c_int, _P(C.c_void_p), _P(C.c_size_t), _P(C.c_uint64)]),
    "b200c_ipc_export": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, _P(b200c_ipc_handle)]),
    "b200c_ipc_open": (C.c_int, [C.c_void_p, _P(b200c_ipc_handle), _P(C.c_void_p)]),
    "b200c_ipc_close": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200c_copy_segments_async": (C.c_int, [C.c_void_p, _P(b200c_copy_seg), C.c_int, C.c_void_p, C.c_uint64, C.c_void_p,
                                            C.c_uint64, C.c_uint, C.c_int, C.c_int]),
    "b200c_copy_segments_after": (C.c_int, [C.c_void_p, C.c_int, _P(b200c_copy_seg), C.c_int, C.c_void_p, C.c_uint64, C.c_void_p,
                                            C.c_uint64, C.c_uint, C.c_int, C.c_int]),
    "b200c_wait_flags": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_uint64, C.c_uint, C.c_int]),
    "b200c_signal_flags": (C.c_int, [C.c_void_p, _P(C.c_void_p), C.c_int, C.c_uint64]),
    "b200c_exchange_status": (C.c_int, [C.c_void_p, _P(C.c_int)]),
    "b200c_stream_join": (C.c_int, [C.c_void_p]),
    "b200c_dev_alloc": (C.c_int, [C.c_void_p, C.c_size_t, _P(C.c_void_p)]),
    "b200c_dev_free": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200c_host_alloc_pinned": (C.c_int, [C.c_size_t, _P(C.c_void_p)]),
    "b200c_host_free_pinned": (C.c_int, [C.c_void_p]),
    "b200c_dev_memset": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_size_t]),
    "b200c_memcpy_h2d": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "b200c_memcpy_d2h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
}

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc", "libb200const.so")
_lib = None


def bind(lib, symbols, prefix_from="b200c_", prefix_to="b200c_"):
    """Attach restype/argtypes; a missing symbol is an error."""
    for name, (res, args) in symbols.items():
        real = prefix_to + name[len(prefix_from):]
        fn = getattr(lib, real)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    return lib


def load():
    """Load libb200const.so (built by __graft_entry__.build / csrc/build.sh)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'`. "
                "There is no CPU implementation to fall back to.")
        _lib = bind(C.CDLL(LIB_PATH), SYMBOLS)
    return _lib
