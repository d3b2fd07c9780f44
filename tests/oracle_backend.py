"""ctypes wrapper of the CPU oracle (oracle/liboracle.so) exposing the same backend interface as
npu_plugin_b200.const.CudaBackend, so a ContentAttr can be folded on either side."""
import ctypes as C
import os
import subprocess

import numpy as np

from npu_plugin_b200 import _cabi as A
from npu_plugin_b200 import const as K

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "oracle", "liboracle.so")
_P = C.POINTER


def build():
    subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle")])


def _load():
    src = os.path.join(ROOT, "oracle", "const_oracle.cpp")
    if not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        build()
    lib = C.CDLL(LIB)
    lib.orc_last_error.restype = C.c_char_p
    lib.orc_set_threads.restype = C.c_int
    lib.orc_set_threads.argtypes = [C.c_int]
    lib.orc_infer_type.argtypes = [_P(A.b200c_type), _P(A.b200c_xform), C.c_int, _P(A.b200c_type)]
    lib.orc_insert_position.argtypes = [_P(C.c_int32), C.c_int, C.c_int32, _P(C.c_int)]
    lib.orc_total_alloc_size.restype = C.c_int64
    lib.orc_total_alloc_size.argtypes = [_P(A.b200c_type)]
    lib.orc_fold.argtypes = [_P(A.b200c_type), C.c_void_p, C.c_size_t, C.c_int, _P(A.b200c_xform), C.c_int,
                             C.c_void_p, C.c_size_t, _P(C.c_size_t), _P(A.b200c_type)]
    lib.orc_count_nonsparse_per_oc.argtypes = [_P(A.b200c_type), C.c_void_p, C.c_size_t, C.c_int, _P(A.b200c_xform),
                                               C.c_int, _P(C.c_int64), C.c_int64]
    lib.orc_swizzle.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_uint32]
    lib.orc_deswizzle.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_uint32]
    lib.orc_btc_bound.argtypes = [C.c_size_t, _P(C.c_size_t)]
    lib.orc_btc_compress.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, _P(C.c_size_t)]
    lib.orc_btc_decompress.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, _P(C.c_size_t)]
    lib.orc_f32_to_f16.restype = C.c_uint16
    lib.orc_f32_to_f16.argtypes = [C.c_float]
    lib.orc_f16_to_f32.restype = C.c_float
    lib.orc_f16_to_f32.argtypes = [C.c_uint16]
    lib.orc_f32_to_bf16.restype = C.c_uint16
    lib.orc_f32_to_bf16.argtypes = [C.c_float]
    return lib


class OracleBackend:
    name = "oracle"

    def __init__(self):
        self.lib = _load()

    def _err(self):
        return self.lib.orc_last_error()

    def set_threads(self, n):
        return self.lib.orc_set_threads(n)

    def infer_type(self, base_type, transforms):
        keep = []
        out = K.out_type_slot(K.max_q_of(base_type, transforms), keep)
        bt = base_type.to_c(keep)
        ch = K.chain_to_c(transforms, keep)
        K.raise_for(self.lib.orc_infer_type(C.byref(bt), ch, len(transforms), C.byref(out)), self._err())
        return K.NDType.from_c(out)

    def insert_position(self, kinds, new_kind):
        arr = (C.c_int32 * max(1, len(kinds)))(*kinds)
        pos = C.c_int()
        K.raise_for(self.lib.orc_insert_position(arr, len(kinds), new_kind, C.byref(pos)), self._err())
        return pos.value

    def fold(self, base_type, data, is_splat, transforms):
        keep = []
        bt = base_type.to_c(keep)
        ch = K.chain_to_c(transforms, keep)
        final = self.infer_type(base_type, transforms)
        cap = max(final.getTotalAllocSize(), 1)
        out = np.zeros(cap, dtype=np.uint8)
        ot = K.out_type_slot(K.max_q_of(base_type, transforms), keep)
        nb = C.c_size_t()
        buf = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        rc = self.lib.orc_fold(C.byref(bt), buf.ctypes.data, buf.size, int(is_splat), ch, len(transforms),
                               out.ctypes.data, cap, C.byref(nb), C.byref(ot))
        K.raise_for(rc, self._err())
        t = K.NDType.from_c(ot)
        return K.Content(t, out[:max(t.getTotalAllocSize(), nb.value)], nb.value)

    def count_nonsparse_per_oc(self, base_type, data, is_splat, transforms):
        keep = []
        bt = base_type.to_c(keep)
        ch = K.chain_to_c(transforms, keep)
        t = self.infer_type(base_type, transforms)
        oc = t.shape[0]
        counts = (C.c_int64 * max(1, oc))()
        buf = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        rc = self.lib.orc_count_nonsparse_per_oc(C.byref(bt), buf.ctypes.data, buf.size, int(is_splat), ch,
                                                 len(transforms), counts, oc)
        K.raise_for(rc, self._err())
        return [counts[i] for i in range(oc)]

    def swizzle(self, data, key):
        buf = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        out = np.zeros_like(buf)
        K.raise_for(self.lib.orc_swizzle(buf.ctypes.data, buf.size, out.ctypes.data, key), self._err())
        return out

    def deswizzle(self, data, key):
        buf = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        out = np.zeros_like(buf)
        K.raise_for(self.lib.orc_deswizzle(buf.ctypes.data, buf.size, out.ctypes.data, key), self._err())
        return out

    def btc_bound(self, n):
        b = C.c_size_t()
        self.lib.orc_btc_bound(n, C.byref(b))
        return b.value

    def btc_compress(self, data):
        buf = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        cap = self.btc_bound(buf.size)
        out = np.zeros(cap, dtype=np.uint8)
        n = C.c_size_t()
        rc = self.lib.orc_btc_compress(buf.ctypes.data, buf.size, out.ctypes.data, cap, C.byref(n))
        K.raise_for(rc, self._err())
        return out[:n.value], rc == A.NOT_SMALLER

    def btc_decompress(self, stream, n_out):
        buf = np.ascontiguousarray(stream).view(np.uint8).reshape(-1)
        out = np.zeros(max(1, n_out), dtype=np.uint8)
        n = C.c_size_t()
        rc = self.lib.orc_btc_decompress(buf.ctypes.data, buf.size, out.ctypes.data, n_out, C.byref(n))
        K.raise_for(rc, self._err())
        return out[:n.value]
