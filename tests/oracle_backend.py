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
    lib.orc_synth_fill.argtypes = [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_double, C.c_double, C.c_uint64,
                                   C.c_uint64]
    lib.orc_digest64.restype = C.c_uint64
    lib.orc_digest64.argtypes = [C.c_void_p, C.c_uint64]
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
        n = K.quick_q_of(base_type, transforms)
        for attempt in (0, 1):
            keep = []
            out = K.out_type_slot(n, keep)
            bt = base_type.to_c(keep)
            ch = K.chain_to_c(transforms, keep)
            rc = self.lib.orc_infer_type(C.byref(bt), ch, len(transforms), C.byref(out))
            if rc != A.OK and attempt == 0 and out.nq > n:  # the type needs more room than the first guess: it says how much
                n = int(out.nq)
                continue
            K.raise_for(rc, self._err())
            return K.NDType.from_c(out)

    def detect_splat(self, data, elem_bytes):
        """detectSplatElementWise (content.cpp:103-118) in numpy."""
        buf = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        if buf.size == 0:
            return False
        if buf.size < elem_bytes:
            raise K.ConstError("The data must contain at least one element")
        if buf.size % elem_bytes:
            raise K.ConstError("The data array has unexpected length")
        rows = buf.reshape(-1, elem_bytes)
        return bool((rows == rows[0]).all())

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
        ot = K.out_type_slot(max(K.q_slots_of(final), K.quick_q_of(base_type, transforms)), keep)
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

    # resident contents: for the CPU oracle "resident" memory is host memory
    def fold_resident(self, base_type, data, is_splat, transforms):
        if isinstance(data, K.ResidentContent):
            data = data.buf
        c = self.fold(base_type, data, is_splat, transforms)
        raw = np.array(c.copyTo(), copy=True)
        return K.ResidentContent(self, c.getType(), raw, raw.size, c.bytesWritten)

    def resident_to_host(self, rc):
        return rc.buf

    def free_resident(self, rc):
        rc.buf = None

    def synth_fill(self, count, dtype, dist, p0, p1, seed, stream_id):
        """CPU twin of b200c_synth_fill: the same bytes as the device generator."""
        out = np.zeros(int(count) * A.dtype_bits(dtype) // 8, dtype=np.uint8)
        rc = self.lib.orc_synth_fill(out.ctypes.data, int(count), dtype, dist, p0, p1, seed, stream_id)
        if rc != 0:
            raise ValueError("orc_synth_fill: bad arguments")
        return out

    def synth_of(self, decl, seed):
        dt, dist, p0, p1 = decl.synth
        return self.synth_fill(decl.nbytes * 8 // A.dtype_bits(dt), dt, dist, p0, p1, seed, decl.stream)

    def digest64(self, data):
        buf = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        return int(self.lib.orc_digest64(buf.ctypes.data if buf.size else None, buf.size))


class OracleShardFolder:
    """CPU stand-in for npu_plugin_b200.blob.ShardFolder with the same interface: "pointers" are addresses
    of host memory, folding and compression run in the oracle.  Lets the sharded whole-model routine run
    on CPU ranks (gloo) with real folded bytes."""

    def __init__(self, backend, decls):
        from npu_plugin_b200.blob import MIN_COMPRESS_BYTES, SEGMENT_ALIGN
        self.b, self.decls = backend, decls
        self.folded_offsets, self.folded_sizes = [], []
        at = 0
        for d in decls:
            size = backend.infer_type(d.base_type, d.transforms).getTotalAllocSize()
            self.folded_offsets.append(at)
            self.folded_sizes.append(size)
            at = (at + size + SEGMENT_ALIGN - 1) // SEGMENT_ALIGN * SEGMENT_ALIGN
        self.folded_bytes = max(at, 1)
        self.comp_idx = [i for i, d in enumerate(decls) if d.compress and self.folded_sizes[i] >= MIN_COMPRESS_BYTES]

    @staticmethod
    def _view(ptr, n):
        return np.ctypeslib.as_array((C.c_ubyte * max(1, n)).from_address(ptr))[:n]

    def fold(self, data_ptrs, folded_ptr, data_on_device=True, side_ptrs=None, max_batch_bytes=None):
        for i, d in enumerate(self.decls):
            x = self._view(data_ptrs[i], d.nbytes)
            ts = d.transforms
            for t in ts:
                if t.kind == A.X_QUANTIZE_SYNTH:
                    oc = d.base_type.shape[0]
                    t.side0, t.side1 = np.zeros(oc, np.float32), np.zeros(oc, np.int32)
            out = self.b.fold(d.base_type, x, d.is_splat, ts).copyTo()
            self._view(folded_ptr + self.folded_offsets[i], self.folded_sizes[i])[:out.size] = out

    def compress_inplace(self, folded_ptr):
        size, flag = list(self.folded_sizes), [False] * len(self.decls)
        for i in self.comp_idx:
            slot = self._view(folded_ptr + self.folded_offsets[i], self.folded_sizes[i])
            stream, not_smaller = self.b.btc_compress(slot.copy())
            if not not_smaller:
                slot[:stream.size] = stream
                size[i], flag[i] = stream.size, True
        return [(i, self.folded_offsets[i], size[i], flag[i]) for i in range(len(self.decls))]
