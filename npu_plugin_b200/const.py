"""Host-side mirror of the reference's Const dialect API for Python callers.

Names follow vpux::Const (src/vpux_compiler/tblgen/vpux/compiler/dialect/const/attributes.td:72-107):
ContentAttr with its builder methods (convertElemType, quantCast, dequantize, rescale, add, reorder,
padWithZero, subview, bitPack, getSparsityMap, sparsify, swizzleConstant, reshape, ...), Content
(getType, isSplat, copyTo, getValues) and DeclareOp.getContent().  The arithmetic runs in
libb200const.so on the GPU; this module only marshals descriptors.

A `backend` object supplies infer_type / insert_position / fold / ...; the default is the CUDA
library.  Tests pass the CPU oracle's backend to run the same chain on both sides.
"""
import ctypes as C

import numpy as np

from . import _cabi as A


class ConstError(RuntimeError):
    """The reference would have raised VPUX_THROW here; the message is the reference-style text."""


class Unsupported(RuntimeError):
    pass


class CudaError(RuntimeError):
    pass


def raise_for(rc, msg):
    if rc in (A.OK, A.NOT_SMALLER):
        return rc
    text = msg.decode() if isinstance(msg, bytes) else str(msg)
    if rc == A.ERR_THROW:
        raise ConstError(text)
    if rc == A.ERR_UNSUPPORTED:
        raise Unsupported(text)
    if rc in (A.ERR_CUDA, A.ERR_NOMEM):
        raise CudaError(text)
    raise ValueError(f"b200c error {rc}: {text}")


# --------------------------------------------------------------------------- DimsOrder
class DimsOrder(tuple):
    """Permutation, outermost memory dim first (DimsOrder::toPermutation,
    src/vpux_compiler/src/core/attributes/dims_order.cpp)."""

    @staticmethod
    def fromCode(code):
        digits = []
        while code:
            digits.append((code & 0xF) - 1)
            code >>= 4
        return DimsOrder(reversed(digits))

    @staticmethod
    def fromNumDims(n):
        return DimsOrder(range(n))

    def code(self):
        c = 0
        for d in self:
            c = (c << 4) | (d + 1)
        return c

    def dimPos(self, d):
        return self.index(d)


DimsOrder.C = DimsOrder((0,))
DimsOrder.NC = DimsOrder((0, 1))
DimsOrder.CHW = DimsOrder((0, 1, 2))
DimsOrder.HWC = DimsOrder((1, 2, 0))
DimsOrder.NCHW = DimsOrder((0, 1, 2, 3))
DimsOrder.NHWC = DimsOrder((0, 2, 3, 1))
DimsOrder.NHCW = DimsOrder((0, 2, 1, 3))
DimsOrder.OIYX = DimsOrder.NCHW
DimsOrder.OYXI = DimsOrder.NHWC
DimsOrder.YXOI = DimsOrder((2, 3, 0, 1))
DimsOrder.NCDHW = DimsOrder((0, 1, 2, 3, 4))
DimsOrder.NDHWC = DimsOrder((0, 2, 3, 4, 1))


# --------------------------------------------------------------------------- element types
class Quant:
    """mlir::quant::UniformQuantizedType / UniformQuantizedPerAxisType."""

    def __init__(self, kind, storage, expressed, scales, zps, axis=0, qmin=None, qmax=None):
        self.kind = kind
        self.storage = storage  # normalised storage integer dtype (si8/ui8/si4/ui4)
        self.expressed = expressed
        self.scales = [float(s) for s in scales]
        self.zps = [int(z) for z in zps]
        self.axis = int(axis)
        bits = A.dtype_bits(storage)
        signed = A.dtype_class(storage) == A.CLS_SINT
        self.qmin = int(qmin) if qmin is not None else (-(1 << (bits - 1)) if signed else 0)
        self.qmax = int(qmax) if qmax is not None else ((1 << (bits - 1)) - 1 if signed else (1 << bits) - 1)

    def __eq__(self, o):
        return isinstance(o, Quant) and (self.kind, self.storage, self.expressed, self.scales, self.zps, self.axis,
                                         self.qmin, self.qmax) == (o.kind, o.storage, o.expressed, o.scales, o.zps,
                                                                   o.axis, o.qmin, o.qmax)

    def __repr__(self):
        return (f"Quant(kind={self.kind}, storage={self.storage:#x}, axis={self.axis}, n={len(self.scales)}, "
                f"range=[{self.qmin},{self.qmax}])")


def UniformQuantizedType(storage, expressed, scale, zeroPoint, qmin=None, qmax=None):
    return Quant(A.Q_PER_TENSOR, storage, expressed, [scale], [zeroPoint], 0, qmin, qmax)


def UniformQuantizedPerAxisType(storage, expressed, scales, zeroPoints, axis, qmin=None, qmax=None):
    return Quant(A.Q_PER_AXIS, storage, expressed, scales, zeroPoints, axis, qmin, qmax)


def _np_dtype(dt):
    m = {A.F64: np.float64, A.F32: np.float32, A.F16: np.float16, A.BF16: np.uint16, A.I8: np.uint8,
         A.SI8: np.int8, A.UI8: np.uint8, A.I16: np.uint16, A.SI16: np.int16, A.UI16: np.uint16, A.I32: np.uint32,
         A.SI32: np.int32, A.UI32: np.uint32, A.I64: np.uint64, A.SI64: np.int64, A.UI64: np.uint64}
    return np.dtype(m[dt])


class NDType:
    """shape + element type (+ DimsOrder): the part of vpux::NDTypeInterface constants use."""

    def __init__(self, shape, elem, order=None):
        self.shape = tuple(int(s) for s in shape)
        self.quant = elem if isinstance(elem, Quant) else None
        self.dtype = elem.storage if isinstance(elem, Quant) else int(elem)
        self.order = DimsOrder(order) if order is not None else DimsOrder.fromNumDims(len(self.shape))

    @property
    def rank(self):
        return len(self.shape)

    def getNumElements(self):
        n = 1
        for s in self.shape:
            n *= s
        return n

    def getElemTypeSize(self):
        return A.dtype_bits(self.dtype)

    def getTotalAllocSize(self):
        n = 1 if self.rank == 0 else self.getNumElements()
        return (self.getElemTypeSize() * n + 7) // 8

    def getMemShape(self):
        return tuple(self.shape[d] for d in self.order)

    def getElementType(self):
        return self.quant if self.quant is not None else self.dtype

    def __eq__(self, o):
        return isinstance(o, NDType) and (self.shape, self.dtype, self.quant, tuple(self.order)) == (
            o.shape, o.dtype, o.quant, tuple(o.order))

    def __repr__(self):
        return f"NDType({self.shape}, {self.dtype:#x}, order={tuple(self.order)}, quant={self.quant})"

    # ---- marshalling
    def to_c(self, keep):
        t = A.b200c_type()
        t.dtype = self.dtype
        t.rank = self.rank
        for k, s in enumerate(self.shape):
            t.shape[k] = s
        for k, d in enumerate(self.order):
            t.order[k] = d
        if self.quant is not None:
            q = self.quant
            t.qkind, t.qaxis, t.qexpressed = q.kind, q.axis, q.expressed
            t.qmin, t.qmax = q.qmin, q.qmax
            t.nq = len(q.scales)
            sc = (C.c_double * max(1, len(q.scales)))(*q.scales)
            zp = (C.c_int64 * max(1, len(q.zps)))(*q.zps)
            keep.extend([sc, zp])
            t.scales = C.cast(sc, C.POINTER(C.c_double))
            t.zps = C.cast(zp, C.POINTER(C.c_int64))
        return t

    @staticmethod
    def from_c(t):
        shape = [t.shape[k] for k in range(t.rank)]
        order = [t.order[k] for k in range(t.rank)]
        elem = t.dtype
        if t.qkind != A.Q_NONE:
            elem = Quant(t.qkind, t.dtype, t.qexpressed, [t.scales[i] for i in range(t.nq)],
                         [t.zps[i] for i in range(t.nq)], t.qaxis, t.qmin, t.qmax)
        return NDType(shape, elem, order)


def out_type_slot(max_q, keep):
    """A b200c_type with caller storage for up to max_q quantisation parameters."""
    t = A.b200c_type()
    sc = (C.c_double * max(1, max_q))()
    zp = (C.c_int64 * max(1, max_q))()
    keep.extend([sc, zp])
    t.nq = max_q
    t.scales = C.cast(sc, C.POINTER(C.c_double))
    t.zps = C.cast(zp, C.POINTER(C.c_int64))
    return t


# --------------------------------------------------------------------------- transformations
_NAMES = {A.X_CONVERT_ELEM_TYPE: "ConvertElemType", A.X_QUANT_CAST: "QuantCast", A.X_DEQUANTIZE: "Dequantize",
          A.X_RESCALE: "Rescale", A.X_ADD: "Add", A.X_REORDER: "Reorder", A.X_SUBVIEW: "SubView",
          A.X_PAD_WITH_ZERO: "PadWithZero", A.X_BIT_PACK: "BitPack", A.X_GET_SPARSITY_MAP: "GetSparsityMap",
          A.X_SPARSIFY: "Sparsify", A.X_SWIZZLE_CONSTANT: "SwizzleConstant", A.X_RESHAPE: "Reshape",
          A.X_CHANGE_SHAPE_AND_ELEM_TYPE: "ChangeShapeAndElemType", A.X_BROADCAST: "Broadcast",
          A.X_TRANSPOSE: "Transpose", A.X_REVERSE: "Reverse", A.X_EXPAND_DILATED: "ExpandDilated", A.X_RELOCATE_WEIGHTS_TABLE: "RelocateWeightsTable",
          A.X_QUANTIZE_SYNTH: "QuantizeSynth"}


class Transform:
    """One Const::TransformAttrInterface instance."""

    def __init__(self, kind, a=(), b=(), f=0.0, i0=0, i1=0, elem=None, aux=None, side0=None, side1=None):
        self.kind, self.a, self.b, self.f, self.i0, self.i1 = kind, tuple(a), tuple(b), float(f), int(i0), int(i1)
        self.elem, self.aux, self.side0, self.side1 = elem, (None if aux is None else [int(v) for v in aux]), side0, side1

    def getTransformationName(self):
        return _NAMES[self.kind]

    def key(self):
        """Value identity of the transformation (MLIR attributes are uniqued by value)."""
        e = self.elem
        ek = (e.kind, e.storage, e.expressed, tuple(e.scales), tuple(e.zps), e.axis, e.qmin, e.qmax) if isinstance(e, Quant) else e
        return (self.kind, self.a, self.b, self.f, self.i0, self.i1, ek, None if self.aux is None else tuple(self.aux))

    def __eq__(self, o):
        return isinstance(o, Transform) and self.key() == o.key()

    def __hash__(self):
        return hash(self.key())

    def __repr__(self):
        return f"#const.{_NAMES[self.kind]}"

    @staticmethod
    def _ptr(side):
        if side is None:
            return None
        if isinstance(side, np.ndarray):
            return side.ctypes.data
        return int(side)

    def to_c(self, keep):
        x = A.b200c_xform()
        x.kind = self.kind
        n = max(len(self.a), len(self.b))
        x.n = n
        for k, v in enumerate(self.a):
            x.a[k] = v
        for k, v in enumerate(self.b):
            x.b[k] = v
        x.f, x.i0, x.i1 = self.f, self.i0, self.i1
        if self.elem is not None:
            x.type = NDType((), self.elem).to_c(keep)
        if self.aux is not None:
            arr = (C.c_int64 * max(1, len(self.aux)))(*self.aux)
            keep.append(arr)
            x.aux = C.cast(arr, C.POINTER(C.c_int64))
            x.naux = len(self.aux)
        x.side0 = self._ptr(self.side0)
        x.side1 = self._ptr(self.side1)
        return x


def chain_to_c(transforms, keep):
    arr = (A.b200c_xform * max(1, len(transforms)))()
    for i, t in enumerate(transforms):
        arr[i] = t.to_c(keep)
    return arr


def quick_q_of(base_type, transforms):
    """First guess for the parameter storage of a chain's output type: the longest parameter list that goes in,
    or the largest extent named anywhere (a per-axis list is as long as one dimension)."""
    m = max([1] + list(base_type.shape))
    if base_type.quant is not None:
        m = max(m, len(base_type.quant.scales))
    for t in transforms:
        for v in list(t.a) + list(t.b) + [t.i1]:
            m = max(m, abs(int(v)))
        if isinstance(t.elem, Quant):
            m = max(m, len(t.elem.scales))
    return min(m, 1 << 24) + 64


def infer_type_through(entry, last_error, base_type, transforms):
    """b200c_infer_type behind `entry`, with parameter storage sized by quick_q_of and, when the library answers
    that the output type needs more (it reports how many in the type's nq), once more with that."""
    n = quick_q_of(base_type, transforms)
    for attempt in (0, 1):
        keep = []
        out = out_type_slot(n, keep)
        bt = base_type.to_c(keep)
        ch = chain_to_c(transforms, keep)
        rc = entry(C.byref(bt), ch, len(transforms), C.byref(out))
        if rc == A.ERR_CAPACITY and attempt == 0 and out.nq > n:
            n = int(out.nq)
            continue
        raise_for(rc, last_error())
        return NDType.from_c(out)


def q_slots_of(ndtype):
    """Parameter storage an output type slot needs when the type is already known."""
    return max(1, len(ndtype.quant.scales)) if ndtype.quant is not None else 1


# --------------------------------------------------------------------------- Content
class Content:
    """Result of ContentAttr.fold(): the folded type plus the bytes Content::copyTo writes."""

    def __init__(self, ndtype, raw, written, splat=False):
        self._type, self._raw, self._written, self._splat = ndtype, raw, written, splat

    def getType(self):
        return self._type

    def copyTo(self, buf=None):
        """Bytes copyTo writes into a zero-initialised buffer of getTotalAllocSize bytes."""
        if buf is None:
            return self._raw
        b = np.frombuffer(buf, dtype=np.uint8) if not isinstance(buf, np.ndarray) else buf.view(np.uint8).reshape(-1)
        b[:self._written] = self._raw[:self._written]
        return buf

    @property
    def bytesWritten(self):
        return self._written

    def getValues(self, np_dtype=None):
        dt = np.dtype(np_dtype) if np_dtype is not None else _np_dtype(self._type.dtype)
        if self._type.getElemTypeSize() < 8:
            raise ConstError(f"Unsupported storage type of size '{self._type.getElemTypeSize()}' bits.")
        vals = self._raw[:self._type.getNumElements() * _np_dtype(self._type.dtype).itemsize].view(
            _np_dtype(self._type.dtype))
        return vals.astype(dt) if dt != vals.dtype else vals


class ResidentContent:
    """A folded constant whose bytes stay where the backend computes (device memory for the CUDA backend): the
    folded type, the byte count copyTo writes, and the buffer.  to_content() brings the bytes to the host."""

    def __init__(self, backend, ndtype, buf, nbytes, written):
        self.backend, self.type, self.buf, self.nbytes, self.written = backend, ndtype, buf, int(nbytes), int(written)
        self._released = False

    def type_as_base(self):
        """The type a base content of these bytes has: shape, storage element type and order (quantisation
        parameters are not part of a base content; the next QuantCast of a chain re-attaches them)."""
        return NDType(self.type.shape, self.type.dtype, self.type.order)

    def to_content(self):
        raw = self.backend.resident_to_host(self)
        return Content(self.type, raw, self.written)

    def release(self):
        if not self._released:
            self._released = True
            self.backend.free_resident(self)


# --------------------------------------------------------------------------- backend (CUDA library)
class CudaBackend:
    """Calls libb200const.so; one b200c_ctx per backend object."""

    name = "b200"

    def __init__(self, device=0):
        self.lib = A.load()
        h = C.c_void_p()
        raise_for(self.lib.b200c_create(device, C.byref(h)), self.lib.b200c_last_error())
        self.ctx = h
        self.device = device

    def close(self):
        if self.ctx:
            self.lib.b200c_destroy(self.ctx)
            self.ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _err(self):
        return self.lib.b200c_last_error()

    # host-only entry points
    def infer_type(self, base_type, transforms):
        return infer_type_through(self.lib.b200c_infer_type, self._err, base_type, transforms)

    def insert_position(self, kinds, new_kind):
        arr = (C.c_int32 * max(1, len(kinds)))(*kinds)
        pos = C.c_int()
        raise_for(self.lib.b200c_insert_position(arr, len(kinds), new_kind, C.byref(pos)), self._err())
        return pos.value

    # compute entry points
    def fold(self, base_type, data, is_splat, transforms):
        keep = []
        bt = base_type.to_c(keep)
        ch = chain_to_c(transforms, keep)
        final = self.infer_type(base_type, transforms)
        # the folded Content can be larger than the attribute's type says only for Sparsify<false>
        # (never: it is smaller); the inferred size is therefore a safe capacity.
        cap = max(final.getTotalAllocSize(), 1)
        out = np.zeros(cap, dtype=np.uint8)
        ot = out_type_slot(max(q_slots_of(final), quick_q_of(base_type, transforms)), keep)
        nb = C.c_size_t()
        buf = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        rc = self.lib.b200c_fold(self.ctx, C.byref(bt), buf.ctypes.data, buf.size, int(is_splat), 0, ch,
                                 len(transforms), out.ctypes.data, cap, 0, C.byref(nb), C.byref(ot), 0)
        raise_for(rc, self._err())
        t = NDType.from_c(ot)
        return Content(t, out[:max(t.getTotalAllocSize(), nb.value)], nb.value)

    def fold_resident(self, base_type, data, is_splat, transforms):
        """fold() + copyTo() with the result left in device memory.  `data` is a host array or a ResidentContent
        (a cached folded prefix, read where it lies)."""
        keep = []
        bt = base_type.to_c(keep)
        ch = chain_to_c(transforms, keep)
        final = self.infer_type(base_type, transforms)
        cap = max(final.getTotalAllocSize(), 1)
        out = self.dev_alloc(cap)
        ot = out_type_slot(max(q_slots_of(final), quick_q_of(base_type, transforms)), keep)
        nb = C.c_size_t()
        try:
            self.fill_zero(out, cap)
            if isinstance(data, ResidentContent):
                src, n, on_dev = data.buf, data.nbytes, 1
            else:
                buf = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
                src, n, on_dev = buf.ctypes.data, buf.size, 0
            rc = self.lib.b200c_fold(self.ctx, C.byref(bt), src, n, int(is_splat), on_dev, ch, len(transforms), out, cap, 1,
                                     C.byref(nb), C.byref(ot), 0)
            raise_for(rc, self._err())
        except Exception:
            self.dev_free(out)
            raise
        t = NDType.from_c(ot)
        return ResidentContent(self, t, out, max(t.getTotalAllocSize(), nb.value), nb.value)

    def resident_to_host(self, rc):
        return self.download(rc.buf, rc.nbytes)

    def free_resident(self, rc):
        self.dev_free(rc.buf)

    def count_nonsparse_per_oc(self, base_type, data, is_splat, transforms):
        keep = []
        bt = base_type.to_c(keep)
        ch = chain_to_c(transforms, keep)
        t = self.infer_type(base_type, [x for x in transforms])
        oc = t.shape[0]
        counts = (C.c_int64 * max(1, oc))()
        buf = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        rc = self.lib.b200c_count_nonsparse_per_oc(self.ctx, C.byref(bt), buf.ctypes.data, buf.size, int(is_splat), 0,
                                                   ch, len(transforms), counts, oc)
        raise_for(rc, self._err())
        return [counts[i] for i in range(oc)]

    def btc_bound(self, n):
        b = C.c_size_t()
        raise_for(self.lib.b200c_btc_bound(n, C.byref(b)), self._err())
        return b.value

    def btc_compress(self, data):
        """Returns (stream bytes, not_smaller flag)."""
        buf = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        cap = self.btc_bound(buf.size)
        out = np.zeros(cap, dtype=np.uint8)
        n = C.c_size_t()
        rc = self.lib.b200c_btc_compress(self.ctx, buf.ctypes.data, buf.size, 0, out.ctypes.data, cap, 0, C.byref(n))
        raise_for(rc, self._err())
        return out[:n.value], rc == A.NOT_SMALLER

    def btc_decompress(self, stream, n_out):
        buf = np.ascontiguousarray(stream).view(np.uint8).reshape(-1)
        out = np.zeros(max(1, n_out), dtype=np.uint8)
        n = C.c_size_t()
        rc = self.lib.b200c_btc_decompress(self.ctx, buf.ctypes.data, buf.size, 0, out.ctypes.data, n_out, 0,
                                           C.byref(n))
        raise_for(rc, self._err())
        return out[:n.value]

    def launch_count(self):
        return self.lib.b200c_launch_count(self.ctx)

    def synchronize(self):
        raise_for(self.lib.b200c_synchronize(self.ctx), self._err())

    def detect_splat(self, data, elem_bytes):
        """detectSplatElementWise (content.cpp:103-137) on a host array."""
        buf = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        flag = C.c_int()
        raise_for(self.lib.b200c_detect_splat(self.ctx, buf.ctypes.data if buf.size else None, buf.size, elem_bytes, 0,
                                              C.byref(flag)), self._err())
        return bool(flag.value)

    # ---- device memory and the multi-GPU exchange (thin wrappers; pointers are plain integers)
    def dev_alloc(self, nbytes):
        p = C.c_void_p()
        raise_for(self.lib.b200c_dev_alloc(self.ctx, max(1, int(nbytes)), C.byref(p)), self._err())
        return p.value

    def dev_free(self, ptr):
        if ptr:
            self.lib.b200c_dev_free(self.ctx, ptr)

    def pinned_alloc(self, nbytes):
        p = C.c_void_p()
        raise_for(self.lib.b200c_host_alloc_pinned(max(1, int(nbytes)), C.byref(p)), self._err())
        return p.value

    def pinned_free(self, ptr):
        if ptr:
            self.lib.b200c_host_free_pinned(ptr)

    def upload(self, dev_ptr, array):
        a = np.ascontiguousarray(array).view(np.uint8).reshape(-1)
        raise_for(self.lib.b200c_memcpy_h2d(self.ctx, dev_ptr, a.ctypes.data, a.size), self._err())

    def download(self, dev_ptr, nbytes):
        out = np.zeros(int(nbytes), np.uint8)
        raise_for(self.lib.b200c_memcpy_d2h(self.ctx, out.ctypes.data, dev_ptr, out.size), self._err())
        return out

    def fill_zero(self, dev_ptr, nbytes):
        raise_for(self.lib.b200c_dev_memset(self.ctx, dev_ptr, 0, int(nbytes)), self._err())
        self.synchronize()

    def synth_fill(self, dev_ptr, count, dtype, dist, p0, p1, seed, stream_id):
        raise_for(self.lib.b200c_synth_fill(self.ctx, dev_ptr, int(count), dtype, dist, p0, p1, seed, stream_id), self._err())

    def digest64(self, ptrs, sizes):
        n = len(ptrs)
        if n == 0:
            return []
        pa = (C.c_void_p * n)(*ptrs)
        sa = (C.c_size_t * n)(*sizes)
        out = (C.c_uint64 * n)()
        raise_for(self.lib.b200c_digest64_batch(self.ctx, n, pa, sa, out), self._err())
        return [int(v) for v in out]

    def ipc_export(self, dev_ptr, nbytes):
        h = A.b200c_ipc_handle()
        raise_for(self.lib.b200c_ipc_export(self.ctx, dev_ptr, int(nbytes), C.byref(h)), self._err())
        return bytes(h)

    def ipc_open(self, desc):
        h = A.b200c_ipc_handle.from_buffer_copy(desc)
        p = C.c_void_p()
        raise_for(self.lib.b200c_ipc_open(self.ctx, C.byref(h), C.byref(p)), self._err())
        return p.value

    def ipc_close(self, mapped):
        self.lib.b200c_ipc_close(self.ctx, mapped)

    def copy_segments_async(self, segs, wait_flag=None, wait_value=0, done_flag=None, done_value=0, timeout_ms=5000,
                            mode=0, ctas=64, after_ticket=None):
        """segs: (src pointer, dst pointer, bytes) triples; see b200c_copy_segments_async.  With after_ticket the
        copies are ordered after that compression ticket only (b200c_copy_segments_after)."""
        n = len(segs)
        arr = (A.b200c_copy_seg * max(1, n))()
        for i, (src, dst, nb) in enumerate(segs):
            arr[i].src, arr[i].dst, arr[i].n = src, dst, nb
        if after_ticket is not None:
            raise_for(self.lib.b200c_copy_segments_after(self.ctx, after_ticket, arr, n, wait_flag, wait_value, done_flag,
                                                         done_value, timeout_ms, mode, ctas), self._err())
            return
        raise_for(self.lib.b200c_copy_segments_async(self.ctx, arr, n, wait_flag, wait_value, done_flag, done_value,
                                                     timeout_ms, mode, ctas), self._err())

    def wait_flags(self, flags_ptr, count, value, timeout_ms=5000, on_transfer_stream=False):
        raise_for(self.lib.b200c_wait_flags(self.ctx, flags_ptr, count, value, timeout_ms, int(on_transfer_stream)), self._err())

    def signal_flags(self, targets, value):
        arr = (C.c_void_p * max(1, len(targets)))(*targets)
        raise_for(self.lib.b200c_signal_flags(self.ctx, arr, len(targets), value), self._err())

    def stream_join(self):
        raise_for(self.lib.b200c_stream_join(self.ctx), self._err())

    def exchange_status(self):
        st = C.c_int()
        raise_for(self.lib.b200c_exchange_status(self.ctx, C.byref(st)), self._err())
        return st.value


_default_backend = None


def default_backend():
    global _default_backend
    if _default_backend is None:
        _default_backend = CudaBackend(0)
    return _default_backend


# --------------------------------------------------------------------------- ContentAttr
def valid_raw_buffer(base_type, raw):
    """The buffer rule ContentAttr::verify applies to a dense resource (content.cpp:76-86, through
    mlir::DenseElementsAttr::isValidRawBuffer): the bytes hold every element of the type, or exactly one element
    (a splat).  One-bit elements are packed eight to a byte, and a single byte is a splat only when it is 0x00 or
    0xFF.  Sub-byte elements wider than one bit are held packed here (the layout Content keeps them in), where
    MLIR's attribute storage spends a byte on each.  Returns (valid, detected splat)."""
    bits, n = base_type.getElemTypeSize(), base_type.getNumElements()
    nbytes = int(raw.size) * raw.itemsize
    splat = n == 1
    if bits == 1:
        if nbytes == 1 and int(raw.reshape(-1).view(np.uint8)[0]) in (0x00, 0xFF):
            return True, True
        return nbytes == (n + 7) // 8, splat
    if nbytes == (bits + 7) // 8:
        return True, True
    return nbytes == (bits * n + 7) // 8, splat


class ContentAttr:
    """Const::ContentAttr: base content + ordered transformation list + inferred final type."""

    def __init__(self, base, base_type, is_splat, transforms, backend):
        self._base, self._baseType, self._isSplat = base, base_type, is_splat
        self._transforms = list(transforms)
        self._backend = backend

    @staticmethod
    def get(base, base_type=None, is_splat=None, backend=None):
        """base: numpy array holding the dense (or single splat) element(s); base_type: NDType
        (defaults to the array's shape and dtype)."""
        if base is None:
            raise ConstError("Got NULL 'baseContent' in 'ContentAttr'")
        arr = np.ascontiguousarray(base)
        if base_type is None:
            m = {np.dtype(np.float32): A.F32, np.dtype(np.float16): A.F16, np.dtype(np.float64): A.F64,
                 np.dtype(np.int8): A.SI8, np.dtype(np.uint8): A.UI8, np.dtype(np.int16): A.SI16,
                 np.dtype(np.uint16): A.UI16, np.dtype(np.int32): A.SI32, np.dtype(np.uint32): A.UI32,
                 np.dtype(np.int64): A.SI64, np.dtype(np.uint64): A.UI64}
            base_type = NDType(arr.shape, m[arr.dtype])
        if base_type.quant is not None:  # every plain element type here is an integer or a float
            raise ConstError(f"Got unsupported element type for 'baseContent' in 'ContentAttr' : '{base_type.getElementType()}'")
        valid, detected = valid_raw_buffer(base_type, arr)
        nbytes, bits = arr.size * arr.itemsize, base_type.getElemTypeSize()
        if is_splat is None:
            is_splat = detected and base_type.getNumElements() != 1
        elif is_splat:  # the caller says one element: any value of it is taken
            valid = nbytes == (bits + 7) // 8
        else:
            valid = nbytes == base_type.getTotalAllocSize()
        if not valid:
            raise ConstError(f"Size of dense resource buffer '{nbytes}' in 'baseContent' doesn't match its type '{base_type}'")
        return ContentAttr(arr, base_type, bool(is_splat), [], backend or default_backend())

    @staticmethod
    def getDenseResource(raw, base_type, backend=None):
        """A dense resource (mlir::DenseResourceElementsAttr) as base content.  Its blob is opaque to MLIR, so the
        reference looks at the bytes itself (detectSplatManually, content.cpp:120-137): empty data is no splat, a
        buffer of exactly one element is one, and otherwise all elements are compared with the first
        (detectSplatElementWise, content.cpp:103-118) -- here by the backend's probe, a device kernel on the CUDA
        backend.  A splat keeps its first element only, as the reference's take_front(elementSize)."""
        backend = backend or default_backend()
        if raw is None:
            raise ConstError("Got NULL 'baseContent' in 'ContentAttr'")
        arr = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        attr = ContentAttr.get(arr, base_type, backend=backend)  # the size check; a one-element buffer is a splat already
        bits = base_type.getElemTypeSize()
        if attr._isSplat or arr.size == 0 or bits % 8 != 0:
            return attr
        elem = bits // 8
        if backend.detect_splat(arr, elem):
            splat = base_type.getNumElements() != 1
            return ContentAttr(arr[:elem].copy(), base_type, splat, [], backend)
        return attr

    # -- accessors
    def getBaseContent(self):
        return self._base

    def getTransformations(self):
        return list(self._transforms)

    def getType(self):
        return self._backend.infer_type(self._baseType, self._transforms)

    def withBackend(self, backend):
        return ContentAttr(self._base, self._baseType, self._isSplat, self._transforms, backend)

    # -- ContentAttr::addTransformation (content.cpp:305-331)
    def addTransformation(self, t):
        kinds = [x.kind for x in self._transforms]
        pos = self._backend.insert_position(kinds, t.kind)
        ts = list(self._transforms)
        ts.insert(pos, t)
        out = ContentAttr(self._base, self._baseType, self._isSplat, ts, self._backend)
        out.getType()  # inferFinalType runs when the attribute is built; errors surface here
        # with background folding enabled for this context, the new attribute is folded ahead of time (content.cpp:320-328)
        from .cache import ConstantFoldingCacheManager, FoldingRequest
        mgr = ConstantFoldingCacheManager.getInstance()
        if mgr.contains(self._backend):
            mgr.get(self._backend).enqueueRequest(FoldingRequest(out, t))
        return out

    def key(self):
        """Value identity: the base content object, its type and splat flag, and the transformation list."""
        bt = self._baseType
        return (id(self._base), bt.shape, bt.dtype, tuple(bt.order), self._isSplat, tuple(t.key() for t in self._transforms))

    # -- ContentAttr::stripTransformationsFrom / getLastTransformationsFrom (content.cpp:342-369): the rightmost
    #    occurrence of the transformation splits the list
    def _rightmost(self, t):
        for i in range(len(self._transforms) - 1, -1, -1):
            if self._transforms[i] == t:
                return i
        return None

    def stripTransformationsFrom(self, t):
        i = self._rightmost(t)
        if i is None:
            return None
        return ContentAttr(self._base, self._baseType, self._isSplat, self._transforms[:i], self._backend)

    def getLastTransformationsFrom(self, t):
        i = self._rightmost(t)
        return [] if i is None else list(self._transforms[i:])

    # -- builder methods (attributes.td:72-107)
    def convertElemType(self, elem):
        return self.addTransformation(Transform(A.X_CONVERT_ELEM_TYPE, elem=elem))

    def quantCast(self, quant=None):
        return self.addTransformation(Transform(A.X_QUANT_CAST, elem=quant))

    def dequantize(self):
        return self.addTransformation(Transform(A.X_DEQUANTIZE))

    def rescale(self, scale):
        return self.addTransformation(Transform(A.X_RESCALE, f=scale))

    def add(self, bias):
        return self.addTransformation(Transform(A.X_ADD, f=bias))

    def reorder(self, order):
        return self.addTransformation(Transform(A.X_REORDER, a=tuple(order)))

    def transpose(self, order):
        return self.addTransformation(Transform(A.X_TRANSPOSE, a=tuple(order)))

    def reshape(self, shape):
        return self.addTransformation(Transform(A.X_RESHAPE, b=tuple(shape)))

    def changeShapeAndElemType(self, shape, elem):
        return self.addTransformation(Transform(A.X_CHANGE_SHAPE_AND_ELEM_TYPE, b=tuple(shape), elem=elem))

    def subview(self, offset, shape):
        return self.addTransformation(Transform(A.X_SUBVIEW, a=tuple(offset), b=tuple(shape)))

    def padWithZero(self, padBefore, padAfter):
        return self.addTransformation(Transform(A.X_PAD_WITH_ZERO, a=tuple(padBefore), b=tuple(padAfter)))

    def broadcast(self, axis, value):
        return self.addTransformation(Transform(A.X_BROADCAST, i0=axis, i1=value))

    def reverse(self, axis):
        return self.addTransformation(Transform(A.X_REVERSE, i0=axis))

    def expandDilated(self, dilations):
        return self.addTransformation(Transform(A.X_EXPAND_DILATED, a=tuple(dilations)))

    def relocateWeightsTablePointers(self, weightsPtr, sparsityPtr, offsets, weightsElemBitSize=0, numElems=None,
                                     alignment=0):
        """relocate_weights_table.cpp:205-213; numElems/alignment stand for the CompressionSchemeAttr."""
        return self.addTransformation(Transform(A.X_RELOCATE_WEIGHTS_TABLE, a=tuple(offsets), b=tuple(weightsPtr),
                                                i0=sparsityPtr, i1=weightsElemBitSize, aux=numElems, f=alignment))

    def bitPack(self, width):
        return self.addTransformation(Transform(A.X_BIT_PACK, i0=width))

    def getSparsityMap(self):
        return self.addTransformation(Transform(A.X_GET_SPARSITY_MAP))

    def sparsify(self, compressOutputType, numActualElements=None):
        return self.addTransformation(Transform(A.X_SPARSIFY, i0=int(bool(compressOutputType)), aux=numActualElements))

    def swizzleConstant(self, swizzleKey, arch=3):
        return self.addTransformation(Transform(A.X_SWIZZLE_CONSTANT, i0=swizzleKey, i1=arch))

    def quantizeSynth(self, scheme):
        """Synthetic per-output-channel quantiser (no reference counterpart); the per-channel
        scales / zero points land in the returned attribute's `.sideScales` / `.sideZeroPoints`."""
        oc = self.getType().shape[0]
        s0 = np.zeros(oc, dtype=np.float32)
        s1 = np.zeros(oc, dtype=np.int32)
        out = self.addTransformation(Transform(A.X_QUANTIZE_SYNTH, i0=scheme, side0=s0, side1=s1))
        return out

    @property
    def sideScales(self):
        for t in self._transforms:
            if t.kind == A.X_QUANTIZE_SYNTH:
                return t.side0
        return None

    @property
    def sideZeroPoints(self):
        for t in self._transforms:
            if t.kind == A.X_QUANTIZE_SYNTH:
                return t.side1
        return None

    # -- ContentAttr::fold (content.cpp:167-193) + copyTo
    def fold(self, bypassCache=False):
        if not bypassCache:
            from .cache import ConstantFoldingCacheManager, FailedContent
            mgr = ConstantFoldingCacheManager.getInstance()
            if mgr.contains(self._backend):
                hit = mgr.get(self._backend).getContent(self)
                if isinstance(hit, FailedContent):
                    raise hit.error
                if hit is not None:
                    return hit.to_content()
        return self._backend.fold(self._baseType, self._base, self._isSplat, self._transforms)

    def countNonSparseElementsPerOC(self):
        return self._backend.count_nonsparse_per_oc(self._baseType, self._base, self._isSplat, self._transforms)


class DeclareOp:
    """Const::DeclareOp (src/vpux_compiler/src/dialect/const/ops.cpp): a result type plus a ContentAttr.

    getContent() folds the attribute (ops.cpp:88-91 via getContentAttr().fold()); the verifier compares the
    attribute's inferred type with the result type (ops.cpp:164-193); serialize() appends the copyTo bytes to an
    ELF constants section and getBinarySize() is the folded type's total alloc size (ops.cpp:97-118)."""

    def __init__(self, result_type, contentAttr, swizzled=False, loc=None):
        self._type, self._attr, self._swizzled, self.loc = result_type, contentAttr, bool(swizzled), loc
        self.verify()

    def getContentAttr(self):
        return self._attr

    def getType(self):
        return self._type

    def getContent(self):
        return self._attr.fold()

    def fold(self):
        """DeclareOp::fold: the op folds to its attribute."""
        return self._attr

    def verify(self):
        attr_type, op_type = self._attr.getType(), self._type
        # for a type with swizzling the shape check is skipped: the content may have been flattened
        if not self._swizzled and tuple(op_type.shape) != tuple(attr_type.shape):
            raise ConstError(f"'Const.Declare' has mismatch in value shape '{list(attr_type.shape)}' and result shape "
                             f"'{list(op_type.shape)}'")
        if op_type.getElementType() != attr_type.getElementType():
            attr_is_integer = attr_type.quant is None and A.dtype_class(attr_type.dtype) in (A.CLS_INT, A.CLS_SINT, A.CLS_UINT)
            if op_type.quant is None and not attr_is_integer:
                raise ConstError(f"'Const.Declare' has mismatch in value element type '{attr_type.getElementType()}' and "
                                 f"result element type '{op_type.getElementType()}'")
        if tuple(op_type.order) != tuple(attr_type.order):
            raise ConstError(f"'Const.Declare' has mismatch in value DimsOrder '{tuple(attr_type.order)}' and result "
                             f"DimsOrder '{tuple(op_type.order)}'")

    def getBinarySize(self):
        return self.getContent().getType().getTotalAllocSize()

    def serialize(self, section):
        """Appends the constant's bytes to `section` (a bytearray): copyTo into a zero-initialised buffer of the
        folded type's size."""
        cnt = self.getContent()
        buf = np.zeros(cnt.getType().getTotalAllocSize(), np.uint8)
        cnt.copyTo(buf)
        section += buf.tobytes()
        return len(buf)


def constant_folding_pass(ops):
    """ConstantFoldingPass::safeRunOnFunc (src/vpux_compiler/src/dialect/const/passes/constant_folding.cpp:27-77):
    every DeclareOp is replaced by one whose base content holds the folded bytes and whose list is empty -- except
    for sub-byte element types (more than 1 and fewer than 8 bits), which a dense attribute cannot store: those
    keep the packed bytes as a [1,1,1,N] ui8 base plus ChangeShapeAndElemType back to the original shape and
    element type.  A quantised result is stored under its normalised storage integer type."""
    out = []
    for op in ops:
        attr = op.getContentAttr()
        content = op.getContent()
        ctype = content.getType()
        nbytes = ctype.getTotalAllocSize()
        buf = np.zeros(nbytes, np.uint8)
        content.copyTo(buf)
        bits = ctype.getElemTypeSize()
        if 1 < bits < 8:
            base_type = NDType((1, 1, 1, nbytes), A.UI8, ctype.order)
            orig = op.getType()
            new_attr = ContentAttr.get(buf, base_type, is_splat=False, backend=attr._backend).changeShapeAndElemType(
                orig.shape, orig.getElementType())
        else:
            base_type = NDType(ctype.shape, ctype.dtype, ctype.order)  # quantised: the normalised storage type
            new_attr = ContentAttr.get(buf, base_type, is_splat=False, backend=attr._backend)
        out.append(DeclareOp(op.getType(), new_attr, swizzled=op._swizzled, loc=op.loc))
    return out
