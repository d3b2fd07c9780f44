"""The step after folding: constant fusion and the constants-section writers.

fuse_constants -- the weight table, weights, weights sparsity map and activation window of one NCE task
become one flat constant (FuseConstants, src/vpux_compiler/src/dialect/VPUIP/passes/fuse_constants.cpp:82-176,
src/vpux_compiler/src/utils/constant_fusion.cpp).  The reference folds each part and appends its values to a
byte vector element by element; here the parts are folded by ONE batched call whose outputs are adjacent
ranges of the fused buffer on the device ("concatenate after fold" without a concatenation pass), and the
fused bytes come back with one copy.

write_section -- the constants section of the blob: every constant's live bytes gathered from the
512-byte-slotted blob into one dense buffer, each segment aligned to 8 bytes and zero-padded as the graph-schema
writer does (serializeBinaryData, src/vpux_compiler/src/dialect/VPUIP/graph-schema/export.cpp:465-479), or with no
padding as the ELF writer does (Const::DeclareOp::serialize, src/vpux_compiler/src/dialect/const/ops.cpp:97-108).
One launch of the library's segment-copy kernel moves all of them.
"""
import ctypes as C

import numpy as np

from . import _cabi as A
from .const import NDType, chain_to_c, raise_for


class FusedConstant:
    """type: NDType of the fused constant ([1,1,1,N] ui8 or f16); data: its bytes; views[k]: (offset, size) in
    elements of the fused type where part k lives (None for an absent part), i.e. the SubView that replaces it."""

    def __init__(self, ndtype, data, views):
        self.type, self.data, self.views = ndtype, data, views


def _part_kind(t):
    """How populateFusedConstantBuffer reads a folded part of type t (fuse_constants.cpp:103-150)."""
    if t.quant is not None:
        return "quant"
    if t.dtype == A.UI8 or t.dtype == A.I8:
        return "u8"
    if t.dtype == A.F16:
        return "f16"
    if t.dtype == A.SI32:
        return "si32"
    if A.dtype_bits(t.dtype) == 1:
        return "i1"
    raise ValueError("Unsupported data type for constant")


def fuse_constants(backend, weight_table=None, weights=None, weights_sm=None, activation_window=None):
    """Each argument is a ContentAttr (npu_plugin_b200.const) or None."""
    parts = [weight_table, weights, weights_sm, activation_window]
    present = [p for p in parts if p is not None]
    types = [p.getType() for p in present]
    kinds = [_part_kind(t) for t in types]
    sizes = [t.getTotalAllocSize() for t in types]
    total = sum(sizes)
    lib, ctx = backend.lib, backend.ctx
    fused_dev = backend.dev_alloc(max(1, total))
    staged, keep = [], []
    try:
        backend.fill_zero(fused_dev, max(1, total))
        n = len(present)
        items = (A.b200c_fold_item * max(1, n))()
        at = 0
        for k, (p, size) in enumerate(zip(present, sizes)):
            raw = np.ascontiguousarray(p.getBaseContent()).view(np.uint8).reshape(-1)
            d = backend.dev_alloc(max(1, raw.size))
            staged.append(d)
            backend.upload(d, raw)
            bt = p._baseType.to_c(keep)
            ch = chain_to_c(p.getTransformations(), keep)
            keep += [bt, ch]
            it = items[k]
            it.base = C.pointer(bt)
            it.data = d
            it.nbytes = raw.size
            it.is_splat = int(p._isSplat)
            it.n = len(p.getTransformations())
            it.chain = C.cast(ch, C.POINTER(A.b200c_xform))
            it.out = fused_dev + at
            it.out_cap = size
            at += size
        if n:
            raise_for(lib.b200c_fold_batch(ctx, items, n, 1, 1, 0), lib.b200c_last_error())
        data = backend.download(fused_dev, total)
    finally:
        backend.dev_free(fused_dev)
        for d in staged:
            backend.dev_free(d)
    joint_f16 = sum(s for s, k in zip(sizes, kinds) if k == "f16")
    if joint_f16 * 2 > total:
        t, es = NDType((1, 1, 1, total // 2), A.F16), 2
    else:
        t, es = NDType((1, 1, 1, total), A.UI8), 1
    views, off, j = [], 0, 0
    for p in parts:
        if p is None:
            views.append(None)
            continue
        views.append((off, sizes[j] // es))
        off += sizes[j] // es
        j += 1
    return FusedConstant(t, data, views)


class Section:
    """offsets[i] / sizes[i]: where constant i lies in `data` (a numpy uint8 array on the host)."""

    def __init__(self, data, offsets, sizes, compressed):
        self.data, self.offsets, self.sizes, self.compressed = data, offsets, sizes, compressed


def section_layout(sizes, align=8):
    offs, at = [], 0
    for s in sizes:
        offs.append(at)
        at += (s + align - 1) // align * align if align > 1 else s
    return offs, at


def write_section(backend, blob_ptr, table, align=8, copy_mode=0):
    """table: [(constant index, blob offset, size, compressed)] as ShardedFolder.collect returns it.  Gathers the
    live bytes of every constant into one dense section on the device (one copy-kernel launch), then brings it to
    the host.  align=8: the graph-schema layout; align=1: the ELF layout."""
    sizes = [size for _, _, size, _ in table]
    offs, total = section_layout(sizes, align)
    dev = backend.dev_alloc(max(1, total))
    try:
        backend.fill_zero(dev, max(1, total))
        backend.copy_segments_async([(blob_ptr + off, dev + o, size) for (_, off, size, _), o in zip(table, offs)], mode=copy_mode)
        backend.synchronize()
        data = backend.download(dev, total)
    finally:
        backend.dev_free(dev)
    return Section(data, offs, sizes, [bool(c) for _, _, _, c in table])
