"""Stand-ins for a memory checker, and the host-side fault cases of the allocator.

Guard words: every device output buffer of the calls below is followed by 512 canary bytes which must be
intact afterwards -- fold (reorders, padding, swizzled outputs whose size is rounded up to 512, BitPack,
the sparsity transformations), the batched fold, all forms of compress and decompress.  An out-of-bounds
store of a kernel shows up as a changed canary without any fault on the GPU.

Allocator: the library's scratch arena takes its blocks from an allocator the caller installs
(b200c_set_allocator).  An allocator that has no memory makes the call fail with B200C_ERR_NOMEM; the
context stays usable and gives the oracle's bytes once memory is available again.
"""
import ctypes as C

import numpy as np
import pytest

from npu_plugin_b200 import _cabi as A
from npu_plugin_b200.blob import ConstantDecl, ShardFolder
from npu_plugin_b200.const import (ContentAttr, CudaBackend, DimsOrder, NDType, UniformQuantizedPerAxisType,
                                   UniformQuantizedType, chain_to_c, raise_for)

pytestmark = pytest.mark.gpu

GUARD = 512
CANARY = 0xA5


class Guarded:
    """A device buffer of `n` bytes followed by the canary."""

    def __init__(self, gpu, n):
        self.gpu, self.n = gpu, n
        self.ptr = gpu.dev_alloc(n + GUARD)
        gpu.upload(self.ptr, np.full(n + GUARD, CANARY, np.uint8))

    def check(self, what):
        tail = self.gpu.download(self.ptr + self.n, GUARD)
        assert (tail == CANARY).all(), f"{what}: bytes behind the output buffer were overwritten"

    def bytes(self, n=None):
        return self.gpu.download(self.ptr, self.n if n is None else n)

    def free(self):
        self.gpu.dev_free(self.ptr)


def _chains(rng):
    """(name, base array, base type, chain builder) covering every kernel family."""
    w = rng.normal(0, 0.05, (48, 40, 3, 3)).astype(np.float32)
    q = UniformQuantizedPerAxisType(A.SI8, A.F32, [1.0] * 48, [0] * 48, 0, -127, 127)
    yield "quantise+reorder+swizzle", w, lambda a: (a.quantizeSynth(A.QSYNTH_SYM_I8).convertElemType(A.SI8).quantCast(q)
                                                    .reorder(DimsOrder.OYXI).swizzleConstant(5, 3))
    h = rng.normal(0, 0.02, (37, 64, 1, 1)).astype(np.float16)
    qu = UniformQuantizedPerAxisType(A.UI8, A.F16, [1.0] * 37, [0] * 37, 0, 0, 15)
    yield "u4 bitpack", h, lambda a: (a.quantizeSynth(A.QSYNTH_ASYM_U4).convertElemType(A.UI8).quantCast(qu)
                                      .reorder(DimsOrder.NHWC).bitPack(4))
    s = rng.integers(-127, 128, (24, 48, 1, 1)).astype(np.int8)
    s[rng.random(s.shape) < 0.5] = 0
    yield "sparsity map", s, lambda a: a.getSparsityMap().swizzleConstant(5, 3)
    yield "sparsify", s, lambda a: a.sparsify(False).swizzleConstant(5, 3)
    c = rng.integers(-127, 128, (20, 3, 7, 7)).astype(np.int8)
    qt = UniformQuantizedType(A.SI8, A.F16, 0.01, 3, -127, 127)
    yield "reorder+pad", c, lambda a: a.quantCast(qt).reorder(DimsOrder.OYXI).padWithZero((0, 0, 0, 0), (0, 13, 0, 0))
    t = rng.integers(0, 255, (5, 6, 7)).astype(np.uint8)
    yield "subview+transpose", t, lambda a: a.subview((1, 2, 3), (3, 3, 4)).reorder((2, 0, 1))
    d = rng.integers(0, 16, (33, 100, 1, 1)).astype(np.uint8)
    qd = UniformQuantizedPerAxisType(A.UI8, A.F16, [0.01 + 0.001 * k for k in range(33)], [k % 16 for k in range(33)], 0, 0, 15)
    yield "dequantise", d, lambda a: a.quantCast(qd).dequantize().convertElemType(A.F16)


def test_fold_outputs_stay_inside_their_buffers(gpu, oracle):
    rng = np.random.default_rng(31)
    for name, base, build in _chains(rng):
        attr_g = build(ContentAttr.get(base, backend=gpu))
        attr_o = build(ContentAttr.get(base, backend=oracle))
        want = attr_o.fold().copyTo()
        transforms = attr_g.getTransformations()
        bt = attr_g._baseType
        keep = []
        ctype, chain = bt.to_c(keep), chain_to_c(transforms, keep)
        cap = max(gpu.infer_type(bt, transforms).getTotalAllocSize(), 1)
        out = Guarded(gpu, cap)
        src = gpu.dev_alloc(base.nbytes)
        # with the output on the device the quantiser's per-channel tables are device buffers too
        sides = []
        for k, t in enumerate(transforms):
            if t.kind == A.X_QUANTIZE_SYNTH:
                sides = [Guarded(gpu, 4 * base.shape[0]), Guarded(gpu, 4 * base.shape[0])]
                chain[k].side0, chain[k].side1 = sides[0].ptr, sides[1].ptr
        try:
            gpu.upload(src, np.ascontiguousarray(base).view(np.uint8).reshape(-1))
            nb = C.c_size_t()
            rc = gpu.lib.b200c_fold(gpu.ctx, C.byref(ctype), src, base.nbytes, 0, 1, chain, len(transforms), out.ptr, cap, 1,
                                    C.byref(nb), None, 0)
            raise_for(rc, gpu.lib.b200c_last_error())
            out.check(name)
            for g in sides:
                g.check(name + " (per-channel table)")
            assert np.array_equal(out.bytes(nb.value), want.reshape(-1).view(np.uint8)[:nb.value]), name
            if sides:
                assert np.array_equal(sides[0].bytes().view(np.float32), attr_o.sideScales), name
        finally:
            gpu.dev_free(src)
            out.free()
            for g in sides:
                g.free()


def test_batched_fold_and_compress_stay_inside_their_slots(gpu, oracle):
    """The whole-model path: every slot of the blob is followed by a canary-filled gap (slots are 512-byte
    aligned; sizes here leave part of the last 512 bytes unused) and the blob by a guard."""
    rng = np.random.default_rng(32)
    decls, data = [], []
    for k, (o, i, y, x) in enumerate([(40, 24, 3, 3), (17, 96, 1, 1), (64, 3, 7, 7), (33, 31, 1, 1)]):
        w = np.clip(np.rint(rng.laplace(0, 10, (o, i, y, x))), -127, 127).astype(np.int8)
        w[rng.random(w.shape) < 0.2] = 0
        a = ContentAttr.get(w, backend=gpu).quantCast(UniformQuantizedType(A.SI8, A.F16, 0.01, 0, -127, 127)).reorder(DimsOrder.OYXI)
        decls.append(ConstantDecl(f"c{k}", a._baseType, a.getTransformations(), w.nbytes, compress=True))
        data.append(w)
    folder = ShardFolder(gpu, decls)
    blob = Guarded(gpu, folder.folded_bytes)
    ins = [gpu.dev_alloc(w.nbytes) for w in data]
    try:
        for p, w in zip(ins, data):
            gpu.upload(p, w.view(np.uint8).reshape(-1))
        folder.fold(ins, blob.ptr, True)
        segs = folder.compress_inplace(blob.ptr)
        blob.check("batched fold + in-place compression")
        got = blob.bytes()
        for (i, off, size, comp), w, d in zip(segs, data, decls):
            end = off + folder.folded_sizes[i]
            nxt = folder.folded_offsets[i + 1] if i + 1 < len(decls) else folder.folded_bytes
            if not comp:
                assert (got[end:nxt] == CANARY).all(), f"slot {i}: bytes between the slots were overwritten"
            folded = oracle.fold(d.base_type, w, False, d.transforms).copyTo().reshape(-1).view(np.uint8)
            live = got[off:off + size]
            if comp:
                assert np.array_equal(gpu.btc_decompress(live, folded.size), folded)
            else:
                assert np.array_equal(live, folded)
    finally:
        for p in ins:
            gpu.dev_free(p)
        blob.free()


def test_compress_and_decompress_stay_inside_their_buffers(gpu):
    rng = np.random.default_rng(33)
    x = np.clip(np.rint(rng.laplace(0, 5, 300_007)), -127, 127).astype(np.int8).view(np.uint8)
    x[rng.random(x.size) < 0.3] = 0
    bound = gpu.btc_bound(x.size)
    src, out, back = gpu.dev_alloc(x.size), Guarded(gpu, bound), Guarded(gpu, x.size)
    try:
        gpu.upload(src, x)
        n = C.c_size_t()
        rc = gpu.lib.b200c_btc_compress(gpu.ctx, src, x.size, 1, out.ptr, bound, 1, C.byref(n))
        raise_for(rc, gpu.lib.b200c_last_error())
        out.check("compress")
        stream = out.bytes(n.value)
        m = C.c_size_t()
        rc = gpu.lib.b200c_btc_decompress(gpu.ctx, out.ptr, n.value, 1, back.ptr, x.size, 1, C.byref(m))
        raise_for(rc, gpu.lib.b200c_last_error())
        back.check("decompress")
        assert m.value == x.size and np.array_equal(back.bytes(), x)
        # the allocation-free form writes the same stream into a guarded buffer
        gpu.upload(out.ptr, np.full(bound + GUARD, CANARY, np.uint8))
        rc = gpu.lib.b200c_btc_compress_noalloc(gpu.device, src, x.size, out.ptr, bound, None, C.byref(n))
        raise_for(rc, gpu.lib.b200c_last_error())
        out.check("compress_noalloc")
        assert np.array_equal(out.bytes(n.value), stream)
    finally:
        gpu.dev_free(src)
        out.free()
        back.free()


def test_allocator_failure_is_reported_and_the_context_recovers(oracle):
    import torch
    gpu = CudaBackend(0)  # a context of its own: its arena is empty, so the first call has to allocate
    state = {"fail": True, "allocs": 0, "frees": 0, "live": {}}

    def alloc(user, nbytes):
        if state["fail"]:
            return None
        state["allocs"] += 1
        p = torch.cuda.caching_allocator_alloc(nbytes, 0)
        state["live"][p] = nbytes
        return p

    def free(user, p):
        state["frees"] += 1
        torch.cuda.caching_allocator_delete(p)
        del state["live"][p]

    alloc_c, free_c = A.ALLOC_FN(alloc), A.FREE_FN(free)
    raise_for(gpu.lib.b200c_set_allocator(gpu.ctx, C.cast(alloc_c, C.c_void_p), C.cast(free_c, C.c_void_p), None),
              gpu.lib.b200c_last_error())
    rng = np.random.default_rng(34)
    w = rng.normal(0, 1, (8, 6, 3, 3)).astype(np.float32)
    build = lambda be: ContentAttr.get(w, backend=be).convertElemType(A.F16).reorder(DimsOrder.OYXI).swizzleConstant(5, 3)
    keep = []
    attr = build(gpu)
    bt, tr = attr._baseType, attr.getTransformations()
    ctype, chain = bt.to_c(keep), chain_to_c(tr, keep)
    cap = gpu.infer_type(bt, tr).getTotalAllocSize()
    out = np.zeros(cap, np.uint8)
    nb = C.c_size_t()
    call = lambda: gpu.lib.b200c_fold(gpu.ctx, C.byref(ctype), w.ctypes.data, w.nbytes, 0, 0, chain, len(tr), out.ctypes.data, cap, 0,
                                      C.byref(nb), None, 0)
    assert call() == A.ERR_NOMEM
    assert b"allocator" in gpu.lib.b200c_last_error()
    assert call() == A.ERR_NOMEM  # still failing, still no crash
    state["fail"] = False
    assert call() == A.OK
    assert state["allocs"] >= 1
    assert np.array_equal(out[:nb.value], build(oracle).fold().copyTo().reshape(-1).view(np.uint8)[:nb.value])
    # removing the allocator hands every block back to it
    raise_for(gpu.lib.b200c_set_allocator(gpu.ctx, None, None, None), gpu.lib.b200c_last_error())
    assert state["frees"] == state["allocs"] and not state["live"]
    assert call() == A.OK  # now on the CUDA allocator
    gpu.close()
