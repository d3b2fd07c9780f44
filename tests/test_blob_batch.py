"""The batched whole-model entry point (b200c_fold_batch) against per-constant folds and the oracle."""
import ctypes as C

import numpy as np
import pytest

from npu_plugin_b200 import _cabi as A
from npu_plugin_b200.blob import ConstantDecl, ShardFolder, partition
from npu_plugin_b200.const import DimsOrder, NDType, Transform, UniformQuantizedPerAxisType, raise_for

gpu_only = pytest.mark.gpu


def linear_decl(name, o, i):
    q = UniformQuantizedPerAxisType(A.SI8, A.F16, [1.0] * o, [0] * o, 0, -127, 127)
    chain = [Transform(A.X_QUANTIZE_SYNTH, i0=A.QSYNTH_SYM_I8), Transform(A.X_CONVERT_ELEM_TYPE, elem=A.SI8),
             Transform(A.X_QUANT_CAST, elem=q), Transform(A.X_REORDER, a=DimsOrder.NHWC),
             Transform(A.X_SWIZZLE_CONSTANT, i0=5, i1=3)]
    return ConstantDecl(name, NDType((o, i, 1, 1), A.F16), chain, o * i * 2)


class DevBuf:
    def __init__(self, gpu, nbytes):
        self.gpu, self.n = gpu, nbytes
        p = C.c_void_p()
        raise_for(gpu.lib.b200c_dev_alloc(gpu.ctx, max(1, nbytes), C.byref(p)), gpu.lib.b200c_last_error())
        self.ptr = p.value

    def upload(self, arr):
        a = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
        raise_for(self.gpu.lib.b200c_memcpy_h2d(self.gpu.ctx, self.ptr, a.ctypes.data, a.size), self.gpu.lib.b200c_last_error())

    def download(self, n=None):
        out = np.zeros(self.n if n is None else n, np.uint8)
        raise_for(self.gpu.lib.b200c_memcpy_d2h(self.gpu.ctx, out.ctypes.data, self.ptr, out.size), self.gpu.lib.b200c_last_error())
        return out

    def free(self):
        self.gpu.lib.b200c_dev_free(self.gpu.ctx, self.ptr)


@gpu_only
def test_batched_fold_matches_single_folds_and_oracle(gpu, oracle):
    rng = np.random.default_rng(11)
    shapes = [(64, 256), (48, 1024), (16, 4096), (40, 11008), (128, 64), (7, 20000), (33, 100)]
    decls = [linear_decl(f"w{k}", o, i) for k, (o, i) in enumerate(shapes)]
    decls.append(ConstantDecl("gain", NDType((512,), A.F16), [], 1024, compress=False))
    data = [rng.normal(0, 0.02, d.nbytes // 2).astype(np.float16) for d in decls]
    # an int8 constant with small values: this one does compress
    small = np.clip(np.rint(rng.laplace(0, 3, (64, 1024, 1, 1))), -127, 127).astype(np.int8)
    qs = UniformQuantizedPerAxisType(A.SI8, A.F16, [1.0] * 64, [0] * 64, 0, -127, 127)
    decls.append(ConstantDecl("small", NDType((64, 1024, 1, 1), A.SI8),
                              [Transform(A.X_QUANT_CAST, elem=qs), Transform(A.X_REORDER, a=DimsOrder.NHWC)], small.size))
    data.append(small)
    folder = ShardFolder(gpu, decls)
    ins = [DevBuf(gpu, d.nbytes) for d in decls]
    for b, x in zip(ins, data):
        b.upload(x)
    scales = [DevBuf(gpu, 4 * d.base_type.shape[0]) if d.transforms else None for d in decls]
    zps = [DevBuf(gpu, 4 * d.base_type.shape[0]) if d.transforms else None for d in decls]
    side = [(s.ptr, z.ptr) if s else None for s, z in zip(scales, zps)]
    out_a, out_b = DevBuf(gpu, folder.folded_bytes), DevBuf(gpu, folder.folded_bytes)
    folder.fold([b.ptr for b in ins], out_a.ptr, True, side)
    raise_for(gpu.lib.b200c_synchronize(gpu.ctx), gpu.lib.b200c_last_error())
    batched_scales = [s.download() if s else None for s in scales]
    folder.fold_one_by_one([b.ptr for b in ins], out_b.ptr, True, side)
    raise_for(gpu.lib.b200c_synchronize(gpu.ctx), gpu.lib.b200c_last_error())
    a, b = out_a.download(), out_b.download()
    for i, d in enumerate(decls):
        off, size = folder.folded_offsets[i], folder.folded_sizes[i]
        ref = oracle.fold(d.base_type, data[i], False, d.transforms).copyTo()
        assert np.array_equal(a[off:off + size], ref), d.name
        assert np.array_equal(b[off:off + size], ref), d.name
        if d.transforms:
            assert np.array_equal(batched_scales[i], scales[i].download()), d.name
    # host input through the same entry point, issued in bounded groups
    host = [np.ascontiguousarray(x) for x in data]
    out_c = DevBuf(gpu, folder.folded_bytes)
    folder.fold([h.ctypes.data for h in host], out_c.ptr, False, side, max_batch_bytes=200_000)
    raise_for(gpu.lib.b200c_synchronize(gpu.ctx), gpu.lib.b200c_last_error())
    c = out_c.download()
    for i in range(len(decls)):
        off, size = folder.folded_offsets[i], folder.folded_sizes[i]
        assert np.array_equal(c[off:off + size], a[off:off + size])
    # batched compression keeps incompressible segments as they are and reports it
    blob = DevBuf(gpu, folder.blob_bound)
    segs = folder.compress(out_a.ptr, blob.ptr, folder.blob_bound)
    raw = blob.download()
    for i, off, size, compressed in segs:
        folded = a[folder.folded_offsets[i]:folder.folded_offsets[i] + folder.folded_sizes[i]]
        stream, not_smaller = oracle.btc_compress(folded)
        assert compressed == (not not_smaller)
        expect = stream if compressed else folded
        assert size == expect.size and np.array_equal(raw[off:off + size], expect), decls[i].name
    assert any(c for _, _, _, c in segs) and not all(c for _, _, _, c in segs)
    # in-place form: streams replace the head of their own segment, the rest is not touched
    inplace = folder.compress_inplace(out_b.ptr)
    after = out_b.download()
    assert len(inplace) == len(decls)
    for i, off, size, compressed in inplace:
        folded = a[off:off + folder.folded_sizes[i]]
        if i in folder.comp_idx:
            stream, not_smaller = oracle.btc_compress(folded)
            assert compressed == (not not_smaller), decls[i].name
        else:
            assert not compressed
        if compressed:
            assert size == stream.size and np.array_equal(after[off:off + size], stream), decls[i].name
            assert np.array_equal(gpu.btc_decompress(after[off:off + size], folded.size), folded)
        else:
            assert size == folded.size and np.array_equal(after[off:off + size], folded), decls[i].name
    for x in ins + [out_a, out_b, out_c, blob] + [s for s in scales + zps if s]:
        x.free()


def test_partition_is_deterministic_and_balanced():
    decls = [linear_decl(f"t{k}", o, i) for k, (o, i) in enumerate([(4096, 4096)] * 8 + [(11008, 4096)] * 4 + [(32000, 4096)])]
    for world in (1, 2, 4, 8):
        owner = partition(decls, world)
        assert owner == partition(decls, world)
        load = [sum(d.nbytes for d, o in zip(decls, owner) if o == r) for r in range(world)]
        assert max(load) - min(load) <= max(d.nbytes for d in decls)


@gpu_only
def test_many_small_constants_in_one_batch(gpu, oracle):
    """Enough items for the planning threads, mixing every batched kernel family: fused quantiser
    (register and staged), tile transposes, sparsity map and sparsify (size known only on the
    device), dequantize rows.  Every output and every reported size must equal the oracle's."""
    rng = np.random.default_rng(21)
    decls, data = [], []
    q8 = lambda o: UniformQuantizedPerAxisType(A.SI8, A.F16, [1.0] * o, [0] * o, 0, -127, 127)
    for k in range(96):
        kind = k % 6
        if kind == 0:
            o, i = int(rng.integers(4, 40)), int(rng.choice([64, 256, 1040, 4096]))
            decls.append(linear_decl(f"lin{k}", o, i))
            data.append(rng.normal(0, 0.02, o * i).astype(np.float16))
        elif kind == 1:
            o, i = int(rng.integers(2, 24)), int(rng.choice([16, 32, 64]))
            x = rng.integers(-127, 128, (o, i, 3, 3)).astype(np.int8)
            decls.append(ConstantDecl(f"conv{k}", NDType(x.shape, A.SI8),
                                      [Transform(A.X_QUANT_CAST, elem=q8(o)), Transform(A.X_REORDER, a=DimsOrder.NHWC)], x.size))
            data.append(x)
        elif kind in (2, 3):
            o, i = int(rng.integers(3, 50)), int(rng.choice([16, 128, 1024]))
            x = rng.integers(-127, 128, (o, i, 1, 1)).astype(np.int8)
            x[rng.random(x.shape) < 0.5] = 0
            first = Transform(A.X_GET_SPARSITY_MAP) if kind == 2 else Transform(A.X_SPARSIFY, i0=0)
            chain = [first] + ([Transform(A.X_SWIZZLE_CONSTANT, i0=5, i1=3)] if k % 4 < 2 else [])
            decls.append(ConstantDecl(f"sp{k}", NDType(x.shape, A.SI8), chain, x.size, compress=False))
            data.append(x)
        elif kind == 4:
            o, i = int(rng.integers(2, 30)), int(rng.choice([48, 4096]))
            x = rng.integers(0, 256, (o, i)).astype(np.uint8)
            qt = UniformQuantizedPerAxisType(A.UI8, A.F16, list(rng.uniform(0.001, 0.1, o)), list(map(int, rng.integers(0, 255, o))), 0, 0, 255)
            decls.append(ConstantDecl(f"dq{k}", NDType(x.shape, A.UI8),
                                      [Transform(A.X_QUANT_CAST, elem=qt), Transform(A.X_DEQUANTIZE)], x.size, compress=False))
            data.append(x)
        else:
            x = rng.normal(0, 1, (int(rng.integers(1, 9)), 33)).astype(np.float16)
            decls.append(ConstantDecl(f"gain{k}", NDType(x.shape, A.F16), [], x.nbytes, compress=False))
            data.append(x)
    folder = ShardFolder(gpu, decls)
    ins = [DevBuf(gpu, d.nbytes) for d in decls]
    for b, x in zip(ins, data):
        b.upload(x)
    has_q = [any(t.kind == A.X_QUANTIZE_SYNTH for t in d.transforms) for d in decls]
    scales = [DevBuf(gpu, 4 * d.base_type.shape[0]) if q else None for d, q in zip(decls, has_q)]
    zps = [DevBuf(gpu, 4 * d.base_type.shape[0]) if q else None for d, q in zip(decls, has_q)]
    side = [(s.ptr, z.ptr) if s else None for s, z in zip(scales, zps)]
    out = DevBuf(gpu, folder.folded_bytes)
    for _ in range(2):  # the second pass reuses the marshalled items and the warmed-up pool
        folder.fold([b.ptr for b in ins], out.ptr, True, side)
        raise_for(gpu.lib.b200c_synchronize(gpu.ctx), gpu.lib.b200c_last_error())
        a = out.download()
        for i, d in enumerate(decls):
            ref = oracle.fold(d.base_type, data[i], False, d.transforms).copyTo().view(np.uint8).ravel()
            off = folder.folded_offsets[i]
            assert folder._items[i].out_bytes == ref.size, (d.name, folder._items[i].out_bytes, ref.size)
            assert np.array_equal(a[off:off + ref.size], ref), d.name
    for b in ins + [out] + [s for s in scales + zps if s]:
        b.free()


def test_weighted_partition_follows_the_shares():
    from npu_plugin_b200.blob import gather_aware_weights
    decls = [ConstantDecl(f"c{k}", NDType((4,), A.F16), [], 1000 + 37 * (k % 11)) for k in range(400)]
    total = sum(d.nbytes for d in decls)
    for world in (2, 4, 8):
        w = gather_aware_weights(world, compute_seconds=5.0, transfer_seconds=9.0)
        assert abs(sum(w) - 1.0) < 1e-9 and abs(w[0] - 9.0 / 14.0) < 1e-9
        owner = partition(decls, world, w)
        for r in range(world):
            share = sum(d.nbytes for d, o in zip(decls, owner) if o == r) / total
            assert abs(share - w[r]) < 0.02, (world, r, share, w[r])
    # cheap transfers: an equal split
    assert gather_aware_weights(4, 5.0, 0.1) == [0.25] * 4
    assert gather_aware_weights(1, 5.0, 9.0) == [1.0]


@gpu_only
def test_two_contexts_fold_concurrently(oracle):
    """Calls on different contexts may run at the same time (the reference folds from many threads):
    two host threads, each with a context of its own, fold different constants and both match the oracle."""
    import threading
    from npu_plugin_b200.const import ContentAttr, CudaBackend
    rng = np.random.default_rng(33)
    ws = [rng.normal(0, 0.02, (48, 2048, 1, 1)).astype(np.float16) for _ in range(2)]
    results, errors = [None, None], []

    def build(backend, w):
        a = ContentAttr.get(w, NDType(w.shape, A.F16), backend=backend).quantizeSynth(A.QSYNTH_SYM_I8)
        q = UniformQuantizedPerAxisType(A.SI8, A.F16, [1.0] * 48, [0] * 48, 0, -127, 127)
        return a.convertElemType(A.SI8).quantCast(q).reorder(DimsOrder.NHWC).swizzleConstant(5, 3)

    def work(k):
        try:
            be = CudaBackend(0)
            for _ in range(20):
                results[k] = build(be, ws[k]).fold().copyTo()
        except Exception as e:  # surfaced below
            errors.append(e)

    threads = [threading.Thread(target=work, args=(k,)) for k in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for k in range(2):
        assert np.array_equal(results[k], build(oracle, ws[k]).fold().copyTo())


@gpu_only
def test_sparsity_batch_over_densities_and_shapes(gpu, oracle):
    """GetSparsityMap and Sparsify of the same weights in one batch (the map kernel then also counts for the
    Sparsify), over densities from all-sparse to all-dense, a non-zero sparse value, channel lengths with and
    without the shared-count form, swizzled and plain, with and without numActualElements."""
    from npu_plugin_b200.const import UniformQuantizedType
    rng = np.random.default_rng(29)
    cases = []  # (weights, zero point or None, swizzle)
    for k, (oc, work, density, zp, swz) in enumerate([
            (64, 1024, 0.5, None, True), (48, 1024, 0.0, None, True), (48, 1024, 1.0, None, True), (33, 1024, 0.05, None, False),
            (40, 1024, 0.95, 7, True), (17, 16, 0.5, None, True), (24, 48, 0.4, None, False), (9, 2000, 0.5, None, True),
            (5, 4096, 0.7, 3, True), (128, 128, 0.5, None, True), (31, 512, 0.02, None, True), (6, 3072, 0.5, None, True)]):
        w = rng.integers(-127, 128, (oc, work, 1, 1)).astype(np.int8)
        fill = 0 if zp is None else zp
        w[w == fill] = fill + 1
        w[rng.random(w.shape) >= density] = fill
        cases.append((w, zp, swz))
    decls, data = [], []
    for k, (w, zp, swz) in enumerate(cases):
        pre = [] if zp is None else [Transform(A.X_QUANT_CAST, elem=UniformQuantizedType(A.SI8, A.F16, 0.1, zp, -128, 127))]
        tail = [Transform(A.X_SWIZZLE_CONSTANT, i0=5, i1=3)] if swz else []
        bt = NDType(w.shape, A.SI8)
        decls.append(ConstantDecl(f"map{k}", bt, pre + [Transform(A.X_GET_SPARSITY_MAP)] + tail, w.size, compress=False))
        data.append(w)
        if k % 2:  # numActualElements given: the per-channel counts of the data
            counts = [int(c) for c in (w.reshape(w.shape[0], -1) != (0 if zp is None else zp)).sum(axis=1)]
            sp = Transform(A.X_SPARSIFY, i0=1, aux=counts)
        else:
            sp = Transform(A.X_SPARSIFY, i0=0)
        decls.append(ConstantDecl(f"vals{k}", bt, pre + [sp] + tail, w.size, compress=False))
        data.append(w)
    folder = ShardFolder(gpu, decls)
    ins = [DevBuf(gpu, d.nbytes) for d in decls]
    out = DevBuf(gpu, folder.folded_bytes)
    try:
        for b, x in zip(ins, data):
            b.upload(x)
        for _ in range(2):  # the second pass runs over a used arena and a dirty output buffer
            gpu.upload(out.ptr, np.full(folder.folded_bytes, 0xCD, np.uint8))
            folder.fold([b.ptr for b in ins], out.ptr, True)
            gpu.synchronize()
            got = out.download()
            for i, (d, x) in enumerate(zip(decls, data)):
                want = oracle.fold(d.base_type, x, False, d.transforms)
                wb = want.copyTo().reshape(-1).view(np.uint8)
                n = want.bytesWritten
                off = folder.folded_offsets[i]
                assert np.array_equal(got[off:off + n], wb[:n]), d.name
    finally:
        for b in ins:
            b.free()
        out.free()
