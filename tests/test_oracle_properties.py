"""The CPU oracle against plain numpy statements of what each transformation means.

The oracle restates the reference's loops; these tests restate the *definitions* (a transpose, a slice, a pad, a
bit pack ...) with numpy on seeded random shapes, so a slip in the oracle's index arithmetic cannot hide behind a
GPU implementation that made the same slip.  CPU only.
"""
import itertools

import numpy as np
import pytest

from npu_plugin_b200 import _cabi as A
from npu_plugin_b200.const import ContentAttr, NDType, UniformQuantizedPerAxisType, UniformQuantizedType

DTYPES = [(A.UI8, np.uint8), (A.SI8, np.int8), (A.F16, np.float16), (A.SI32, np.int32), (A.F32, np.float32)]


def _rand(rng, shape, npdt):
    if np.issubdtype(npdt, np.floating):
        return rng.normal(0, 4, shape).astype(npdt)
    info = np.iinfo(npdt)
    return rng.integers(max(info.min, -100), min(info.max, 100) + 1, shape).astype(npdt)


def _shapes(rng, n, max_rank=5, max_extent=6):
    for _ in range(n):
        rank = int(rng.integers(1, max_rank + 1))
        yield tuple(int(rng.integers(1, max_extent + 1)) for _ in range(rank))


def test_reorder_is_a_transpose_of_memory(oracle):
    rng = np.random.default_rng(1)
    for shape in _shapes(rng, 40):
        dt, npdt = DTYPES[int(rng.integers(len(DTYPES)))]
        x = _rand(rng, shape, npdt)
        perm = tuple(int(p) for p in rng.permutation(len(shape)))
        c = ContentAttr.get(x, NDType(shape, dt), backend=oracle).reorder(perm).fold()
        assert c.getType().shape == shape and tuple(c.getType().order) == perm
        assert c.copyTo().tobytes() == np.ascontiguousarray(np.transpose(x, perm)).tobytes()
        # a second reorder composes: the bytes are the transpose by the new order of the logical tensor
        perm2 = tuple(int(p) for p in rng.permutation(len(shape)))
        c2 = ContentAttr.get(x, NDType(shape, dt), backend=oracle).reorder(perm).reorder(perm2).fold()
        assert c2.copyTo().tobytes() == np.ascontiguousarray(np.transpose(x, perm2)).tobytes()


def test_transpose_permutes_the_logical_shape(oracle):
    rng = np.random.default_rng(2)
    for shape in _shapes(rng, 25, max_rank=4):
        x = _rand(rng, shape, np.float32)
        perm = tuple(int(p) for p in rng.permutation(len(shape)))
        c = ContentAttr.get(x, NDType(shape, A.F32), backend=oracle).transpose(perm).fold()
        want = np.transpose(x, perm)
        assert c.getType().shape == want.shape
        assert np.array_equal(c.getValues().reshape(want.shape), want)


def test_subview_is_a_slice_and_pad_is_a_pad(oracle):
    rng = np.random.default_rng(3)
    for shape in _shapes(rng, 40, max_rank=4):
        dt, npdt = DTYPES[int(rng.integers(len(DTYPES)))]
        x = _rand(rng, shape, npdt)
        off = [int(rng.integers(0, s)) for s in shape]
        ext = [int(rng.integers(1, s - o + 1)) for s, o in zip(shape, off)]
        c = ContentAttr.get(x, NDType(shape, dt), backend=oracle).subview(off, ext).fold()
        sl = tuple(slice(o, o + e) for o, e in zip(off, ext))
        assert c.copyTo().tobytes() == np.ascontiguousarray(x[sl]).tobytes()
        before = [int(rng.integers(0, 3)) for _ in shape]
        after = [int(rng.integers(0, 3)) for _ in shape]
        c = ContentAttr.get(x, NDType(shape, dt), backend=oracle).padWithZero(before, after).fold()
        assert c.copyTo().tobytes() == np.pad(x, list(zip(before, after))).tobytes()


def test_pad_of_a_quantised_tensor_fills_with_the_zero_point(oracle):
    rng = np.random.default_rng(4)
    x = rng.integers(0, 256, (3, 4, 2, 2)).astype(np.uint8)
    q = UniformQuantizedType(A.UI8, A.F32, 0.1, 77, 0, 255)
    c = ContentAttr.get(x, backend=oracle).quantCast(q).padWithZero((0, 1, 0, 0), (0, 2, 1, 0)).fold()
    assert c.copyTo().tobytes() == np.pad(x, ((0, 0), (1, 2), (0, 1), (0, 0)), constant_values=77).tobytes()
    qa = UniformQuantizedPerAxisType(A.UI8, A.F32, [0.1, 0.2, 0.3], [5, 6, 7], 0, 0, 255)
    c = ContentAttr.get(x, backend=oracle).quantCast(qa).padWithZero((0, 0, 0, 0), (0, 3, 0, 0)).fold()
    want = np.concatenate([x, np.broadcast_to(np.array([5, 6, 7], np.uint8).reshape(3, 1, 1, 1), (3, 3, 2, 2))], axis=1)
    assert c.copyTo().tobytes() == want.tobytes()


def test_value_transformations_follow_their_formulas(oracle):
    rng = np.random.default_rng(5)
    x = rng.integers(0, 256, (4, 6, 1, 1)).astype(np.uint8)
    scales, zps = [0.5, 0.25, 2.0, 0.125], [0, 128, 3, 255]
    qa = UniformQuantizedPerAxisType(A.UI8, A.F32, scales, zps, 0, 0, 255)
    c = ContentAttr.get(x, backend=oracle).quantCast(qa).dequantize().fold()
    want = ((x.astype(np.int64) - np.array(zps).reshape(4, 1, 1, 1)) * np.array(scales, np.float64).reshape(4, 1, 1, 1)).astype(np.float32)
    assert np.array_equal(c.getValues().reshape(x.shape), want)
    f = rng.normal(0, 3, (5, 7)).astype(np.float32)
    c = ContentAttr.get(f, backend=oracle).rescale(0.3).add(1.5).fold()
    assert np.array_equal(c.getValues().reshape(f.shape), f * np.float32(0.3) + np.float32(1.5))
    c = ContentAttr.get(f, backend=oracle).convertElemType(A.F16).fold()
    assert np.array_equal(c.copyTo().view(np.float16).reshape(f.shape), f.astype(np.float16))


def test_bit_pack_and_sub_byte_copy_out(oracle):
    rng = np.random.default_rng(6)
    v = rng.integers(0, 16, 64).astype(np.uint8)
    c = ContentAttr.get(v, NDType((64,), A.UI8), backend=oracle).bitPack(4).fold()
    assert np.array_equal(c.copyTo(), v[0::2] | (v[1::2] << 4))            # low nibble first
    c = ContentAttr.get(v, NDType((64,), A.UI8), backend=oracle).convertElemType(A.UI4).fold()
    assert np.array_equal(c.copyTo(), (v[0::2] << 4) | v[1::2])            # first element in the high nibble
    b = rng.integers(0, 2, 64).astype(np.uint8)
    c = ContentAttr.get(b, NDType((64,), A.UI8), backend=oracle).convertElemType(A.I1).fold()
    assert np.array_equal(c.copyTo(), np.packbits(b, bitorder="big"))      # first element in the top bit


def test_sparsity_map_and_sparsify_layout(oracle):
    rng = np.random.default_rng(7)
    for oc, work, density in [(3, 16, 0.5), (5, 40, 0.3), (2, 128, 0.9), (4, 200, 0.05)]:
        w = rng.integers(1, 128, (oc, work, 1, 1)).astype(np.int8)
        w[rng.random(w.shape) >= density] = 0
        c = ContentAttr.get(w, backend=oracle).getSparsityMap().fold()
        row_bits = (work + 127) // 128 * 128
        assert c.getType().shape == (oc, 1, 1, row_bits)
        want = np.zeros((oc, row_bits), np.uint8)
        want[:, :work] = w.reshape(oc, work) != 0
        assert np.array_equal(c.copyTo(), np.packbits(want, axis=1, bitorder="little").reshape(-1))
        c = ContentAttr.get(w, backend=oracle).sparsify(False).fold()
        out = c.copyTo()
        chunks = []
        for ch in w.reshape(oc, work):
            kept = ch[ch != 0].view(np.uint8)
            chunks.append(np.concatenate([kept, np.zeros(-kept.size % 16, np.uint8)]))  # channel starts are 16-byte aligned
        want = np.concatenate(chunks)
        assert c.bytesWritten == want.size and np.array_equal(out[:want.size], want)
        counts = ContentAttr.get(w, backend=oracle).countNonSparseElementsPerOC()
        assert list(counts) == [int((ch != 0).sum()) for ch in w.reshape(oc, work)]


def test_swizzle_rotates_chunks_inside_512_byte_blocks(oracle):
    rng = np.random.default_rng(8)
    for key, n in itertools.product(range(6), (512, 1536, 5000, 40000)):
        x = rng.integers(0, 256, n).astype(np.uint8)
        c = ContentAttr.get(x, NDType((n, 1, 1, 1), A.UI8), backend=oracle).swizzleConstant(key, 3).fold()
        total = (n + 511) // 512 * 512
        out = c.copyTo()
        assert out.size == total
        padded = np.concatenate([x, np.zeros(total - n, np.uint8)])
        want = np.empty(total, np.uint8)
        for a in range(0, total, 16):
            block = (a >> 9) & 63
            stagger = (block & ((1 << key) - 1)) << (9 - key)
            to = (a & ~511) + ((a + stagger) & 511)
            want[to:to + 16] = padded[a:a + 16]
        assert np.array_equal(out, want), (key, n)


def test_broadcast_and_reverse(oracle):
    rng = np.random.default_rng(9)
    x = rng.integers(0, 100, (1, 3, 1, 4)).astype(np.uint8)
    c = ContentAttr.get(x, backend=oracle).broadcast(0, 5).broadcast(2, 2).fold()
    assert c.copyTo().tobytes() == np.ascontiguousarray(np.broadcast_to(x, (5, 3, 2, 4))).tobytes()
    y = rng.normal(0, 1, (2, 3, 4)).astype(np.float32)
    for axis in range(2):  # the last dim cannot be the axis
        c = ContentAttr.get(y, backend=oracle).reverse(axis).fold()
        # Reverse<axis>: everything behind the axis is reversed as one run
        run = int(np.prod(y.shape[axis + 1:]))
        assert np.array_equal(c.getValues().reshape(-1, run), y.reshape(-1, run)[:, ::-1])
