"""Parity of the CUDA library (through the C ABI) with the CPU oracle on seeded inputs.

Integer, packed, sparsity-map, swizzled and compressed bytes must be bit-exact; float outputs are
compared bit-exactly too (the tolerance the task allows, 1 fp16 ulp, is stated where it would apply
but is not needed: both sides use the same double -> float -> half rounding sequence).
"""
import numpy as np
import pytest

from npu_plugin_b200 import _cabi as A
from npu_plugin_b200.const import (ConstError, ContentAttr, DimsOrder, NDType, Transform, UniformQuantizedPerAxisType,
                                   UniformQuantizedType)

pytestmark = pytest.mark.gpu

FP16_ULP_TOLERANCE = 0  # allowed: 1 ulp; achieved and asserted: 0


def both(attr_builder, gpu, oracle):
    """Fold the same attribute on both sides; returns (gpu content, oracle content)."""
    return attr_builder(gpu).fold(), attr_builder(oracle).fold()


def assert_same(cg, co):
    assert cg.getType() == co.getType(), (cg.getType(), co.getType())
    assert cg.bytesWritten == co.bytesWritten
    g, o = cg.copyTo(), co.copyTo()
    assert g.shape == o.shape
    if not np.array_equal(g, o):
        bad = np.flatnonzero(g != o)
        raise AssertionError(f"{bad.size} bytes differ, first at {bad[0]}: gpu={g[bad[0]]} oracle={o[bad[0]]}")


# ------------------------------------------------------------------ config 1
# Single Conv weight: f32 [256,256,3,3] N(0,0.05) -> per-channel symmetric int8 -> OIYX->OYXI ->
# pad I to a multiple of 16 -> swizzle key 5.  589,824-byte blob + 256 f32 scales.
def cfg1_attr(backend, w, pad_i=0):
    O, I, Y, X = w.shape
    a = ContentAttr.get(w, NDType(w.shape, A.F32), backend=backend).quantizeSynth(A.QSYNTH_SYM_I8)
    q = UniformQuantizedPerAxisType(A.SI8, A.F32, [1.0] * O, [0] * O, 0, -127, 127)
    a = a.convertElemType(A.SI8).quantCast(q).reorder(DimsOrder.OYXI)
    a = a.padWithZero((0, 0, 0, 0), (0, pad_i, 0, 0)).swizzleConstant(5, 3)
    return a


@pytest.mark.parametrize("shape,pad", [((256, 256, 3, 3), 0), ((64, 3, 7, 7), 13), ((32, 24, 1, 1), 8)])
def test_cfg1_conv_weight(gpu, oracle, shape, pad):
    rng = np.random.default_rng(1)
    w = rng.normal(0, 0.05, shape).astype(np.float32)
    ag, ao = cfg1_attr(gpu, w, pad), cfg1_attr(oracle, w, pad)
    cg, co = ag.fold(), ao.fold()
    assert_same(cg, co)
    assert np.array_equal(ag.sideScales, ao.sideScales)
    if shape == (256, 256, 3, 3):
        assert cg.bytesWritten == 589824
    # independent numpy restatement of the whole chain
    O = shape[0]
    amax = np.abs(w.reshape(O, -1)).max(axis=1)
    scale = (amax / np.float32(127)).astype(np.float32)
    qv = np.clip(np.rint(w / scale[:, None, None, None]), -127, 127).astype(np.int8)
    nhwc = np.transpose(qv, (0, 2, 3, 1))
    nhwc = np.pad(nhwc, ((0, 0), (0, 0), (0, 0), (0, pad)))
    flat = nhwc.reshape(-1).view(np.uint8)
    padded = np.zeros((flat.size + 511) // 512 * 512, np.uint8)
    padded[:flat.size] = flat
    assert np.array_equal(oracle.deswizzle(cg.copyTo(), 5), padded)
    assert np.array_equal(ag.sideScales, scale)


# ------------------------------------------------------------------ config 2
# int4 weight-only linear: f16 [O,I] N(0,0.02) -> per-channel asymmetric u4 -> BitPack -> NHWC [O,I,1,1];
# and the Dequantize leg back to f16.
def cfg2_pack_attr(backend, w):
    O, I = w.shape
    a = ContentAttr.get(w.reshape(O, I, 1, 1), NDType((O, I, 1, 1), A.F16), backend=backend)
    a = a.quantizeSynth(A.QSYNTH_ASYM_U4)
    q = UniformQuantizedPerAxisType(A.UI8, A.F16, [1.0] * O, [0] * O, 0, 0, 15)
    # BitPack is LAST, so the Reorder added after it lands in front of it (content.cpp:268-299)
    return a.convertElemType(A.UI8).quantCast(q).bitPack(4).reorder(DimsOrder.NHWC)


@pytest.mark.parametrize("shape", [(64, 256), (300, 4096)])
def test_cfg2_int4_pack_and_dequant(gpu, oracle, shape):
    rng = np.random.default_rng(2)
    w = rng.normal(0, 0.02, shape).astype(np.float16)
    ag, ao = cfg2_pack_attr(gpu, w), cfg2_pack_attr(oracle, w)
    assert [t.getTransformationName() for t in ag.getTransformations()][-2:] == ["Reorder", "BitPack"]
    cg, co = ag.fold(), ao.fold()
    assert_same(cg, co)
    assert cg.bytesWritten == shape[0] * shape[1] // 2
    assert np.array_equal(ag.sideScales, ao.sideScales) and np.array_equal(ag.sideZeroPoints, ao.sideZeroPoints)
    # numpy restatement
    wf = w.astype(np.float32)
    mn, mx = wf.min(axis=1), wf.max(axis=1)
    scale = ((mx - mn) / np.float32(15)).astype(np.float32)
    zp = np.clip(np.rint(-mn / scale), 0, 15).astype(np.float32)
    qv = np.clip(np.rint(wf / scale[:, None]) + zp[:, None], 0, 15).astype(np.uint8)
    packed = (qv[:, 0::2] | (qv[:, 1::2] << 4)).reshape(-1)
    assert np.array_equal(cg.copyTo(), packed)

    # dequantize leg: u8 values -> QuantCast(per-axis scale, zp) -> Dequantize (expressed f16)
    O, I = shape
    qt = UniformQuantizedPerAxisType(A.UI8, A.F16, [float(s) for s in ag.sideScales],
                                     [int(z) for z in ag.sideZeroPoints], 0, 0, 15)

    def deq(backend):
        return ContentAttr.get(qv.reshape(O, I, 1, 1), NDType((O, I, 1, 1), A.UI8), backend=backend) \
            .quantCast(qt).reorder(DimsOrder.NHWC).dequantize()

    dg, do = deq(gpu).fold(), deq(oracle).fold()
    assert dg.getType().dtype == A.F16
    assert_same(dg, do)
    # round trip: |w - dequant(quant(w))| <= scale/2 (+ f16 rounding)
    back = dg.getValues().astype(np.float32).reshape(O, I)
    assert np.all(np.abs(back - wf) <= scale[:, None] * 0.5 + 1e-3)


# ------------------------------------------------------------------ config 3
# sparse int8 1x1 conv weight: map (1 bit/elem, per-channel 128-bit padding) and compacted values
# (per-channel 16-byte alignment), both swizzled.
@pytest.mark.parametrize("shape", [(1024, 1024, 1, 1), (37, 24, 3, 3), (5, 8, 1, 1)])
def test_cfg3_sparse_weights(gpu, oracle, shape):
    rng = np.random.default_rng(3)
    w = rng.integers(-127, 128, shape, dtype=np.int8)
    w[rng.random(shape) < 0.5] = 0

    def base(b):
        return ContentAttr.get(w, NDType(shape, A.SI8), backend=b)

    mg, mo = both(lambda b: base(b).getSparsityMap().swizzleConstant(5, 3), gpu, oracle)
    assert_same(mg, mo)
    counts_g, counts_o = base(gpu).countNonSparseElementsPerOC(), base(oracle).countNonSparseElementsPerOC()
    assert counts_g == counts_o == [int(np.count_nonzero(w[o])) for o in range(shape[0])]
    sg, so = both(lambda b: base(b).sparsify(True, counts_o).swizzleConstant(5, 3), gpu, oracle)
    assert_same(sg, so)
    # Sparsify<false> folds to the same bytes (the attribute type differs, the content does not)
    fg, fo = both(lambda b: base(b).sparsify(False).swizzleConstant(5, 3), gpu, oracle)
    assert_same(fg, fo)
    assert np.array_equal(fg.copyTo(), sg.copyTo())
    # the map really marks the non-zeros
    work = shape[1] * shape[2] * shape[3]
    bits = np.unpackbits(oracle.deswizzle(mg.copyTo(), 5), bitorder="little")
    per_oc = (work + 127) // 128 * 128
    assert np.array_equal(bits[:shape[0] * per_oc].reshape(shape[0], per_oc)[:, :work], (w.reshape(shape[0], -1) != 0))


@pytest.mark.parametrize("dtype,npdt", [(A.F16, np.float16), (A.F32, np.float32), (A.UI8, np.uint8)])
def test_sparsity_other_types(gpu, oracle, dtype, npdt):
    rng = np.random.default_rng(33)
    shape = (6, 16, 2, 2)
    w = (rng.integers(-3, 4, shape)).astype(npdt) if npdt != np.uint8 else rng.integers(0, 4, shape).astype(np.uint8)
    if npdt != np.uint8:
        w.reshape(-1)[5] = -0.0  # negative zero counts as sparse (float comparison)

    def base(b):
        a = ContentAttr.get(w, NDType(shape, dtype), backend=b)
        if dtype == A.UI8:
            a = a.quantCast(UniformQuantizedType(A.UI8, A.F32, 0.5, 2, 0, 255))
        return a

    assert_same(*both(lambda b: base(b).getSparsityMap(), gpu, oracle))
    assert_same(*both(lambda b: base(b).sparsify(False), gpu, oracle))


# ------------------------------------------------------------------ config 4
# ResNet-50-shaped int8 weights -> QuantCast -> OYXI (-> pad for the stem) -> block compression.
RESNET_SHAPES = [(64, 3, 7, 7), (64, 64, 1, 1), (64, 64, 3, 3), (256, 64, 1, 1), (128, 128, 3, 3), (512, 2048, 1, 1),
                 (1000, 2048, 1, 1)]


def laplace_i8(rng, shape, b=12.0, zeros=0.1):
    x = np.clip(np.rint(rng.laplace(0, b, shape)), -127, 127).astype(np.int8)
    x[rng.random(shape) < zeros] = 0
    return x


@pytest.mark.parametrize("shape", RESNET_SHAPES)
def test_cfg4_resnet_fold_and_compress(gpu, oracle, shape):
    rng = np.random.default_rng(4 + shape[0] + shape[1])
    w = laplace_i8(rng, shape)
    pad = (-shape[1]) % 16 if shape[1] < 16 else 0

    def chain(b):
        q = UniformQuantizedType(A.SI8, A.F16, 0.01, 0, -127, 127)
        a = ContentAttr.get(w, NDType(shape, A.SI8), backend=b).quantCast(q).reorder(DimsOrder.OYXI)
        if pad:
            a = a.padWithZero((0, 0, 0, 0), (0, pad, 0, 0))
        return a

    cg, co = both(chain, gpu, oracle)
    assert_same(cg, co)
    folded = cg.copyTo()
    sg, ns_g = gpu.btc_compress(folded)
    so, ns_o = oracle.btc_compress(folded)
    assert ns_g == ns_o
    assert np.array_equal(sg, so), "compressed stream differs from the oracle encoder"
    assert len(sg) % 32 == 0 and len(sg) <= gpu.btc_bound(folded.size)
    assert np.array_equal(oracle.btc_decompress(sg, folded.size), folded)
    assert np.array_equal(gpu.btc_decompress(sg, folded.size), folded)


# ------------------------------------------------------------------ config 5 (shape analogue)
# 7B-style linear: f16 [O,I] -> symmetric int8 -> Reorder NHWC -> swizzle(5) -> compression
@pytest.mark.parametrize("shape", [(128, 512), (96, 1000)])
def test_cfg5_linear_chain(gpu, oracle, shape):
    rng = np.random.default_rng(5)
    w = rng.normal(0, 0.02, shape).astype(np.float16)
    O, I = shape

    def chain(b):
        a = ContentAttr.get(w.reshape(O, I, 1, 1), NDType((O, I, 1, 1), A.F16), backend=b)
        a = a.quantizeSynth(A.QSYNTH_SYM_I8).convertElemType(A.SI8)
        a = a.quantCast(UniformQuantizedPerAxisType(A.SI8, A.F16, [1.0] * O, [0] * O, 0, -127, 127))
        return a.reorder(DimsOrder.NHWC).swizzleConstant(5, 3)

    ag, ao = chain(gpu), chain(oracle)
    cg, co = ag.fold(), ao.fold()
    assert_same(cg, co)
    assert np.array_equal(ag.sideScales, ao.sideScales)
    sg, ns_g = gpu.btc_compress(cg.copyTo())
    so, ns_o = oracle.btc_compress(cg.copyTo())
    assert ns_g == ns_o and np.array_equal(sg, so)


# ------------------------------------------------------------------ codec
@pytest.mark.parametrize("n", [1, 63, 64, 65, 4095, 4096, 4097, 50176, 100000])
@pytest.mark.parametrize("kind", ["const", "ramp", "sparse", "small", "noise"])
def test_codec_parity_and_roundtrip(gpu, oracle, n, kind):
    rng = np.random.default_rng(n)
    if kind == "const":
        x = np.full(n, 1, np.uint8)
    elif kind == "ramp":
        x = (np.arange(n) % 7 + 100).astype(np.uint8)
    elif kind == "sparse":
        x = rng.integers(0, 256, n).astype(np.uint8)
        x[rng.random(n) < 0.8] = 0
    elif kind == "small":
        x = rng.integers(-5, 6, n).astype(np.int8).view(np.uint8)
    else:
        x = rng.integers(0, 256, n).astype(np.uint8)
    sg, ns_g = gpu.btc_compress(x)
    so, ns_o = oracle.btc_compress(x)
    assert ns_g == ns_o
    assert np.array_equal(sg, so)
    assert np.array_equal(gpu.btc_decompress(sg, n), x)
    assert np.array_equal(oracle.btc_decompress(sg, n), x)
    assert ns_g == (n <= len(sg))


def test_codec_every_mode_and_field_width(gpu, oracle):
    """Blocks built so that every record form occurs -- RAW, CONST, PACKU and PACKS with each field width from 1 to 7,
    SPARSE -- shuffled, so that the blocks of one iteration of the emit kernel mix all forms, at several lengths
    (a ragged tail, block counts around the kernel's 128-block iterations and 1024-block shares)."""
    rng = np.random.default_rng(99)
    blocks = []
    for rep in range(40):
        for w in range(1, 8):
            lo = int(rng.integers(40, 100)) if w < 7 else 100
            blocks.append((lo + rng.integers(0, 1 << w, 64)).astype(np.uint8))            # PACKU, width w
            blocks[-1][:2] = (lo, lo + (1 << w) - 1)
            half = 1 << (w - 1)
            b = rng.integers(-half, half, 64).astype(np.int8)
            b[:2] = (-half, half - 1)
            blocks.append(b.view(np.uint8))                                               # PACKS, width w
        blocks.append(rng.integers(0, 256, 64).astype(np.uint8))                          # RAW
        blocks.append(np.full(64, int(rng.integers(0, 256)), np.uint8))                   # CONST
        sp = rng.integers(1, 256, 64).astype(np.uint8)
        sp[rng.random(64) < 0.85] = 0
        blocks.append(sp)                                                                 # SPARSE
    order = rng.permutation(len(blocks))
    x_all = np.concatenate([blocks[i] for i in order])
    modes = set()
    for n in (x_all.size, 64 * 127, 64 * 128 + 5, 64 * 1024, 64 * 1025 - 1, 64 * 300 + 37):
        x = np.resize(x_all, n)
        sg, ns_g = gpu.btc_compress(x)
        so, ns_o = oracle.btc_compress(x)
        assert ns_g == ns_o and np.array_equal(sg, so), f"stream of {n} bytes differs from the oracle encoder"
        assert np.array_equal(gpu.btc_decompress(sg, n), x)
        assert np.array_equal(oracle.btc_decompress(sg, n), x)
    # the forms really occur: walk the records of the first stream
    so, _ = oracle.btc_compress(x_all)
    nblocks = (x_all.size + 63) // 64
    nsuper = (nblocks + 63) // 64
    at = 32 + 4 * nsuper
    for _ in range(nblocks):
        h = int(so[at])
        mode, w = h >> 5, h & 31
        modes.add((mode, w))
        at += {0: 65, 1: 2, 2: 2 + 8 * w, 3: 1 + 8 * w}.get(mode, 9 + int(np.unpackbits(so[at + 1:at + 9]).sum()))
    assert {(0, 0), (1, 0), (4, 0)} <= modes
    assert {(2, w) for w in range(1, 8)} <= modes and {(3, w) for w in range(1, 8)} <= modes


def test_truncated_and_malformed_streams_are_rejected(backend):
    """A stream cut anywhere -- inside the header, the index, a record, the mask of a SPARSE record -- or with an
    unassigned mode in a record header is reported as an error; the decoder looks at no byte behind the end of the
    stream it was given (the size of a SPARSE record is only read once its mask is known to be inside)."""
    from npu_plugin_b200.const import ConstError
    rng = np.random.default_rng(5)
    x = rng.integers(1, 256, 64 * 70).astype(np.uint8)
    x[rng.random(x.size) < 0.85] = 0          # every block becomes a SPARSE record
    stream, not_smaller = backend.btc_compress(x)
    assert not not_smaller
    assert np.array_equal(backend.btc_decompress(stream, x.size), x)
    first_record = 32 + 4 * 2                  # header + two index entries (70 blocks)
    assert stream[first_record] >> 5 == 4
    for cut in (0, 10, 31, 33, first_record, first_record + 1, first_record + 5, first_record + 8, first_record + 9,
                stream.size // 2, stream.size - 40):
        with pytest.raises(ConstError):
            backend.btc_decompress(stream[:cut].copy(), x.size)
    for bad_mode in (5, 6, 7):
        broken = stream.copy()
        broken[first_record] = (bad_mode << 5) | (broken[first_record] & 31)
        with pytest.raises(ConstError):
            backend.btc_decompress(broken, x.size)


# ------------------------------------------------------------------ random chains
def random_chain(rng, backend, base, btype, splat=False):
    """A random mix of index and value transformations over one base tensor (same draws for both backends)."""
    a = ContentAttr.get(base, btype, is_splat=splat, backend=backend)
    shape = list(btype.shape)
    r = len(shape)
    quant = False
    for _ in range(int(rng.integers(1, 7))):
        op = int(rng.integers(0, 8))
        if op == 0:  # reorder
            a = a.reorder(DimsOrder(rng.permutation(r).tolist()))
        elif op == 1:  # subview
            off = [int(rng.integers(0, s)) for s in shape]
            shp = [int(rng.integers(1, s - o + 1)) for s, o in zip(shape, off)]
            a = a.subview(off, shp)
            shape = shp
        elif op == 2:  # pad
            before = [int(rng.integers(0, 3)) for _ in shape]
            after = [int(rng.integers(0, 3)) for _ in shape]
            if quant == "axis":
                before[0] = after[0] = 0 if r != 4 else before[0]
            a = a.padWithZero(before, after)
            shape = [s + b + c for s, b, c in zip(shape, before, after)]
        elif op == 3:
            a = a.rescale(float(rng.choice([0.5, 2.0, 0.1, -3.0])))
        elif op == 4:
            a = a.add(float(rng.choice([0.0, 1.0, -7.5, 100.0])))
        elif op == 5 and not quant and a.getType().dtype in (A.UI8, A.SI8):
            dt = a.getType().dtype
            zp = 3 if dt == A.UI8 else -2
            if r == 4 and rng.random() < 0.5:
                n = shape[0]
                a = a.quantCast(UniformQuantizedPerAxisType(dt, A.F32, [0.25 * (i + 1) for i in range(n)], [zp] * n, 0))
                quant = "axis"
            else:
                a = a.quantCast(UniformQuantizedType(dt, A.F16, 0.125, zp))
                quant = "tensor"
        elif op == 6 and quant:
            a = a.dequantize()
            quant = False
        elif op == 7 and not quant:
            a = a.convertElemType(int(rng.choice([A.F32, A.F16, A.SI32, A.F64, A.SI16])))
    return a


@pytest.mark.parametrize("seed", range(60))
def test_random_chains(gpu, oracle, seed):
    rng = np.random.default_rng(1000 + seed)
    r = int(rng.integers(1, 6))
    shape = [int(rng.integers(1, 7)) for _ in range(r)]
    kind = int(rng.integers(0, 4))
    if kind == 0:
        base, dt = rng.integers(0, 20, shape).astype(np.uint8), A.UI8
    elif kind == 1:
        base, dt = rng.integers(-20, 20, shape).astype(np.int8), A.SI8
    elif kind == 2:
        base, dt = rng.integers(-50, 50, shape).astype(np.float32), A.F32
    else:
        base, dt = (rng.integers(-50, 50, shape) * 0.5).astype(np.float16), A.F16
    splat = rng.random() < 0.15
    if splat:
        base = base.reshape(-1)[:1].copy()
    btype = NDType(shape, dt)

    def run(backend):
        state = np.random.default_rng(seed)  # identical draws on both sides
        try:
            return random_chain(state, backend, base, btype, splat).fold(), None
        except ConstError as e:
            return None, str(e)

    (cg, eg), (co, eo) = run(gpu), run(oracle)
    assert (eg is None) == (eo is None), (eg, eo)
    if eg is None:
        assert_same(cg, co)


# ------------------------------------------------------------------ data-dependent errors
def test_checked_cast_errors(gpu, oracle):
    # f32 300.0 -> si8 is out of range at copy-out (checked_cast.hpp:106-117)
    for backend in (gpu, oracle):
        a = ContentAttr.get(np.array([1.0, 300.0], np.float32), NDType((2,), A.F32), backend=backend)
        with pytest.raises(ConstError):
            a.convertElemType(A.SI8).fold()
        # si32 16777217 -> f32 is inexact (checked_cast.hpp:119-125)
        b = ContentAttr.get(np.array([16777217], np.int32), NDType((1,), A.SI32), backend=backend)
        with pytest.raises(ConstError):
            b.rescale(1.0).fold()
        # negative value into BitPack's uint8 read
        c = ContentAttr.get(np.array([-1, 2], np.int8), NDType((2,), A.SI8), backend=backend)
        with pytest.raises(ConstError):
            c.bitPack(4).fold()
        # splat into BitPack, odd count
        with pytest.raises(ConstError):
            ContentAttr.get(np.array([1], np.int8), NDType((4,), A.SI8), is_splat=True, backend=backend).bitPack(4).fold()
        with pytest.raises(ConstError):
            ContentAttr.get(np.array([1, 2, 3], np.int8), NDType((3,), A.SI8), backend=backend).bitPack(4).fold()
        # per-axis zero points that differ cannot be sparsified (sparsity.cpp:19-22)
        q = UniformQuantizedPerAxisType(A.UI8, A.F32, [1.0, 1.0], [1, 2], 0)
        d = ContentAttr.get(np.zeros((2, 8, 1, 1), np.uint8), NDType((2, 8, 1, 1), A.UI8), backend=backend).quantCast(q)
        with pytest.raises(ConstError):
            d.getSparsityMap().fold()
    # after an error the context keeps working
    ok = ContentAttr.get(np.array([1.0, 2.0], np.float32), NDType((2,), A.F32), backend=gpu).convertElemType(A.SI8).fold()
    assert list(ok.copyTo()) == [1, 2]


def test_empty_and_tiny(gpu, oracle):
    for shape in [(0,), (1,), (1, 1, 1, 1), (2, 0, 3)]:
        w = np.zeros(shape, np.float32)
        assert_same(*both(lambda b: ContentAttr.get(w, NDType(shape, A.F32), backend=b).convertElemType(A.F16), gpu, oracle))


# ------------------------------------------------------------------ fused quantiser edge cases
# The single-pass kernel replaces the per-element IEEE division and rint by an FMA-corrected
# reciprocal and a magic-constant rounding; these rows are built to sit on rounding ties and at the
# edges of the float range, for every kernel variant (warp rows, register rows, staged rows, scalar tails).
@pytest.mark.parametrize("npdt,dt", [(np.float16, A.F16), (np.float32, A.F32)])
@pytest.mark.parametrize("scheme", [A.QSYNTH_SYM_I8, A.QSYNTH_ASYM_U4])
@pytest.mark.parametrize("rowlen", [16, 100, 1024, 1040, 4096, 11008, 20000])
def test_fused_quantiser_ties_and_extremes(gpu, oracle, npdt, dt, scheme, rowlen):
    rng = np.random.default_rng(rowlen + scheme)
    rows = 9
    w = rng.normal(0, 1, (rows, rowlen)).astype(np.float32)
    # row 0: exact multiples of amax/254 -> quotients on .5 ties
    amax = 3.96875
    k = rng.integers(-254, 255, rowlen)
    w[0] = (k * (amax / 254.0))
    w[0, 0] = amax
    # row 1: all zero (scale falls back to 1); row 2: a single non-zero
    w[1] = 0
    w[2] = 0
    w[2, rowlen // 2] = -0.5
    # row 3: tiny magnitudes; row 4: large magnitudes
    w[3] *= 1e-6
    w[4] *= 1000.0 if npdt == np.float16 else 1e30
    # row 5: constant row (asymmetric scale is zero -> 1)
    w[5] = 0.37
    if npdt == np.float32:
        w[6] *= 1e-38  # subnormal products
        w[7, ::3] = np.float32(1e-45)
    w = w.astype(npdt)
    store = A.SI8 if scheme == A.QSYNTH_SYM_I8 else A.UI8
    qmin, qmax = (-127, 127) if scheme == A.QSYNTH_SYM_I8 else (0, 15)

    def chain(b, swz, pack):
        a = ContentAttr.get(w.reshape(rows, rowlen, 1, 1), NDType((rows, rowlen, 1, 1), dt), backend=b)
        a = a.quantizeSynth(scheme).convertElemType(store)
        a = a.quantCast(UniformQuantizedPerAxisType(store, A.F32, [1.0] * rows, [0] * rows, 0, qmin, qmax))
        if pack:
            return a.bitPack(4)
        return a.swizzleConstant(5, 3) if swz else a

    for swz, pack in [(False, False), (True, False)] + ([(False, True)] if scheme == A.QSYNTH_ASYM_U4 and rowlen % 2 == 0 else []):
        ag, ao = chain(gpu, swz, pack), chain(oracle, swz, pack)
        assert_same(ag.fold(), ao.fold())
        assert np.array_equal(ag.sideScales, ao.sideScales) and np.array_equal(ag.sideZeroPoints, ao.sideZeroPoints)


# ------------------------------------------------------------------ byte-moving views (tile kernel bodies)
# Reorders and copies that change no value take vectorised bodies in the tile kernel: block transposes
# with 3x3 kernels (register byte permutes), other kernel sizes and element widths (32-bit pieces),
# unaligned extents (scalar pieces), with and without the swizzle rotation and a leading SubView that
# breaks the 16-byte alignment of the source.
@pytest.mark.parametrize("shape", [(64, 64, 3, 3), (40, 512, 3, 3), (7, 48, 3, 3), (16, 20, 3, 3), (8, 32, 7, 7),
                                   (12, 6, 5, 5), (5, 3, 2, 2), (300, 16, 1, 1), (3, 1000, 1, 1)])
@pytest.mark.parametrize("dt,npdt", [(A.SI8, np.int8), (A.F16, np.float16), (A.F32, np.float32), (A.F64, np.float64)])
@pytest.mark.parametrize("swizzle", [False, True])
def test_reorder_moves_bytes(gpu, oracle, shape, dt, npdt, swizzle):
    rng = np.random.default_rng(11)
    w = rng.integers(-100, 100, shape).astype(npdt)

    def build(backend):
        a = ContentAttr.get(w, NDType(shape, dt), backend=backend).reorder(DimsOrder.OYXI)
        return a.swizzleConstant(5, 3) if swizzle else a

    cg, co = both(build, gpu, oracle)
    assert_same(cg, co)
    if not swizzle:
        want = np.ascontiguousarray(w.transpose(0, 2, 3, 1)).view(np.uint8).ravel()
        assert np.array_equal(cg.copyTo().ravel()[:want.size], want)


@pytest.mark.parametrize("off", [1, 3, 16])
@pytest.mark.parametrize("chan", [64, 20])
@pytest.mark.parametrize("inner", [False, True])
def test_reorder_after_subview(gpu, oracle, off, chan, inner):
    rng = np.random.default_rng(12)
    shape = (40 + off, chan + (off if inner else 0), 3, 3)
    w = rng.integers(-100, 100, shape).astype(np.int8)
    lo = (off, off if inner else 0, 0, 0)

    def build(backend):
        a = ContentAttr.get(w, NDType(shape, A.SI8), backend=backend).subview(lo, (40, chan, 3, 3))
        return a.reorder(DimsOrder.OYXI)

    cg, co = both(build, gpu, oracle)
    assert_same(cg, co)
    want = np.ascontiguousarray(w[lo[0]:, lo[1]:].transpose(0, 2, 3, 1)).view(np.uint8).ravel()
    assert np.array_equal(cg.copyTo().ravel(), want)


# ------------------------------------------------------------------ Broadcast / Reverse / ExpandDilated
@pytest.mark.parametrize("dt,npdt", [(A.SI8, np.int8), (A.UI8, np.uint8), (A.F16, np.float16), (A.F32, np.float32)])
@pytest.mark.parametrize("order", [None, DimsOrder.NHWC])
def test_remaining_transforms_match_oracle(gpu, oracle, dt, npdt, order):
    rng = np.random.default_rng(31)
    shape = (3, 4, 5, 6)
    w = rng.integers(0, 100, shape).astype(npdt)

    def base(backend):
        a = ContentAttr.get(w, NDType(shape, dt), backend=backend)
        return a.reorder(order) if order is not None else a

    builders = [
        lambda b: base(b).reverse(0),
        lambda b: base(b).reverse(2),
        lambda b: base(b).add(1.0).reverse(1) if dt in (A.F16, A.F32) else base(b).reverse(1),
        lambda b: base(b).expandDilated((2, 3)),
        lambda b: base(b).subview((0, 1, 0, 0), (3, 2, 5, 6)).expandDilated((1, 2)),
        lambda b: base(b).subview((0, 0, 0, 0), (1, 4, 5, 6)).broadcast(0, 4),
        lambda b: base(b).subview((0, 1, 0, 0), (3, 1, 5, 6)).broadcast(1, 5).reverse(1),
        lambda b: base(b).subview((0, 0, 2, 0), (3, 4, 1, 6)).broadcast(2, 3).padWithZero((0, 0, 1, 0), (0, 0, 0, 2)),
    ]
    for k, build in enumerate(builders):
        cg, co = build(gpu).fold(), build(oracle).fold()
        try:
            assert_same(cg, co)
        except AssertionError as e:
            raise AssertionError(f"builder {k}: {e}")


def test_expand_dilated_quantised_fill(gpu, oracle):
    rng = np.random.default_rng(32)
    w = rng.integers(0, 255, (2, 3, 3, 3)).astype(np.uint8)
    q = UniformQuantizedType(A.UI8, A.F16, 0.5, 128, 0, 255)

    def build(backend):
        return ContentAttr.get(w, NDType(w.shape, A.UI8), backend=backend).quantCast(q).expandDilated((2, 2))

    cg, co = both(build, gpu, oracle)
    assert_same(cg, co)
    assert cg.copyTo().reshape(2, 3, 5, 5)[0, 0, 1, 1] == 128  # the gaps hold the zero point


# ------------------------------------------------------------------ RelocateWeightsTable
@pytest.mark.parametrize("offsets,ptrs", [((0, 0), (1000, 1000)), ((0, 16, 32), (4096, 8192, 12288)), ((0, 8, 8, 40), (64, 128, 192, 256))])
@pytest.mark.parametrize("compressed", [False, True])
def test_relocate_weights_table(gpu, oracle, offsets, ptrs, compressed):
    rng = np.random.default_rng(41)
    OC = 48
    table = np.zeros((OC, 1, 1, 4), np.int32)
    table[:, 0, 0, 0] = 512 + 144 * np.arange(OC)      # weights pointers, constant step
    table[:, 0, 0, 1] = 7000 + 32 * np.arange(OC)      # sparsity pointers
    table[::5, 0, 0, 1] = 0xFFFFFF                      # channels without a sparsity map keep the marker
    table[:, 0, 0, 2:] = rng.integers(-1000, 1000, (OC, 2))
    table[5, 0, 0, 1] = 7000 + 32                       # keep entries 0 and 1 regular: they define the steps
    table[0, 0, 0, 1] = 7000
    num = [int(v) for v in rng.integers(1, 300, OC)] if compressed else None

    def build(backend):
        a = ContentAttr.get(table, NDType(table.shape, A.SI32), backend=backend)
        return a.relocateWeightsTablePointers(ptrs, 90000, offsets, 8 if compressed else 0, num, 0)

    cg, co = both(build, gpu, oracle)
    assert_same(cg, co)
    got = cg.getValues().reshape(OC, 4)
    assert np.array_equal(got[:, 2:], table[:, 0, 0, 2:])
    assert got[0, 0] == ptrs[0] and (got[10::5, 1] == 0xFFFFFF).all()


# ------------------------------------------------------------------ exhaustive small reorders
def _all_small_reorders():
    import itertools
    cases = []
    for rank in range(1, 6):
        shape = [2, 3, 4, 2, 3][:rank]
        for perm in itertools.permutations(range(rank)):
            cases.append((tuple(shape), perm))
    return cases


@pytest.mark.gpu
def test_every_permutation_of_small_tensors(gpu, oracle):
    """Every memory permutation of every rank up to 5 at extents of at most 4 (153 permutations), for 1-, 2- and
    4-byte elements, plain and followed by SwizzleConstant, folded in one batched call and compared with the oracle
    byte for byte -- the index arithmetic of the view composer and of the tile / generic kernels has no case left
    that only large shapes would reach."""
    from npu_plugin_b200.blob import ConstantDecl, ShardFolder
    rng = np.random.default_rng(17)
    decls, data = [], []
    for (shape, perm), (dt, npdt) in itertools_product(_all_small_reorders(), [(A.UI8, np.uint8), (A.F16, np.float16), (A.SI32, np.int32)]):
        x = rng.integers(0, 100, shape).astype(npdt)
        for swz in (False, True):
            chain = [Transform(A.X_REORDER, a=perm)] + ([Transform(A.X_SWIZZLE_CONSTANT, i0=5, i1=3)] if swz else [])
            if swz:
                # SwizzleConstant flattens to [N,1,1,1] under the input's order and the reference rejects the
                # combinations where that order does not fit the new shape: those are not folds
                try:
                    oracle.infer_type(NDType(shape, dt), chain)
                except ConstError:
                    continue
            decls.append(ConstantDecl(f"p{len(decls)}", NDType(shape, dt), chain, x.nbytes, compress=False))
            data.append(x)
    folder = ShardFolder(gpu, decls)
    total_in = sum(x.nbytes for x in data)
    src, out = gpu.dev_alloc(total_in + 16 * len(data)), gpu.dev_alloc(folder.folded_bytes)
    try:
        ptrs, at = [], 0
        for x in data:
            gpu.upload(src + at, x)
            ptrs.append(src + at)
            at += (x.nbytes + 15) // 16 * 16
        gpu.fill_zero(out, folder.folded_bytes)
        folder.fold(ptrs, out, True)
        gpu.synchronize()
        got = gpu.download(out, folder.folded_bytes)
        for i, (d, x) in enumerate(zip(decls, data)):
            want = oracle.fold(d.base_type, x, False, d.transforms).copyTo().reshape(-1).view(np.uint8)
            off = folder.folded_offsets[i]
            assert np.array_equal(got[off:off + want.size], want), f"{d.base_type.shape} perm {d.transforms[0].a} dtype {d.base_type.dtype}"
    finally:
        gpu.dev_free(src)
        gpu.dev_free(out)


def itertools_product(a, b):
    import itertools
    return itertools.product(a, b)
