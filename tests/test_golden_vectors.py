"""Known-answer tests taken from the reference's own unit and lit tests for the Const dialect.

Each case cites the reference test it restates (paths inside openvinotoolkit/npu_plugin):
  UT  = tests/unit/vpux_compiler/dialect/const/content_tests.cpp
  LIT = tests/lit/NPU/dialect/const/passes/
They run against the CPU oracle everywhere (this pins the oracle) and, on the GPU box, against the
CUDA library through the C ABI.
"""
import numpy as np
import pytest

from npu_plugin_b200 import _cabi as A
from npu_plugin_b200.const import (ConstError, ContentAttr, DimsOrder, NDType, UniformQuantizedPerAxisType,
                                   UniformQuantizedType)


def attr(backend, vals, shape, dtype, np_dtype=None, splat=False):
    arr = np.asarray(vals, dtype=np_dtype)
    return ContentAttr.get(arr, NDType(shape, dtype), is_splat=splat, backend=backend)


def iota(n, np_dtype):
    return np.arange(n).astype(np_dtype)


# UT:98-121 FromDenseElementsAttr / :356-378 CopyTo style: no transformation
def test_from_dense_and_copy_to(backend):
    vals = iota(24, np.float32)
    c = attr(backend, vals, (1, 2, 3, 4), A.F32).fold()
    assert c.getType() == NDType((1, 2, 3, 4), A.F32)
    assert np.array_equal(c.getValues(), vals)
    assert c.copyTo().tobytes() == vals.tobytes()


# UT:419-446 CopyTo_I4: first element lands in the high nibble
def test_copy_to_i4(backend):
    c = attr(backend, [1, 7, 10, 15], (4,), A.I8, np.uint8).convertElemType(A.I4).fold()
    assert c.getType().getTotalAllocSize() == 2
    assert list(c.copyTo()) == [0x17, 0xAF]


# UT:448-477 CopyTo_I1: first element lands in the most significant bit
def test_copy_to_i1(backend):
    vals = [0, 0, 0, 1, 0, 0, 1, 1, 1, 1, 1, 1, 1, 1, 1, 0]
    c = attr(backend, vals, (16,), A.I8, np.uint8).convertElemType(A.I1).fold()
    assert list(c.copyTo()) == [0x13, 0xFE]


# UT:479-503, :505-527 Splat_CopyTo_FP32 / U8
def test_splat_copy_to(backend):
    c = attr(backend, [1.0], (8,), A.F32, np.float32, splat=True).fold()
    assert np.array_equal(c.copyTo().view(np.float32), np.ones(8, np.float32))
    c = attr(backend, [1], (8,), A.I8, np.uint8, splat=True).fold()
    assert list(c.copyTo()) == [1] * 8


# UT:529-553 Splat_CopyTo_I4 and :555-579 Splat_CopyTo_I1
def test_splat_copy_to_subbyte(backend):
    c = attr(backend, [10], (4,), A.I8, np.uint8, splat=True).convertElemType(A.I4).fold()
    assert list(c.copyTo()) == [0xAA, 0xAA]
    c = attr(backend, [1], (16,), A.I8, np.uint8, splat=True).convertElemType(A.I1).fold()
    assert list(c.copyTo()) == [0xFF, 0xFF]


# UT:581-606 ConvertElemType f32 -> si32, :608-635 splat
def test_convert_elem_type(backend):
    vals = iota(24, np.float32)
    c = attr(backend, vals, (1, 2, 3, 4), A.F32).convertElemType(A.SI32).fold()
    assert c.getType() == NDType((1, 2, 3, 4), A.SI32)
    assert np.array_equal(c.getValues(np.int32), np.arange(24, dtype=np.int32))
    c = attr(backend, [4.0], (1, 2, 3, 4), A.F32, np.float32, splat=True).convertElemType(A.SI32).fold()
    assert np.array_equal(c.getValues(np.int32), np.full(24, 4, np.int32))


# UT:663-693 Add, and Rescale (CA/rescale.cpp:64-78)
def test_add_and_rescale(backend):
    vals = iota(24, np.float32)
    c = attr(backend, vals, (1, 2, 3, 4), A.F32).add(10).fold()
    assert np.array_equal(c.getValues(), vals + np.float32(10))
    c = attr(backend, vals, (1, 2, 3, 4), A.F32).rescale(0.1).fold()
    assert np.array_equal(c.getValues(), vals * np.float32(0.1))


# UT:695-724 QuantCast leaves the values alone
def test_quant_cast(backend):
    vals = iota(16, np.uint8)
    q = UniformQuantizedType(A.UI8, A.F32, 0.078431372549019607, 128, 0, 255)
    c = attr(backend, vals, (1, 16), A.UI8).quantCast(q).fold()
    assert c.getType().quant == q
    assert np.array_equal(c.copyTo(), vals)


# UT:726-764 Dequantize, scale 2/254
def test_dequantize(backend):
    vals = np.array([((i % 3) - 1) * 127 for i in range(16)], dtype=np.int8)
    q = UniformQuantizedType(A.SI8, A.F32, 2.0 / 254.0, 0, -127, 127)
    c = attr(backend, vals, (1, 16), A.SI8).quantCast(q).dequantize().fold()
    assert c.getType() == NDType((1, 16), A.F32)
    exp = np.array([float((i % 3) - 1) for i in range(16)], dtype=np.float32)
    np.testing.assert_allclose(c.getValues(), exp, rtol=4 * np.finfo(np.float32).eps)  # EXPECT_FLOAT_EQ = 4 ulp
    # the exact reference arithmetic: float((q - zp) * double scale)
    exact = ((vals.astype(np.int64) - 0).astype(np.float64) * (2.0 / 254.0)).astype(np.float32)
    assert np.array_equal(c.getValues(), exact)


# UT:766-797 Reshape is metadata only
def test_reshape(backend):
    vals = iota(18, np.float32)
    c = attr(backend, vals, (1, 9, 2), A.F32).reshape((1, 3, 3, 2)).fold()
    assert c.getType().shape == (1, 3, 3, 2)
    assert np.array_equal(c.getValues(), vals)


# UT:868-903 Reorder NCHW -> NHWC, :905-942 ReorderAfterReshape
@pytest.mark.parametrize("reshape_first", [False, True])
def test_reorder(backend, reshape_first):
    N, Cc, H, W = 1, 2, 2, 2
    vals = iota(N * Cc * H * W, np.float32)
    if reshape_first:
        a = attr(backend, vals, (N, Cc * H * W), A.F32).reshape((N, Cc, H, W))
    else:
        a = attr(backend, vals, (N, Cc, H, W), A.F32)
    c = a.reorder(DimsOrder.NHWC).fold()
    assert c.getType().order == DimsOrder.NHWC and c.getType().shape == (N, Cc, H, W)
    out = c.getValues()
    for n in range(N):
        for ch in range(Cc):
            for h in range(H):
                for w in range(W):
                    assert out[ch + w * Cc + h * Cc * W + n * Cc * W * H] == vals[w + h * W + ch * W * H + n * W * H * Cc]


def check_padded(out, exp, buf, pad, zp, act_off=0, orig_off=0):
    """checkPaddedBuffer, UT:55-80"""
    IC, IH, IW = buf
    PC, PH, PW = pad
    for c in range(IC + 2 * PC):
        for h in range(IH + 2 * PH):
            for w in range(IW + 2 * PW):
                ni = w + h * (IW + 2 * PW) + c * (IW + 2 * PW) * (IH + 2 * PH) + act_off
                if c < PC or c >= IC + PC or h < PH or h >= IH + PH or w < PW or w >= IW + PW:
                    assert out[ni] == zp, (c, h, w)
                else:
                    oi = (w - PW) + (h - PH) * IW + (c - PC) * IW * IH + orig_off
                    assert out[ni] == exp[oi], (c, h, w)


# UT:944-972 Pad, :974-1000 PadSplat
def test_pad(backend):
    vals = iota(6, np.int32)
    c = attr(backend, vals, (1, 2, 3), A.SI32).padWithZero((1, 1, 1), (1, 1, 1)).fold()
    assert c.getType().shape == (3, 4, 5)
    check_padded(c.getValues(np.int32), vals, (1, 2, 3), (1, 1, 1), 0)
    c = attr(backend, [42], (1, 2, 3), A.SI32, np.int32, splat=True).padWithZero((1, 1, 1), (1, 1, 1)).fold()
    check_padded(c.getValues(np.int32), np.full(6, 42, np.int32), (1, 2, 3), (1, 1, 1), 0)


# UT:1002-1045 PadUniformQuant: the pad value is the zero point (128); storage stays f32, copy-out gives u8
def test_pad_uniform_quant(backend):
    OC, IC, IH, IW = 2, 1, 2, 3
    vals = iota(OC * IC * IH * IW, np.float32)
    q = UniformQuantizedType(A.UI8, A.F32, 0.078431372549019607, 128, 0, 255)
    a = attr(backend, vals, (OC, IC, IH, IW), A.F32).convertElemType(A.UI8).quantCast(q)
    c = a.padWithZero((0, 2, 2, 2), (0, 2, 2, 2)).fold()
    out = c.copyTo()  # ui8 bytes
    for oc in range(OC):
        check_padded(out, vals, (IC, IH, IW), (2, 2, 2), 128, oc * (IC + 4) * (IW + 4) * (IH + 4), oc * IC * IW * IH)


# UT:1047-1106 PadPerAxisQuant: padded channels take the edge scales/zero points
def test_pad_per_axis_quant(backend):
    OC, IC, IH, IW = 2, 1, 2, 3
    vals = iota(OC * IC * IH * IW, np.float32)
    zp = 127
    q = UniformQuantizedPerAxisType(A.UI8, A.F32, [0.5, 0.5], [zp, zp], 0, 0, 255)
    a = attr(backend, vals, (OC, IC, IH, IW), A.F32).convertElemType(A.UI8).quantCast(q)
    a = a.padWithZero((2, 2, 2, 2), (2, 2, 2, 2))
    t = a.getType()
    assert t.shape == (6, 5, 6, 7) and t.quant.zps == [zp] * 6 and t.quant.scales == [0.5] * 6
    out = a.fold().copyTo()
    ch = IC * IW * IH
    exp = np.concatenate([np.full(ch * 2, zp, np.float32), vals, np.full(ch * 2, zp, np.float32)])
    for oc in range(OC + 4):
        check_padded(out, exp, (IC, IH, IW), (2, 2, 2), zp, oc * (IC + 4) * (IW + 4) * (IH + 4), oc * ch)


# UT:1108-1149 SubView, :1203-1231 SubViewSplat
def test_subview(backend):
    vals = iota(6, np.int32)
    c = attr(backend, vals, (1, 2, 3), A.SI32).subview((0, 1, 1), (1, 1, 1)).fold()
    assert c.getType().shape == (1, 1, 1)
    assert c.getValues(np.int32)[0] == vals[1 + 1 * 3]
    c = attr(backend, vals, (1, 2, 3), A.SI32).subview((0, 0, 1), (1, 2, 2)).fold()
    assert list(c.getValues(np.int32)) == [1, 2, 4, 5]
    c = attr(backend, [42], (1, 2, 3), A.SI32, np.int32, splat=True).subview((0, 1, 1), (1, 1, 1)).fold()
    assert c.getValues(np.int32)[0] == 42


# UT:1151-1201 SubViewI1: packed bits, bit k of a byte is element k (LSB first)
def test_subview_i1(backend):
    IC, IH, IW = 1, 7, 5
    bits = np.array([i % 2 for i in range(IC * IH * IW)], dtype=np.uint8)
    packed = np.packbits(bits, bitorder="little")
    a = ContentAttr.get(packed, NDType((IC, IH, IW), A.I1), is_splat=False, backend=backend)
    for off, shp in [((0, 1, 1), (1, 1, 1)), ((0, 2, 1), (1, 3, 4))]:
        c = a.subview(off, shp).fold()
        raw = c.copyTo()
        ref = bits.reshape(IC, IH, IW)[off[0]:off[0] + shp[0], off[1]:off[1] + shp[1], off[2]:off[2] + shp[2]]
        got = np.unpackbits(raw, bitorder="little")[:ref.size]
        assert np.array_equal(got, ref.reshape(-1))


# UT:1233-1262 BitPack: low nibble first
def test_bit_pack(backend):
    a = attr(backend, [1, 2, 3, 4, 5, 6], (1, 2, 3), A.SI8, np.int8).bitPack(4)
    assert a.getType() == NDType((1, 2, 3), A.SI4)
    assert list(a.fold().copyTo()) == [0x21, 0x43, 0x65]


# UT:1264-1306 BitPackQuant
def test_bit_pack_quant(backend):
    q = UniformQuantizedType(A.SI8, A.F32, 1.0, 0, -4, 3)
    a = attr(backend, [1, 2, 3, 1, 2, 3], (1, 2, 3), A.SI8, np.int8).quantCast(q).bitPack(4)
    assert a.getType().quant == UniformQuantizedType(A.SI4, A.F32, 1.0, 0, -4, 3)
    assert list(a.fold().copyTo()) == [0x21, 0x13, 0x32]


# UT:1308-1340 Transpose 512x40
def test_transpose(backend):
    N, Cc = 512, 40
    vals = iota(N * Cc, np.float32)
    c = attr(backend, vals, (N, Cc), A.F32).transpose((1, 0)).fold()
    assert c.getType().shape == (Cc, N)
    assert np.array_equal(c.getValues().reshape(Cc, N), vals.reshape(N, Cc).T)


# UT:1342-1393 BitPackIsLast: ordering and the errors of late insertions
def test_bit_pack_is_last(backend):
    a = attr(backend, [1, 2, 3, 4, 5, 6], (1, 1, 2, 3), A.SI8, np.int8).bitPack(4)
    names = [t.getTransformationName() for t in a.add(17.0).getTransformations()]
    assert names == ["Add", "BitPack"]
    names = [t.getTransformationName() for t in a.add(17.0).broadcast(1, 42).getTransformations()]
    assert names == ["Add", "Broadcast", "BitPack"]
    with pytest.raises(ConstError):
        a.dequantize()
    a.convertElemType(A.SI32)
    a.padWithZero((0, 1, 2, 3), (0, 3, 2, 1))
    a.reorder(DimsOrder.NHWC)
    a.rescale(19.0)
    a.reshape((1, 2, 3))
    a.subview((0, 0, 0, 0), (1, 1, 2, 3))
    a.transpose(DimsOrder.NHWC)
    with pytest.raises(ConstError):
        a.swizzleConstant(5, 3)
    assert a.quantCast(UniformQuantizedType(A.SI8, A.F32, 0.078431372549019607, 0, -4, 3)) is not None


# UT:1446-1481 GetSparsityMap, :1483-1527 quantised (zero point 7)
def test_get_sparsity_map(backend):
    vals = [0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 0, 11, 0, 13, 14, 15]
    a = attr(backend, vals, (1, 1, 2, 8), A.UI8, np.uint8).getSparsityMap()
    assert a.getType() == NDType((1, 1, 1, 128), A.I1)
    raw = a.fold().copyTo()
    assert len(raw) == 16 and list(raw[:2]) == [0xFE, 0xEB] and not raw[2:].any()
    vals = [7, 0, 1, 2, 3, 4, 5, 6, 7, 8, 7, 10, 7, 12, 13, 14]
    q = UniformQuantizedType(A.UI8, A.F32, 1.0, 7, 0, 14)
    raw = attr(backend, vals, (1, 1, 2, 8), A.UI8, np.uint8).quantCast(q).getSparsityMap().fold().copyTo()
    assert list(raw[:2]) == [0xFE, 0xEA] and not raw[2:].any()


SPARSE_IN = [0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 0, 11, 0, 13, 14, 15,
             16, 0, 18, 19, 20, 0, 22, 23, 24, 25, 26, 0, 0, 29, 30, 31]
SPARSE_OUT = [1, 2, 3, 4, 5, 6, 7, 8, 9, 11, 13, 14, 15, 0, 0, 0,
              16, 18, 19, 20, 22, 23, 24, 25, 26, 29, 30, 31, 0, 0, 0, 0]


# UT:1529-1553 Sparsify
def test_sparsify(backend):
    a = attr(backend, SPARSE_IN, (2, 1, 2, 8), A.UI8, np.uint8).sparsify(False)
    assert a.getType() == NDType((2, 1, 2, 8), A.UI8)  # attribute type is unchanged for compressOutputType=false
    c = a.fold()
    assert c.getType() == NDType((32, 1, 1, 1), A.UI8)  # the folded content is flat u8
    assert list(c.copyTo()[:32]) == SPARSE_OUT
    b = attr(backend, SPARSE_IN, (2, 1, 2, 8), A.UI8, np.uint8)
    assert b.countNonSparseElementsPerOC() == [13, 12]
    c2 = b.sparsify(True, [13, 12]).fold()
    assert c2.getType() == NDType((32, 1, 1, 1), A.UI8) and list(c2.copyTo()) == SPARSE_OUT


# UT:1555-1603 SparsifyQuantized (zero point 16)
def test_sparsify_quantized(backend):
    vals = [16, 1, 2, 3, 4, 5, 6, 7, 8, 9, 16, 11, 16, 13, 14, 15,
            16, 16, 18, 19, 20, 16, 22, 23, 24, 25, 26, 16, 16, 29, 30, 31]
    exp = [1, 2, 3, 4, 5, 6, 7, 8, 9, 11, 13, 14, 15, 0, 0, 0,
           18, 19, 20, 22, 23, 24, 25, 26, 29, 30, 31, 0, 0, 0, 0, 0]
    q = UniformQuantizedType(A.UI8, A.F32, 1.0, 16, 0, 31)
    c = attr(backend, vals, (2, 1, 2, 8), A.UI8, np.uint8).quantCast(q).sparsify(False).fold()
    assert list(c.copyTo()[:32]) == exp


# UT:1605-1637 PositionRequirement
def test_position_requirement(backend):
    a = attr(backend, iota(9, np.float32), (1, 1, 3, 3), A.F32).rescale(10.0)
    a = a.swizzleConstant(5, 3).sparsify(False).convertElemType(A.F16)
    names = [t.getTransformationName() for t in a.getTransformations()]
    assert names == ["Rescale", "ConvertElemType", "Sparsify", "SwizzleConstant"]


# LIT constant_folding.mlir:212-222 ConstFoldI4: f16 {1,0,1,2} -> si4 -> bytes [16, 18]
def test_lit_const_fold_i4(backend):
    q = UniformQuantizedType(A.SI4, A.F16, 0.0039215686274509803, 0)
    a = attr(backend, [1.0, 0.0, 1.0, 2.0], (1, 4, 1, 1), A.F16, np.float16)
    a = a.convertElemType(A.SI4).quantCast(q).reorder(DimsOrder.YXOI)
    c = a.fold()
    assert c.getType().getTotalAllocSize() == 2
    assert list(c.copyTo()) == [16, 18]


# LIT constant_folding.mlir:12-30 ConstFold chain on a splat: -1.0 -> f16 -> ui8 must fail the range check
# of the lazy conversion only when values are read; with 129 (QuantConstFold, :34-52) it folds.
def test_lit_quant_const_fold(backend):
    q = UniformQuantizedType(A.UI8, A.F16, 0.0039215686274509803, 0)
    a = attr(backend, [129], (16, 3, 1, 1), A.UI8, np.uint8, splat=True).quantCast(q).reorder(DimsOrder.YXOI)
    c = a.fold()
    assert c.getType().order == DimsOrder.YXOI
    assert list(c.copyTo()) == [129] * 48
    d = a.dequantize().fold()  # inserted before nothing LAST: Dequantize goes at the end
    # expressed type is f16: f32 storage (one rounding) then f16 at copy-out (second rounding)
    exp = np.float16(np.float32(np.float64(129) * 0.0039215686274509803))
    assert d.getType().dtype == A.F16
    assert np.array_equal(d.getValues(), np.full(48, exp, np.float16))


# LIT constant_folding_37XX.mlir:13-35: splat-true i1 100x1x1x384 swizzled -> 40960 bits, all 0xFF
def test_lit_swizzle_subbyte_splat(backend):
    a = ContentAttr.get(np.array([1], np.uint8), NDType((100, 1, 1, 384), A.I1), is_splat=True, backend=backend)
    a = a.swizzleConstant(5, 3)
    assert a.getType() == NDType((40960, 1, 1, 1), A.I1)
    raw = a.fold().copyTo()
    assert len(raw) == 5120 and (raw == 0xFF).all()


# LIT constant_folding_37XX.mlir:46-62: long chain then swizzle; first bytes 0x01 00 00 ...
def test_lit_swizzle_after_chain(backend):
    q = UniformQuantizedType(A.UI8, A.F16, 1.0, 0, 0, 254)
    a = attr(backend, [1.0], (32, 1, 1, 1), A.F16, np.float16, splat=True)
    a = a.convertElemType(A.UI8).quantCast(q).reorder(DimsOrder.NHWC).reorder(DimsOrder.NCHW)
    a = a.reshape((32, 1, 1, 1)).padWithZero((0, 0, 0, 0), (0, 15, 0, 0)).reorder(DimsOrder.NHWC)
    a = a.subview((0, 0, 0, 0), (16, 16, 1, 1)).swizzleConstant(5, 3)
    assert a.getType().shape == (512, 1, 1, 1) and a.getType().dtype == A.UI8
    raw = a.fold().copyTo()
    # before swizzling: 16 rows of [1, 0 x15]; 256 bytes -> padded to 512; block 0 has stagger 0
    exp = np.zeros(512, np.uint8)
    exp[0:256:16] = 1
    assert np.array_equal(raw, exp)


# LIT constant_folding_37XX.mlir:66-75: 3 bytes -> reshape/broadcast -> 768 bytes after swizzle alignment
def test_lit_swizzle_shape_mismatch(backend):
    a = attr(backend, [1, 2, 3], (1, 1, 3, 1), A.UI8, np.uint8).swizzleConstant(5, 3)
    assert a.getType() == NDType((512, 1, 1, 1), A.UI8)
    raw = a.fold().copyTo()
    assert list(raw[:3]) == [1, 2, 3] and not raw[3:].any()


# tests/unit/vpux_compiler/utils/swizzling_test.cpp:35-100: deswizzle(swizzle(x)) == x for keys 0..5,
# aligned and unaligned sizes; swizzled != x once the buffer exceeds the pattern stride (512 B) and key > 0.
@pytest.mark.parametrize("key", [0, 1, 2, 3, 4, 5])
@pytest.mark.parametrize("size", [512, 1024, 4096, 16384, 50176, 1000, 5000])
def test_swizzle_roundtrip(backend, oracle, key, size):
    rng = np.random.default_rng(key * 100 + size)
    x = rng.integers(0, 256, size, dtype=np.uint8)
    a = ContentAttr.get(x, NDType((size, 1, 1, 1), A.UI8), backend=backend).swizzleConstant(key, 3)
    raw = a.fold().copyTo()
    padded = np.zeros((size + 511) // 512 * 512, np.uint8)
    padded[:size] = x
    assert len(raw) == len(padded)
    assert np.array_equal(oracle.deswizzle(raw, key), padded)
    if key > 0 and len(padded) > 512:
        assert not np.array_equal(raw, padded)
    if key == 0:
        assert np.array_equal(raw, padded)


# The swizzle address rule itself, independent of both implementations
# (swizzle_transform.hpp:58-80 + CA/swizzle_transform.cpp:41-79): chunk at address a moves to
# (a & ~511) + ((a + ((a>>9 & mask) << (9-key))) & 511).
@pytest.mark.parametrize("key", [1, 3, 5])
def test_swizzle_address_rule(backend, key):
    size = 8192
    x = np.arange(size, dtype=np.uint32).astype(np.uint8) ^ (np.arange(size) >> 8).astype(np.uint8)
    raw = ContentAttr.get(x, NDType((size, 1, 1, 1), A.UI8), backend=backend).swizzleConstant(key, 3).fold().copyTo()
    exp = np.zeros(size, np.uint8)
    for a in range(0, size, 16):
        stagger = ((a >> 9) & 63 & ((1 << key) - 1)) << (9 - key)
        dst = (a & ~511) + ((a + stagger) & 511)
        exp[dst:dst + 16] = x[a:a + 16]
    assert np.array_equal(raw, exp)


# ---- the remaining transformations: Broadcast, Reverse, ExpandDilated --------------------------------
# LIT constant_folding.mlir:108-205 broadcastNonSplat*: the broadcast axis is tiled, whatever lies inside it repeats
@pytest.mark.parametrize("vals,shape,steps,final,want", [
    ([1, 2, 3], (1, 3, 1, 1), [(0, 3)], (1, 9, 1, 1), [1, 2, 3, 1, 2, 3, 1, 2, 3]),          # PreChannel :110-119
    ([1, 2, 3], (1, 3, 1, 1), [(2, 3)], (1, 9, 1, 1), [1, 1, 1, 2, 2, 2, 3, 3, 3]),          # PostChannel :124-133
    ([1, 2, 3, 4, 5, 6], (1, 3, 1, 2), [(2, 2)], None, [1, 2, 1, 2, 3, 4, 3, 4, 5, 6, 5, 6]),  # MiddleChannel :138-149
    (list(range(1, 13)), (1, 3, 2, 2), [(2, 4)], None,
     [1, 2, 3, 4, 1, 2, 3, 4, 5, 6, 7, 8, 5, 6, 7, 8, 9, 10, 11, 12, 9, 10, 11, 12]),       # MiddleChannelNone1 :154-164
])
def test_lit_broadcast_non_splat(backend, vals, shape, steps, final, want):
    a = attr(backend, vals, (len(vals),), A.I8, np.uint8).reshape(shape)
    for axis, value in steps:
        a = a.broadcast(axis, value)
    if final is not None:
        a = a.reshape(final)
    assert list(a.fold().copyTo()) == want


# LIT constant_folding.mlir:168-205 broadcastNonSplatTwoDims / MultiDims (f32 -> f16, two broadcasts)
@pytest.mark.parametrize("shape,steps", [((1, 1, 1, 4), [(1, 4), (2, 4)]), ((1, 1, 4, 1), [(1, 4), (3, 4)])])
def test_lit_broadcast_two_dims(backend, shape, steps):
    base = np.array([1, 2, 3, 4], np.float32).reshape(shape)
    a = attr(backend, base, shape, A.F32).convertElemType(A.F16).reshape(shape)
    for axis, value in steps:
        a = a.broadcast(axis, value)
    c = a.fold()
    assert c.getType().shape == (1, 4, 4, 4)
    assert np.array_equal(c.getValues().reshape(1, 4, 4, 4), np.broadcast_to(base, (1, 4, 4, 4)).astype(np.float16))


# UT:792-868 ReverseCWise / ReverseNWise: everything behind the axis is reversed as one run
@pytest.mark.parametrize("axis", [0, 1])
def test_reverse(backend, axis):
    N, Cc, H, W = 2, 3, 4, 5
    vals = iota(N * Cc * H * W, np.float32)
    c = attr(backend, vals, (N, Cc, H, W), A.F32).reverse(axis).fold()
    assert c.getType() == NDType((N, Cc, H, W), A.F32)
    run = {0: Cc * H * W, 1: H * W}[axis]
    assert np.array_equal(c.getValues().reshape(-1, run), vals.reshape(-1, run)[:, ::-1])


def test_reverse_errors(backend):
    with pytest.raises(ConstError):  # the last dim cannot be the axis (reverse.cpp:64-65)
        attr(backend, iota(6, np.float32), (2, 3), A.F32).reverse(1).fold()
    with pytest.raises(ConstError):  # si32 is not among the handled element types (reverse.cpp:103-116)
        attr(backend, iota(6, np.int32), (2, 3), A.SI32).reverse(0).fold()


# UT:1395-1442 ExpandDilated: 5x5 kernels, dilation 3 -> 13x13 with zeros between the taps
def test_expand_dilated(backend):
    OC, IC, KY, KX, d = 2, 2, 5, 5, 3
    vals = iota(OC * IC * KY * KX, np.int32)
    c = attr(backend, vals, (OC, IC, KY, KX), A.SI32).expandDilated((d, d)).fold()
    dK = KY + (KY - 1) * (d - 1)
    assert c.getType() == NDType((OC, IC, dK, dK), A.SI32)
    want = np.zeros((OC, IC, dK, dK), np.int32)
    want[:, :, ::d, ::d] = vals.reshape(OC, IC, KY, KX)
    assert np.array_equal(c.getValues().reshape(want.shape), want)


# UT:119-134 FromEmptyDenseElementsAttr: a tensor with no elements folds to a content with no values
def test_from_empty_dense(backend):
    c = attr(backend, [], (0,), A.F32, np.float32).fold()
    assert c.getType() == NDType((0,), A.F32)
    assert c.getValues().size == 0 and c.copyTo().size == 0


# UT:348-370 ConvertStorageElemType: getValues<int32_t>() of f32 storage converts element by element
def test_convert_storage_elem_type(backend):
    vals = iota(24, np.float32)
    c = attr(backend, vals, (1, 2, 3, 4), A.F32).fold()
    assert c.getType() == NDType((1, 2, 3, 4), A.F32)
    assert list(c.getValues(np.int32)) == list(range(24))


# UT:608-634 ConvertElemTypeSplat: the single stored element is converted, the content stays a splat of 24 elements
def test_convert_elem_type_splat(backend):
    c = attr(backend, [4.0], (1, 2, 3, 4), A.F32, np.float32, splat=True).convertElemType(A.SI32).fold()
    assert c.getType() == NDType((1, 2, 3, 4), A.SI32)
    assert list(c.getValues(np.int32)) == [4] * 24
    assert c.copyTo().view(np.int32).tolist() == [4] * 24


# UT:636-662 ConvertElemTypeSubByte: u8 {0,1,2} read as i1 gives {false,true,true}; three 1-bit elements do not fill
# a byte, so copying them out is refused (Content::copySubByteContent: elements per byte must be a power of two)
def test_convert_elem_type_sub_byte(backend):
    a = attr(backend, [0, 1, 2], (3,), A.UI8, np.uint8).convertElemType(A.I1)
    assert a.getType() == NDType((3,), A.I1)
    with pytest.raises(ConstError, match="Invalid number of elements per byte"):
        a.fold().copyTo()
    # the same conversion on eight elements packs the low bit of each (getValues<int8_t>() & 1), first element in
    # the most significant bit: 2 contributes 0, 7 contributes 1
    c = attr(backend, [0, 1, 2, 0, 0, 7, 0, 1], (8,), A.UI8, np.uint8).convertElemType(A.I1).fold()
    assert list(c.copyTo()) == [0b01000101]


# UT:1482-1530 GetSparsityMapQuantized: the zero point (7) is the sparse value
def test_get_sparsity_map_quantized(backend):
    vals = [7, 0, 1, 2, 3, 4, 5, 6, 7, 8, 7, 10, 7, 12, 13, 14]
    q = UniformQuantizedType(A.UI8, A.F32, 1.0, 7, 0, 14)
    c = attr(backend, vals, (1, 1, 2, 8), A.UI8, np.uint8).quantCast(q).getSparsityMap().fold()
    assert c.getType() == NDType((1, 1, 1, 128), A.I1)
    out = c.copyTo()
    assert out.size == 16 and list(out[:2]) == [0xFE, 0xEA] and not out[2:].any()


# UT:1639-1667 ChangeShapeAndElemType: shape and (quantised) element type change, the values stay
def test_change_shape_and_elem_type(backend):
    vals = iota(16, np.uint8)
    q = UniformQuantizedType(A.UI8, A.F32, 0.078431372549019607, 128, 0, 255)
    a = attr(backend, vals, (2, 1, 1, 8), A.UI8).changeShapeAndElemType((1, 2, 1, 8), q)
    assert a.getType() == NDType((1, 2, 1, 8), q)
    c = a.fold()
    assert c.getType() != NDType((2, 1, 1, 8), A.UI8)
    assert list(c.getValues(np.uint8)) == list(range(16))


# UT:1669-1711 ChangeShapeAndElemTypePerAxisQuant: the quantised axis moves with the reshape
def test_change_shape_and_elem_type_per_axis(backend):
    vals = iota(16, np.uint8)
    q1 = UniformQuantizedPerAxisType(A.UI8, A.F16, [0.5, 0.5], [127, 127], 0, 0, 255)
    q2 = UniformQuantizedPerAxisType(A.UI8, A.F16, [0.5, 0.5], [127, 127], 1, 0, 255)
    a1 = attr(backend, vals, (2, 1, 1, 8), A.UI8).quantCast(q1)
    a2 = a1.changeShapeAndElemType((1, 2, 1, 8), q2)
    assert a1.getType() != a2.getType()
    c1, c2 = a1.fold(), a2.fold()
    assert c1.getType() == NDType((2, 1, 1, 8), q1) and c2.getType() == NDType((1, 2, 1, 8), q2)
    assert list(c1.getValues(np.uint8)) == list(range(16)) and list(c2.getValues(np.uint8)) == list(range(16))


# UT:1713-1737 ChangeShapeAndElemTypeFloat: f32 storage under an si32 type is converted when the values are read
def test_change_shape_and_elem_type_float(backend):
    vals = iota(16, np.float32)
    a = attr(backend, vals, (2, 1, 1, 8), A.F32).changeShapeAndElemType((1, 2, 1, 8), A.SI32)
    assert a.getType() == NDType((1, 2, 1, 8), A.SI32)
    c = a.fold()
    assert list(c.getValues(np.int32)) == list(range(16))
    assert c.copyTo().view(np.int32).tolist() == list(range(16))


# UT:1739-1765 GetTransformationsRange and :1767-1796 ...DuplicatedTransformations: the list is cut at the last
# occurrence of a transformation (equal transformations are one uniqued object in the reference)
def test_get_transformations_range(backend):
    a = attr(backend, iota(10, np.float32), (10,), A.F32).add(1.0).reshape((2, 5)).subview((0, 0), (1, 5))
    ts = a.getTransformations()
    assert [t.getTransformationName() for t in ts] == ["Add", "Reshape", "SubView"]
    head = a.stripTransformationsFrom(ts[1])
    assert [t.getTransformationName() for t in head.getTransformations()] == ["Add"]
    assert [t.getTransformationName() for t in a.getLastTransformationsFrom(ts[1])] == ["Reshape", "SubView"]
    # the stripped attribute folds to the head's result, the full one to the first row of it
    assert np.array_equal(head.fold().getValues(), iota(10, np.float32) + 1)
    assert np.array_equal(a.fold().getValues(), (iota(10, np.float32) + 1)[:5])
    d = attr(backend, iota(10, np.float32), (10,), A.F32).add(1.0).reshape((2, 5)).reshape((2, 5)).subview((0, 0), (1, 5))
    ts = d.getTransformations()
    assert len(ts) == 4 and ts[1] == ts[2]
    for which in (ts[1], ts[2]):  # either Reshape reaches the same result
        assert [t.getTransformationName() for t in d.stripTransformationsFrom(which).getTransformations()] == ["Add", "Reshape"]
        assert [t.getTransformationName() for t in d.getLastTransformationsFrom(which)] == ["Reshape", "SubView"]


# LIT constant_folding.mlir:56-107 I1SubviewConstFold{Splat,NotSplat,NonSplat}: SubView on 1-bit content (bit k of a
# byte is element k) -- a splat stays a splat, a dense one is cut bit by bit
def test_lit_i1_subview(backend):
    splat = ContentAttr.get(np.array([1], np.uint8), NDType((1, 32, 3, 3), A.I1), is_splat=True, backend=backend)
    c = splat.subview((0, 16, 0, 0), (1, 16, 3, 3)).fold()
    assert c.getType() == NDType((1, 16, 3, 3), A.I1)
    assert list(c.copyTo()) == [0xFF] * 18  # dense<true> : tensor<1x16x3x3xi1>, 144 bits
    row = np.packbits(np.array([1, 0, 1, 0], np.uint8), bitorder="little")
    c = ContentAttr.get(row, NDType((1, 4), A.I1), is_splat=False, backend=backend).subview((0, 2), (1, 2)).fold()
    assert list(np.unpackbits(c.copyTo(), bitorder="little")[:2]) == [1, 0]  # dense<[[true, false]]>
    bits = np.array([0] * 8 + [1] * 8 + [0, 1] * 4 + [1, 0] * 4, np.uint8)
    dense = ContentAttr.get(np.packbits(bits, bitorder="little"), NDType((1, 32, 1, 1), A.I1), is_splat=False, backend=backend)
    c = dense.subview((0, 16, 0, 0), (1, 16, 1, 1)).fold()
    assert c.getType() == NDType((1, 16, 1, 1), A.I1)
    assert list(np.unpackbits(c.copyTo(), bitorder="little")) == [0, 1] * 4 + [1, 0] * 4
