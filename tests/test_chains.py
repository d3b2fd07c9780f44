"""The chain builders (npu_plugin_b200.chains) against hand-computed results, on the CPU oracle and on the GPU."""
import numpy as np
import pytest

from npu_plugin_b200 import _cabi as A
from npu_plugin_b200 import chains
from npu_plugin_b200.const import ContentAttr, DimsOrder, NDType, UniformQuantizedPerAxisType, UniformQuantizedType


def kinds(attr):
    return [t.kind for t in attr.getTransformations()]


def test_align_convolution_weights(backend):
    rng = np.random.default_rng(1)
    w = rng.integers(-100, 100, (8, 3, 3, 3)).astype(np.int8)
    a = chains.align_convolution_weights(ContentAttr.get(w, backend=backend), alignment=16)
    assert kinds(a) == [A.X_RESHAPE, A.X_PAD_WITH_ZERO]
    assert a.getType().shape == (8, 1, 1, 32)
    want = np.zeros((8, 32), np.int8)
    want[:, :27] = w.reshape(8, 27)
    assert np.array_equal(a.fold().copyTo().view(np.int8).reshape(8, 32), want)
    # C-major convolution: flattened in NCHW order, result laid out NHWC
    c = chains.align_convolution_weights(ContentAttr.get(w, backend=backend), alignment=16, is_cmajor_conv=True)
    assert kinds(c) == [A.X_REORDER, A.X_RESHAPE, A.X_PAD_WITH_ZERO, A.X_REORDER]
    assert np.array_equal(c.fold().copyTo().view(np.int8).reshape(8, 32), want)  # [O,1,1,I] NHWC has the same memory order
    # already aligned: untouched
    w16 = rng.integers(-100, 100, (4, 16, 1, 1)).astype(np.int8)
    same = ContentAttr.get(w16, backend=backend)
    assert chains.align_convolution_weights(same) is same


def test_align_depthwise_weights(backend):
    rng = np.random.default_rng(2)
    w = rng.normal(0, 1, (6, 1, 3, 3)).astype(np.float16)
    a = chains.align_depthwise_weights(ContentAttr.get(w, backend=backend), (6, 9, 1, 1), 7)
    assert a.getType().shape == (6, 16, 1, 1) and tuple(a.getType().order) == tuple(DimsOrder.NHWC)
    want = np.zeros((6, 16), np.float16)
    want[:, :9] = w.reshape(6, 9)
    assert np.array_equal(a.fold().copyTo().view(np.float16).reshape(6, 16), want)


def test_weights_to_u8(backend):
    rng = np.random.default_rng(3)
    w = rng.integers(-128, 128, (4, 8, 1, 1)).astype(np.int8)
    q = UniformQuantizedType(A.SI8, A.F16, 0.02, -3)
    qu = UniformQuantizedType(A.UI8, A.F16, 0.02, 125)
    a = chains.weights_to_u8(ContentAttr.get(w, backend=backend).quantCast(q), qu)
    assert kinds(a)[-5:] == [A.X_QUANT_CAST, A.X_CONVERT_ELEM_TYPE, A.X_ADD, A.X_CONVERT_ELEM_TYPE, A.X_QUANT_CAST]
    assert a.getType().quant == qu
    assert np.array_equal(a.fold().copyTo().reshape(w.shape), (w.astype(np.int16) + 128).astype(np.uint8))


def test_sparsify_weights_and_flatten(backend):
    rng = np.random.default_rng(4)
    w = rng.integers(-127, 128, (16, 32, 1, 1)).astype(np.int8)
    w[rng.random(w.shape) < 0.6] = 0
    q = UniformQuantizedPerAxisType(A.SI8, A.F16, [0.1] * 16, [0] * 16, 0)
    base = ContentAttr.get(w, backend=backend).quantCast(q).reorder(DimsOrder.OYXI)
    vals, smap, counts = chains.sparsify_weights(base)
    assert counts == [int(np.count_nonzero(w[o])) for o in range(16)]
    assert kinds(vals) == [A.X_QUANT_CAST, A.X_SPARSIFY] and kinds(smap) == [A.X_QUANT_CAST, A.X_GET_SPARSITY_MAP]
    bits = np.unpackbits(smap.fold().copyTo().reshape(16, -1), axis=1, bitorder="little")[:, :32]
    assert np.array_equal(bits.astype(bool), w.reshape(16, 32) != 0)
    folded = vals.fold()
    raw, at = folded.copyTo(), 0
    for o in range(16):
        nz = w[o].reshape(-1)[w[o].reshape(-1) != 0]
        assert np.array_equal(raw[at:at + nz.size].view(np.int8), nz)
        at += (nz.size + 15) // 16 * 16
    flat = chains.flatten_sparse_weights(vals, counts)
    assert flat.getType().shape == (at, 1, 1, 1)
    assert np.array_equal(flat.fold().copyTo()[:at], raw[:at])
    assert chains.flatten_sparse_weights(base, counts) is base


def test_sparse_identity_filter(backend):
    vals, smap, counts = chains.sparse_identity_filter(16, 16, A.F16, backend=backend)
    assert counts == [1] * 16
    raw = vals.fold().copyTo().view(np.float16)
    assert np.array_equal(raw[::8][:16], np.ones(16, np.float16))  # one element per channel, 16-byte aligned runs
    bits = np.unpackbits(smap.fold().copyTo().reshape(16, -1), axis=1, bitorder="little")[:, :16]
    assert np.array_equal(bits, np.eye(16, dtype=np.uint8))
    qv, _, qc = chains.sparse_identity_filter(16, 16, UniformQuantizedType(A.UI8, A.F16, 1.0, 0), backend=backend)
    assert qc == [1] * 16 and np.array_equal(qv.fold().copyTo()[::16][:16], np.ones(16, np.uint8))


def test_hwtest_default_weights(backend):
    w = (np.arange(2 * 4 * 1 * 2).reshape(2, 4, 1, 2) % 16).astype(np.uint8)
    q4 = UniformQuantizedType(A.UI4, A.F16, 0.5, 0, 0, 15)
    a = chains.hwtest_default_weights(ContentAttr.get(w, backend=backend), q4)
    assert kinds(a) == [A.X_REORDER, A.X_QUANT_CAST, A.X_BIT_PACK]
    oyxi = np.transpose(w, (0, 2, 3, 1)).reshape(-1)
    want = (oyxi[0::2] & 0xF) | ((oyxi[1::2] & 0xF) << 4)
    assert np.array_equal(a.fold().copyTo(), want.astype(np.uint8))
    plain = chains.hwtest_default_weights(ContentAttr.get(w, backend=backend))
    assert kinds(plain) == [A.X_REORDER]


def test_attach_swizzle_once(backend):
    w = np.arange(1024, dtype=np.uint8).reshape(4, 256, 1, 1)
    a = chains.attach_swizzle(ContentAttr.get(w, backend=backend))
    assert kinds(a) == [A.X_SWIZZLE_CONSTANT]
    assert chains.attach_swizzle(a) is a
    assert a.fold().copyTo().size == 1024


# tests/lit/NPU/dialect/IE/passes/convert_weights_to_u8.mlir:9-32 (@Conv): dense<-1.0> 3x3x3x3 f16 with
# [ConvertElemType<si8>, QuantCast<i8<-127:127> per axis 0>] becomes u8<0:254> with zero points 127 through
# [..., QuantCast<>, ConvertElemType<i32>, Add<127.0>, ConvertElemType<ui8>, QuantCast<new type>]
def test_weights_to_u8_on_the_lit_case(oracle):
    scales = [0.010680671751968504, 0.0081200787401574797, 0.010596087598425197]
    q_old = UniformQuantizedPerAxisType(A.SI8, A.F16, scales, [0, 0, 0], 0, -127, 127)
    q_new = UniformQuantizedPerAxisType(A.UI8, A.F16, scales, [127, 127, 127], 0, 0, 254)
    base = ContentAttr.get(np.array([-1.0], np.float16), NDType((3, 3, 3, 3), A.F16), backend=oracle)
    assert base._isSplat
    a = chains.weights_to_u8(base.convertElemType(A.SI8).quantCast(q_old), q_new)
    ts = a.getTransformations()
    assert [t.getTransformationName() for t in ts] == ["ConvertElemType", "QuantCast", "QuantCast", "ConvertElemType", "Add",
                                                        "ConvertElemType", "QuantCast"]
    assert ts[0].elem == A.SI8 and ts[2].elem is None and ts[3].elem == A.I32 and ts[4].f == 127.0 and ts[5].elem == A.UI8
    assert a.getType() == NDType((3, 3, 3, 3), q_new)
    raw = a.fold().copyTo()
    assert raw.size == 81 and (raw == 126).all()  # -1 - (-127)
    # the library's own type inference (host code) accepts the same list
    from test_abi_and_host import HostOnly
    assert HostOnly().infer_type(base._baseType, ts) == a.getType()


# tests/lit/NPU/conversion/passes/IE2VPU/convert_IE_to_VPU_NCE_37XX.mlir:210-229 (@ConvToNCE4channels): weights
# 16x4x1x1 f16 NHWC become 16x1x1x16 through [Reorder<NHWC>, Reshape<[16,1,1,4]>, PadWithZero<[0,0,0,0],[0,0,0,12]>]
def test_align_convolution_weights_on_the_lit_case(oracle):
    base = ContentAttr.get(np.array([1.0], np.float16), NDType((16, 4, 1, 1), A.F16), backend=oracle).reorder(DimsOrder.NHWC)
    a = chains.align_convolution_weights(base, alignment=chains.VPU_WEIGHT_SET_BYTE_ALIGNMENT)
    ts = a.getTransformations()
    assert [t.getTransformationName() for t in ts] == ["Reorder", "Reshape", "PadWithZero"]
    assert ts[1].b == (16, 1, 1, 4) and ts[2].a == (0, 0, 0, 0) and ts[2].b == (0, 0, 0, 12)
    assert a.getType() == NDType((16, 1, 1, 16), A.F16, DimsOrder.NHWC)
    got = a.fold().copyTo().view(np.float16).reshape(16, 16)
    assert (got[:, :4] == 1.0).all() and (got[:, 4:] == 0.0).all()


# tests/lit/NPU/dialect/VPU/passes/sparsify_weights_30XX.mlir:30-51 (@SparsifyPaddedConv): 16x15x1x1 f16 ones padded
# to 16x32x1x1 NHWC -> folded base + [Sparsify<false>], a 16x1x1x128 i1 map from [GetSparsityMap], numElems = 15
def test_sparsify_weights_on_the_lit_case(oracle):
    base = (ContentAttr.get(np.array([1.0], np.float16), NDType((16, 15, 1, 1), A.F16), backend=oracle)
            .reorder(DimsOrder.NHWC).padWithZero((0, 0, 0, 0), (0, 17, 0, 0)))
    vals, smap, counts = chains.sparsify_weights(base)
    assert counts == [15] * 16
    assert [t.getTransformationName() for t in vals.getTransformations()] == ["Sparsify"]
    assert [t.getTransformationName() for t in smap.getTransformations()] == ["GetSparsityMap"]
    assert vals._baseType == NDType((16, 32, 1, 1), A.F16, DimsOrder.NHWC) and not vals._isSplat
    assert vals.getType() == NDType((16, 32, 1, 1), A.F16, DimsOrder.NHWC)
    assert smap.getType() == NDType((16, 1, 1, 128), A.I1)
    bits = np.unpackbits(smap.fold().copyTo().reshape(16, 16), axis=1, bitorder="little")
    assert (bits[:, :15] == 1).all() and (bits[:, 15:] == 0).all()
    raw = vals.fold().copyTo().view(np.float16)
    assert raw.size >= 16 * 16 and (raw[:16 * 16].reshape(16, 16)[:, :15] == 1.0).all() and (raw[:16 * 16].reshape(16, 16)[:, 15] == 0.0).all()
    # late in the pipeline the type becomes the flat compressed one: 16 runs of 15 f16 = 30 bytes, each padded to 32
    flat = chains.flatten_sparse_weights(vals, counts)
    assert flat.getType().shape == (16 * 32, 1, 1, 1) and flat.getType().dtype == A.UI8


# tests/lit/NPU/dialect/VPU/passes/lower_unaligned_sparsity_ops_37XX.mlir:28-33,74-79: the identity filter of a lowered
# sparsity op is an f32 16x16x1x1 constant with [ConvertElemType<ui8>, QuantCast<q>, Reorder<NHWC>, Sparsify<false>]
# (or [ConvertElemType<f16>, Reorder<NHWC>, Sparsify<false>]), its map 16x1x1x128 i1, numElems = 1 per channel
def test_sparse_identity_filter_on_the_lit_cases(oracle):
    names = lambda a: [t.getTransformationName() for t in a.getTransformations()]
    q = UniformQuantizedType(A.UI8, A.F16, 1.0, 0)
    vals, smap, counts = chains.sparse_identity_filter(16, 16, q, order=DimsOrder.NHWC, backend=oracle)
    assert names(vals) == ["ConvertElemType", "QuantCast", "Reorder", "Sparsify"]
    assert names(smap) == ["ConvertElemType", "QuantCast", "Reorder", "GetSparsityMap"]
    assert vals._baseType == NDType((16, 16, 1, 1), A.F32) and counts == [1] * 16
    assert vals.getType() == NDType((16, 16, 1, 1), q, DimsOrder.NHWC) and smap.getType() == NDType((16, 1, 1, 128), A.I1)
    vals, smap, counts = chains.sparse_identity_filter(16, 16, A.F16, order=DimsOrder.NHWC, backend=oracle)
    assert names(vals) == ["ConvertElemType", "Reorder", "Sparsify"] and names(smap) == ["ConvertElemType", "Reorder", "GetSparsityMap"]
    assert vals.getType() == NDType((16, 16, 1, 1), A.F16, DimsOrder.NHWC) and smap.getType() == NDType((16, 1, 1, 128), A.I1)
    assert counts == [1] * 16
