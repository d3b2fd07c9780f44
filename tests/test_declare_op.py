"""Const::DeclareOp and the constant-folding pass on the host mirror: the verifier's rules
(src/vpux_compiler/src/dialect/const/ops.cpp:164-193), getContent / serialize / getBinarySize, and the pass's
re-typing of folded constants including the sub-byte case the reference pins in
tests/lit/NPU/dialect/const/passes/constant_folding.mlir:212-222 (bytes [16, 18] typed 1x1x1x2xui8)."""
import numpy as np
import pytest

from npu_plugin_b200 import _cabi as A
from npu_plugin_b200.const import (ConstError, ContentAttr, DeclareOp, DimsOrder, NDType, UniformQuantizedType,
                                   constant_folding_pass)


def test_constant_folding_of_a_4bit_constant(backend):
    # ConstFoldI4: f16 {1,0,1,2} -> ConvertElemType<si4> -> QuantCast<i4:f16> -> Reorder<YXOI>
    w = np.array([1.0, 0.0, 1.0, 2.0], np.float16).reshape(1, 4, 1, 1)
    q = UniformQuantizedType(A.SI4, A.F16, 0.0039215686274509803, 0)
    attr = ContentAttr.get(w, backend=backend).convertElemType(A.SI4).quantCast(q).reorder(DimsOrder.YXOI)
    op = DeclareOp(NDType((1, 4, 1, 1), q, DimsOrder.YXOI), attr)
    (folded,) = constant_folding_pass([op])
    new_attr = folded.getContentAttr()
    # the TYPE of the stored dense attribute: 1x1x1x2xui8 in YXOI order, holding the two packed bytes
    assert new_attr._baseType.shape == (1, 1, 1, 2) and new_attr._baseType.dtype == A.UI8
    assert tuple(new_attr._baseType.order) == tuple(DimsOrder.YXOI)
    assert new_attr.getBaseContent().tolist() == [16, 18]
    assert [t.kind for t in new_attr.getTransformations()] == [A.X_CHANGE_SHAPE_AND_ELEM_TYPE]
    # the op keeps its result type, and the attribute infers back to it
    assert folded.getType() == op.getType()
    assert new_attr.getType().shape == (1, 4, 1, 1) and new_attr.getType().quant == q
    assert folded.getContent().copyTo().tolist() == [16, 18]


def test_constant_folding_of_plain_and_quantised_constants(backend):
    # ConstFold: dense<-1.0> f32 splat -> f16 -> ui8?? would throw on -1; use the quantised u8 chain on 3.0 instead
    q = UniformQuantizedType(A.UI8, A.F16, 0.5, 0)
    a = (ContentAttr.get(np.array([3.0], np.float32), NDType((16, 3, 1, 1), A.F32), is_splat=True, backend=backend)
         .convertElemType(A.F16).convertElemType(A.UI8).quantCast(q).dequantize().reorder(DimsOrder.YXOI))
    op = DeclareOp(NDType((16, 3, 1, 1), A.F16, DimsOrder.YXOI), a)
    (f,) = constant_folding_pass([op])
    assert not f.getContentAttr().getTransformations()
    assert f.getContentAttr()._baseType == NDType((16, 3, 1, 1), A.F16, DimsOrder.YXOI)
    assert np.array_equal(f.getContent().copyTo().view(np.float16), np.full(48, 1.5, np.float16))
    # a quantised result is stored under its storage integer type; the op keeps the quantised type
    w = np.arange(24, dtype=np.uint8).reshape(2, 3, 2, 2)
    aq = ContentAttr.get(w, backend=backend).quantCast(q).reorder(DimsOrder.NHWC)
    (fq,) = constant_folding_pass([DeclareOp(NDType((2, 3, 2, 2), q, DimsOrder.NHWC), aq)])
    assert fq.getContentAttr()._baseType == NDType((2, 3, 2, 2), A.UI8, DimsOrder.NHWC)
    assert fq.getType().quant == q
    assert np.array_equal(fq.getContent().copyTo().reshape(2, 2, 2, 3), np.transpose(w, (0, 2, 3, 1)))


def test_declare_op_verifier_and_serialize(backend):
    w = np.arange(12, dtype=np.float32).reshape(3, 4)
    a = ContentAttr.get(w, backend=backend)
    with pytest.raises(ConstError, match="mismatch in value shape"):
        DeclareOp(NDType((4, 3), A.F32), a)
    with pytest.raises(ConstError, match="mismatch in value element type"):
        DeclareOp(NDType((3, 4), A.F16), a)
    with pytest.raises(ConstError, match="mismatch in value DimsOrder"):
        DeclareOp(NDType((3, 4), A.F32, (1, 0)), a)
    # an integer attribute under a quantised result type is accepted; so is a shape mismatch of a swizzled constant
    q = UniformQuantizedType(A.UI8, A.F16, 1.0, 0)
    DeclareOp(NDType((3, 4), q), ContentAttr.get(w.astype(np.uint8), backend=backend))
    sw = ContentAttr.get(np.arange(100, dtype=np.uint8).reshape(1, 100, 1, 1), backend=backend).swizzleConstant(5, 3)
    with pytest.raises(ConstError):
        DeclareOp(NDType((1, 100, 1, 1), A.UI8), sw)
    op = DeclareOp(NDType((1, 100, 1, 1), A.UI8), sw, swizzled=True)
    assert op.getBinarySize() == 512
    section = bytearray(b"xyz")
    assert op.serialize(section) == 512 and len(section) == 515
    assert section[3:3 + 16] == bytes(range(16))
    assert op.fold() is sw and op.getContentAttr() is sw


# ContentAttr::verify (content.cpp:61-99) on the cases of tests/lit/NPU/dialect/const/passes/content.mlir:70-136: a dense
# resource is accepted when it holds every element or exactly one (a splat), refused with the reference's text otherwise
def test_content_attr_verifies_its_base_buffer(oracle):
    from npu_plugin_b200.const import ConstError, UniformQuantizedType
    t = NDType((1, 3, 1, 1), A.F32)
    ok = ContentAttr.get(np.array([1, 2, 3], np.uint32).view(np.float32), t, backend=oracle)   # ParsePrintDenseResource
    assert ok.getType() == t and not ok._isSplat
    with pytest.raises(ConstError, match="Size of dense resource buffer '8' in 'baseContent' doesn't match its type"):
        ContentAttr.get(np.array([2, 3], np.uint32), t, backend=oracle)                            # ...NoAlignment
    with pytest.raises(ConstError, match="Size of dense resource buffer '16' in 'baseContent' doesn't match its type"):
        ContentAttr.get(np.array([1, 2, 3, 4], np.uint32), t, backend=oracle)                      # ...WrongDataSize
    splat = ContentAttr.get(np.array([1], np.uint32).view(np.float32), NDType((2, 3, 1, 1), A.F32), backend=oracle)
    assert splat._isSplat                                                                          # ...Splat
    raw = splat.fold().copyTo()
    assert np.array_equal(raw.view(np.uint32), np.full(6, 1, np.uint32))
    # one-bit elements: packed eight to a byte; a single byte is a splat only as 0x00 or 0xFF
    bits = NDType((4, 8), A.I1)
    assert not ContentAttr.get(np.array([1, 2, 3, 4], np.uint8), bits, backend=oracle)._isSplat
    assert ContentAttr.get(np.array([0xFF], np.uint8), bits, backend=oracle)._isSplat
    with pytest.raises(ConstError, match="Size of dense resource buffer '1'"):
        ContentAttr.get(np.array([0x0F], np.uint8), bits, backend=oracle)
    # a type of one element is never flagged as a splat; a missing or quantised base is refused
    assert not ContentAttr.get(np.array([5.0], np.float32), backend=oracle)._isSplat
    with pytest.raises(ConstError, match="Got NULL 'baseContent'"):
        ContentAttr.get(None, t, backend=oracle)
    with pytest.raises(ConstError, match="Got unsupported element type"):
        ContentAttr.get(np.zeros(3, np.uint8), NDType((3,), UniformQuantizedType(A.UI8, A.F32, 1.0, 0)), backend=oracle)
    # the caller's own splat flag is checked against the size as well
    with pytest.raises(ConstError, match="Size of dense resource buffer '12'"):
        ContentAttr.get(np.zeros(3, np.float32), t, is_splat=True, backend=oracle)
    with pytest.raises(ConstError, match="Size of dense resource buffer '4'"):
        ContentAttr.get(np.zeros(1, np.float32), t, is_splat=False, backend=oracle)


# tests/unit/vpux_compiler/dialect/const/content_tests.cpp:160-320: a dense resource that holds every element is no
# splat, one that holds a single element or only equal elements is (and folds to that value everywhere), an empty one
# is not
def test_dense_resource_splat_detection(oracle):
    t = NDType((1, 2, 3, 4), A.F32)
    vals = np.arange(24, dtype=np.float32)
    dense = ContentAttr.getDenseResource(vals, t, backend=oracle)
    assert not dense._isSplat and np.array_equal(dense.fold().copyTo().view(np.float32), vals)
    one = ContentAttr.getDenseResource(np.array([4.0], np.float32), t, backend=oracle)
    assert one._isSplat and (one.fold().copyTo().view(np.float32) == 4.0).all() and one.fold().copyTo().size == 96
    equal = ContentAttr.getDenseResource(np.full(24, -4.0, np.float32), t, backend=oracle)
    assert equal._isSplat and equal.getBaseContent().size == 4
    assert (equal.fold().copyTo().view(np.float32) == -4.0).all() and equal.fold().copyTo().size == 96
    empty = ContentAttr.getDenseResource(np.zeros(0, np.float32), NDType((0,), A.F32), backend=oracle)
    assert not empty._isSplat and empty.getType() == NDType((0,), A.F32)
    # equal bytes are not equal elements: 0x0101 0x0101 ... is a splat of 16-bit elements, 0x01 0x02 0x01 0x02 too,
    # but a single differing byte is noticed
    pat = np.tile(np.array([1, 2], np.uint8), 50)
    assert ContentAttr.getDenseResource(pat, NDType((50,), A.UI16), backend=oracle)._isSplat
    pat[37] = 3
    assert not ContentAttr.getDenseResource(pat, NDType((50,), A.UI16), backend=oracle)._isSplat
    # a splat behaves as one downstream: BitPack refuses it (bit_pack.cpp:109)
    from npu_plugin_b200.const import ConstError
    with pytest.raises(ConstError, match="splat"):
        ContentAttr.getDenseResource(np.full(8, 3, np.int8), NDType((8,), A.SI8), backend=oracle).bitPack(4).fold()
