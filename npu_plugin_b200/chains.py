"""The chain builders: the callers of the ContentAttr API that assemble the transformation lists the
hot path folds.  Each function restates one call site of the reference compiler on the host-side
ContentAttr mirror (npu_plugin_b200.const), so that a workload or a test asks for "the aligned weights
of this convolution" instead of hand-assembling the list.

  align_depthwise_weights      getAlignedConstWeights, src/vpux_compiler/src/dialect/VPU/utils/const_utils.cpp:101-119
  align_convolution_weights    alignConvWeightsTensor,  src/vpux_compiler/src/dialect/VPU/utils/const_utils.cpp:246-283
  weights_to_u8                ConvertWeightsToU8 ConstRewriter, src/vpux_compiler/src/dialect/IE/passes/convert_weights_to_u8.cpp:85-101
  sparsify_weights             SparsifyWeightsPass, src/vpux_compiler/src/dialect/VPU/transforms/passes/sparsify_weights.cpp:108-164
  flatten_sparse_weights       compressConstWeightsType, src/vpux_compiler/src/dialect/VPUIP/passes/flatten_sparse_weights_types.cpp:41-73
  sparse_identity_filter       createFilter, src/vpux_compiler/src/dialect/VPU/transforms/passes/lower_sparsity_ops.cpp:209-250
  hwtest_default_weights       generateDefaultWeightsAttr, src/vpux_translate_utils/src/hwtest/hwtest_utils.cpp:184-197
  attach_swizzle               Swizzling::attachSwizzleTransformation, src/vpux_compiler/src/dialect/VPUIP/passes/swizzling.cpp:469-500
"""
import numpy as np

from . import _cabi as A
from .const import ContentAttr, DimsOrder, NDType, Quant, Transform

VPU_WEIGHT_SET_BYTE_ALIGNMENT = 16  # nce_invariant.hpp:39
SWIZZLING_KEY_5 = 5
ARCH_VPUX37XX = 3


def align_depthwise_weights(weights, flat_shape, padding):
    """Depthwise weights flattened to flat_shape = [OC, IC*KY*KX / ..., 1, 1]-style 4D shape and padded along
    dim 1 by `padding`: reorder(NCHW) -> reshape -> padWithZero -> reorder(NHWC)."""
    return (weights.reorder(DimsOrder.NCHW).reshape(tuple(flat_shape))
            .padWithZero((0, 0, 0, 0), (0, padding, 0, 0)).reorder(DimsOrder.NHWC))


def align_convolution_weights(weights, alignment=16, is_cmajor_conv=False):
    """Weights [OC, IC, KY, KX] whose IC*KY*KX is not a multiple of `alignment` become [OC, 1, 1, aligned]:
    (reorder(NCHW) for the C-major convolution ->) reshape -> padWithZero on the last dim (-> reorder(NHWC)).
    Returns the attribute unchanged when no padding is needed, as the reference returns the original filter."""
    OC, IC, KY, KX = weights.getType().shape
    remainder = (IC * KY * KX) % alignment
    if remainder == 0:
        return weights
    padding = alignment - remainder
    flat = (OC, 1, 1, IC * KY * KX)
    a = weights.reorder(DimsOrder.NCHW).reshape(flat) if is_cmajor_conv else weights.reshape(flat)
    a = a.padWithZero((0, 0, 0, 0), (0, 0, 0, padding))
    return a.reorder(DimsOrder.NHWC) if is_cmajor_conv else a


def weights_to_u8(weights, new_quant):
    """Signed-int8 quantised weights re-based to unsigned: quantCast() -> convertElemType(i32, signless as the
    reference's getInt32Type) -> add(-storageMin) -> convertElemType(ui8) -> quantCast(new type).  `new_quant` is the
    u8 quantised type (zero points shifted by -storageMin by the caller's type converter).  The list is the one
    tests/lit/NPU/dialect/IE/passes/convert_weights_to_u8.mlir:25-32 checks."""
    old = weights.getType().quant
    if old is None:
        raise ValueError("weights_to_u8: the constant is not quantised")
    return (weights.quantCast().convertElemType(A.I32).add(float(-old.qmin)).convertElemType(A.UI8).quantCast(new_quant))


def sparsify_weights(weights, backend=None):
    """The weights constant of a sparsifiable operation becomes a pair (sparsified values, sparsity map) plus the
    per-output-channel counts that go into the compression scheme.  As in the pass, the original chain is folded
    first and its bytes become the base of a fresh attribute (so later passes do not fold it again); a quantised
    result keeps its quantised type through quantCast."""
    backend = backend or weights._backend
    content = weights.fold()
    folded_type = content.getType()
    counts = weights.countNonSparseElementsPerOC()
    base_elem = folded_type.dtype
    raw = np.array(content.copyTo(), copy=True)
    fresh = ContentAttr.get(raw, NDType(folded_type.shape, base_elem, folded_type.order), is_splat=False, backend=backend)
    if folded_type.quant is not None:
        fresh = fresh.quantCast(folded_type.quant)
    return fresh.sparsify(False), fresh.getSparsityMap(), counts


def flatten_sparse_weights(attr, num_elems):
    """Late in the pipeline the Sparsify transformation is rewritten to Sparsify<true, numElems> so that the
    attribute's type is the flat compressed one."""
    ts = []
    found = False
    for t in attr.getTransformations():
        if t.kind == A.X_SPARSIFY:
            t = Transform(A.X_SPARSIFY, i0=1, aux=[int(v) for v in num_elems])
            found = True
        ts.append(t)
    if not found:
        return attr
    return ContentAttr(attr._base, attr._baseType, attr._isSplat, ts, attr._backend)


def sparse_identity_filter(OC, IC, elem, order=DimsOrder.OYXI, backend=None):
    """The identity filter of a lowered sparsity op: ones on the diagonal of an [OC, IC, 1, 1] f32 constant ->
    (convertElemType(ui8) -> quantCast(q) | convertElemType(f16)) -> reorder -> sparsify(false), with its sparsity map
    and per-channel counts.  elem: a Quant, A.F16 or A.F32."""
    content = np.zeros((OC, IC, 1, 1), np.float32)
    flat = content.reshape(-1)
    for oc in range(OC):
        if oc * IC + oc < flat.size:
            flat[oc * IC + oc] = 1.0
    attr = ContentAttr.get(content, NDType((OC, IC, 1, 1), A.F32), backend=backend)
    if isinstance(elem, Quant):
        attr = attr.convertElemType(A.UI8).quantCast(elem)
    elif elem == A.F16:
        attr = attr.convertElemType(A.F16)
    if tuple(order) != tuple(DimsOrder.fromNumDims(4)):
        attr = attr.reorder(order)
    return attr.sparsify(False), attr.getSparsityMap(), attr.countNonSparseElementsPerOC()


def hwtest_default_weights(weights, quant=None):
    """Hardware-test weights: reorder(OYXI) -> quantCast(type with the constant's storage) -> bitPack(4) for 4-bit
    storage."""
    a = weights.reorder(DimsOrder.OYXI)
    if quant is not None:
        storage = a.getType().dtype
        q = Quant(quant.kind, storage, quant.expressed, quant.scales, quant.zps, quant.axis, quant.qmin, quant.qmax)
        a = a.quantCast(q)
        if A.dtype_bits(quant.storage) == 4:
            a = a.bitPack(4)
    return a


def attach_swizzle(attr, key=SWIZZLING_KEY_5, arch=ARCH_VPUX37XX):
    """Adds SwizzleConstant unless the list already holds one (a constant shared by several NCE tasks)."""
    if any(t.kind == A.X_SWIZZLE_CONSTANT for t in attr.getTransformations()):
        return attr
    return attr.swizzleConstant(key, arch)
