// Type inference for transformation chains: each attribute's inferOutputType and
// ContentAttr::inferFinalType / getInsertionPosition of the reference, on the MLIR-free model of
// ctype.h.  Reference files are under src/vpux_compiler/src/dialect/const/attributes/ unless a
// longer path is given.
#include "ctype.h"

#include <algorithm>
#include <numeric>

namespace b200c {

// ---------------------------------------------------------------------------- descriptors
TensorType typeFromC(const b200c_type& c, bool elemOnly) {
    TensorType t;
    if (!dtValid(c.dtype)) throw BadArg("unknown element type code");
    t.dtype = c.dtype;
    if (!elemOnly) {
        if (c.rank < 0 || c.rank > B200C_MAX_RANK) throw BadArg("rank out of range");
        t.shape.assign(c.shape, c.shape + c.rank);
        t.order.resize(c.rank);
        std::vector<bool> seen(c.rank, false);
        for (int k = 0; k < c.rank; ++k) {
            const int d = c.order[k];
            if (d >= c.rank || seen[d]) throw BadArg("order is not a permutation");
            seen[d] = true;
            t.order[k] = d;
            if (c.shape[k] < 0) throw BadArg("negative dimension");
        }
    }
    if (c.qkind != B200C_Q_NONE) {
        if (c.qkind != B200C_Q_PER_TENSOR && c.qkind != B200C_Q_PER_AXIS) throw BadArg("unknown quantisation kind");
        if (!dtIsInt(c.dtype)) throw BadArg("quantised type needs an integer storage type");
        if (dtClass(c.dtype) == B200C_CLS_INT) throw BadArg("quantised storage must be the normalised signed/unsigned integer");
        if (c.nq < 1 || c.scales == nullptr || c.zps == nullptr) throw BadArg("missing quantisation parameters");
        if (c.qkind == B200C_Q_PER_TENSOR && c.nq != 1) throw BadArg("per-tensor quantisation takes one scale");
        t.q.kind = c.qkind;
        t.q.axis = c.qaxis;
        t.q.expressed = c.qexpressed;
        t.q.qmin = c.qmin;
        t.q.qmax = c.qmax;
        t.q.scales = c.scales;  // borrowed for the duration of the call
        t.q.zps = c.zps;
        t.q.n = static_cast<size_t>(c.nq);
    }
    return t;
}

void typeToC(const TensorType& t, b200c_type* c) {
    double* sc = const_cast<double*>(c->scales);
    int64_t* zp = const_cast<int64_t*>(c->zps);
    const int64_t cap = c->nq;
    c->dtype = t.dtype;
    c->rank = t.rank();
    for (int k = 0; k < B200C_MAX_RANK; ++k) {
        c->shape[k] = k < t.rank() ? t.shape[k] : 0;
        c->order[k] = k < t.rank() ? static_cast<uint8_t>(t.order[k]) : 0;
    }
    c->qkind = t.q.kind;
    c->qaxis = t.q.axis;
    c->qexpressed = t.q.expressed;
    c->qmin = t.q.qmin;
    c->qmax = t.q.qmax;
    c->nq = static_cast<int64_t>(t.q.n);
    if (t.quantized()) {
        if (sc == nullptr || zp == nullptr || cap < c->nq) {
            throw Capacity("output type needs caller storage for " + std::to_string(c->nq) + " quantisation parameters");
        }
        if (sc != t.q.scales) std::copy(t.q.scales, t.q.scales + t.q.n, sc);
        if (zp != t.q.zps) std::copy(t.q.zps, t.q.zps + t.q.n, zp);
    }
}

Transformation xformFromC(const b200c_xform& c) {
    Transformation x;
    x.kind = c.kind;
    if (c.n < 0 || c.n > B200C_MAX_RANK) throw BadArg("transformation array length out of range");
    x.a.assign(c.a, c.a + c.n);
    x.b.assign(c.b, c.b + c.n);
    x.f = c.f;
    x.i0 = c.i0;
    x.i1 = c.i1;
    x.hasType = c.type.dtype != 0;
    if (x.hasType) x.type = typeFromC(c.type, /*elemOnly=*/true);
    x.hasAux = c.aux != nullptr;
    if (x.hasAux) {
        if (c.naux < 0) throw BadArg("negative aux length");
        x.aux.assign(c.aux, c.aux + c.naux);
    }
    x.side0 = c.side0;
    x.side1 = c.side1;
    return x;
}

// ---------------------------------------------------------------------------- type edits
// validateQuantElemType (src/vpux_compiler/src/utils/quantization.cpp:23-45)
static void checkPerAxis(const TensorType& t) {
    if (t.q.kind != B200C_Q_PER_AXIS) return;
    if (t.q.axis < 0 || t.q.axis >= t.rank()) {
        refThrow("Quantized axis '%d' is out of main type rank '%d'", t.q.axis, t.rank());
    }
    if (static_cast<size_t>(t.shape[t.q.axis]) != t.q.n) {
        refThrow("Number of scales '%zu' in per-axis quantized type do not match the quantized dimension size '%lld'",
                 t.q.n, static_cast<long long>(t.shape[t.q.axis]));
    }
}

// Where a per-axis dimension lands after a reshape that only adds/removes unit dims
// (getQuantizedAxis, src/vpux_compiler/src/utils/types.cpp:128-165).  Returns -1 when it cannot be traced.
static int axisAfterReshape(int axis, const Dims& from, const Dims& to) {
    if (axis < 0 || static_cast<size_t>(axis) >= from.size()) return -1;
    size_t leadFrom = 0, leadTo = 0;
    while (leadFrom < from.size() && from[leadFrom] == 1) ++leadFrom;
    while (leadTo < to.size() && to[leadTo] == 1) ++leadTo;
    if (leadFrom == from.size() || leadTo == to.size()) return axis;
    std::vector<int64_t> f, t;
    std::copy_if(from.begin(), from.end(), std::back_inserter(f), [](int64_t v) { return v != 1; });
    std::copy_if(to.begin(), to.end(), std::back_inserter(t), [](int64_t v) { return v != 1; });
    if (f != t) return -1;
    const int shift = static_cast<int>(leadTo) - static_cast<int>(leadFrom);
    if (axis < -shift || axis + shift >= static_cast<int>(to.size())) return -1;
    return axis + shift;
}

// changeShape (type_interfaces.cpp:176-196): identity order follows the new rank, any other order must fit
TensorType withShape(const TensorType& in, const Dims& shape) {
    TensorType out = in;
    out.shape = shape;
    if (in.identityOrder()) {
        out.setIdentityOrder();
    } else if (shape.size() != in.shape.size()) {
        refThrow("Order is incompatible with the new shape");
    }
    if (in.q.kind == B200C_Q_PER_AXIS) {
        const int moved = axisAfterReshape(in.q.axis, in.shape, shape);
        if (moved >= 0) out.q.axis = moved;
    }
    checkPerAxis(out);
    return out;
}

// changeShapeElemType (type_interfaces.cpp:217-233)
TensorType withShapeAndElem(const TensorType& in, const Dims& shape, int dtype, const QuantInfo& q) {
    TensorType out = in;
    out.shape = shape;
    if (in.identityOrder()) {
        out.setIdentityOrder();
    } else if (shape.size() != in.shape.size()) {
        refThrow("Order is incompatible with the new shape");
    }
    out.dtype = dtype;
    out.q = q;
    checkPerAxis(out);
    return out;
}

static TensorType withElem(const TensorType& in, int dtype, const QuantInfo& q) {
    TensorType out = in;
    out.dtype = dtype;
    out.q = q;
    checkPerAxis(out);
    return out;
}

// pad() with expandScalesAndZP (type_interfaces.cpp:295-321, quantization.cpp:56-100)
static TensorType padded(const TensorType& in, const Dims& before, const Dims& after) {
    if (before.size() != after.size()) refThrow("Got non consistent 'padBefore' and 'padAfter' values");
    if (before.size() != in.shape.size()) refThrow("Paddings and input shape are not consistent");
    TensorType out = in;
    for (int d = 0; d < in.rank(); ++d) out.shape[d] += before[d] + after[d];
    if (in.q.kind == B200C_Q_PER_AXIS) {
        const int64_t front = before[in.q.axis], back = after[in.q.axis];
        if (front != 0 || back != 0) {
            if (front < 0 || back < 0) throw BadArg("negative padding on the quantised axis");
            if (in.q.n == 0) refThrow("Can't get value for expand scales.");
            if (!in.q.zpsAllEqual()) refThrow("All zero points should be equal");
            std::vector<double> sc(static_cast<size_t>(front), in.q.scales[0]);
            sc.insert(sc.end(), in.q.scales, in.q.scales + in.q.n);
            sc.insert(sc.end(), static_cast<size_t>(back), in.q.scales[in.q.n - 1]);
            std::vector<int64_t> zp(static_cast<size_t>(front), in.q.zps[0]);
            zp.insert(zp.end(), in.q.zps, in.q.zps + in.q.n);
            zp.insert(zp.end(), static_cast<size_t>(back), in.q.zps[in.q.n - 1]);
            out.q.own(std::move(sc), std::move(zp));
        }
    }
    checkPerAxis(out);
    return out;
}

// extractDenseTile with tileScalesAndZP (type_interfaces.cpp:263-279, quantization.cpp:106-130)
static TensorType tiled(const TensorType& in, const Dims& offset, const Dims& shape) {
    TensorType out = in;
    out.shape = shape;
    if (in.q.kind == B200C_Q_PER_AXIS) {
        if (offset.size() != shape.size()) refThrow("Offsets doesn't match shape");
        const int64_t lo = offset[in.q.axis], n = shape[in.q.axis];
        if (!(lo == 0 && static_cast<size_t>(n) == in.q.n)) {
            if (lo < 0 || n < 0 || static_cast<size_t>(lo + n) > in.q.n) {
                refThrow("Invalid slice of the quantization parameters");
            }
            out.q.scales = in.q.scales + lo;  // a window into the same table
            out.q.zps = in.q.zps + lo;
            out.q.n = static_cast<size_t>(n);
        }
    }
    checkPerAxis(out);
    return out;
}

// getSparsifyValue (src/vpux_compiler/src/utils/sparsity.cpp:12-26)
int64_t sparsifyValue(const TensorType& t) {
    if (t.q.kind == B200C_Q_NONE) return 0;
    if (t.q.kind == B200C_Q_PER_AXIS && !t.q.zpsAllEqual()) refThrow("Not all zero-points are equal");
    return t.q.zps[0];
}

// ---------------------------------------------------------------------------- inferOutputType
TensorType inferOne(const Transformation& x, const TensorType& in) {
    switch (x.kind) {
    case B200C_X_CONVERT_ELEM_TYPE:  // convert_elem_type.cpp:68-73
        if (!x.hasType) throw BadArg("ConvertElemType needs an element type");
        if (in.quantized()) refThrow("Can't convert quantized element type to the requested element type");
        return withElem(in, x.type.dtype, QuantInfo());

    case B200C_X_QUANT_CAST:  // quant_cast.cpp:61-75
        if (x.hasType) {
            if (!x.type.quantized()) throw BadArg("QuantCast needs a quantised element type (or none)");
            if (in.quantized() || in.dtype != x.type.dtype) {
                refThrow("Can't cast element type to the quantized element type: storage types differ");
            }
            return withElem(in, x.type.dtype, x.type.q);
        }
        if (!in.quantized()) refThrow("Unable to restore storage type from non-quantized type");
        return withElem(in, in.dtype, QuantInfo());

    case B200C_X_DEQUANTIZE:  // dequantize.cpp:23-28
        if (!in.quantized()) refThrow("Got non quantized type in 'DequantizeAttr'");
        if (!dtIsFloat(in.q.expressed)) throw BadArg("expressed type of the quantised type is not a float type");
        return withElem(in, in.q.expressed, QuantInfo());

    case B200C_X_RESCALE:  // rescale.cpp:55-57
    case B200C_X_ADD:      // add.cpp:52-54
    case B200C_X_REVERSE:  // reverse.cpp:50-52
        return in;
    case B200C_X_RELOCATE_WEIGHTS_TABLE:  // relocate_weights_table.cpp:114-116
        if (x.a.empty() || x.a.size() != x.b.size()) throw BadArg("RelocateWeightsTable: one weights pointer per cluster offset");
        return in;

    case B200C_X_REORDER: {  // reorder.cpp:67-73
        if (static_cast<int>(x.a.size()) != in.rank()) refThrow("DimsOrder doesn't match type");
        TensorType out = in;
        std::vector<bool> seen(in.rank(), false);
        for (int k = 0; k < in.rank(); ++k) {
            const int64_t d = x.a[k];
            if (d < 0 || d >= in.rank() || seen[d]) throw BadArg("Reorder: not a permutation");
            seen[d] = true;
            out.order[k] = static_cast<int>(d);
        }
        return out;
    }

    case B200C_X_SUBVIEW: {  // subview.cpp:105-117
        if (!(in.bits() >= 8 || in.bits() == 1)) {
            refThrow("SubViewAttr does not support sub-byte element types except i1");
        }
        if (static_cast<int>(x.b.size()) != in.rank()) {
            refThrow("View shape and input shape are not consistent in 'SubViewAttr'");
        }
        for (int d = 0; d < in.rank(); ++d) {
            if (x.a[d] < 0 || x.b[d] < 0 || x.a[d] + x.b[d] > in.shape[d]) throw BadArg("SubView: tile out of bounds");
        }
        return tiled(in, x.a, x.b);
    }

    case B200C_X_PAD_WITH_ZERO:  // pad_with_zero.cpp:98-102
        for (size_t d = 0; d < x.a.size(); ++d) {
            if (x.a[d] < 0 || x.b[d] < 0) throw BadArg("PadWithZero: negative padding");
        }
        return padded(in, x.a, x.b);

    case B200C_X_BIT_PACK: {  // bit_pack.cpp:75-102: same signedness, `width` bits, quant parameters kept
        if (!in.quantized() && dtIsFloat(in.dtype)) refThrow("Bit pack does not support float inputs.");
        if (!dtIsInt(in.dtype)) refThrow("Got unsupported input element type in bitpack");
        if (x.i0 != 1 && x.i0 != 4 && x.i0 != 8) throw BadArg("BitPack: unsupported width");
        TensorType out = in;
        out.dtype = B200C_DTYPE(dtClass(in.dtype), static_cast<int>(x.i0));
        return out;
    }

    case B200C_X_GET_SPARSITY_MAP: {  // get_sparsity_map.cpp:68-75; shape rule nce_sparsity.cpp:637-644
        if (in.rank() != 4) refThrow("Expected data shape to be 4D, while shape has rank %d", in.rank());
        const int64_t perOC = in.shape[1] * in.shape[2] * in.shape[3];
        TensorType out = withShape(in, {in.shape[0], 1, 1, roundUp(perOC, 128)});
        out.setIdentityOrder();
        return withElem(out, B200C_I1, QuantInfo());
    }

    case B200C_X_SPARSIFY: {  // sparsify.cpp:94-111
        if (x.i0 == 0) return in;
        if (!x.hasAux) refThrow("Missing number of actual elements");
        const int64_t elemBytes = in.bits() / 8;
        int64_t bytes = 0;
        for (int64_t n : x.aux) {
            if (n < 0) refThrow("Got negative elem number value '%lld' in 'numActualElements'", static_cast<long long>(n));
            bytes += roundUp(n * elemBytes, kWeightSetAlign);
        }
        return withShapeAndElem(in, {bytes, 1, 1, 1}, B200C_UI8, QuantInfo());
    }

    case B200C_X_SWIZZLE_CONSTANT: {  // swizzle_transform.cpp:126-148
        if (x.i1 != kArchVPUX37XX) refThrow("Architecture %lld does not support swizzling", static_cast<long long>(x.i1));
        const int64_t bytes = roundUp(in.allocBytes(), kSwizzleSizeAlign);
        if (in.bits() == 1) return withShape(in, {bytes * 8, 1, 1, 1});
        if (!in.quantized() && in.dtype == B200C_F16) return withShape(in, {bytes / 2, 1, 1, 1});
        return withShapeAndElem(in, {bytes, 1, 1, 1}, B200C_UI8, QuantInfo());
    }

    case B200C_X_RESHAPE: {  // reshape.cpp:73-76
        int64_t n = 1;
        for (auto d : x.b) n *= d;
        if (n != in.count()) throw BadArg("Reshape: element count changes");
        return withShape(in, x.b);
    }

    case B200C_X_CHANGE_SHAPE_AND_ELEM_TYPE:  // change_shape_and_elem_type.cpp:84-88
        if (!x.hasType) throw BadArg("ChangeShapeAndElemType needs an element type");
        return withShapeAndElem(in, x.b, x.type.dtype, x.type.q);

    case B200C_X_BROADCAST: {  // broadcast.cpp:62-78
        if (x.i0 < 0 || x.i0 >= in.rank()) throw BadArg("Broadcast: axis out of range");
        if (x.i1 < in.shape[x.i0]) {
            refThrow("Value cannot be broadcasted due to new value's size is less than old one: %lld < %lld",
                     static_cast<long long>(x.i1), static_cast<long long>(in.shape[x.i0]));
        }
        Dims none(in.rank(), 0), after(in.rank(), 0);
        after[x.i0] = x.i1 - in.shape[x.i0];
        return padded(in, none, after);
    }

    case B200C_X_TRANSPOSE: {  // transpose.cpp:67-86
        if (static_cast<int>(x.a.size()) != in.rank()) refThrow("DimsOrder doesn't match type");
        Dims shape(in.rank());
        std::vector<bool> seen(in.rank(), false);
        for (int k = 0; k < in.rank(); ++k) {
            const int64_t d = x.a[k];
            if (d < 0 || d >= in.rank() || seen[d]) throw BadArg("Transpose: not a permutation");
            seen[d] = true;
            shape[k] = in.shape[d];
        }
        QuantInfo q = in.q;
        if (q.kind == B200C_Q_PER_AXIS) q.axis = static_cast<int>(x.a[q.axis]);
        return withShapeAndElem(in, shape, in.dtype, q);
    }

    case B200C_X_QUANTIZE_SYNTH:
        if (in.quantized() || !dtIsFloat(in.dtype)) refThrow("QuantizeSynth expects a float tensor");
        if (x.i0 != B200C_QSYNTH_SYM_I8 && x.i0 != B200C_QSYNTH_ASYM_U4) throw BadArg("QuantizeSynth: unknown scheme");
        return in;

    case B200C_X_EXPAND_DILATED: {  // expand_dilated.cpp:78-82, getDilatedType (utils/dilated_utils.cpp:11-34)
        if (in.rank() != 4) refThrow("Got invalid tensor rank '4'");
        if (x.a.size() < 2) throw BadArg("ExpandDilated needs two dilations");
        if (x.a[0] < 1 || x.a[1] < 1) throw BadArg("ExpandDilated: dilations must be positive");
        Dims shape = in.shape;
        shape[2] = in.shape[2] + (in.shape[2] - 1) * (x.a[0] - 1);
        shape[3] = in.shape[3] + (in.shape[3] - 1) * (x.a[1] - 1);
        return withShape(in, shape);
    }
    default:
        throw BadArg("unknown transformation kind " + std::to_string(x.kind));
    }
}

TensorType inferChain(const TensorType& base, const std::vector<Transformation>& chain) {
    TensorType t = base;
    checkPerAxis(t);
    for (const auto& x : chain) t = inferOne(x, t);
    return t;
}

// ---------------------------------------------------------------------------- ordering
PositionReq positionOf(int kind) {
    switch (kind) {
    case B200C_X_GET_SPARSITY_MAP:  // get_sparsity_map.cpp:113-115
    case B200C_X_SPARSIFY:          // sparsify.cpp:192-194
        return PositionReq::PreferredLast;
    case B200C_X_BIT_PACK:          // bit_pack.cpp:136-138
    case B200C_X_SWIZZLE_CONSTANT:  // swizzle_transform.cpp:245-247
        return PositionReq::Last;
    default:
        return PositionReq::None;
    }
}

bool acceptsSubByteStorage(int kind) {  // subview.cpp:317-319, swizzle_transform.cpp:259-261
    return kind == B200C_X_SUBVIEW || kind == B200C_X_SWIZZLE_CONSTANT;
}

// content.cpp:268-299: [NONE]* then [PREFERRED_LAST]* then at most one [LAST]; stable within a class
int insertPosition(const std::vector<int>& kinds, int newKind) {
    const int n = static_cast<int>(kinds.size());
    if (n == 0) return 0;
    const PositionReq incoming = positionOf(newKind);
    if (incoming == PositionReq::Last) {
        if (positionOf(kinds.back()) == PositionReq::Last) {
            refThrow("Existing transformation with LAST position requirement");
        }
        return n;
    }
    int pos = n;
    while (pos > 0) {
        const PositionReq r = positionOf(kinds[pos - 1]);
        const bool stayBehind = r == PositionReq::None ||
                                (r == PositionReq::PreferredLast && incoming == PositionReq::PreferredLast);
        if (stayBehind) break;
        --pos;
    }
    return pos;
}

}  // namespace b200c
