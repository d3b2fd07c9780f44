//
// b200_bridge.cpp -- in-tree adapter between the Const dialect and the B200 shim (include/b200const.h).
//
// Where it goes: src/vpux_compiler/src/dialect/const/utils/b200_bridge.cpp, compiled into the compiler
// library when the build is configured with -DENABLE_B200_CONST_FOLDING=ON and linked against
// libb200const.so.  It cannot be compiled in the repository that ships this file (MLIR/LLVM, OpenVINO
// and TBB are absent there); it is written against the reference's own headers so that a maintainer can
// review it line by line.  The two call sites it serves are shown in patches/README.md:
//
//   Const::ContentAttr::fold           (src/vpux_compiler/src/dialect/const/attributes/content.cpp:167-193)
//   BitCompactorCodec::compress        (src/vpux_compiler/src/utils/bit_compactor_codec.cpp:15-42)
//
// and, for whole-model export, serializeBinaryData (src/vpux_compiler/src/dialect/VPUIP/graph-schema/export.cpp:453-493).
//
// Contract kept: fold() returns a Const::Content that owns a temp buffer holding exactly the bytes the
// reference's transformation loop would have produced followed by copyTo-style conversion to the folded
// type's element type (so getValues<T>() and copyTo() of the result behave as before); every
// data-dependent VPUX_THROW of the CPU path comes back as B200C_ERR_THROW with the same message and is
// re-thrown here; "not smaller" from the codec is mlir::failure().
//

#include "vpux/compiler/dialect/const/utils/b200_bridge.hpp"

#include "vpux/compiler/core/attributes/dims_order.hpp"
#include "vpux/compiler/dialect/VPUIP/attributes.hpp"
#include "vpux/compiler/dialect/const/attributes/content.hpp"
#include "vpux/compiler/dialect/const/utils/constant_folding_cache.hpp"
#include "vpux/compiler/dialect/const/utils/content.hpp"
#include "vpux/compiler/utils/attributes.hpp"
#include "vpux/compiler/utils/quantization.hpp"
#include "vpux/compiler/utils/types.hpp"
#include "vpux/utils/core/error.hpp"

#include <mlir/Dialect/Quant/QuantTypes.h>
#include <mlir/IR/BuiltinAttributes.h>
#include <mlir/IR/DialectResourceBlobManager.h>

#include <b200const.h>

#include <deque>
#include <mutex>

using namespace vpux;

namespace {

//
// Device contexts: one per calling thread (fold() is called from the export's parallel loop, from the
// background folding threads and from multithreaded passes; a context serialises its own calls).
//

b200c_ctx* threadContext() {
    struct Holder {
        b200c_ctx* ctx = nullptr;
        Holder() {
            const char* dev = std::getenv("IE_NPU_B200_DEVICE");
            const int rc = b200c_create(dev != nullptr ? std::atoi(dev) : 0, &ctx);
            VPUX_THROW_UNLESS(rc == B200C_OK, "B200 constant folding: {0}", b200c_last_error());
        }
        ~Holder() {
            b200c_destroy(ctx);
        }
    };
    static thread_local Holder holder;
    return holder.ctx;
}

[[noreturn]] void rethrow(int rc) {
    // B200C_ERR_THROW carries the text the CPU path would have put into VPUX_THROW
    VPUX_THROW("{0}{1}", rc == B200C_ERR_THROW ? "" : "B200 constant folding: ", b200c_last_error());
}

//
// Types
//

int32_t lowerElemType(mlir::Type type) {
    if (const auto qType = type.dyn_cast<mlir::quant::QuantizedType>()) {
        return lowerElemType(normalizeQuantStorageType(qType));
    }
    if (type.isF64()) return B200C_F64;
    if (type.isF32()) return B200C_F32;
    if (type.isF16()) return B200C_F16;
    if (type.isBF16()) return B200C_BF16;
    if (const auto intType = type.dyn_cast<mlir::IntegerType>()) {
        const int cls = intType.isSigned() ? B200C_CLS_SINT : (intType.isUnsigned() ? B200C_CLS_UINT : B200C_CLS_INT);
        return B200C_DTYPE(cls, static_cast<int>(intType.getWidth()));
    }
    VPUX_THROW("B200 constant folding: unsupported element type '{0}'", type);
}

// Owns the scale / zero-point arrays a b200c_type points to.
struct TypeStorage {
    std::deque<std::vector<double>> scales;
    std::deque<std::vector<int64_t>> zps;
};

void lowerQuant(mlir::Type elemType, b200c_type& out, TypeStorage& keep) {
    out.qkind = B200C_Q_NONE;
    if (const auto uniform = elemType.dyn_cast<mlir::quant::UniformQuantizedType>()) {
        out.qkind = B200C_Q_PER_TENSOR;
        keep.scales.push_back({uniform.getScale()});
        keep.zps.push_back({uniform.getZeroPoint()});
        out.qexpressed = lowerElemType(uniform.getExpressedType());
        out.qmin = uniform.getStorageTypeMin();
        out.qmax = uniform.getStorageTypeMax();
    } else if (const auto perAxis = elemType.dyn_cast<mlir::quant::UniformQuantizedPerAxisType>()) {
        out.qkind = B200C_Q_PER_AXIS;
        out.qaxis = perAxis.getQuantizedDimension();
        keep.scales.emplace_back(perAxis.getScales().begin(), perAxis.getScales().end());
        keep.zps.emplace_back(perAxis.getZeroPoints().begin(), perAxis.getZeroPoints().end());
        out.qexpressed = lowerElemType(perAxis.getExpressedType());
        out.qmin = perAxis.getStorageTypeMin();
        out.qmax = perAxis.getStorageTypeMax();
    } else {
        return;
    }
    out.nq = static_cast<int64_t>(keep.scales.back().size());
    out.scales = keep.scales.back().data();
    out.zps = keep.zps.back().data();
}

void lowerOrder(DimsOrder order, uint8_t* out) {
    const auto perm = order.toPermutation();  // perm[k] = logical dim at memory position k, outermost first
    for (size_t k = 0; k < perm.size(); ++k) {
        out[k] = static_cast<uint8_t>(perm[k].ind());
    }
}

b200c_type lowerType(vpux::NDTypeInterface type, TypeStorage& keep) {
    b200c_type t;
    std::memset(&t, 0, sizeof(t));
    const auto shape = type.getShape();
    VPUX_THROW_UNLESS(shape.size() <= B200C_MAX_RANK, "B200 constant folding: rank {0} is not supported", shape.size());
    t.dtype = lowerElemType(type.getElementType());
    t.rank = static_cast<int32_t>(shape.size());
    for (size_t k = 0; k < shape.size(); ++k) {
        t.shape[k] = shape[Dim(k)];
    }
    lowerOrder(type.getDimsOrder(), t.order);
    lowerQuant(type.getElementType(), t, keep);
    return t;
}

// element type only (ConvertElemType, QuantCast, ChangeShapeAndElemType)
b200c_type lowerElemOnly(mlir::Type elemType, TypeStorage& keep) {
    b200c_type t;
    std::memset(&t, 0, sizeof(t));
    if (elemType != nullptr) {
        t.dtype = lowerElemType(elemType);
        lowerQuant(elemType, t, keep);
    }
    return t;
}

mlir::Type raiseElemType(mlir::MLIRContext* ctx, const b200c_type& t) {
    mlir::Type storage;
    const int bits = B200C_DTYPE_BITS(t.dtype);
    switch (B200C_DTYPE_CLASS(t.dtype)) {
    case B200C_CLS_FLOAT:
        storage = bits == 64 ? mlir::Type(mlir::Float64Type::get(ctx))
                             : (bits == 32 ? mlir::Type(mlir::Float32Type::get(ctx)) : mlir::Type(mlir::Float16Type::get(ctx)));
        break;
    case B200C_CLS_BFLOAT:
        storage = mlir::BFloat16Type::get(ctx);
        break;
    case B200C_CLS_SINT:
        storage = mlir::IntegerType::get(ctx, bits, mlir::IntegerType::Signed);
        break;
    case B200C_CLS_UINT:
        storage = mlir::IntegerType::get(ctx, bits, mlir::IntegerType::Unsigned);
        break;
    default:
        storage = mlir::IntegerType::get(ctx, bits, mlir::IntegerType::Signless);
        break;
    }
    return storage;
}

//
// rawDataOf / isSplat: the base ElementsAttr as (bytes, splat flag), as wrapBaseContent reads it
// (content.cpp:143-159).  For a dense resource the "all elements equal" test of detectSplatElementWise
// (content.cpp:103-126) runs on the device.
//

struct RawBase {
    ArrayRef<char> data;
    bool isSplat = false;
};

RawBase rawDataOf(mlir::ElementsAttr baseContent) {
    RawBase raw;
    if (const auto dense = mlir::dyn_cast<mlir::DenseElementsAttr>(baseContent)) {
        raw.data = dense.getRawData();
        raw.isSplat = dense.isSplat();
        return raw;
    }
    const auto resource = mlir::cast<mlir::DenseResourceElementsAttr>(baseContent);
    raw.data = resource.getRawHandle().getBlob()->getData();
    if (raw.data.empty()) {
        return raw;  // empty data is not a splat
    }
    bool singleElementSplat = false;
    std::ignore = mlir::DenseElementsAttr::isValidRawBuffer(baseContent.getShapedType(), raw.data, singleElementSplat);
    if (singleElementSplat) {
        raw.isSplat = true;
        return raw;
    }
    const auto elemBytes = static_cast<int>(vpux::getElemTypeSize(baseContent.getShapedType()).to<Byte>().count());
    int flag = 0;
    const int rc = b200c_detect_splat(threadContext(), raw.data.data(), raw.data.size(), elemBytes, /*data_on_device=*/0, &flag);
    if (rc != B200C_OK) {
        rethrow(rc);
    }
    if (flag != 0) {
        raw.data = raw.data.take_front(static_cast<size_t>(elemBytes));
        raw.isSplat = true;
    }
    return raw;
}

//
// lower(getTransformations()): one b200c_xform per attribute, all 19 mnemonics of
// src/vpux_compiler/tblgen/vpux/compiler/dialect/const/attributes.td:131-620
//

struct Lowered {
    std::vector<b200c_xform> chain;
    TypeStorage types;
    std::deque<std::vector<int64_t>> aux;
};

void putArray(ArrayRef<int64_t> values, int64_t* dst, int32_t* n) {
    VPUX_THROW_UNLESS(values.size() <= B200C_MAX_RANK, "B200 constant folding: rank {0} is not supported", values.size());
    for (size_t k = 0; k < values.size(); ++k) {
        dst[k] = values[k];
    }
    *n = std::max<int32_t>(*n, static_cast<int32_t>(values.size()));
}

void putOrder(mlir::AffineMapAttr order, int64_t* dst, int32_t* n) {
    const auto perm = DimsOrder::fromAffineMap(order.getValue()).toPermutation();
    for (size_t k = 0; k < perm.size(); ++k) {
        dst[k] = perm[k].ind();
    }
    *n = static_cast<int32_t>(perm.size());
}

void lower(ArrayRef<Const::TransformAttrInterface> transformations, Lowered& out) {
    out.chain.reserve(transformations.size());
    for (const auto& attr : transformations) {
        b200c_xform x;
        std::memset(&x, 0, sizeof(x));
        if (const auto a = attr.dyn_cast<Const::ConvertElemTypeAttr>()) {
            x.kind = B200C_X_CONVERT_ELEM_TYPE;
            x.type = lowerElemOnly(a.getElemType(), out.types);
        } else if (const auto a = attr.dyn_cast<Const::QuantCastAttr>()) {
            x.kind = B200C_X_QUANT_CAST;
            x.type = lowerElemOnly(a.getElemType(), out.types);  // null element type: strip the quantisation
        } else if (attr.isa<Const::DequantizeAttr>()) {
            x.kind = B200C_X_DEQUANTIZE;
        } else if (const auto a = attr.dyn_cast<Const::RescaleAttr>()) {
            x.kind = B200C_X_RESCALE;
            x.f = a.getScale().getValueAsDouble();
        } else if (const auto a = attr.dyn_cast<Const::AddAttr>()) {
            x.kind = B200C_X_ADD;
            x.f = a.getBias().getValueAsDouble();
        } else if (const auto a = attr.dyn_cast<Const::ReorderAttr>()) {
            x.kind = B200C_X_REORDER;
            putOrder(a.getOrder(), x.a, &x.n);
        } else if (const auto a = attr.dyn_cast<Const::SubViewAttr>()) {
            x.kind = B200C_X_SUBVIEW;
            putArray(parseIntArrayAttr<int64_t>(a.getOffset()), x.a, &x.n);
            putArray(parseIntArrayAttr<int64_t>(a.getShape()), x.b, &x.n);
        } else if (const auto a = attr.dyn_cast<Const::PadWithZeroAttr>()) {
            x.kind = B200C_X_PAD_WITH_ZERO;
            putArray(parseIntArrayAttr<int64_t>(a.getPadBefore()), x.a, &x.n);
            putArray(parseIntArrayAttr<int64_t>(a.getPadAfter()), x.b, &x.n);
        } else if (const auto a = attr.dyn_cast<Const::BitPackAttr>()) {
            x.kind = B200C_X_BIT_PACK;
            x.i0 = a.getWidth().getInt();
        } else if (attr.isa<Const::GetSparsityMapAttr>()) {
            x.kind = B200C_X_GET_SPARSITY_MAP;
        } else if (const auto a = attr.dyn_cast<Const::SparsifyAttr>()) {
            x.kind = B200C_X_SPARSIFY;
            x.i0 = a.getCompressOutputType().getValue() ? 1 : 0;
            if (a.getNumActualElements() != nullptr) {
                const auto values = a.getNumActualElements().getValues<int64_t>();
                out.aux.emplace_back(values.begin(), values.end());
                x.aux = out.aux.back().data();
                x.naux = static_cast<int64_t>(out.aux.back().size());
            }
        } else if (const auto a = attr.dyn_cast<Const::SwizzleConstantAttr>()) {
            x.kind = B200C_X_SWIZZLE_CONSTANT;
            x.i0 = a.getSwizzleKey().getInt();
            x.i1 = a.getArch().getInt();
        } else if (const auto a = attr.dyn_cast<Const::ReshapeAttr>()) {
            x.kind = B200C_X_RESHAPE;
            putArray(parseIntArrayAttr<int64_t>(a.getShape()), x.b, &x.n);
        } else if (const auto a = attr.dyn_cast<Const::ChangeShapeAndElemTypeAttr>()) {
            x.kind = B200C_X_CHANGE_SHAPE_AND_ELEM_TYPE;
            putArray(parseIntArrayAttr<int64_t>(a.getShape()), x.b, &x.n);
            x.type = lowerElemOnly(a.getElemType(), out.types);
        } else if (const auto a = attr.dyn_cast<Const::BroadcastAttr>()) {
            x.kind = B200C_X_BROADCAST;
            x.i0 = a.getAxis().getInt();
            x.i1 = a.getValue().getInt();
        } else if (const auto a = attr.dyn_cast<Const::TransposeAttr>()) {
            x.kind = B200C_X_TRANSPOSE;
            putOrder(a.getOrder(), x.a, &x.n);
        } else if (const auto a = attr.dyn_cast<Const::ReverseAttr>()) {
            x.kind = B200C_X_REVERSE;
            x.i0 = a.getAxis().getInt();
        } else if (const auto a = attr.dyn_cast<Const::ExpandDilatedAttr>()) {
            x.kind = B200C_X_EXPAND_DILATED;
            putArray(parseIntArrayAttr<int64_t>(a.getDilations()), x.a, &x.n);
        } else if (const auto a = attr.dyn_cast<Const::RelocateWeightsTableAttr>()) {
            x.kind = B200C_X_RELOCATE_WEIGHTS_TABLE;
            const auto weightsPtr = parseIntArrayAttr<int64_t>(a.getWeightsPtr());
            const auto offsets = parseIntArrayAttr<int64_t>(a.getOffsets());
            VPUX_THROW_UNLESS(weightsPtr.size() == offsets.size(), "RelocateWeightsTable: {0} pointers for {1} clusters",
                              weightsPtr.size(), offsets.size());
            putArray(offsets, x.a, &x.n);
            putArray(weightsPtr, x.b, &x.n);
            x.i0 = static_cast<int32_t>(*a.getSparsityPtr().getValue().getRawData());
            x.i1 = a.getWeightsElemBitSize() != nullptr ? a.getWeightsElemBitSize().getInt() : 0;
            if (const auto scheme = a.getWeightsCompression()) {
                const auto numElems = scheme.getNumElems().getValues<int64_t>();
                out.aux.emplace_back(numElems.begin(), numElems.end());
                x.aux = out.aux.back().data();
                x.naux = static_cast<int64_t>(out.aux.back().size());
                x.f = scheme.getAlignment() != nullptr ? static_cast<double>(scheme.getAlignment().getInt()) : 0.0;
            }
        } else {
            VPUX_THROW("B200 constant folding: transformation '{0}' has no lowering", attr.getTransformationName());
        }
        out.chain.push_back(x);
    }
}

// the folded type reported by the shim, raised back to an NDTypeInterface (shape, storage element type, order;
// the quantisation parameters are taken from the attribute's own inferred type, which the shim's
// b200c_infer_type is tested to agree with)
vpux::NDTypeInterface raiseType(mlir::MLIRContext* ctx, const b200c_type& t, vpux::NDTypeInterface inferred) {
    SmallVector<int64_t> shape(t.shape, t.shape + t.rank);
    SmallVector<uint32_t> perm(t.order, t.order + t.rank);
    const auto order = DimsOrder::fromPermutation(to_small_vector(perm | transformed([](uint32_t d) {
                                                                       return Dim(d);
                                                                   })));
    mlir::Type elemType = raiseElemType(ctx, t);
    if (t.qkind != B200C_Q_NONE) {
        elemType = inferred.getElementType();
    }
    return mlir::RankedTensorType::get(shape, elemType, vpux::getTensorAttr(ctx, order, nullptr))
            .cast<vpux::NDTypeInterface>();
}

}  // namespace

//
// foldOnB200: what ContentAttr::fold calls instead of its transformation loop
//

Const::Content vpux::Const::foldOnB200(Const::ContentAttr attr) {
    const auto baseContent = attr.getBaseContent();
    const auto baseType = baseContent.getShapedType().cast<vpux::NDTypeInterface>();
    const auto raw = rawDataOf(baseContent);

    Lowered lowered;
    lower(attr.getTransformations(), lowered);
    TypeStorage baseKeep;
    const b200c_type base = lowerType(baseType, baseKeep);

    // the folded Content's type can differ from the attribute's inferred type (Sparsify<false>): the shim
    // reports it; capacity is the inferred type's size, which is never smaller
    const auto inferred = attr.getType();
    const auto capacity = static_cast<size_t>(inferred.getTotalAllocSize().count());

    b200c_type outType;
    std::memset(&outType, 0, sizeof(outType));
    const auto maxQuant = static_cast<size_t>(std::max<int64_t>(inferred.getShape().totalSize(), 1)) + 64;
    std::vector<double> outScales(maxQuant);
    std::vector<int64_t> outZps(maxQuant);
    outType.scales = outScales.data();
    outType.zps = outZps.data();
    outType.nq = static_cast<int64_t>(maxQuant);

    // Content::allocTempBuffer with the folded element type as storage: the result needs no further conversion
    std::vector<char> bytes(capacity, 0);
    size_t written = 0;
    const int rc = b200c_fold(threadContext(), &base, raw.data.data(), raw.data.size(), raw.isSplat ? 1 : 0,
                              /*data_on_device=*/0, lowered.chain.data(), static_cast<int>(lowered.chain.size()), bytes.data(),
                              capacity, /*out_on_device=*/0, &written, &outType, /*flags=*/0);
    if (rc != B200C_OK) {
        rethrow(rc);
    }

    const auto foldedType = raiseType(baseContent.getContext(), outType, inferred);
    auto content = Const::Content::allocTempBuffer(foldedType, foldedType.getElementType(), /*isSplat=*/false);
    auto dst = content.getRawTempBuf();
    VPUX_THROW_UNLESS(dst.size() >= written, "B200 constant folding: folded {0} bytes into a buffer of {1}", written,
                      dst.size());
    std::memcpy(dst.data(), bytes.data(), written);
    return content;
}

//
// compressOnB200: what BitCompactorCodec::compress calls instead of btc27::BitCompactor
// (the stream is the shim's own block format; see include/b200const.h)
//

mlir::FailureOr<std::vector<uint8_t>> vpux::compressOnB200(std::vector<uint8_t>& data, const Logger& log) {
    VPUX_THROW_WHEN(data.empty(), "BitCompactorCodec::compress: Empty input data vector");
    size_t bound = 0;
    b200c_btc_bound(data.size(), &bound);
    std::vector<uint8_t> stream(bound, 0);
    size_t size = 0;
    const int rc = b200c_btc_compress(threadContext(), data.data(), data.size(), /*in_on_device=*/0, stream.data(), bound,
                                      /*out_on_device=*/0, &size);
    if (rc == B200C_NOT_SMALLER) {
        log.nest().trace("BitCompactorCodec::compress: uncompressedDataSize <= compressedSize");
        return mlir::failure();
    }
    if (rc != B200C_OK) {
        rethrow(rc);
    }
    VPUX_THROW_WHEN(size > bound, "Compression would lead to buffer overflow");
    stream.resize(size);
    return stream;
}

//
// Cache hand-off: the folding cache (constant_folding_cache.cpp:78-108) stores Const::Content values keyed by
// ContentAttr.  Results of foldOnB200 are ordinary Content objects, so background folding
// (constant_folding_in_background.cpp:20-55) keeps working unchanged: its worker threads call fold(bypassCache =
// true) -> foldOnB200 and publish the result with cache.addContent(attr, content); each worker owns one device
// context through threadContext().  Partial-fold reuse (an attribute whose list extends a cached one) is served
// by folding the remaining transformations over the cached Content's bytes:
//

Const::Content vpux::Const::foldOnB200From(Const::Content cached, ArrayRef<Const::TransformAttrInterface> remaining) {
    // the cached Content is the folded result of a prefix: wrap its bytes as a new base and fold the rest
    const auto type = cached.getType();
    std::vector<char> bytes(static_cast<size_t>(type.getTotalAllocSize().count()), 0);
    cached.copyTo(MutableArrayRef(bytes.data(), bytes.size()));

    Lowered lowered;
    lower(remaining, lowered);
    TypeStorage keep;
    b200c_type base = lowerType(type, keep);
    base.qkind = B200C_Q_NONE;  // a base content carries its storage type; the first QuantCast of `remaining` re-tags it

    auto finalType = type;
    for (const auto& attr : remaining) {
        finalType = attr.inferOutputType(finalType);
    }
    const auto capacity = static_cast<size_t>(finalType.getTotalAllocSize().count());
    std::vector<char> out(capacity, 0);
    size_t written = 0;
    const int rc = b200c_fold(threadContext(), &base, bytes.data(), bytes.size(), /*is_splat=*/0, 0, lowered.chain.data(),
                              static_cast<int>(lowered.chain.size()), out.data(), capacity, 0, &written, nullptr, 0);
    if (rc != B200C_OK) {
        rethrow(rc);
    }
    auto content = Const::Content::allocTempBuffer(finalType, finalType.getElementType(), false);
    std::memcpy(content.getRawTempBuf().data(), out.data(), written);
    return content;
}
