/*
 * b200const.hpp -- header-only C++17 host layer over the C ABI of b200const.h.
 *
 * It mirrors the part of the reference's C++ interface that constant folding goes through --
 * vpux::Const::ContentAttr with its builder methods and fold(), and vpux::Const::Content with
 * getType(), getValues<T>() and copyTo()
 * (src/vpux_compiler/include/vpux/compiler/dialect/const/attributes/content.hpp,
 *  src/vpux_compiler/include/vpux/compiler/dialect/const/utils/content.hpp) -- with the same method
 * names, argument meaning and error behaviour (a failing call throws b200::Const::Error carrying the
 * text the reference would have put into VPUX_THROW).  MLIR types are replaced by small value types
 * (NDType, DimsOrder, QuantParams).  Everything here only marshals descriptors: all arithmetic runs
 * in the library's CUDA kernels, and there is no CPU path.
 */
#ifndef B200CONST_HPP_
#define B200CONST_HPP_

#include "b200const.h"

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace b200 {
namespace Const {

class Error : public std::runtime_error {
public:
    Error(int code, const std::string& what): std::runtime_error(what), _code(code) {
    }
    int code() const {  // one of B200C_ERR_*
        return _code;
    }

private:
    int _code;
};

inline void check(int rc) {
    if (rc < 0) throw Error(rc, b200c_last_error());
}

// vpux::DimsOrder: perm[k] = logical dimension stored at memory position k (outermost first)
struct DimsOrder {
    std::vector<uint8_t> perm;
    static DimsOrder identity(int rank) {
        DimsOrder o;
        for (int k = 0; k < rank; ++k) o.perm.push_back(static_cast<uint8_t>(k));
        return o;
    }
    static DimsOrder fromPermutation(std::initializer_list<int> p) {
        DimsOrder o;
        for (int d : p) o.perm.push_back(static_cast<uint8_t>(d));
        return o;
    }
    static DimsOrder NCHW() {
        return identity(4);
    }
    static DimsOrder NHWC() {
        return fromPermutation({0, 2, 3, 1});
    }
    static DimsOrder OIYX() {
        return identity(4);
    }
    static DimsOrder OYXI() {
        return fromPermutation({0, 2, 3, 1});
    }
    bool operator==(const DimsOrder& o) const {
        return perm == o.perm;
    }
};

// mlir::quant::UniformQuantizedType / UniformQuantizedPerAxisType
struct QuantParams {
    int kind = B200C_Q_NONE;
    int axis = 0;
    int expressed = B200C_F32;
    int64_t qmin = 0, qmax = 0;
    std::vector<double> scales;
    std::vector<int64_t> zps;
    static QuantParams perTensor(int expressed, double scale, int64_t zp, int64_t qmin, int64_t qmax) {
        QuantParams q;
        q.kind = B200C_Q_PER_TENSOR;
        q.expressed = expressed;
        q.scales = {scale};
        q.zps = {zp};
        q.qmin = qmin;
        q.qmax = qmax;
        return q;
    }
    static QuantParams perAxis(int expressed, std::vector<double> scales, std::vector<int64_t> zps, int axis, int64_t qmin,
                               int64_t qmax) {
        QuantParams q;
        q.kind = B200C_Q_PER_AXIS;
        q.expressed = expressed;
        q.scales = std::move(scales);
        q.zps = std::move(zps);
        q.axis = axis;
        q.qmin = qmin;
        q.qmax = qmax;
        return q;
    }
};

// vpux::NDTypeInterface of a constant: shape, element type (storage integer for quantised types), order
struct NDType {
    int dtype = 0;
    std::vector<int64_t> shape;
    DimsOrder order;
    QuantParams quant;

    NDType() = default;
    NDType(std::vector<int64_t> s, int dt): dtype(dt), shape(std::move(s)), order(DimsOrder::identity(static_cast<int>(shape.size()))) {
    }
    NDType(std::vector<int64_t> s, int dt, DimsOrder o): dtype(dt), shape(std::move(s)), order(std::move(o)) {
    }
    NDType(std::vector<int64_t> s, int storage, QuantParams q): dtype(storage), shape(std::move(s)),
            order(DimsOrder::identity(static_cast<int>(shape.size()))), quant(std::move(q)) {
    }
    int getRank() const {
        return static_cast<int>(shape.size());
    }
    int64_t getNumElements() const {
        int64_t n = 1;
        for (auto d : shape) n *= d;
        return n;
    }
    // the POD form; borrows the scale / zero-point storage of *this
    b200c_type toC() const {
        if (shape.size() > B200C_MAX_RANK) throw Error(B200C_ERR_INVALID, "rank above B200C_MAX_RANK");
        b200c_type t;
        std::memset(&t, 0, sizeof(t));
        t.dtype = dtype;
        t.rank = getRank();
        for (int k = 0; k < t.rank; ++k) {
            t.shape[k] = shape[k];
            t.order[k] = order.perm[k];
        }
        t.qkind = quant.kind;
        t.qaxis = quant.axis;
        t.qexpressed = quant.expressed;
        t.qmin = quant.qmin;
        t.qmax = quant.qmax;
        t.nq = static_cast<int64_t>(quant.scales.size());
        t.scales = quant.scales.data();
        t.zps = quant.zps.data();
        return t;
    }
    static NDType fromC(const b200c_type& t) {
        NDType r;
        r.dtype = t.dtype;
        r.shape.assign(t.shape, t.shape + t.rank);
        r.order.perm.assign(t.order, t.order + t.rank);
        r.quant.kind = t.qkind;
        r.quant.axis = t.qaxis;
        r.quant.expressed = t.qexpressed;
        r.quant.qmin = t.qmin;
        r.quant.qmax = t.qmax;
        if (t.qkind != B200C_Q_NONE) {
            r.quant.scales.assign(t.scales, t.scales + t.nq);
            r.quant.zps.assign(t.zps, t.zps + t.nq);
        }
        return r;
    }
    int64_t getTotalAllocSize() const {  // NDTypeInterface::getTotalAllocSize
        const b200c_type t = toC();
        return b200c_total_alloc_size(&t);
    }
};

// One device context (stream + scratch memory); calls on one context are serialised.
class Backend {
public:
    explicit Backend(int device = 0) {
        check(b200c_create(device, &_ctx));
    }
    ~Backend() {
        b200c_destroy(_ctx);
    }
    Backend(const Backend&) = delete;
    Backend& operator=(const Backend&) = delete;
    b200c_ctx* ctx() const {
        return _ctx;
    }

private:
    b200c_ctx* _ctx = nullptr;
};

// vpux::Const::Content after fold(): the folded bytes in the layout copyTo() produces, on the host
class Content {
public:
    Content(NDType type, std::vector<uint8_t> bytes): _type(std::move(type)), _bytes(std::move(bytes)) {
    }
    const NDType& getType() const {
        return _type;
    }
    // Const::Content::copyTo(MutableArrayRef<char>)
    void copyTo(void* dst, size_t cap) const {
        if (cap < _bytes.size()) throw Error(B200C_ERR_CAPACITY, "Const::Content::copyTo: buffer too small");
        std::memcpy(dst, _bytes.data(), _bytes.size());
    }
    const std::vector<uint8_t>& getRawBytes() const {
        return _bytes;
    }
    // values of byte-sized, non-quantised element types
    template <typename T>
    std::vector<T> getValues() const {
        if (_bytes.size() % sizeof(T) != 0) throw Error(B200C_ERR_INVALID, "getValues: element size does not divide the buffer");
        std::vector<T> v(_bytes.size() / sizeof(T));
        std::memcpy(v.data(), _bytes.data(), _bytes.size());
        return v;
    }

private:
    NDType _type;
    std::vector<uint8_t> _bytes;
};

// Result of constant fusion: the [1,1,1,N] ui8 or f16 constant that replaces the weight table, weights, weights
// sparsity map and activation window of one NCE task; views[k] = (offset, size) in elements of the fused type where
// part k lives -- the SubView that replaces it -- or (-1, -1) for an absent part.
struct FusedConstant {
    NDType type;
    std::vector<uint8_t> data;
    std::vector<std::pair<int64_t, int64_t>> views;
};

// vpux::Const::ContentAttr: a base content plus an ordered transformation list.  The builder methods
// return a new attribute, as the reference's do; a transformation is inserted at the position
// getInsertionPosition gives it (content.cpp:268-299).
class ContentAttr {
public:
    // ContentAttr::get(baseContent): `data` is copied.  The checks of ContentAttr::verify (content.cpp:61-99) run here:
    // the buffer holds every element of the type, or exactly one (a splat -- taken as one even when isSplat was
    // left false, the rule mlir::DenseElementsAttr::isValidRawBuffer applies to a dense resource; a single byte of
    // one-bit elements only as 0x00 or 0xFF).  Sub-byte elements are held packed.
    static ContentAttr get(const void* data, size_t nbytes, NDType baseType, bool isSplat = false) {
        if (data == nullptr) throw Error(B200C_ERR_THROW, "Got NULL 'baseContent' in 'ContentAttr'");
        if (baseType.quant.kind != B200C_Q_NONE) {
            throw Error(B200C_ERR_THROW, "Got unsupported element type for 'baseContent' in 'ContentAttr'");
        }
        const size_t bits = static_cast<size_t>(B200C_DTYPE_BITS(baseType.dtype));
        const size_t count = static_cast<size_t>(baseType.getNumElements());
        const size_t one = (bits + 7) / 8, all = (bits * count + 7) / 8;
        bool valid = isSplat ? nbytes == one : nbytes == all;
        if (!isSplat && !valid && nbytes == one && count != 1) {
            const uint8_t byte = *static_cast<const uint8_t*>(data);
            valid = isSplat = bits != 1 || byte == 0x00 || byte == 0xFF;
        }
        if (!valid) {
            throw Error(B200C_ERR_THROW, "Size of dense resource buffer '" + std::to_string(nbytes) +
                                                 "' in 'baseContent' doesn't match its type");
        }
        ContentAttr a;
        a._base = std::move(baseType);
        a._data = std::make_shared<std::vector<uint8_t>>(static_cast<const uint8_t*>(data),
                                                         static_cast<const uint8_t*>(data) + nbytes);
        a._splat = isSplat;
        return a;
    }
    template <typename T>
    static ContentAttr get(const std::vector<T>& values, NDType baseType, bool isSplat = false) {
        return get(values.data(), values.size() * sizeof(T), std::move(baseType), isSplat);
    }

    ContentAttr convertElemType(int dtype) const {
        Step s(B200C_X_CONVERT_ELEM_TYPE);
        s.type.dtype = dtype;
        return add(std::move(s));
    }
    ContentAttr quantCast(const QuantParams& q, int storage) const {  // quantCast(nullptr) = quantCast()
        Step s(B200C_X_QUANT_CAST);
        s.type.dtype = storage;
        s.type.quant = q;
        return add(std::move(s));
    }
    ContentAttr quantCast() const {
        return add(Step(B200C_X_QUANT_CAST));
    }
    ContentAttr dequantize() const {
        return add(Step(B200C_X_DEQUANTIZE));
    }
    ContentAttr rescale(double scale) const {
        Step s(B200C_X_RESCALE);
        s.x.f = scale;
        return add(std::move(s));
    }
    ContentAttr add(double bias) const {
        Step s(B200C_X_ADD);
        s.x.f = bias;
        return add(std::move(s));
    }
    ContentAttr reorder(const DimsOrder& order) const {
        Step s(B200C_X_REORDER);
        s.x.n = static_cast<int32_t>(order.perm.size());
        for (size_t k = 0; k < order.perm.size(); ++k) s.x.a[k] = order.perm[k];
        return add(std::move(s));
    }
    ContentAttr transpose(const DimsOrder& order) const {
        Step s(B200C_X_TRANSPOSE);
        s.x.n = static_cast<int32_t>(order.perm.size());
        for (size_t k = 0; k < order.perm.size(); ++k) s.x.a[k] = order.perm[k];
        return add(std::move(s));
    }
    ContentAttr reshape(const std::vector<int64_t>& shape) const {
        Step s(B200C_X_RESHAPE);
        fill(s.x.b, shape, &s.x.n);
        return add(std::move(s));
    }
    ContentAttr subview(const std::vector<int64_t>& offset, const std::vector<int64_t>& shape) const {
        Step s(B200C_X_SUBVIEW);
        fill(s.x.a, offset, &s.x.n);
        fill(s.x.b, shape, &s.x.n);
        return add(std::move(s));
    }
    ContentAttr padWithZero(const std::vector<int64_t>& padBefore, const std::vector<int64_t>& padAfter) const {
        Step s(B200C_X_PAD_WITH_ZERO);
        fill(s.x.a, padBefore, &s.x.n);
        fill(s.x.b, padAfter, &s.x.n);
        return add(std::move(s));
    }
    ContentAttr broadcast(int64_t axis, int64_t value) const {
        Step s(B200C_X_BROADCAST);
        s.x.i0 = axis;
        s.x.i1 = value;
        return add(std::move(s));
    }
    ContentAttr reverse(int64_t axis) const {
        Step s(B200C_X_REVERSE);
        s.x.i0 = axis;
        return add(std::move(s));
    }
    ContentAttr expandDilated(const std::vector<int64_t>& dilations) const {
        Step s(B200C_X_EXPAND_DILATED);
        fill(s.x.a, dilations, &s.x.n);
        return add(std::move(s));
    }
    // numElems / alignment stand for the VPUIP::CompressionSchemeAttr (empty = no weights compression)
    ContentAttr relocateWeightsTablePointers(const std::vector<int32_t>& weightsPtr, uint64_t sparsityPtr,
                                             const std::vector<int64_t>& offsets, uint64_t weightsElemBitSize = 0,
                                             const std::vector<int64_t>& numElems = {}, int64_t alignment = 0) const {
        Step s(B200C_X_RELOCATE_WEIGHTS_TABLE);
        if (weightsPtr.size() != offsets.size()) throw Error(B200C_ERR_INVALID, "one weights pointer per cluster offset");
        fill(s.x.a, offsets, &s.x.n);
        fill(s.x.b, std::vector<int64_t>(weightsPtr.begin(), weightsPtr.end()), &s.x.n);
        s.x.i0 = static_cast<int64_t>(sparsityPtr);
        s.x.i1 = static_cast<int64_t>(weightsElemBitSize);
        s.x.f = static_cast<double>(alignment);
        s.aux = numElems;
        return add(std::move(s));
    }
    // ContentAttr::changeShapeAndElemType(newShape, newElemType); q != nullptr: a quantised element type
    ContentAttr changeShapeAndElemType(const std::vector<int64_t>& shape, int dtype, const QuantParams* q = nullptr) const {
        Step s(B200C_X_CHANGE_SHAPE_AND_ELEM_TYPE);
        fill(s.x.b, shape, &s.x.n);
        s.type = q ? NDType({}, dtype, *q) : NDType({}, dtype);
        return add(std::move(s));
    }
    ContentAttr bitPack(int64_t width) const {
        Step s(B200C_X_BIT_PACK);
        s.x.i0 = width;
        return add(std::move(s));
    }
    ContentAttr getSparsityMap() const {
        return add(Step(B200C_X_GET_SPARSITY_MAP));
    }
    // sparsify(compressOutputType, numActualElements): numActualElements may be empty
    ContentAttr sparsify(bool compressOutputType, const std::vector<int64_t>& numActualElements = {}) const {
        Step s(B200C_X_SPARSIFY);
        s.x.i0 = compressOutputType ? 1 : 0;
        s.aux = numActualElements;
        return add(std::move(s));
    }
    ContentAttr swizzleConstant(uint64_t swizzleKey, uint64_t arch) const {
        Step s(B200C_X_SWIZZLE_CONSTANT);
        s.x.i0 = static_cast<int64_t>(swizzleKey);
        s.x.i1 = static_cast<int64_t>(arch);
        return add(std::move(s));
    }

    // Every Sparsify of the list rewritten in place to Sparsify<true, numElems>, so that the attribute's type is the
    // flat compressed one (compressConstWeightsType,
    // src/vpux_compiler/src/dialect/VPUIP/passes/flatten_sparse_weights_types.cpp:41-73)
    ContentAttr withCompressedSparsify(const std::vector<int64_t>& numElems) const {
        ContentAttr r = *this;
        for (Step& s : r._steps) {
            if (s.x.kind == B200C_X_SPARSIFY) {
                s.x.i0 = 1;
                s.aux = numElems;
            }
        }
        return r;
    }

    const NDType& getBaseType() const {
        return _base;
    }
    bool isSplat() const {
        return _splat;
    }
    size_t getNumTransformations() const {
        return _steps.size();
    }
    int getTransformationKind(size_t i) const {
        return _steps[i].x.kind;
    }
    // Two transformations with equal parameters are one uniqued attribute object in the reference, so the two
    // methods below cut the list at the LAST transformation equal to transformation i of this attribute
    // (ContentAttr::stripTransformationsFrom / getLastTransformationsFrom, attributes.td:72-107).
    bool sameTransformation(size_t i, size_t j) const {
        const Step &a = _steps[i], &b = _steps[j];
        const b200c_xform &x = a.x, &y = b.x;
        if (x.kind != y.kind || x.n != y.n || x.f != y.f || x.i0 != y.i0 || x.i1 != y.i1) return false;
        for (int k = 0; k < x.n; ++k)
            if (x.a[k] != y.a[k] || x.b[k] != y.b[k]) return false;
        const QuantParams &p = a.type.quant, &q = b.type.quant;
        return a.type.dtype == b.type.dtype && p.kind == q.kind && p.axis == q.axis && p.expressed == q.expressed &&
               p.qmin == q.qmin && p.qmax == q.qmax && p.scales == q.scales && p.zps == q.zps && a.aux == b.aux;
    }
    // the attribute without transformation i's last equal and everything behind it
    ContentAttr stripTransformationsFrom(size_t i) const {
        ContentAttr r = *this;
        r._steps.erase(r._steps.begin() + static_cast<std::ptrdiff_t>(lastEqual(i)), r._steps.end());
        return r;
    }
    // kinds of the transformations from transformation i's last equal on
    std::vector<int> getLastTransformationsFrom(size_t i) const {
        std::vector<int> kinds;
        for (size_t k = lastEqual(i); k < _steps.size(); ++k) kinds.push_back(_steps[k].x.kind);
        return kinds;
    }

    // ContentAttr::getType(): inferFinalType over the list (pure host code in the library)
    NDType getType() const {
        Marshalled m(*this);
        b200c_type out;
        std::memset(&out, 0, sizeof(out));
        std::vector<double> scales(maxQuantEntries());
        std::vector<int64_t> zps(scales.size());
        out.scales = scales.data();
        out.zps = zps.data();
        out.nq = static_cast<int64_t>(scales.size());
        check(b200c_infer_type(&m.base, m.chain.data(), static_cast<int>(m.chain.size()), &out));
        return NDType::fromC(out);
    }

    // ContentAttr::fold() + Content::copyTo() on the device behind `be`
    Content fold(const Backend& be) const {
        Marshalled m(*this);
        const NDType finalType = getType();
        size_t cap = static_cast<size_t>(finalType.getTotalAllocSize());
        std::vector<uint8_t> out(cap ? cap : 1);
        size_t written = 0;
        check(b200c_fold(be.ctx(), &m.base, _data->data(), _data->size(), _splat ? 1 : 0, /*data_on_device=*/0,
                         m.chain.data(), static_cast<int>(m.chain.size()), out.data(), cap, /*out_on_device=*/0, &written,
                         nullptr, 0));
        out.resize(written);
        return Content(finalType, std::move(out));
    }

    // FuseConstants (src/vpux_compiler/src/dialect/VPUIP/passes/fuse_constants.cpp:82-176,
    // src/vpux_compiler/src/utils/constant_fusion.cpp): parts[k] is the weight table, the weights, the weights sparsity
    // map and the activation window (nullptr = absent).  The reference folds each part and appends its values to a byte
    // vector; here ONE batched call folds the parts into adjacent ranges of the fused buffer on the device and one copy
    // brings the bytes back.  The fused type is f16 when f16 parts hold more than half of the bytes, else ui8.
    static FusedConstant fuse(const Backend& be, const std::vector<const ContentAttr*>& parts) {
        std::vector<const ContentAttr*> present;
        for (const ContentAttr* p : parts)
            if (p != nullptr) present.push_back(p);
        std::vector<Marshalled> descs;
        descs.reserve(present.size());  // the items point into these
        std::vector<size_t> sizes;
        size_t total = 0, f16Bytes = 0;
        for (const ContentAttr* p : present) {
            const NDType t = p->getType();
            const int bits = B200C_DTYPE_BITS(t.dtype);
            const bool known = t.quant.kind != B200C_Q_NONE || t.dtype == B200C_UI8 || t.dtype == B200C_I8 || t.dtype == B200C_F16 ||
                               t.dtype == B200C_SI32 || bits == 1;
            if (!known) throw Error(B200C_ERR_THROW, "Unsupported data type for constant");
            const size_t size = static_cast<size_t>(t.getTotalAllocSize());
            if (t.quant.kind == B200C_Q_NONE && t.dtype == B200C_F16) f16Bytes += size;
            sizes.push_back(size);
            total += size;
            descs.emplace_back(*p);
        }
        struct DeviceBuffer {
            b200c_ctx* ctx;
            void* ptr = nullptr;
            ~DeviceBuffer() {
                if (ptr) b200c_dev_free(ctx, ptr);
            }
        } fused{be.ctx()};
        check(b200c_dev_alloc(be.ctx(), total ? total : 1, &fused.ptr));
        check(b200c_dev_memset(be.ctx(), fused.ptr, 0, total ? total : 1));
        std::vector<b200c_fold_item> items(present.size());
        size_t at = 0;
        for (size_t k = 0; k < present.size(); ++k) {
            b200c_fold_item& it = items[k];
            std::memset(&it, 0, sizeof(it));
            it.base = &descs[k].base;
            it.data = present[k]->_data->data();
            it.nbytes = present[k]->_data->size();
            it.is_splat = present[k]->_splat ? 1 : 0;
            it.n = static_cast<int32_t>(descs[k].chain.size());
            it.chain = descs[k].chain.data();
            it.out = static_cast<uint8_t*>(fused.ptr) + at;
            it.out_cap = sizes[k];
            at += sizes[k];
        }
        if (!items.empty()) {
            check(b200c_fold_batch(be.ctx(), items.data(), static_cast<int>(items.size()), /*data_on_device=*/0, /*out_on_device=*/1, 0));
        }
        FusedConstant r;
        r.data.resize(total);
        if (total) check(b200c_memcpy_d2h(be.ctx(), r.data.data(), fused.ptr, total));
        const size_t es = f16Bytes * 2 > total ? 2 : 1;
        r.type = NDType({1, 1, 1, static_cast<int64_t>(total / es)}, es == 2 ? B200C_F16 : B200C_UI8);
        int64_t off = 0;
        size_t j = 0;
        for (const ContentAttr* p : parts) {
            if (p == nullptr) {
                r.views.emplace_back(-1, -1);
                continue;
            }
            const int64_t n = static_cast<int64_t>(sizes[j++] / es);
            r.views.emplace_back(off, n);
            off += n;
        }
        return r;
    }

    // vpux::countNonSparseElementsPerOC on the folded content
    std::vector<int64_t> countNonSparseElementsPerOC(const Backend& be) const {
        Marshalled m(*this);
        const NDType t = getType();
        std::vector<int64_t> counts(t.shape.empty() ? 0 : static_cast<size_t>(t.shape[0]));
        check(b200c_count_nonsparse_per_oc(be.ctx(), &m.base, _data->data(), _data->size(), _splat ? 1 : 0, 0, m.chain.data(),
                                           static_cast<int>(m.chain.size()), counts.data(), static_cast<int64_t>(counts.size())));
        return counts;
    }

private:
    struct Step {
        b200c_xform x;
        NDType type;               // owns the quantisation arrays x.type points to
        std::vector<int64_t> aux;  // owns x.aux
        explicit Step(int kind) {
            std::memset(&x, 0, sizeof(x));
            x.kind = kind;
        }
    };
    // the C descriptors of an attribute; pointers refer to storage owned by the attribute
    struct Marshalled {
        b200c_type base;
        std::vector<b200c_xform> chain;
        explicit Marshalled(const ContentAttr& a): base(a._base.toC()) {
            for (const Step& s : a._steps) {
                b200c_xform x = s.x;
                if (s.type.dtype != 0 || s.type.quant.kind != B200C_Q_NONE) x.type = s.type.toC();  // element type only
                x.aux = s.aux.empty() ? nullptr : s.aux.data();
                x.naux = static_cast<int64_t>(s.aux.size());
                chain.push_back(x);
            }
        }
    };

    static void fill(int64_t* dst, const std::vector<int64_t>& v, int32_t* n) {
        if (v.size() > B200C_MAX_RANK) throw Error(B200C_ERR_INVALID, "rank above B200C_MAX_RANK");
        for (size_t k = 0; k < v.size(); ++k) dst[k] = v[k];
        *n = static_cast<int32_t>(v.size());
    }
    // room for the per-axis parameters of any type the list can produce (the quantised axis can grow
    // through PadWithZero and Broadcast)
    size_t maxQuantEntries() const {
        int64_t n = 1;
        for (auto d : _base.shape) n = std::max<int64_t>(n, d);
        for (const Step& s : _steps) {
            n = std::max<int64_t>(n, static_cast<int64_t>(s.type.quant.scales.size()));
            int64_t grow = std::max<int64_t>(0, s.x.i1);
            for (int k = 0; k < B200C_MAX_RANK; ++k) grow = std::max(grow, std::max(s.x.a[k], s.x.b[k]));
            n += grow;
        }
        return static_cast<size_t>(std::min<int64_t>(n, int64_t(1) << 24) + 64);
    }
    size_t lastEqual(size_t i) const {
        if (i >= _steps.size()) throw Error(B200C_ERR_INVALID, "transformation index out of range");
        size_t last = i;
        for (size_t k = i + 1; k < _steps.size(); ++k)
            if (sameTransformation(i, k)) last = k;
        return last;
    }
    // ContentAttr::addTransformation: insert at getInsertionPosition, then re-check the final type
    ContentAttr add(Step s) const {
        std::vector<int32_t> kinds;
        for (const Step& t : _steps) kinds.push_back(t.x.kind);
        int pos = 0;
        check(b200c_insert_position(kinds.data(), static_cast<int>(kinds.size()), s.x.kind, &pos));
        ContentAttr r = *this;
        r._steps.insert(r._steps.begin() + pos, std::move(s));
        (void)r.getType();  // throws what inferOutputType would
        return r;
    }

    NDType _base;
    std::shared_ptr<std::vector<uint8_t>> _data;
    bool _splat = false;
    std::vector<Step> _steps;
};

// vpux::Const::DeclareOp (src/vpux_compiler/src/dialect/const/ops.cpp): a result type plus a ContentAttr.
// The constructor runs the op's verifier (ops.cpp:164-193): shape (skipped for a swizzled result type, whose
// content may have been flattened), element type (a mismatch is accepted when the result type is quantised or
// the attribute's element type is an integer) and DimsOrder must agree with the attribute's inferred type.
class DeclareOp {
public:
    DeclareOp(NDType resultType, ContentAttr attr, bool swizzled = false)
            : _type(std::move(resultType)), _attr(std::move(attr)), _swizzled(swizzled) {
        verify();
    }
    const ContentAttr& getContentAttr() const {
        return _attr;
    }
    const NDType& getType() const {
        return _type;
    }
    bool isSwizzled() const {
        return _swizzled;
    }
    // DeclareOp::getContent(): fold of the attribute
    Content getContent(const Backend& be) const {
        return _attr.fold(be);
    }
    // DeclareOp::getBinarySize (ops.cpp:114-118)
    size_t getBinarySize() const {
        return static_cast<size_t>(_attr.getType().getTotalAllocSize());
    }
    // DeclareOp::serialize (ops.cpp:97-108): the copyTo bytes in a zero-initialised buffer of the folded type's size
    // are appended to the section
    void serialize(const Backend& be, std::vector<uint8_t>& section) const {
        const Content cnt = getContent(be);
        const size_t size = static_cast<size_t>(cnt.getType().getTotalAllocSize());
        const size_t at = section.size();
        section.resize(at + size, 0);
        cnt.copyTo(section.data() + at, size);
    }
    void verify() const {
        const NDType attrType = _attr.getType();
        if (!_swizzled && attrType.shape != _type.shape) {
            throw Error(B200C_ERR_THROW, "'Const.Declare' has mismatch in value shape and result shape");
        }
        const bool sameElem = attrType.dtype == _type.dtype && attrType.quant.kind == _type.quant.kind &&
                              attrType.quant.scales == _type.quant.scales && attrType.quant.zps == _type.quant.zps &&
                              attrType.quant.axis == _type.quant.axis && attrType.quant.qmin == _type.quant.qmin &&
                              attrType.quant.qmax == _type.quant.qmax;
        if (!sameElem) {
            const int cls = B200C_DTYPE_CLASS(attrType.dtype);
            const bool attrIsInteger = attrType.quant.kind == B200C_Q_NONE &&
                                       (cls == B200C_CLS_INT || cls == B200C_CLS_SINT || cls == B200C_CLS_UINT);
            if (_type.quant.kind == B200C_Q_NONE && !attrIsInteger) {
                throw Error(B200C_ERR_THROW, "'Const.Declare' has mismatch in value element type and result element type");
            }
        }
        if (!(attrType.order == _type.order)) {
            throw Error(B200C_ERR_THROW, "'Const.Declare' has mismatch in value DimsOrder and result DimsOrder");
        }
    }

private:
    NDType _type;
    ContentAttr _attr;
    bool _swizzled;
};

// One op of ConstantFoldingPass::safeRunOnFunc
// (src/vpux_compiler/src/dialect/const/passes/constant_folding.cpp:27-77): the folded bytes become the base content
// of a new DeclareOp with the same result type.  A sub-byte element type (more than 1, fewer than 8 bits) cannot be
// the storage of a dense attribute: its packed bytes are kept as [1,1,1,N] ui8 plus ChangeShapeAndElemType back to
// the op's shape and element type.  A quantised result is stored under its normalised storage integer.
inline DeclareOp foldConstant(const Backend& be, const DeclareOp& op) {
    const Content content = op.getContent(be);
    const NDType& ct = content.getType();
    const size_t size = static_cast<size_t>(ct.getTotalAllocSize());
    std::vector<uint8_t> buf(size, 0);
    content.copyTo(buf.data(), size);
    const int bits = B200C_DTYPE_BITS(ct.dtype);
    if (bits > 1 && bits < 8) {
        NDType base({1, 1, 1, static_cast<int64_t>(size)}, B200C_UI8, ct.order);
        const NDType& orig = op.getType();
        ContentAttr a = ContentAttr::get(buf.data(), size, base)
                                .changeShapeAndElemType(orig.shape, orig.dtype, orig.quant.kind != B200C_Q_NONE ? &orig.quant : nullptr);
        return DeclareOp(orig, std::move(a), op.isSwizzled());
    }
    NDType base(ct.shape, ct.dtype, ct.order);  // quantisation parameters dropped: the storage integer type
    return DeclareOp(op.getType(), ContentAttr::get(buf.data(), size, base), op.isSwizzled());
}

// detectSplatElementWise, run by the reference when it wraps a dense resource
// (src/vpux_compiler/src/dialect/const/attributes/content.cpp:103-137): true when all elements are equal
inline bool detectSplat(const Backend& be, const void* data, size_t nbytes, int elemBytes) {
    int flag = 0;
    check(b200c_detect_splat(be.ctx(), data, nbytes, elemBytes, /*data_on_device=*/0, &flag));
    return flag != 0;
}

// vpux::BitCompactorCodec::compress (src/vpux_compiler/src/utils/bit_compactor_codec.cpp:15-42):
// returns false (mlir::failure) when the stream would not be smaller than the input
inline bool compress(const Backend& be, const std::vector<uint8_t>& data, std::vector<uint8_t>* stream) {
    size_t bound = 0, n = 0;
    check(b200c_btc_bound(data.size(), &bound));
    stream->resize(bound);
    const int rc = b200c_btc_compress(be.ctx(), data.data(), data.size(), 0, stream->data(), bound, 0, &n);
    check(rc);
    if (rc == B200C_NOT_SMALLER) {
        stream->clear();
        return false;
    }
    stream->resize(n);
    return true;
}

inline std::vector<uint8_t> decompress(const Backend& be, const std::vector<uint8_t>& stream, size_t originalSize) {
    std::vector<uint8_t> out(originalSize ? originalSize : 1);
    size_t n = 0;
    check(b200c_btc_decompress(be.ctx(), stream.data(), stream.size(), 0, out.data(), originalSize, 0, &n));
    out.resize(n);
    return out;
}

inline FusedConstant fuseConstants(const Backend& be, const ContentAttr* weightTable, const ContentAttr* weights,
                                   const ContentAttr* weightsSparsityMap, const ContentAttr* activationWindow) {
    return ContentAttr::fuse(be, {weightTable, weights, weightsSparsityMap, activationWindow});
}

// The constants section of a blob: every op's bytes (DeclareOp::serialize) one after the other, each start aligned
// to `align` bytes and the gap zero-filled -- 8 for the graph-schema writer (serializeBinaryData,
// src/vpux_compiler/src/dialect/VPUIP/graph-schema/export.cpp:465-479), 1 for the ELF writer (ops.cpp:97-108).
// offsets receives where every constant starts.
inline std::vector<uint8_t> writeSection(const Backend& be, const std::vector<DeclareOp>& ops, size_t align, std::vector<size_t>* offsets) {
    std::vector<uint8_t> section;
    if (offsets) offsets->clear();
    for (const DeclareOp& op : ops) {
        if (offsets) offsets->push_back(section.size());
        op.serialize(be, section);
        if (align > 1) section.resize((section.size() + align - 1) / align * align, 0);
    }
    return section;
}

// The chain builders: the callers of the ContentAttr API that assemble the transformation lists the hot path folds.
// Each function restates one call site of the reference compiler on the ContentAttr mirror above.
namespace chains {

constexpr int64_t VPU_WEIGHT_SET_BYTE_ALIGNMENT = 16;  // nce_invariant.hpp:39

// getAlignedConstWeights (src/vpux_compiler/src/dialect/VPU/utils/const_utils.cpp:101-119): depthwise weights
// flattened to flatShape and padded along dim 1
inline ContentAttr alignDepthwiseWeights(const ContentAttr& weights, const std::vector<int64_t>& flatShape, int64_t padding) {
    return weights.reorder(DimsOrder::NCHW())
            .reshape(flatShape)
            .padWithZero({0, 0, 0, 0}, {0, padding, 0, 0})
            .reorder(DimsOrder::NHWC());
}

// alignConvWeightsTensor (const_utils.cpp:246-283): [OC, IC, KY, KX] whose IC*KY*KX is not a multiple of the
// alignment becomes [OC, 1, 1, aligned]; returned unchanged when no padding is needed
inline ContentAttr alignConvolutionWeights(const ContentAttr& weights, int64_t alignment = VPU_WEIGHT_SET_BYTE_ALIGNMENT,
                                           bool isCMajorConv = false) {
    const std::vector<int64_t> shape = weights.getType().shape;
    if (shape.size() != 4 || alignment <= 0) throw Error(B200C_ERR_INVALID, "alignConvolutionWeights: 4D weights and a positive alignment");
    const int64_t row = shape[1] * shape[2] * shape[3];
    const int64_t remainder = row % alignment;
    if (remainder == 0) return weights;
    const std::vector<int64_t> flat{shape[0], 1, 1, row};
    ContentAttr a = isCMajorConv ? weights.reorder(DimsOrder::NCHW()).reshape(flat) : weights.reshape(flat);
    a = a.padWithZero({0, 0, 0, 0}, {0, 0, 0, alignment - remainder});
    return isCMajorConv ? a.reorder(DimsOrder::NHWC()) : a;
}

// ConvertWeightsToU8 ConstRewriter (src/vpux_compiler/src/dialect/IE/passes/convert_weights_to_u8.cpp:85-101):
// signed quantised weights re-based to unsigned; newQuant is the u8 type with the shifted zero points
inline ContentAttr weightsToU8(const ContentAttr& weights, const QuantParams& newQuant) {
    const NDType t = weights.getType();
    if (t.quant.kind == B200C_Q_NONE) throw Error(B200C_ERR_INVALID, "weightsToU8: the constant is not quantised");
    return weights.quantCast()
            .convertElemType(B200C_I32)  // signless, as the reference's getInt32Type
            .add(static_cast<double>(-t.quant.qmin))
            .convertElemType(B200C_UI8)
            .quantCast(newQuant, B200C_UI8);
}

struct SparseWeights {
    ContentAttr values;           // ...Sparsify<false>
    ContentAttr map;              // ...GetSparsityMap
    std::vector<int64_t> counts;  // countNonSparseElementsPerOC, for the compression scheme
};

// SparsifyWeightsPass (src/vpux_compiler/src/dialect/VPU/transforms/passes/sparsify_weights.cpp:108-164): the
// original list is folded first and its bytes become the base of a fresh attribute (later passes do not fold it
// again); a quantised result keeps its type through quantCast
inline SparseWeights sparsifyWeights(const Backend& be, const ContentAttr& weights) {
    const Content content = weights.fold(be);
    const NDType& folded = content.getType();
    std::vector<int64_t> counts = weights.countNonSparseElementsPerOC(be);
    const size_t size = static_cast<size_t>(folded.getTotalAllocSize());
    std::vector<uint8_t> buf(size, 0);
    content.copyTo(buf.data(), size);
    ContentAttr fresh = ContentAttr::get(buf.data(), size, NDType(folded.shape, folded.dtype, folded.order));
    if (folded.quant.kind != B200C_Q_NONE) fresh = fresh.quantCast(folded.quant, folded.dtype);
    return SparseWeights{fresh.sparsify(false), fresh.getSparsityMap(), std::move(counts)};
}

// compressConstWeightsType (flatten_sparse_weights_types.cpp:41-73); an attribute without Sparsify comes back as it is
inline ContentAttr flattenSparseWeights(const ContentAttr& attr, const std::vector<int64_t>& numElems) {
    return attr.withCompressedSparsify(numElems);
}

// createFilter (src/vpux_compiler/src/dialect/VPU/transforms/passes/lower_sparsity_ops.cpp:209-250): ones on the
// diagonal of an [OC, IC, 1, 1] f32 constant -> (ui8 + quantCast | f16) -> reorder -> Sparsify<false>, with its
// sparsity map and counts.  quant != nullptr: a quantised ui8 filter; otherwise dtype is B200C_F16 or B200C_F32.
inline SparseWeights sparseIdentityFilter(const Backend& be, int64_t OC, int64_t IC, int dtype, const QuantParams* quant = nullptr,
                                          const DimsOrder& order = DimsOrder::OYXI()) {
    std::vector<float> content(static_cast<size_t>(OC * IC), 0.0f);
    for (int64_t oc = 0; oc < OC; ++oc) {
        if (oc * IC + oc < OC * IC) content[static_cast<size_t>(oc * IC + oc)] = 1.0f;
    }
    ContentAttr attr = ContentAttr::get(content, NDType({OC, IC, 1, 1}, B200C_F32));
    if (quant != nullptr) {
        attr = attr.convertElemType(B200C_UI8).quantCast(*quant, B200C_UI8);
    } else if (dtype == B200C_F16) {
        attr = attr.convertElemType(B200C_F16);
    }
    if (!(order == DimsOrder::identity(4))) attr = attr.reorder(order);
    return SparseWeights{attr.sparsify(false), attr.getSparsityMap(), attr.countNonSparseElementsPerOC(be)};
}

// generateDefaultWeightsAttr (src/vpux_translate_utils/src/hwtest/hwtest_utils.cpp:184-197): reorder(OYXI) ->
// quantCast(the type, under the constant's own storage) -> bitPack(4) when the type's storage has 4 bits
inline ContentAttr hwtestDefaultWeights(const ContentAttr& weights, const QuantParams* quant = nullptr, int quantStorage = 0) {
    ContentAttr a = weights.reorder(DimsOrder::OYXI());
    if (quant != nullptr) {
        a = a.quantCast(*quant, a.getType().dtype);
        if (B200C_DTYPE_BITS(quantStorage) == 4) a = a.bitPack(4);
    }
    return a;
}

// Swizzling::attachSwizzleTransformation (src/vpux_compiler/src/dialect/VPUIP/passes/swizzling.cpp:469-500): a
// constant shared by several NCE tasks gets the transformation once
inline ContentAttr attachSwizzle(const ContentAttr& attr, uint64_t swizzleKey = 5, uint64_t arch = 3) {
    for (size_t i = 0; i < attr.getNumTransformations(); ++i) {
        if (attr.getTransformationKind(i) == B200C_X_SWIZZLE_CONSTANT) return attr;
    }
    return attr.swizzleConstant(swizzleKey, arch);
}

}  // namespace chains

}  // namespace Const
}  // namespace b200

#endif /* B200CONST_HPP_ */
