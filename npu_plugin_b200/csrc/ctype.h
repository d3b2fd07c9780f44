// Host-side model of a constant's type and of one transformation, shared by the type-inference
// code and the fold planner.  Mirrors what vpux::NDTypeInterface exposes for ranked tensors
// (src/vpux_compiler/src/core/type_interfaces.cpp) without any MLIR dependency.
#pragma once

#include "../../include/b200const.h"

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>
#include <utility>
#include <initializer_list>

namespace b200c {

// An error the reference would raise with VPUX_THROW; carried to the C ABI as B200C_ERR_THROW.
struct RefThrow : std::runtime_error {
    using std::runtime_error::runtime_error;
};
// Valid in the reference but not built here; B200C_ERR_UNSUPPORTED.
struct NotBuilt : std::runtime_error {
    using std::runtime_error::runtime_error;
};
// Malformed descriptor; B200C_ERR_INVALID.
struct BadArg : std::runtime_error {
    using std::runtime_error::runtime_error;
};
struct CudaFail : std::runtime_error {
    using std::runtime_error::runtime_error;
};
struct NoMem : std::runtime_error {
    using std::runtime_error::runtime_error;
};
struct Capacity : std::runtime_error {
    using std::runtime_error::runtime_error;
};

[[noreturn]] inline void refThrow(const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    throw RefThrow(buf);
}

inline int dtBits(int dt) {
    return B200C_DTYPE_BITS(dt);
}
inline int dtClass(int dt) {
    return B200C_DTYPE_CLASS(dt);
}
inline bool dtIsFloat(int dt) {
    return dtClass(dt) == B200C_CLS_FLOAT || dtClass(dt) == B200C_CLS_BFLOAT;
}
inline bool dtIsInt(int dt) {
    const int c = dtClass(dt);
    return c == B200C_CLS_INT || c == B200C_CLS_SINT || c == B200C_CLS_UINT;
}
inline bool dtValid(int dt) {
    const int b = dtBits(dt);
    switch (dtClass(dt)) {
    case B200C_CLS_FLOAT:
        return b == 16 || b == 32 || b == 64;
    case B200C_CLS_BFLOAT:
        return b == 16;
    case B200C_CLS_INT:
    case B200C_CLS_SINT:
    case B200C_CLS_UINT:
        return b == 1 || b == 4 || b == 8 || b == 16 || b == 32 || b == 64;
    default:
        return false;
    }
}
inline int64_t roundUp(int64_t v, int64_t a) {
    return (v + a - 1) / a * a;
}

// Fixed-capacity vector for shapes, orders and transformation arguments (at most B200C_MAX_RANK
// entries): same interface as the part of std::vector used here, no heap allocation.
template <class T>
class SmallVec {
public:
    SmallVec() = default;
    SmallVec(std::initializer_list<T> l) {
        assign(l.begin(), l.end());
    }
    explicit SmallVec(size_t n, T val = T()) {
        assign(n, val);
    }
    template <class It, class = decltype(*std::declval<It>())>
    SmallVec(It a, It b) {
        assign(a, b);
    }
    SmallVec(const std::vector<T>& v) {
        assign(v.begin(), v.end());
    }
    operator std::vector<T>() const {
        return std::vector<T>(begin(), end());
    }
    size_t size() const {
        return static_cast<size_t>(_n);
    }
    bool empty() const {
        return _n == 0;
    }
    T& operator[](size_t i) {
        return _v[i];
    }
    const T& operator[](size_t i) const {
        return _v[i];
    }
    T* begin() {
        return _v;
    }
    T* end() {
        return _v + _n;
    }
    const T* begin() const {
        return _v;
    }
    const T* end() const {
        return _v + _n;
    }
    const T* data() const {
        return _v;
    }
    T& back() {
        return _v[_n - 1];
    }
    void clear() {
        _n = 0;
    }
    void push_back(const T& x) {
        if (_n >= kCap) throw BadArg("more than B200C_MAX_RANK entries");
        _v[_n++] = x;
    }
    void resize(size_t n, T val = T()) {
        if (n > static_cast<size_t>(kCap)) throw BadArg("more than B200C_MAX_RANK entries");
        for (size_t i = static_cast<size_t>(_n); i < n; ++i) _v[i] = val;
        _n = static_cast<int>(n);
    }
    void assign(size_t n, T val) {
        _n = 0;
        resize(n, val);
    }
    template <class It, class = decltype(*std::declval<It>())>
    void assign(It a, It b) {
        _n = 0;
        for (; a != b; ++a) push_back(static_cast<T>(*a));
    }
    bool operator==(const SmallVec& o) const {
        if (_n != o._n) return false;
        for (int i = 0; i < _n; ++i)
            if (!(_v[i] == o._v[i])) return false;
        return true;
    }
    bool operator!=(const SmallVec& o) const {
        return !(*this == o);
    }

private:
    static constexpr int kCap = B200C_MAX_RANK;
    T _v[kCap] = {};
    int _n = 0;
};
using Dims = SmallVec<int64_t>;

// Quantisation parameters.  The scale / zero-point arrays are views: they either borrow the
// caller's descriptor arrays (valid for the duration of one C ABI call) or point into storage
// owned through the shared pointers, so copying a type never copies the tables.
struct QuantInfo {
    int kind = B200C_Q_NONE;
    int axis = 0;
    int expressed = 0;
    int64_t qmin = 0, qmax = 0;
    const double* scales = nullptr;
    const int64_t* zps = nullptr;
    size_t n = 0;
    std::shared_ptr<std::vector<double>> ownScales;
    std::shared_ptr<std::vector<int64_t>> ownZps;

    void own(std::vector<double> s, std::vector<int64_t> z) {
        ownScales = std::make_shared<std::vector<double>>(std::move(s));
        ownZps = std::make_shared<std::vector<int64_t>>(std::move(z));
        scales = ownScales->data();
        zps = ownZps->data();
        n = ownScales->size();
    }
    bool zpsAllEqual() const {
        for (size_t i = 1; i < n; ++i)
            if (zps[i] != zps[0]) return false;
        return true;
    }
};

struct TensorType {
    int dtype = 0;  // for quantised types: the normalised storage integer
    Dims shape;
    SmallVec<int> order;  // order[k] = logical dim at memory position k, outermost first
    QuantInfo q;

    int rank() const {
        return static_cast<int>(shape.size());
    }
    bool quantized() const {
        return q.kind != B200C_Q_NONE;
    }
    int64_t count() const {
        int64_t n = 1;
        for (auto d : shape) n *= d;
        return n;
    }
    int bits() const {
        return dtBits(dtype);
    }
    bool identityOrder() const {
        for (int k = 0; k < rank(); ++k)
            if (order[k] != k) return false;
        return true;
    }
    void setIdentityOrder() {
        order.resize(shape.size());
        for (size_t k = 0; k < shape.size(); ++k) order[k] = static_cast<int>(k);
    }
    Dims memOrder(const Dims& logical) const {
        Dims m(logical.size());
        for (size_t k = 0; k < logical.size(); ++k) m[k] = logical[order[k]];
        return m;
    }
    Dims memShape() const {
        return memOrder(shape);
    }
    int memPosOf(int logicalDim) const {
        for (int k = 0; k < rank(); ++k)
            if (order[k] == logicalDim) return k;
        throw BadArg("logical dim not in order");
    }
    // getTotalAllocSize: bits x count rounded up to bytes (rank 0 holds one element)
    int64_t allocBytes() const {
        return (static_cast<int64_t>(bits()) * (rank() == 0 ? 1 : count()) + 7) / 8;
    }
};

struct Transformation {
    int kind = 0;
    Dims a, b;
    double f = 0;
    int64_t i0 = 0, i1 = 0;
    bool hasType = false;
    TensorType type;  // element type only (rank 0)
    bool hasAux = false;
    std::vector<int64_t> aux;
    void* side0 = nullptr;
    void* side1 = nullptr;
};

enum class PositionReq { None, PreferredLast, Last };

// descriptor <-> model
TensorType typeFromC(const b200c_type& c, bool elemOnly = false);
void typeToC(const TensorType& t, b200c_type* c);
Transformation xformFromC(const b200c_xform& c);

// inferOutputType of one transformation / of a whole list (ContentAttr::inferFinalType)
TensorType inferOne(const Transformation& x, const TensorType& in);
TensorType inferChain(const TensorType& base, const std::vector<Transformation>& chain);

PositionReq positionOf(int kind);
bool acceptsSubByteStorage(int kind);
int insertPosition(const std::vector<int>& kinds, int newKind);

// helpers the planner also needs
TensorType withShape(const TensorType& in, const Dims& shape);
TensorType withShapeAndElem(const TensorType& in, const Dims& shape, int dtype, const QuantInfo& q);
int64_t sparsifyValue(const TensorType& t);

constexpr int64_t kSwizzleSizeAlign = 512;  // SWIZZLING_SIZE_ALIGNMENT_VPUX37XX
constexpr int kArchVPUX37XX = 3;            // VPU::ArchKind::VPUX37XX
constexpr int64_t kWeightSetAlign = 16;     // VPU_WEIGHT_SET_BYTE_ALIGNMENT (nce_invariant.hpp:39)

}  // namespace b200c
