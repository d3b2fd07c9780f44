// TEST INFRASTRUCTURE -- CPU oracle for the Const-dialect folding path.
//
// A plain C++17 restatement (no MLIR, no OpenVINO) of what the reference
// compiler does when it folds a constant: vpux::Const::Content, the
// transformation attributes' inferOutputType/transform pairs, the fold loop and
// Content::copyTo.  It exists to check the CUDA library and to be timed as the
// CPU baseline; nothing in the product links or calls it.
//
// Reference paths are relative to openvinotoolkit/npu_plugin; CA/ abbreviates
// src/vpux_compiler/src/dialect/const/attributes/, CU/ abbreviates
// src/vpux_compiler/src/dialect/const/utils/.  Parity pins: the known-answer
// vectors of tests/unit/vpux_compiler/dialect/const/content_tests.cpp and the
// lit files under tests/lit/NPU/dialect/const/passes/ (see tests/test_oracle_golden.py).
//
// Loops the reference marks LoopExecPolicy::Parallel run under OpenMP; loops
// that are serial in the reference (BitPack, GetSparsityMap, Sparsify
// compaction, swizzle, sub-byte packing) stay serial, and every materialising
// transformation allocates a fresh buffer, as ContentAttr::fold does.
//
// The descriptor structs of include/b200const.h are reused so that tests can
// hand identical arguments to both sides; no product code is involved.

#include "../include/b200const.h"

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <functional>
#include <limits>
#include <memory>
#include <numeric>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace orc {

// ---------------------------------------------------------------------------
// errors (VPUX_THROW, src/vpux_utils/include/vpux/utils/core/error.hpp:35-43)
// ---------------------------------------------------------------------------
struct Thrown : std::runtime_error {
    using std::runtime_error::runtime_error;
};
struct Unsupported : std::runtime_error {
    using std::runtime_error::runtime_error;
};

[[noreturn]] static void throwf(const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    throw Thrown(buf);
}

// Parallel loop standing in for loop_1d(LoopExecPolicy::Parallel, ...)
// (src/vpux_utils/src/ov/loop.cpp:23-73).  Exceptions are carried out of the region.
template <class F>
static void parallel_for(int64_t n, F&& body) {
    std::string err;
    bool failed = false;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        if (failed) {
            continue;
        }
        try {
            body(i);
        } catch (const std::exception& e) {
#pragma omp critical
            {
                if (!failed) {
                    failed = true;
                    err = e.what();
                }
            }
        }
    }
    if (failed) {
        throw Thrown(err);
    }
}

// ---------------------------------------------------------------------------
// half / bfloat16 (ov::float16 / ov::bfloat16: IEEE binary16 and truncated
// binary32 with round-to-nearest-even from float)
// ---------------------------------------------------------------------------
static inline uint32_t f2u(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    return u;
}
static inline float u2f(uint32_t u) {
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

struct f16 {
    uint16_t bits = 0;
    f16() = default;
    explicit f16(float f) {
        const uint32_t x = f2u(f);
        const uint32_t sign = (x >> 16) & 0x8000u;
        const uint32_t absx = x & 0x7FFFFFFFu;
        uint32_t out;
        if (absx >= 0x7F800000u) {  // inf / nan
            out = 0x7C00u | ((absx > 0x7F800000u) ? (0x0200u | ((absx >> 13) & 0x03FFu)) : 0u);
        } else if (absx >= 0x477FF000u) {  // rounds to >= 65520 -> inf
            out = 0x7C00u;
        } else if (absx >= 0x38800000u) {  // normal half
            const uint32_t mant = absx & 0x007FFFFFu;
            const uint32_t exp = (absx >> 23) - 112u;
            uint32_t h = (exp << 10) | (mant >> 13);
            const uint32_t rem = mant & 0x1FFFu;
            if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) {
                ++h;
            }
            out = h;
        } else if (absx >= 0x33000000u) {  // subnormal half
            const uint32_t exp = absx >> 23;
            const uint32_t mant = (absx & 0x007FFFFFu) | 0x00800000u;
            const uint32_t shift = 126u - exp;  // 14..24
            uint32_t h = mant >> shift;
            const uint32_t rem = mant & ((1u << shift) - 1u);
            const uint32_t half = 1u << (shift - 1u);
            if (rem > half || (rem == half && (h & 1u))) {
                ++h;
            }
            out = h;
        } else {
            out = 0;
        }
        bits = static_cast<uint16_t>(sign | out);
    }
    explicit operator float() const {
        const uint32_t sign = (bits & 0x8000u) << 16;
        const uint32_t exp = (bits >> 10) & 0x1Fu;
        const uint32_t mant = bits & 0x3FFu;
        if (exp == 0) {
            if (mant == 0) {
                return u2f(sign);
            }
            // subnormal: value = mant * 2^-24
            const float v = static_cast<float>(mant) * 5.9604644775390625e-08f;
            return (sign != 0) ? -v : v;
        }
        if (exp == 31) {
            return u2f(sign | 0x7F800000u | (mant << 13));
        }
        return u2f(sign | ((exp + 112u) << 23) | (mant << 13));
    }
};

struct bf16 {
    uint16_t bits = 0;
    bf16() = default;
    explicit bf16(float f) {
        uint32_t x = f2u(f);
        if ((x & 0x7FFFFFFFu) > 0x7F800000u) {
            bits = static_cast<uint16_t>((x >> 16) | 0x0040u);
        } else {
            x += 0x7FFFu + ((x >> 16) & 1u);
            bits = static_cast<uint16_t>(x >> 16);
        }
    }
    explicit operator float() const {
        return u2f(static_cast<uint32_t>(bits) << 16);
    }
};

// ov::float16 compares through float (so -0 == +0, NaN != NaN).
static inline bool operator==(f16 a, f16 b) {
    return static_cast<float>(a) == static_cast<float>(b);
}
static inline bool operator!=(f16 a, f16 b) {
    return !(a == b);
}
static inline bool operator==(bf16 a, bf16 b) {
    return static_cast<float>(a) == static_cast<float>(b);
}
static inline bool operator!=(bf16 a, bf16 b) {
    return !(a == b);
}

// ---------------------------------------------------------------------------
// checked_cast (src/vpux_utils/include/vpux/utils/core/checked_cast.hpp:43-146,
// src/vpux_utils/include/vpux/utils/IE/float16.hpp:25-50)
// ---------------------------------------------------------------------------
template <class T>
struct is_half : std::false_type {};
template <>
struct is_half<f16> : std::true_type {};
template <>
struct is_half<bf16> : std::true_type {};

template <class T>
static const char* tname() {
    if (std::is_same<T, int8_t>::value) return "int8_t";
    if (std::is_same<T, uint8_t>::value) return "uint8_t";
    if (std::is_same<T, int16_t>::value) return "int16_t";
    if (std::is_same<T, uint16_t>::value) return "uint16_t";
    if (std::is_same<T, int32_t>::value) return "int32_t";
    if (std::is_same<T, uint32_t>::value) return "uint32_t";
    if (std::is_same<T, int64_t>::value) return "int64_t";
    if (std::is_same<T, uint64_t>::value) return "uint64_t";
    if (std::is_same<T, float>::value) return "float";
    if (std::is_same<T, double>::value) return "double";
    return "?";
}

template <class Out, class In>
static Out ccast(In v) {
    if constexpr (std::is_same<Out, In>::value) {
        return v;
    } else if constexpr (is_half<In>::value) {
        // half/bfloat source: through float (float16.hpp:25-41)
        if constexpr (is_half<Out>::value) {
            return Out(static_cast<float>(v));
        } else {
            return ccast<Out>(static_cast<float>(v));
        }
    } else if constexpr (is_half<Out>::value) {
        return Out(ccast<float>(v));  // float16.hpp:43-50
    } else if constexpr (std::is_integral<In>::value && std::is_integral<Out>::value) {
        if constexpr (std::is_signed<In>::value && std::is_signed<Out>::value) {
            if (static_cast<int64_t>(v) < static_cast<int64_t>(std::numeric_limits<Out>::lowest()) ||
                static_cast<int64_t>(v) > static_cast<int64_t>(std::numeric_limits<Out>::max())) {
                throwf("Can not safely cast %lld from %s to %s", (long long)v, tname<In>(), tname<Out>());
            }
        } else if constexpr (!std::is_signed<In>::value && !std::is_signed<Out>::value) {
            if (static_cast<uint64_t>(v) > static_cast<uint64_t>(std::numeric_limits<Out>::max())) {
                throwf("Can not safely cast %llu from %s to %s", (unsigned long long)v, tname<In>(), tname<Out>());
            }
        } else if constexpr (!std::is_signed<In>::value && std::is_signed<Out>::value) {
            if (static_cast<uint64_t>(v) > static_cast<uint64_t>(std::numeric_limits<Out>::max())) {
                throwf("Can not safely cast %llu from %s to %s", (unsigned long long)v, tname<In>(), tname<Out>());
            }
        } else {  // signed -> unsigned
            if (v < 0 || static_cast<uint64_t>(v) > static_cast<uint64_t>(std::numeric_limits<Out>::max())) {
                throwf("Can not safely cast %lld from %s to %s", (long long)v, tname<In>(), tname<Out>());
            }
        }
        return static_cast<Out>(v);
    } else if constexpr (std::is_floating_point<In>::value && std::is_integral<Out>::value) {
        // checked_cast.hpp:106-117: range test in the source type, then C truncation
        if (!(v <= static_cast<In>(std::numeric_limits<Out>::max())) ||
            !(v >= static_cast<In>(std::numeric_limits<Out>::lowest()))) {
            throwf("Can not safely cast %g from %s to %s", (double)v, tname<In>(), tname<Out>());
        }
        return static_cast<Out>(v);
    } else if constexpr (std::is_integral<In>::value && std::is_floating_point<Out>::value) {
        // checked_cast.hpp:119-133: must round-trip
        if (static_cast<In>(static_cast<Out>(v)) != v) {
            throwf("Can not safely cast %lld from %s to %s", (long long)v, tname<In>(), tname<Out>());
        }
        return static_cast<Out>(v);
    } else if constexpr (std::is_same<In, double>::value && std::is_same<Out, float>::value) {
        if (static_cast<double>(static_cast<float>(v)) != v) {  // checked_cast.hpp:135-141
            throwf("Can not safely cast %g from double to float", v);
        }
        return static_cast<float>(v);
    } else {
        return static_cast<Out>(v);  // float -> double
    }
}

// ---------------------------------------------------------------------------
// types
// ---------------------------------------------------------------------------
static inline int dbits(int dt) {
    return B200C_DTYPE_BITS(dt);
}
static inline int dcls(int dt) {
    return B200C_DTYPE_CLASS(dt);
}
static inline bool isFloatDt(int dt) {
    return dcls(dt) == B200C_CLS_FLOAT || dcls(dt) == B200C_CLS_BFLOAT;
}
static inline bool isIntDt(int dt) {
    const int c = dcls(dt);
    return c == B200C_CLS_INT || c == B200C_CLS_SINT || c == B200C_CLS_UINT;
}
static inline int64_t alignUp(int64_t v, int64_t a) {
    return (v + a - 1) / a * a;
}

struct Quant {
    int kind = B200C_Q_NONE;
    int axis = 0;
    int expressed = 0;
    int64_t qmin = 0, qmax = 0;
    std::vector<double> scales;
    std::vector<int64_t> zps;
    bool operator==(const Quant& o) const {
        return kind == o.kind && (kind == B200C_Q_NONE || (axis == o.axis && expressed == o.expressed &&
                                                           qmin == o.qmin && qmax == o.qmax && scales == o.scales &&
                                                           zps == o.zps));
    }
};

struct Type {
    int dtype = 0;
    std::vector<int64_t> shape;
    std::vector<int> order;  // order[k] = logical dim at memory position k (0 = outermost)
    Quant q;

    int rank() const {
        return static_cast<int>(shape.size());
    }
    int64_t numElements() const {
        int64_t n = 1;
        for (auto d : shape) n *= d;
        return n;
    }
    int elemBits() const {
        return dbits(dtype);
    }
    bool identityOrder() const {
        for (int k = 0; k < rank(); ++k)
            if (order[k] != k) return false;
        return true;
    }
    // DimsOrder::toMemoryOrder (src/vpux_compiler/src/core/attributes/dims_order.cpp)
    std::vector<int64_t> toMem(const std::vector<int64_t>& logical) const {
        std::vector<int64_t> m(logical.size());
        for (size_t k = 0; k < logical.size(); ++k) m[k] = logical[order[k]];
        return m;
    }
    std::vector<int64_t> memShape() const {
        return toMem(shape);
    }
    // DimsOrder::dimPos: memory position of a logical dim
    int dimPos(int d) const {
        for (int k = 0; k < rank(); ++k)
            if (order[k] == d) return k;
        throwf("Dim %d is not in the order", d);
    }
    // NDTypeInterface::getTotalAllocSize (src/vpux_compiler/src/core/type_interfaces.cpp:148-162):
    // element bits x element count, rounded up to whole bytes; rank 0 -> one element
    int64_t totalAllocSize() const {
        const int64_t bitsTotal = static_cast<int64_t>(elemBits()) * (rank() == 0 ? 1 : numElements());
        return (bitsTotal + 7) / 8;
    }
};

static Type identityOrdered(Type t) {
    t.order.resize(t.shape.size());
    std::iota(t.order.begin(), t.order.end(), 0);
    return t;
}

// validateQuantElemType (src/vpux_compiler/src/utils/quantization.cpp:23-45)
static void validateQuant(const Type& t) {
    if (t.q.kind == B200C_Q_PER_AXIS) {
        if (t.q.axis < 0 || t.q.axis >= t.rank()) {
            throwf("Quantized axis '%d' is out of main type rank '%d'", t.q.axis, t.rank());
        }
        if (static_cast<size_t>(t.shape[t.q.axis]) != t.q.scales.size()) {
            throwf("Number of scales '%zu' in per-axis quantized type do not match the quantized dimension size '%lld'",
                   t.q.scales.size(), (long long)t.shape[t.q.axis]);
        }
    }
}

static Type fromC(const b200c_type& c) {
    Type t;
    if (c.rank < 0 || c.rank > B200C_MAX_RANK) {
        throw Unsupported("rank out of range");
    }
    t.dtype = c.dtype;
    t.shape.assign(c.shape, c.shape + c.rank);
    t.order.resize(c.rank);
    for (int k = 0; k < c.rank; ++k) t.order[k] = c.order[k];
    t.q.kind = c.qkind;
    if (c.qkind != B200C_Q_NONE) {
        t.q.axis = c.qaxis;
        t.q.expressed = c.qexpressed;
        t.q.qmin = c.qmin;
        t.q.qmax = c.qmax;
        t.q.scales.assign(c.scales, c.scales + c.nq);
        t.q.zps.assign(c.zps, c.zps + c.nq);
    }
    return t;
}

static void toC(const Type& t, b200c_type* c) {
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
    c->nq = static_cast<int64_t>(t.q.scales.size());
    if (t.q.kind != B200C_Q_NONE) {
        if (sc == nullptr || zp == nullptr || cap < c->nq) {
            throw Unsupported("output type needs room for quantisation parameters");
        }
        std::copy(t.q.scales.begin(), t.q.scales.end(), sc);
        std::copy(t.q.zps.begin(), t.q.zps.end(), zp);
    }
}

// getMemIndexND / getMemIndex1D (src/vpux_compiler/src/core/attributes/shape.cpp:60-105)
static void memIndexND(int64_t idx1d, const std::vector<int64_t>& memShape, int64_t* nd) {
    for (int k = static_cast<int>(memShape.size()) - 1; k >= 0; --k) {
        nd[k] = idx1d % memShape[k];
        idx1d = (idx1d - nd[k]) / memShape[k];
    }
    if (idx1d != 0) throwf("Memory index 1D is not compatible with memory shape");
}
static int64_t memIndex1D(const int64_t* nd, const std::vector<int64_t>& memShape) {
    int64_t idx = 0, mul = 1;
    for (int k = static_cast<int>(memShape.size()) - 1; k >= 0; --k) {
        if (nd[k] >= memShape[k]) throwf("Memory index ND is not compatible with memory shape");
        idx += nd[k] * mul;
        mul *= memShape[k];
    }
    return idx;
}

// ---------------------------------------------------------------------------
// Content (src/vpux_compiler/include/vpux/compiler/dialect/const/utils/content.hpp:142-310,
// CU/content.cpp)
// ---------------------------------------------------------------------------
struct Content {
    Type type;
    int storage = 0;  // storage element type (never quantised)
    bool splat = false;
    std::shared_ptr<char[]> owned;
    const char* data = nullptr;
    size_t size = 0;

    char* raw() {
        if (!owned) throwf("Temp buffer was not allocated");
        return owned.get();
    }
};

static Content fromRawBuffer(const Type& type, const char* data, size_t size, int storage, bool splat) {
    Content c;
    c.type = type;
    c.data = data;
    c.size = size;
    c.storage = storage;
    c.splat = splat;
    return c;
}

// Content::allocTempBuffer (CU/content.cpp:32-47)
static Content allocTemp(const Type& type, int storage, bool splat) {
    Content c;
    c.type = type;
    c.storage = storage;
    c.splat = splat;
    const int64_t n = splat ? 1 : type.numElements();
    c.size = static_cast<size_t>((static_cast<int64_t>(dbits(storage)) * n + 7) / 8);
    c.owned = std::shared_ptr<char[]>(new char[c.size ? c.size : 1]);
    c.data = c.owned.get();
    return c;
}
// sub-byte overload (CU/content.cpp:49-61)
static Content allocTemp(const Type& type, int storage, bool splat, size_t rawSize) {
    Content c;
    c.type = type;
    c.storage = storage;
    c.splat = splat;
    c.size = rawSize;
    c.owned = std::shared_ptr<char[]>(new char[rawSize ? rawSize : 1]);
    c.data = c.owned.get();
    return c;
}
// Content::moveBuffer (CU/content.cpp:67-81)
static Content moveBuffer(const Type& type, Content&& other) {
    Content c;
    c.type = type;
    c.storage = other.storage;
    c.splat = other.splat;
    c.data = other.data;
    c.size = other.size;
    c.owned = std::move(other.owned);
    other.data = nullptr;
    other.size = 0;
    return c;
}

// Content::dispatchByElemType (content.hpp:253-299): the C++ type used to read or
// write an element type.  Returns a tag; quantised types go by their storage.
enum class CT { U8, U16, U32, U64, I8, I16, I32, I64, F32, F64, F16, BF16 };

static CT dispatchTag(int dtype, bool quantized) {
    const int c = dcls(dtype), b = dbits(dtype);
    if (quantized) {
        if (c == B200C_CLS_SINT && (b == 8 || b == 4)) return CT::I8;
        if (c == B200C_CLS_UINT && (b == 8 || b == 4)) return CT::U8;
        throwf("Unsupported quantized storage type");
    }
    if ((c == B200C_CLS_UINT || c == B200C_CLS_INT)) {
        if (b == 8 || b == 4) return CT::U8;
        if (b == 16) return CT::U16;
        if (b == 32) return CT::U32;
        if (b == 64) return CT::U64;
    } else if (c == B200C_CLS_SINT) {
        if (b == 8 || b == 4) return CT::I8;
        if (b == 16) return CT::I16;
        if (b == 32) return CT::I32;
        if (b == 64) return CT::I64;
    } else if (c == B200C_CLS_FLOAT) {
        if (b == 32) return CT::F32;
        if (b == 64) return CT::F64;
        if (b == 16) return CT::F16;
    } else if (c == B200C_CLS_BFLOAT && b == 16) {
        return CT::BF16;
    }
    throwf("Unsupported element type");
}

template <class F>
static auto withCT(CT t, F&& f) {
    switch (t) {
    case CT::U8: return f(uint8_t(0));
    case CT::U16: return f(uint16_t(0));
    case CT::U32: return f(uint32_t(0));
    case CT::U64: return f(uint64_t(0));
    case CT::I8: return f(int8_t(0));
    case CT::I16: return f(int16_t(0));
    case CT::I32: return f(int32_t(0));
    case CT::I64: return f(int64_t(0));
    case CT::F32: return f(float(0));
    case CT::F64: return f(double(0));
    case CT::F16: return f(f16());
    default: return f(bf16());
    }
}

// Content::getValues<OutT>() (content.hpp:162-174) with ContentRangeBase::getItem (:90-99)
template <class OutT>
struct Values {
    const char* data;
    size_t size;
    bool splat;
    size_t elemSize;
    int64_t count;
    OutT (*cvt)(const char*);

    OutT operator[](int64_t i) const {
        if (splat) return cvt(data);
        const size_t rawIndex = static_cast<size_t>(i) * elemSize;
        if (!(rawIndex < size)) throwf("Out-of-bound access in ContentRangeBase");
        return cvt(data + rawIndex);
    }
};

template <class OutT>
static Values<OutT> getValues(const Content& c) {
    const CT tag = dispatchTag(c.storage, false);
    if (dbits(c.storage) < 8) throwf("Unsupported storage type of size '%d' bits.", dbits(c.storage));
    Values<OutT> v;
    v.data = c.data;
    v.size = c.size;
    v.splat = c.splat;
    v.elemSize = static_cast<size_t>(dbits(c.storage) / 8);
    v.count = c.type.numElements();
    v.cvt = withCT(tag, [](auto dummy) -> OutT (*)(const char*) {
        using InT = decltype(dummy);
        return [](const char* p) -> OutT {
            InT x;
            std::memcpy(&x, p, sizeof(InT));
            return ccast<OutT>(x);
        };
    });
    if (v.splat && v.size != v.elemSize) {
        throwf("Splat data store size '%zu' doesn't match element type size '%zu'", v.size, v.elemSize);
    }
    return v;
}

// Content::copySubByteContent (CU/content.cpp:129-182)
static void copySubByte(const Content& c, char* target, size_t targetSize) {
    const int elemBits = c.type.elemBits();
    if (c.splat) {
        const int numShifts = 8 / elemBits;
        uint8_t byteValue = 0;
        char sub = c.data[0];
        if (dbits(c.storage) == 1) sub &= 1;
        for (int s = 0; s < numShifts; ++s) byteValue = static_cast<uint8_t>((byteValue << elemBits) + sub);
        std::fill(target, target + targetSize, static_cast<char>(byteValue));
        return;
    }
    if (targetSize < c.size) {
        if (targetSize == 0 || c.size % targetSize != 0) {
            throwf("Cannot pack sub-byte elements into buffer: source data size '%zu', target data size '%zu'", c.size,
                   targetSize);
        }
        const auto src = getValues<int8_t>(c);
        const size_t elemPerByte = static_cast<size_t>(src.count) / targetSize;
        if (!(elemPerByte <= 8 && elemPerByte != 0 && (elemPerByte & (elemPerByte - 1)) == 0)) {
            throwf("Invalid number of elements per byte '%zu'", elemPerByte);
        }
        const int bitsPer = static_cast<int>(8 / elemPerByte);
        const char mask = static_cast<char>((1u << bitsPer) - 1u);
        for (size_t idx = 0; idx < static_cast<size_t>(src.count); idx += elemPerByte) {
            uint8_t byte = 0;
            int shift = 0;
            for (int64_t e = static_cast<int64_t>(elemPerByte) - 1; e >= 0; --e) {
                byte |= static_cast<uint8_t>((src[idx + e] & mask) << shift);
                shift += bitsPer;
            }
            target[idx / elemPerByte] = static_cast<char>(byte);
        }
        return;
    }
    std::memcpy(target, c.data, c.size);
}

// Content::copyTo (CU/content.cpp:184-207).  Returns the number of bytes written.
static size_t copyTo(const Content& c, char* target, size_t targetSize) {
    const int elemBits = c.type.elemBits();
    if (elemBits < 8) {
        copySubByte(c, target, targetSize);
        if (c.splat) return targetSize;
        return targetSize < c.size ? targetSize : c.size;
    }
    const bool trivial = c.type.q.kind == B200C_Q_NONE && c.type.dtype == c.storage;
    if (!c.splat && trivial) {
        if (targetSize < c.size) {
            throwf("Byte sizes of the target buffer '%zu' is smaller then storage buffer '%zu' ", targetSize, c.size);
        }
        std::memcpy(target, c.data, c.size);
        return c.size;
    }
    const CT outTag = dispatchTag(c.type.dtype, c.type.q.kind != B200C_Q_NONE);
    return withCT(outTag, [&](auto dummy) -> size_t {
        using ElemT = decltype(dummy);
        const auto range = getValues<ElemT>(c);
        const size_t need = static_cast<size_t>(range.count) * sizeof(ElemT);
        if (targetSize < need) {
            throwf("Buffer with byte size '%zu' is not enough to hold actual elements with '%zu' byte size", targetSize,
                   need);
        }
        parallel_for(range.count, [&](int64_t i) {  // fillBuf, CU/content.cpp:112-125
            const ElemT v = range[i];
            std::memcpy(target + static_cast<size_t>(i) * sizeof(ElemT), &v, sizeof(ElemT));
        });
        return need;
    });
}

// Content::fillWithZero (CU/content.cpp:213-261): "zero" is the zero point
static void fillWithZero(Content& c) {
    char* buf = c.raw();
    if (c.type.q.kind == B200C_Q_NONE) {
        std::memset(buf, 0, c.size);
        return;
    }
    const CT tag = dispatchTag(c.storage, false);
    if (c.type.q.kind == B200C_Q_PER_AXIS) {
        if (c.type.rank() != 4) throwf("Unsupported shape size %d", c.type.rank());
        if (c.type.q.axis != 0) throwf("Only per-channel quantization is supported");
        const auto memShape = c.type.memShape();
        const int64_t OC = c.type.shape[0], IC = c.type.shape[1], H = c.type.shape[2], W = c.type.shape[3];
        for (int64_t oc = 0; oc < OC; ++oc) {
            const int64_t zp = c.type.q.zps[oc];
            withCT(tag, [&](auto dummy) {
                using ElemT = decltype(dummy);
                const ElemT zv = ccast<ElemT>(zp);
                parallel_for(IC * H * W, [&](int64_t i) {
                    const int64_t w = i % W, h = (i / W) % H, ic = i / (W * H);
                    const std::vector<int64_t> logical{oc, ic, h, w};
                    const auto nd = c.type.toMem(logical);
                    const int64_t idx = memIndex1D(nd.data(), memShape);
                    std::memcpy(buf + idx * sizeof(ElemT), &zv, sizeof(ElemT));
                });
                return 0;
            });
        }
    } else {
        const int64_t zp = c.type.q.zps[0];
        withCT(tag, [&](auto dummy) {
            using ElemT = decltype(dummy);
            if (dbits(c.storage) / 8 != static_cast<int>(sizeof(ElemT))) {
                throwf("Temp buffer type mismatch with storage element size");
            }
            const ElemT zv = ccast<ElemT>(zp);
            const size_t n = c.size / sizeof(ElemT);
            for (size_t i = 0; i < n; ++i) std::memcpy(buf + i * sizeof(ElemT), &zv, sizeof(ElemT));
            return 0;
        });
    }
}

// ---------------------------------------------------------------------------
// transformations
// ---------------------------------------------------------------------------
enum class Pos { NONE, PREFERRED_LAST, LAST };

struct Xform {
    int kind = 0;
    std::vector<int64_t> a, b;
    double f = 0;
    int64_t i0 = 0, i1 = 0;
    Type type;
    bool typeNull = false;
    std::vector<int64_t> aux;
    bool hasAux = false;
    void* side0 = nullptr;
    void* side1 = nullptr;
};

static Xform xformFromC(const b200c_xform& c) {
    Xform x;
    x.kind = c.kind;
    x.a.assign(c.a, c.a + std::min<int>(std::max(c.n, 0), B200C_MAX_RANK));
    x.b.assign(c.b, c.b + std::min<int>(std::max(c.n, 0), B200C_MAX_RANK));
    x.f = c.f;
    x.i0 = c.i0;
    x.i1 = c.i1;
    x.typeNull = (c.type.dtype == 0);
    if (!x.typeNull) {
        b200c_type t = c.type;
        t.rank = 0;
        x.type = fromC(t);
    }
    if (c.aux != nullptr) {
        x.aux.assign(c.aux, c.aux + c.naux);
        x.hasAux = true;
    }
    x.side0 = c.side0;
    x.side1 = c.side1;
    return x;
}

static Pos positionRequirement(int kind) {
    switch (kind) {
    case B200C_X_GET_SPARSITY_MAP:  // CA/get_sparsity_map.cpp:113-115
    case B200C_X_SPARSIFY:          // CA/sparsify.cpp:192-194
        return Pos::PREFERRED_LAST;
    case B200C_X_BIT_PACK:          // CA/bit_pack.cpp:136-138
    case B200C_X_SWIZZLE_CONSTANT:  // CA/swizzle_transform.cpp:245-247
        return Pos::LAST;
    default:
        return Pos::NONE;
    }
}

static bool supportsSubByteStorage(int kind) {
    return kind == B200C_X_SUBVIEW || kind == B200C_X_SWIZZLE_CONSTANT;  // CA/subview.cpp:317, CA/swizzle_transform.cpp:259
}

// getInsertionPosition (CA/content.cpp:268-299)
static int insertionPosition(const std::vector<int>& kinds, int newKind) {
    const int n = static_cast<int>(kinds.size());
    if (n == 0) return 0;
    const Pos newReq = positionRequirement(newKind);
    const Pos lastReq = positionRequirement(kinds.back());
    if (newReq == Pos::LAST && lastReq == Pos::LAST) {
        throwf("Existing transformation with LAST position requirement");
    }
    if (newReq == Pos::LAST) return n;
    int it = n;
    for (; it > 0; --it) {
        const Pos r = positionRequirement(kinds[it - 1]);
        if (r == Pos::NONE || (r == Pos::PREFERRED_LAST && newReq == Pos::PREFERRED_LAST)) return it;
    }
    return it;
}

// getQuantizedAxis (src/vpux_compiler/src/utils/types.cpp:128-165)
static bool quantizedAxisAfterReshape(int axis, const std::vector<int64_t>& prev, const std::vector<int64_t>& next,
                                      int* out) {
    if (static_cast<size_t>(axis) >= prev.size()) return false;
    auto notOne = [](int64_t v) { return v != 1; };
    const auto fp = std::find_if(prev.begin(), prev.end(), notOne);
    const auto fn = std::find_if(next.begin(), next.end(), notOne);
    if (fp == prev.end() || fn == next.end()) {
        *out = axis;
        return true;
    }
    const int gap = static_cast<int>((fn - next.begin()) - (fp - prev.begin()));
    std::vector<int64_t> p, q;
    for (auto v : prev)
        if (v != 1) p.push_back(v);
    for (auto v : next)
        if (v != 1) q.push_back(v);
    if (p != q) return false;
    if (axis < -gap || axis + gap >= static_cast<int>(next.size())) return false;
    *out = axis + gap;
    return true;
}

// TensorNDTypeInterface::changeShape / changeShapeElemType (type_interfaces.cpp:176-196,217-233)
static Type changeShape(const Type& in, const std::vector<int64_t>& shape) {
    Type out = in;
    out.shape = shape;
    if (in.identityOrder()) {
        out = identityOrdered(out);
    } else if (in.rank() != static_cast<int>(shape.size())) {
        throwf("Order is incompatible with the new shape");
    }
    if (in.q.kind == B200C_Q_PER_AXIS) {
        int axis = 0;
        if (quantizedAxisAfterReshape(in.q.axis, in.shape, shape, &axis)) out.q.axis = axis;
    }
    validateQuant(out);
    return out;
}
static Type changeShapeElemType(const Type& in, const std::vector<int64_t>& shape, int dtype, const Quant& q) {
    Type out = in;
    out.shape = shape;
    if (in.identityOrder()) {
        out = identityOrdered(out);
    } else if (in.rank() != static_cast<int>(shape.size())) {
        throwf("Order is incompatible with the new shape");
    }
    out.dtype = dtype;
    out.q = q;
    validateQuant(out);
    return out;
}
static Type changeElemType(const Type& in, int dtype, const Quant& q) {
    Type out = in;
    out.dtype = dtype;
    out.q = q;
    validateQuant(out);
    return out;
}

// TensorNDTypeInterface::pad (type_interfaces.cpp:295-321) + expandScalesAndZP (quantization.cpp:56-100)
static Type padType(const Type& in, const std::vector<int64_t>& before, const std::vector<int64_t>& after) {
    if (before.size() != after.size()) throwf("Got non consistent 'padBefore' and 'padAfter' values");
    if (in.shape.size() != before.size()) throwf("Paddings and input shape are not consistent");
    Type out = in;
    for (int d = 0; d < in.rank(); ++d) out.shape[d] = in.shape[d] + before[d] + after[d];
    if (in.q.kind == B200C_Q_PER_AXIS) {
        const int64_t pb = before[in.q.axis], pa = after[in.q.axis];
        if (pb != 0 || pa != 0) {
            if (in.q.scales.empty()) throwf("Can't get value for expand scales.");
            if (!std::equal(in.q.zps.begin() + 1, in.q.zps.end(), in.q.zps.begin())) {
                throwf("All zero points should be equal");
            }
            std::vector<double> s(static_cast<size_t>(pb), in.q.scales.front());
            s.insert(s.end(), in.q.scales.begin(), in.q.scales.end());
            s.insert(s.end(), static_cast<size_t>(pa), in.q.scales.back());
            std::vector<int64_t> z(static_cast<size_t>(pb), in.q.zps.front());
            z.insert(z.end(), in.q.zps.begin(), in.q.zps.end());
            z.insert(z.end(), static_cast<size_t>(pa), in.q.zps.back());
            out.q.scales = s;
            out.q.zps = z;
        }
    }
    validateQuant(out);
    return out;
}

// TensorNDTypeInterface::extractDenseTile (type_interfaces.cpp:263-279) + tileScalesAndZP (quantization.cpp:106-130)
static Type tileType(const Type& in, const std::vector<int64_t>& offsets, const std::vector<int64_t>& shape) {
    Type out = in;
    out.shape = shape;
    if (in.q.kind == B200C_Q_PER_AXIS) {
        if (offsets.size() != shape.size()) throwf("Offsets doesn't match shape");
        const size_t sz = static_cast<size_t>(shape[in.q.axis]);
        const size_t off = static_cast<size_t>(offsets[in.q.axis]);
        if (!(off == 0 && sz == in.q.scales.size())) {
            if (off + sz > in.q.scales.size()) throwf("Invalid slice of quantization parameters");
            out.q.scales.assign(in.q.scales.begin() + off, in.q.scales.begin() + off + sz);
            out.q.zps.assign(in.q.zps.begin() + off, in.q.zps.begin() + off + sz);
        }
    }
    validateQuant(out);
    return out;
}

static int normalizedIntOf(const Type& t) {
    return t.dtype;  // a quantised Type already carries the normalised storage integer
}

static const int64_t SWIZZLE_SIZE_ALIGN = 512;  // SWIZZLING_SIZE_ALIGNMENT_VPUX37XX
static const int ARCH_VPUX37XX = 3;

static Type inferOutputType(const Xform& x, const Type& in) {
    switch (x.kind) {
    case B200C_X_CONVERT_ELEM_TYPE: {  // CA/convert_elem_type.cpp:68-73
        if (in.q.kind != B200C_Q_NONE) throwf("Can't convert quantized element type");
        return changeElemType(in, x.type.dtype, Quant());
    }
    case B200C_X_QUANT_CAST: {  // CA/quant_cast.cpp:61-75
        if (!x.typeNull) {
            if (in.q.kind != B200C_Q_NONE || in.dtype != x.type.dtype) {
                throwf("Can't cast element type to the quantized type");
            }
            return changeElemType(in, x.type.dtype, x.type.q);
        }
        if (in.q.kind == B200C_Q_NONE) throwf("Unable to restore storage type from non-quantized type");
        return changeElemType(in, normalizedIntOf(in), Quant());
    }
    case B200C_X_DEQUANTIZE: {  // CA/dequantize.cpp:23-28
        if (in.q.kind == B200C_Q_NONE) throwf("Got non quantized type in 'DequantizeAttr'");
        return changeElemType(in, in.q.expressed, Quant());
    }
    case B200C_X_RESCALE:  // CA/rescale.cpp:55-57
    case B200C_X_ADD:      // CA/add.cpp:52-54
    case B200C_X_REVERSE:                 // CA/reverse.cpp:50-52
    case B200C_X_RELOCATE_WEIGHTS_TABLE:  // CA/relocate_weights_table.cpp:114-116
        return in;
    case B200C_X_REORDER: {  // CA/reorder.cpp:67-73
        if (static_cast<int>(x.a.size()) != in.rank()) throwf("DimsOrder doesn't match type");
        Type out = in;
        for (int k = 0; k < in.rank(); ++k) out.order[k] = static_cast<int>(x.a[k]);
        return out;
    }
    case B200C_X_SUBVIEW: {  // CA/subview.cpp:105-117
        const int bitsE = in.elemBits();
        if (!(bitsE >= 8 || bitsE == 1)) throwf("SubViewAttr does not support sub-byte element types except i1");
        if (static_cast<int>(x.b.size()) != in.rank()) {
            throwf("View shape and input shape are not consistent in 'SubViewAttr'");
        }
        return tileType(in, x.a, x.b);
    }
    case B200C_X_PAD_WITH_ZERO:  // CA/pad_with_zero.cpp:98-102
        return padType(in, x.a, x.b);
    case B200C_X_BIT_PACK: {  // CA/bit_pack.cpp:75-102
        if (isFloatDt(in.dtype) && in.q.kind == B200C_Q_NONE) throwf("Bit pack does not support float inputs.");
        const int width = static_cast<int>(x.i0);
        if (!isIntDt(in.dtype)) throwf("Got unsupported input element type in bitpack");
        Type out = in;
        // quantised: storage integer of `width` bits with the same signedness, same min/max and parameters
        out.dtype = B200C_DTYPE(dcls(in.dtype), width);
        validateQuant(out);
        return out;
    }
    case B200C_X_GET_SPARSITY_MAP: {  // CA/get_sparsity_map.cpp:68-75, nce_sparsity.cpp:637-644
        if (in.rank() != 4) throwf("Expected data shape to be 4D");
        const int64_t workload = in.shape[1] * in.shape[2] * in.shape[3];
        // changeShape runs first and validates the (possibly per-axis) element type against the new shape
        Type out = changeShape(in, {in.shape[0], 1, 1, alignUp(workload, 128)});
        if (!out.identityOrder()) out = identityOrdered(out);
        return changeElemType(out, B200C_I1, Quant());
    }
    case B200C_X_SPARSIFY: {  // CA/sparsify.cpp:94-111
        if (x.i0 != 0) {
            if (!x.hasAux) throwf("Missing number of actual elements");
            const int64_t eb = in.elemBits() / 8;
            int64_t total = 0;
            for (auto n : x.aux) total += alignUp(n * eb, 16);
            return changeShapeElemType(in, {total, 1, 1, 1}, B200C_UI8, Quant());
        }
        return in;
    }
    case B200C_X_SWIZZLE_CONSTANT: {  // CA/swizzle_transform.cpp:126-148
        if (x.i1 != ARCH_VPUX37XX) throwf("Architecture does not support swizzling");
        const int64_t newSize = alignUp(in.totalAllocSize(), SWIZZLE_SIZE_ALIGN);
        if (in.elemBits() == 1) return changeShape(in, {newSize * 8, 1, 1, 1});
        if (in.q.kind == B200C_Q_NONE && in.dtype == B200C_F16) return changeShape(in, {newSize / 2, 1, 1, 1});
        return changeShapeElemType(in, {newSize, 1, 1, 1}, B200C_UI8, Quant());
    }
    case B200C_X_RESHAPE:  // CA/reshape.cpp:73-76
        return changeShape(in, x.b);
    case B200C_X_CHANGE_SHAPE_AND_ELEM_TYPE:  // CA/change_shape_and_elem_type.cpp:84-88
        return changeShapeElemType(in, x.b, x.type.dtype, x.type.q);
    case B200C_X_BROADCAST: {  // CA/broadcast.cpp:62-78
        const int axis = static_cast<int>(x.i0);
        if (axis < 0 || axis >= in.rank()) throwf("Broadcast axis out of range");
        if (x.i1 < in.shape[axis]) throwf("Value cannot be broadcasted due to new value's size is less than old one");
        std::vector<int64_t> before(in.rank(), 0), after(in.rank(), 0);
        after[axis] = x.i1 - in.shape[axis];
        return padType(in, before, after);
    }
    case B200C_X_TRANSPOSE: {  // CA/transpose.cpp:67-86
        if (static_cast<int>(x.a.size()) != in.rank()) throwf("DimsOrder doesn't match type");
        std::vector<int64_t> shape(in.rank());
        for (int k = 0; k < in.rank(); ++k) shape[k] = in.shape[x.a[k]];
        Quant q = in.q;
        if (q.kind == B200C_Q_PER_AXIS) q.axis = static_cast<int>(x.a[q.axis]);
        return changeShapeElemType(in, shape, in.dtype, q);
    }
    case B200C_X_QUANTIZE_SYNTH: {
        if (!(in.q.kind == B200C_Q_NONE && isFloatDt(in.dtype))) throwf("QuantizeSynth expects a float tensor");
        return in;
    }
    case B200C_X_EXPAND_DILATED: {  // CA/expand_dilated.cpp:78-82, getDilatedType (utils/dilated_utils.cpp:11-34)
        if (in.rank() != 4) throwf("Got invalid tensor rank '4'");
        if (x.a.size() < 2) throw std::invalid_argument("ExpandDilated needs two dilations");
        Type out = in;
        out.shape[2] = in.shape[2] + (in.shape[2] - 1) * (x.a[0] - 1);
        out.shape[3] = in.shape[3] + (in.shape[3] - 1) * (x.a[1] - 1);
        return out;
    }
    default:
        throw Unsupported("transformation kind not restated in the oracle");
    }
}

// ---- Dequantize (CA/dequantize.cpp:47-94; dequantize(), quantization.cpp:633-635) ----
static inline float dequantizeOne(int64_t q, double scale, int64_t zp) {
    return static_cast<float>(static_cast<double>(q - zp) * scale);
}

static Content xDequantize(const Xform& x, Content& in) {
    const Type outType = inferOutputType(x, in.type);
    const bool perAxis = in.type.q.kind == B200C_Q_PER_AXIS;
    Content out = allocTemp(outType, B200C_F32, perAxis ? false : in.splat);
    const auto q = getValues<int64_t>(in);
    float* real = reinterpret_cast<float*>(out.raw());
    const int64_t nOut = static_cast<int64_t>(out.size / sizeof(float));
    if (!perAxis) {
        const double scale = in.type.q.scales[0];
        const int64_t zp = in.type.q.zps[0];
        parallel_for(nOut, [&](int64_t i) { real[i] = dequantizeOne(q[i], scale, zp); });
    } else {
        const int memAxis = in.type.dimPos(in.type.q.axis);
        const auto memShape = in.type.memShape();
        const int64_t inner = memShape[memAxis];
        int64_t outer = 1;
        for (int k = 0; k < in.type.rank(); ++k)
            if (k != memAxis) outer *= memShape[k];
        if (inner == 0) throwf("Inner size is zero");
        if (outer == 0) throwf("Outer size is zero");
        if (static_cast<int64_t>(in.type.q.scales.size()) != inner) throwf("Wrong scales size");
        std::vector<int64_t> outerShape;
        for (int k = 0; k < in.type.rank(); ++k)
            if (k != memAxis) outerShape.push_back(memShape[k]);
        parallel_for(outer * inner, [&](int64_t t) {
            const int64_t outerInd = t / inner, innerInd = t % inner;
            int64_t ond[B200C_MAX_RANK], full[B200C_MAX_RANK];
            memIndexND(outerInd, outerShape, ond);
            int j = 0;
            for (int k = 0; k < in.type.rank(); ++k) full[k] = (k == memAxis) ? innerInd : ond[j++];
            const int64_t i = memIndex1D(full, memShape);
            real[i] = dequantizeOne(q[i], in.type.q.scales[innerInd], in.type.q.zps[innerInd]);
        });
    }
    return out;
}

// ---- Rescale / Add (CA/rescale.cpp:64-78, CA/add.cpp:60-74) ----
static Content xRescaleAdd(const Xform& x, Content& in) {
    Content out = allocTemp(in.type, B200C_F32, in.splat);
    const auto v = getValues<float>(in);
    float* dst = reinterpret_cast<float*>(out.raw());
    const float k = static_cast<float>(x.f);
    const int64_t n = static_cast<int64_t>(out.size / sizeof(float));
    if (x.kind == B200C_X_RESCALE) {
        parallel_for(n, [&](int64_t i) { dst[i] = v[i] * k; });
    } else {
        parallel_for(n, [&](int64_t i) { dst[i] = v[i] + k; });
    }
    return out;
}

// ---- memPermuteTransformation (CU/transformations.cpp:23-70) ----
// memPerm[k] = input memory position feeding output memory position k.
static Content memPermute(Content& in, const Type& outType, const std::vector<int>& memPerm) {
    bool identity = true;
    for (size_t k = 0; k < memPerm.size(); ++k) identity &= (memPerm[k] == static_cast<int>(k));
    if (in.splat || identity) return moveBuffer(outType, std::move(in));

    Content out = allocTemp(outType, in.storage, in.splat);
    char* dst = out.raw();
    if (out.size != in.size) throwf("Storage buffer size mismatch in 'memPermuteTransformation'");
    const size_t es = static_cast<size_t>(dbits(in.storage) / 8);
    const auto inMem = in.type.memShape();
    const auto outMem = outType.memShape();
    const int r = in.type.rank();

    // CU/mem_permute_optimized.cpp:205-237: 1/2/4-byte storage between NCHW<->NHWC or NCDHW<->NDHWC
    auto isOrd = [](const Type& t, std::initializer_list<int> o) {
        return t.rank() == static_cast<int>(o.size()) && std::equal(o.begin(), o.end(), t.order.begin());
    };
    const bool fast4 = (isOrd(in.type, {0, 1, 2, 3}) && isOrd(outType, {0, 2, 3, 1})) ||
                       (isOrd(in.type, {0, 2, 3, 1}) && isOrd(outType, {0, 1, 2, 3}));
    const bool fast5 = (isOrd(in.type, {0, 1, 2, 3, 4}) && isOrd(outType, {0, 2, 3, 4, 1})) ||
                       (isOrd(in.type, {0, 2, 3, 4, 1}) && isOrd(outType, {0, 1, 2, 3, 4}));
    if ((es == 1 || es == 2 || es == 4) && (fast4 || fast5)) {
        // Same loop nest as blob_copy_4d_t / blob_copy_5d_t (:58-125): parallel over N only, channel
        // planes walked with the logical strides of both layouts.
        std::vector<int64_t> inStr(r), outStr(r);  // logical-dim strides in elements
        {
            int64_t s = 1;
            for (int k = r - 1; k >= 0; --k) {
                inStr[in.type.order[k]] = s;
                s *= inMem[k];
            }
            s = 1;
            for (int k = r - 1; k >= 0; --k) {
                outStr[outType.order[k]] = s;
                s *= outMem[k];
            }
        }
        const int64_t N = in.type.shape[0], C = in.type.shape[1];
        int64_t spatial = 1;
        for (int d = 2; d < r; ++d) spatial *= in.type.shape[d];
        std::vector<int64_t> sp(in.type.shape.begin() + 2, in.type.shape.end());
        const char* src = in.data;
        parallel_for(N, [&](int64_t n) {
            for (int64_t c = 0; c < C; ++c) {
                for (int64_t s = 0; s < spatial; ++s) {
                    int64_t rem = s, io = n * inStr[0] + c * inStr[1], oo = n * outStr[0] + c * outStr[1];
                    for (int d = r - 1; d >= 2; --d) {
                        const int64_t cd = rem % sp[d - 2];
                        rem /= sp[d - 2];
                        io += cd * inStr[d];
                        oo += cd * outStr[d];
                    }
                    std::memcpy(dst + oo * es, src + io * es, es);
                }
            }
        });
        return out;
    }

    parallel_for(in.type.numElements(), [&](int64_t inIdx) {
        int64_t ind[B200C_MAX_RANK], ond[B200C_MAX_RANK];
        memIndexND(inIdx, inMem, ind);
        for (int k = 0; k < r; ++k) ond[k] = ind[memPerm[k]];
        const int64_t outIdx = memIndex1D(ond, outMem);
        const size_t ri = static_cast<size_t>(inIdx) * es, ro = static_cast<size_t>(outIdx) * es;
        if (!(ri < in.size)) throwf("Out-of-bound access in 'memPermuteTransformation'");
        if (!(ro < out.size)) throwf("Out-of-bound access in 'memPermuteTransformation'");
        std::memcpy(dst + ro, in.data + ri, es);
    });
    return out;
}

// ---- Reorder (CA/reorder.cpp:75-95) ----
static Content xReorder(const Xform& x, Content& in) {
    const Type outType = inferOutputType(x, in.type);
    std::vector<int> memPerm(in.type.rank());
    for (int k = 0; k < in.type.rank(); ++k) memPerm[k] = in.type.dimPos(outType.order[k]);
    return memPermute(in, outType, memPerm);
}

// ---- Transpose (CA/transpose.cpp:92-100): reorder followed by a reshape ----
static Content xTranspose(const Xform& x, Content& in) {
    const Type outType = inferOutputType(x, in.type);
    // memPerm = inPerm.compose(order): output memory position k reads the memory position of
    // logical dim order[inOrder[k]] ... evaluated as the affine composition (d) -> inPerm(order(d)).
    const int r = in.type.rank();
    std::vector<int> memPerm(r);
    for (int k = 0; k < r; ++k) memPerm[k] = static_cast<int>(x.a[in.type.order[k]]);
    return memPermute(in, outType, memPerm);
}

// ---- SubView (CA/subview.cpp:123-301) ----
static Content xSubView(const Xform& x, Content& in) {
    const Type outType = inferOutputType(x, in.type);
    Content out = allocTemp(outType, in.storage, in.splat);
    char* dst = out.raw();
    if (in.splat) {
        std::memcpy(dst, in.data, std::min(in.size, out.size));
        return out;
    }
    const auto inMem = in.type.memShape();
    const auto outMem = outType.memShape();
    const auto memOff = in.type.toMem(x.a);
    const int r = in.type.rank();
    if (dbits(in.storage) == 1) {  // bit-addressed, LSB first, serial (:145-174)
        std::memset(dst, 0, out.size);
        const int64_t n = outType.numElements();
        for (int64_t o = 0; o < n; ++o) {
            int64_t ond[B200C_MAX_RANK], ind[B200C_MAX_RANK];
            memIndexND(o, outMem, ond);
            for (int k = 0; k < r; ++k) ind[k] = ond[k] + memOff[k];
            const int64_t i = memIndex1D(ind, inMem);
            const bool bit = (in.data[i / 8] & (1 << (i % 8))) != 0;
            if (bit) dst[o / 8] = static_cast<char>(dst[o / 8] | (1 << (o % 8)));
        }
        return out;
    }
    const size_t es = static_cast<size_t>(dbits(in.storage) / 8);
    if (r == 1) {
        std::memcpy(dst, in.data + memOff[0] * es, static_cast<size_t>(outType.numElements()) * es);
        return out;
    }
    parallel_for(outType.numElements(), [&](int64_t o) {
        int64_t ond[B200C_MAX_RANK], ind[B200C_MAX_RANK];
        memIndexND(o, outMem, ond);
        for (int k = 0; k < r; ++k) ind[k] = ond[k] + memOff[k];
        const int64_t i = memIndex1D(ind, inMem);
        if (!(static_cast<size_t>(i) * es < in.size)) throwf("Out-of-bound access in 'SubViewAttr'");
        std::memcpy(dst + static_cast<size_t>(o) * es, in.data + static_cast<size_t>(i) * es, es);
    });
    return out;
}

// ---- PadWithZero (CA/pad_with_zero.cpp:108-262) ----
static Content xPad(const Xform& x, Content& in) {
    const Type outType = inferOutputType(x, in.type);
    Content out = allocTemp(outType, in.storage, false);
    fillWithZero(out);
    char* dst = out.raw();
    const size_t es = static_cast<size_t>(dbits(in.storage) / 8);
    const auto inMem = in.type.memShape();
    const auto outMem = outType.memShape();
    const auto memPad = in.type.toMem(x.a);
    const int r = in.type.rank();
    if (r == 1 && !in.splat) {
        std::memcpy(dst + memPad[0] * es, in.data, static_cast<size_t>(in.type.numElements()) * es);
        return out;
    }
    parallel_for(in.type.numElements(), [&](int64_t i) {
        int64_t ind[B200C_MAX_RANK], ond[B200C_MAX_RANK];
        memIndexND(i, inMem, ind);
        for (int k = 0; k < r; ++k) ond[k] = ind[k] + memPad[k];
        const int64_t o = memIndex1D(ond, outMem);
        const size_t ri = in.splat ? 0 : static_cast<size_t>(i) * es;
        if (!(ri < in.size)) throwf("Out-of-bound access in 'PadWithZeroAttr'");
        if (!(static_cast<size_t>(o) * es < out.size)) throwf("Out-of-bound access in 'PadWithZeroAttr'");
        std::memcpy(dst + static_cast<size_t>(o) * es, in.data + ri, es);
    });
    return out;
}

// ---- Broadcast (CA/broadcast.cpp:84-116) ----
static Content xBroadcast(const Xform& x, Content& in) {
    const Type outType = inferOutputType(x, in.type);
    Content out = allocTemp(outType, in.storage, in.splat);
    char* dst = out.raw();
    if (in.splat) {
        std::memcpy(dst, in.data, in.size);
        return out;
    }
    const auto mem = in.type.memShape();
    const int index = in.type.dimPos(static_cast<int>(x.i0));
    int64_t pre = 1, after = 1;
    for (int k = 0; k < index; ++k) pre *= mem[k];
    for (int k = index; k < in.type.rank(); ++k) after *= mem[k];
    const int64_t expandDim = mem[index];
    if (x.i1 % expandDim) throwf("Can't broadcast from %lld to %lld", (long long)expandDim, (long long)x.i1);
    const int64_t factor = x.i1 / expandDim;
    const int64_t es = dbits(in.storage) / 8;
    const int64_t single = after * es;
    parallel_for(pre * factor, [&](int64_t t) {
        const int64_t p = t / factor, f = t % factor;
        std::memcpy(dst + single * p * factor + single * f, in.data + p * after * es, static_cast<size_t>(single));
    });
    return out;
}

// ---- Reverse (CA/reverse.cpp:55-88, 93-117) ----
// Every run of `spatialDims` consecutive values (in the order getValues yields them) is reversed;
// the result is stored in the C type of the logical element type.
template <class T>
static Content reverseImpl(Content& in, const Type& outType, int64_t axis) {
    Content out = allocTemp(outType, outType.dtype, false);
    T* dst = reinterpret_cast<T*>(out.raw());
    const int rank = in.type.rank();
    if (!(axis >= 0 && axis < rank - 1)) {
        throwf("Const::Content::reverse: got unexpected content dimension %lld", static_cast<long long>(axis));
    }
    int64_t spatial = 1;
    for (int k = rank - 1; k > axis; --k) spatial *= in.type.shape[k];
    const auto v = getValues<T>(in);
    std::vector<T> vals(static_cast<size_t>(v.count));
    for (int64_t i = 0; i < v.count; ++i) vals[static_cast<size_t>(i)] = v[i];
    for (int64_t at = 0; at < v.count; at += spatial) {
        const int64_t end = std::min<int64_t>(at + spatial, v.count);
        std::reverse(vals.begin() + at, vals.begin() + end);
    }
    std::memcpy(dst, vals.data(), vals.size() * sizeof(T));
    return out;
}

static Content xReverse(const Xform& x, Content& in) {
    const Type outType = inferOutputType(x, in.type);
    const int dt = in.type.dtype;  // the normalised storage integer for quantised types
    if (dt == B200C_SI8) return reverseImpl<int8_t>(in, outType, x.i0);
    if (dt == B200C_UI8) return reverseImpl<uint8_t>(in, outType, x.i0);
    if (dt == B200C_F16) return reverseImpl<f16>(in, outType, x.i0);
    if (dt == B200C_BF16) return reverseImpl<bf16>(in, outType, x.i0);
    if (dt == B200C_F32) return reverseImpl<float>(in, outType, x.i0);
    throwf("Unexpected data type");
    return Content();
}

// ---- ExpandDilated (CA/expand_dilated.cpp:88-122) ----
// Raw storage elements are scattered into a zero-filled buffer; indices are computed from the
// logical shapes as if the layout were OIYX, exactly as the reference does.
static Content xExpandDilated(const Xform& x, Content& in) {
    const Type outType = inferOutputType(x, in.type);
    Content out = allocTemp(outType, in.storage, false);
    fillWithZero(out);
    if (dbits(in.storage) < 8) throwf("Unsupported storage type of size '%d' bits.", dbits(in.storage));
    const int64_t es = dbits(in.storage) / 8;
    const int64_t OC = in.type.shape[0], IC = in.type.shape[1], KY = in.type.shape[2], KX = in.type.shape[3];
    const int64_t dKY = outType.shape[2], dKX = outType.shape[3];
    if (in.splat) throw Unsupported("ExpandDilated of a splat reads past its single stored element in the reference");
    char* dst = out.raw();
    for (int64_t oc = 0; oc < OC; ++oc)
        for (int64_t ic = 0; ic < IC; ++ic)
            for (int64_t ky = 0; ky < KY; ++ky)
                for (int64_t kx = 0; kx < KX; ++kx) {
                    const int64_t dky = ky + (x.a[0] - 1) * ky, dkx = kx + (x.a[1] - 1) * kx;
                    const int64_t o = dkx + dky * dKX + ic * dKX * dKY + oc * dKX * dKY * IC;
                    const int64_t i = kx + ky * KX + ic * KX * KY + oc * KX * KY * IC;
                    std::memcpy(dst + o * es, in.data + i * es, static_cast<size_t>(es));
                }
    return out;
}

// ---- RelocateWeightsTable (CA/relocate_weights_table.cpp:122-203) ----
static int32_t checkedI32(int64_t v) {
    if (v < INT32_MIN || v > INT32_MAX) throwf("Can not safely cast");
    return static_cast<int32_t>(v);
}

static Content xRelocateWeightsTable(const Xform& x, Content& in) {
    const int64_t perOC = 4;  // WEIGHT_TABLE_NUM_ELEMENTS_PER_OC
    const Type outType = inferOutputType(x, in.type);
    Content out = allocTemp(outType, B200C_SI32, false);
    int32_t* patched = reinterpret_cast<int32_t*>(out.raw());
    const auto values = getValues<int32_t>(in);
    const int32_t sparsityPtr = static_cast<int32_t>(x.i0);
    const std::vector<int64_t>& offsets = x.a;
    int32_t weightPtrStep = 0, sparsityPtrStep = 0;
    if (values.count >= perOC * 2) {
        weightPtrStep = values[perOC] - values[0];
        sparsityPtrStep = values[perOC + 1] - values[1];
    }
    const int64_t OC = values.count / perOC;
    const int64_t numClusters = static_cast<int64_t>(offsets.size());
    bool segmented = false;
    for (size_t k = 1; k < offsets.size(); ++k) segmented = segmented || offsets[k] != offsets[k - 1];
    auto isNewCluster = [&](int64_t oc, int64_t cur) {
        return segmented && (cur + 1) < numClusters && oc >= offsets[static_cast<size_t>(cur + 1)];
    };
    std::vector<int64_t> steps(static_cast<size_t>(OC));
    if (x.hasAux) {
        if (static_cast<int64_t>(x.aux.size()) != OC) {
            throwf("Invalid weights compression with %zu elements for %lld channels", x.aux.size(), (long long)OC);
        }
        if (x.i1 == 0) throwf("Missing weights element type attribute");
        const int64_t alignment = x.f > 0 ? static_cast<int64_t>(x.f) : 16;
        int64_t off = 0;
        for (int64_t oc = 0, c = 0; oc < OC; ++oc) {
            if (isNewCluster(oc, c)) {
                ++c;
                off = 0;
            }
            steps[static_cast<size_t>(oc)] = off;
            const int64_t bytes = (x.aux[static_cast<size_t>(oc)] * x.i1 + 7) / 8;
            off += (bytes + alignment - 1) / alignment * alignment;
        }
    } else {
        for (int64_t oc = 0, c = 0; oc < OC; ++oc) {
            if (isNewCluster(oc, c)) ++c;
            steps[static_cast<size_t>(oc)] = static_cast<int64_t>(weightPtrStep) * (oc - offsets[static_cast<size_t>(c)]);
        }
    }
    for (int64_t oc = 0, c = 0; oc < OC; ++oc) {
        if (isNewCluster(oc, c)) ++c;
        const int64_t at = oc * perOC;
        patched[at] = checkedI32(x.b[static_cast<size_t>(c)] + steps[static_cast<size_t>(oc)]);
        patched[at + 1] = values[at + 1];
        if (values[at + 1] != 0xFFFFFF) {  // SPARSITY_PTR_WHEN_NO_SPARSITY
            patched[at + 1] = checkedI32(sparsityPtr + (oc - offsets[static_cast<size_t>(c)]) * static_cast<int64_t>(sparsityPtrStep));
        }
        patched[at + 2] = values[at + 2];
        patched[at + 3] = values[at + 3];
    }
    return out;
}

// ---- BitPack (CA/bit_pack.cpp:108-130) ----
static Content xBitPack(const Xform& x, Content& in) {
    if (in.splat) throwf("Bit pack does not support splat inputs.");
    if (x.i0 != 4) throwf("Bit pack does not support any bitwidth except for 4 at this point.");
    const auto v = getValues<uint8_t>(in);
    if (v.count % 2 != 0) throwf("Storage buffer size is odd, which is unexpected for 4 bit packing.");
    const Type outType = inferOutputType(x, in.type);
    Content out = allocTemp(outType, B200C_UI8, false, static_cast<size_t>(outType.totalAllocSize()));
    uint8_t* dst = reinterpret_cast<uint8_t*>(out.raw());
    for (int64_t i = 0; i < v.count; i += 2) {
        const uint8_t lsn = v[i] & 0x0F, msn = v[i + 1] & 0x0F;
        dst[i / 2] = static_cast<uint8_t>((msn << 4) + lsn);
    }
    return out;
}

// getSparsifyValue (src/vpux_compiler/src/utils/sparsity.cpp:12-26)
static int64_t sparsifyValueOf(const Type& t) {
    if (t.q.kind == B200C_Q_PER_TENSOR) return t.q.zps[0];
    if (t.q.kind == B200C_Q_PER_AXIS) {
        if (std::adjacent_find(t.q.zps.begin(), t.q.zps.end(), std::not_equal_to<>()) != t.q.zps.end()) {
            throwf("Not all zero-points are equal");
        }
        return t.q.zps[0];
    }
    return 0;
}

// element C type of the sparsity transforms: si8, ui8, f16, bf16, f32 only
template <class F>
static auto withSparsityElem(int dtype, F&& f) {
    if (dtype == B200C_SI8) return f(int8_t(0));
    if (dtype == B200C_UI8) return f(uint8_t(0));
    if (dtype == B200C_F16) return f(f16());
    if (dtype == B200C_BF16) return f(bf16());
    if (dtype == B200C_F32) return f(float(0));
    throwf("Unexpected weights data type");
}

// ---- GetSparsityMap (CA/get_sparsity_map.cpp:23-107) ----
static Content xGetSparsityMap(const Xform& x, Content& in) {
    const Type outType = inferOutputType(x, in.type);
    const int64_t sv = sparsifyValueOf(in.type);
    return withSparsityElem(in.type.dtype, [&](auto dummy) -> Content {
        using T = decltype(dummy);
        const auto v = getValues<T>(in);
        Content out = allocTemp(outType, B200C_UI1, false);
        fillWithZero(out);
        char* dst = out.raw();
        const size_t inWork = static_cast<size_t>(in.type.shape[1] * in.type.shape[2] * in.type.shape[3]);
        const size_t outWork = static_cast<size_t>(outType.shape[1] * outType.shape[2] * outType.shape[3]);
        const size_t numOC = static_cast<size_t>(outType.shape[0]);
        // StorageType(sparsifyValue): a plain conversion, not a checked one
        T svT;
        if constexpr (is_half<T>::value) {
            svT = T(static_cast<float>(sv));
        } else {
            svT = static_cast<T>(sv);
        }
        for (size_t oc = 0; oc < numOC; ++oc) {
            const size_t start = oc * inWork;
            size_t o = oc * outWork / 8;
            for (size_t i = 0; i < inWork; i += 8) {
                uint8_t byte = 0;
                for (size_t b = 0; b < 8; ++b) {
                    if (v[static_cast<int64_t>(start + i + b)] != svT) byte |= static_cast<uint8_t>(1u << b);
                }
                dst[o++] = static_cast<char>(byte);
            }
        }
        return out;
    });
}

// countNonSparseElementsPerOC (src/vpux_compiler/src/utils/sparsity.cpp:28-72)
static std::vector<int64_t> countNonSparse(const Content& in) {
    const int64_t sv = sparsifyValueOf(in.type);
    return withSparsityElem(in.type.dtype, [&](auto dummy) -> std::vector<int64_t> {
        using T = decltype(dummy);
        const auto v = getValues<T>(in);
        if (in.type.rank() != 4) throwf("Const::Content::sparsify: got unxpected content shape %d", in.type.rank());
        const int64_t OC = in.type.shape[0], work = in.type.shape[1] * in.type.shape[2] * in.type.shape[3];
        const T svT = ccast<T>(sv);
        std::vector<int64_t> elems(static_cast<size_t>(OC), 0);
        parallel_for(OC, [&](int64_t oc) {
            int64_t n = 0;
            for (int64_t i = oc * work; i < (oc + 1) * work; ++i)
                if (!(v[i] == svT)) ++n;
            elems[static_cast<size_t>(oc)] = n;
        });
        return elems;
    });
}

// ---- Sparsify (CA/sparsify.cpp:115-186) ----
static Content xSparsify(const Xform& x, Content& in) {
    const std::vector<int64_t> numElems = x.hasAux ? x.aux : countNonSparse(in);
    const int64_t eb = in.type.elemBits() / 8;
    int64_t total = 0;
    for (auto n : numElems) total += alignUp(n * eb, 16);
    const Type outType = changeShapeElemType(in.type, {total, 1, 1, 1}, B200C_UI8, Quant());
    const int64_t sv = sparsifyValueOf(in.type);
    return withSparsityElem(in.type.dtype, [&](auto dummy) -> Content {
        using T = decltype(dummy);
        Content out = allocTemp(outType, B200C_UI8, false);
        fillWithZero(out);
        char* dst = out.raw();
        const auto v = getValues<T>(in);
        if (in.type.rank() != 4) throwf("Expected 4D input shape.");
        const int64_t OC = in.type.shape[0], work = in.type.shape[1] * in.type.shape[2] * in.type.shape[3];
        const T svT = ccast<T>(sv);
        int64_t o = 0;
        for (int64_t oc = 0; oc < OC; ++oc) {
            for (int64_t i = oc * work; i < (oc + 1) * work; ++i) {
                const T e = v[i];
                if (e == svT) continue;
                if (static_cast<size_t>((o + 1) * static_cast<int64_t>(sizeof(T))) > out.size) {
                    throw Unsupported("Sparsify: numActualElements smaller than the actual count (heap overflow in the reference)");
                }
                std::memcpy(dst + o * sizeof(T), &e, sizeof(T));
                ++o;
            }
            const int64_t ob = o * static_cast<int64_t>(sizeof(T));
            if (ob % 16 != 0) o = alignUp(ob, 16) / static_cast<int64_t>(sizeof(T));
        }
        return out;
    });
}

// ---- swizzle address transform (src/vpux_compiler/include/vpux/compiler/utils/swizzle_transform.hpp:58-80,
//      CA/swizzle_transform.cpp:41-79) ----
static const uint32_t LOG2_CUT_WIDTH = 4, LOG2_CUT_BYTES = 9, MAX_SWIZZLE_KEY = 5;

struct AddressTransform {
    uint32_t mask, shift;
    explicit AddressTransform(uint32_t key) {
        const uint32_t bitsK = key % (MAX_SWIZZLE_KEY + 1u);
        mask = (1u << bitsK) - 1u;
        shift = LOG2_CUT_BYTES - bitsK;
    }
    uint32_t physical(uint32_t dpu) const {
        uint32_t stagger = dpu >> LOG2_CUT_WIDTH;
        stagger &= (1u << 11) - 1u;
        stagger >>= MAX_SWIZZLE_KEY;
        stagger &= mask;
        stagger <<= shift;
        const uint32_t cutMask = (1u << LOG2_CUT_BYTES) - 1u;
        uint32_t phy = (dpu + stagger) & cutMask;
        return phy + (dpu & ~cutMask);
    }
};

static void swizzleBuffer(const char* in, size_t n, char* out, uint32_t key) {
    const AddressTransform at(key);
    const size_t iters = ((n + 15) >> 4);
    uint32_t dpu = 0;
    for (size_t i = 0; i < iters; ++i, dpu += 16) std::memcpy(out + at.physical(dpu), in + dpu, 16);
}
static void deswizzleBuffer(const char* in, size_t n, char* out, uint32_t key) {
    const AddressTransform at(key);
    const size_t iters = ((n + 15) >> 4);
    uint32_t dpu = 0;
    for (size_t i = 0; i < iters; ++i, dpu += 16) std::memcpy(out + dpu, in + at.physical(dpu), 16);
}

// swizzleValues (CA/swizzle_transform.cpp:154-196)
static Content swizzleValues(Content& in, const Type& outType, uint32_t key) {
    const int64_t total = in.type.totalAllocSize();
    const size_t newSize = static_cast<size_t>(alignUp(total, SWIZZLE_SIZE_ALIGN));
    Content out = allocTemp(outType, outType.dtype, false, newSize);
    char* dst = out.raw();
    std::vector<char> vals(newSize);
    copyTo(in, vals.data(), newSize);
    if (newSize > static_cast<size_t>(total)) {
        const char pad = in.splat ? vals[0] : 0;
        std::fill(vals.begin() + total, vals.end(), pad);
    }
    if (in.splat) {
        std::memcpy(dst, vals.data(), newSize);
        return out;
    }
    swizzleBuffer(vals.data(), newSize, dst, key);
    return out;
}

// ---- SwizzleConstant (CA/swizzle_transform.cpp:202-239) ----
static Content xSwizzle(const Xform& x, Content& in) {
    const uint32_t key = static_cast<uint32_t>(x.i0);
    const Type outType = inferOutputType(x, in.type);
    if (in.type.elemBits() != 1) return swizzleValues(in, outType, key);

    if (in.type.numElements() % 8 != 0) throwf("Elements cannot be packed in bytes");
    const int64_t packed = in.type.numElements() / 8;
    Type packedType = changeShapeElemType(in.type, {1, 1, 1, packed}, B200C_UI8, Quant());
    static const char ff = static_cast<char>(0xFF);
    const char* data = in.data;
    size_t size = in.size;
    if (in.splat && in.data[0] == 1) {
        data = &ff;
        size = 1;
    }
    Content packedIn = fromRawBuffer(packedType, data, size, B200C_UI8, in.splat);
    Content packedOut = swizzleValues(packedIn, outType, key);
    Content out = moveBuffer(outType, std::move(packedOut));
    out.storage = in.storage;
    return out;
}

// ---- QuantizeSynth: synthetic per-channel quantiser (no reference counterpart). ----
// Defined here in float arithmetic; the CUDA kernels must reproduce it bit for bit.
//   scheme 0: scale = max|w| / 127 (1 if the row is all zero); q = clamp(rint(w / scale), -127, 127)
//   scheme 1: scale = (max - min) / 15 (1 if zero); zp = clamp(rint(-min / scale), 0, 15);
//             q = clamp(rint(w / scale) + zp, 0, 15)
// Rows are the slices along logical dim 0; the result keeps the input's layout and logical type,
// in f32 storage.
static Content xQuantizeSynth(const Xform& x, Content& in) {
    const Type outType = inferOutputType(x, in.type);
    if (in.splat) throwf("QuantizeSynth does not support splat inputs");
    if (in.type.rank() < 1) throwf("QuantizeSynth expects rank >= 1");
    const auto v = getValues<float>(in);
    Content out = allocTemp(outType, B200C_F32, false);
    float* dst = reinterpret_cast<float*>(out.raw());
    const int64_t OC = in.type.shape[0];
    const auto memShape = in.type.memShape();
    const int r = in.type.rank();
    const int ocPos = in.type.dimPos(0);
    const int64_t total = in.type.numElements();
    const int64_t work = OC ? total / OC : 0;
    int64_t ocStride = 1;
    for (int k = ocPos + 1; k < r; ++k) ocStride *= memShape[k];
    // memory index of the j-th element of row oc (rows need not be contiguous)
    auto rowIndex = [&](int64_t oc, int64_t j) {
        const int64_t inner = j % ocStride, outer = j / ocStride;
        return (outer * OC + oc) * ocStride + inner;
    };
    float* scalesOut = static_cast<float*>(x.side0);
    int32_t* zpsOut = static_cast<int32_t*>(x.side1);
    const int scheme = static_cast<int>(x.i0);
    if (scheme != B200C_QSYNTH_SYM_I8 && scheme != B200C_QSYNTH_ASYM_U4) throwf("Unknown QuantizeSynth scheme");
    parallel_for(OC, [&](int64_t oc) {
        float mx = 0.f, mn = 0.f, amax = 0.f;
        for (int64_t j = 0; j < work; ++j) {
            const float w = v[rowIndex(oc, j)];
            if (j == 0) {
                mx = mn = w;
            } else {
                mx = std::max(mx, w);
                mn = std::min(mn, w);
            }
            amax = std::max(amax, std::fabs(w));
        }
        float scale;
        int32_t zp = 0;
        if (scheme == B200C_QSYNTH_SYM_I8) {
            scale = amax / 127.0f;
            if (!(scale > 0.f)) scale = 1.0f;
        } else {
            scale = (mx - mn) / 15.0f;
            if (!(scale > 0.f)) scale = 1.0f;
            float z = std::nearbyintf(-mn / scale);
            z = std::min(std::max(z, 0.0f), 15.0f);
            zp = static_cast<int32_t>(z);
        }
        if (scalesOut) scalesOut[oc] = scale;
        if (zpsOut) zpsOut[oc] = zp;
        for (int64_t j = 0; j < work; ++j) {
            const int64_t i = rowIndex(oc, j);
            float q = std::nearbyintf(v[i] / scale);
            if (scheme == B200C_QSYNTH_SYM_I8) {
                q = std::min(std::max(q, -127.0f), 127.0f);
            } else {
                q = std::min(std::max(q + static_cast<float>(zp), 0.0f), 15.0f);
            }
            dst[i] = q;
        }
    });
    return out;
}

static Content applyTransform(const Xform& x, Content& in) {
    switch (x.kind) {
    case B200C_X_CONVERT_ELEM_TYPE:           // CA/convert_elem_type.cpp:79-81
    case B200C_X_QUANT_CAST:                  // CA/quant_cast.cpp:81-83
    case B200C_X_RESHAPE:                     // CA/reshape.cpp:82-84
    case B200C_X_CHANGE_SHAPE_AND_ELEM_TYPE:  // CA/change_shape_and_elem_type.cpp:94-96
        return moveBuffer(inferOutputType(x, in.type), std::move(in));
    case B200C_X_DEQUANTIZE:
        return xDequantize(x, in);
    case B200C_X_RESCALE:
    case B200C_X_ADD:
        return xRescaleAdd(x, in);
    case B200C_X_REORDER:
        return xReorder(x, in);
    case B200C_X_TRANSPOSE:
        return xTranspose(x, in);
    case B200C_X_SUBVIEW:
        return xSubView(x, in);
    case B200C_X_PAD_WITH_ZERO:
        return xPad(x, in);
    case B200C_X_BROADCAST:
        return xBroadcast(x, in);
    case B200C_X_REVERSE:
        return xReverse(x, in);
    case B200C_X_EXPAND_DILATED:
        return xExpandDilated(x, in);
    case B200C_X_RELOCATE_WEIGHTS_TABLE:
        return xRelocateWeightsTable(x, in);
    case B200C_X_BIT_PACK:
        return xBitPack(x, in);
    case B200C_X_GET_SPARSITY_MAP:
        return xGetSparsityMap(x, in);
    case B200C_X_SPARSIFY:
        return xSparsify(x, in);
    case B200C_X_SWIZZLE_CONSTANT:
        return xSwizzle(x, in);
    case B200C_X_QUANTIZE_SYNTH:
        return xQuantizeSynth(x, in);
    default:
        throw Unsupported("transformation kind not restated in the oracle");
    }
}

// ContentAttr::fold (CA/content.cpp:167-193)
static Content fold(const Type& baseType, const char* data, size_t nbytes, bool splat, const std::vector<Xform>& chain) {
    Content res = fromRawBuffer(baseType, data, nbytes, baseType.dtype, splat);
    for (const auto& x : chain) {
        if (dbits(res.storage) < 8 && !supportsSubByteStorage(x.kind)) {
            throwf("Unsupported storage type of size '%d' bits.", dbits(res.storage));
        }
        res = applyTransform(x, res);
    }
    return res;
}

// ---------------------------------------------------------------------------
// block codec: CPU encoder / decoder of the library's own stream format
// (stands where BitCompactor is called, src/vpux_compiler/src/utils/bit_compactor_codec.cpp:15-42;
//  the format is NOT BitCompactor's -- its sources are not in the reference tree).
//
// Stream (little endian): 32-byte header { 'B','2','B','C', u32 version = 1, u64 n, u64 nblocks,
// u32 nsuper, u32 0 }, then an index of nsuper u32 values (byte offset, from the start of the
// records, of the first record of every group of 64 blocks), then one record per 64-byte block of
// the input (the last block is zero-extended), then zero bytes up to a multiple of 32.
// Record = 1 header byte (mode in bits 7..5, parameter w in bits 4..0) + payload:
//   mode 0 RAW     : 64 bytes
//   mode 1 CONST   : 1 byte, all 64 bytes equal it
//   mode 2 PACKU   : 1 byte base (the block minimum as unsigned) + 8*w bytes: (b - base) in w bits, w = 1..7
//   mode 3 PACKS   : 8*w bytes: zigzag(int8 b) in w bits, w = 1..7
//   mode 4 SPARSE  : 8-byte mask (bit k of mask byte j = element 8j+k is non-zero) + the non-zero bytes
// Packed fields are laid out per 8-element group: 8 values of w bits, value k at bits [k*w, k*w+w)
// of a little-endian w-byte word.  Mode choice: smallest record; ties go to the smaller mode id.
// ---------------------------------------------------------------------------
namespace codec {
static const size_t HDR = 32;
static const size_t SUPER = 64;
static inline uint8_t zigzag(uint8_t b) {
    const int8_t s = static_cast<int8_t>(b);
    return static_cast<uint8_t>((static_cast<uint8_t>(s) << 1) ^ static_cast<uint8_t>(s >> 7));
}
static inline uint8_t unzigzag(uint8_t z) {
    return static_cast<uint8_t>((z >> 1) ^ static_cast<uint8_t>(-(z & 1)));
}
static inline int bitWidth(uint8_t v) {
    int w = 0;
    while (v) {
        ++w;
        v >>= 1;
    }
    return w;
}
static size_t bound(size_t n) {
    const size_t blocks = (n + 63) / 64;
    const size_t supers = (blocks + SUPER - 1) / SUPER;
    return static_cast<size_t>(alignUp(static_cast<int64_t>(HDR + 4 * supers + blocks * 65), 32));
}
static void put32(uint8_t* p, uint32_t v) {
    for (int i = 0; i < 4; ++i) p[i] = static_cast<uint8_t>(v >> (8 * i));
}
static uint32_t get32(const uint8_t* p) {
    return p[0] | (uint32_t(p[1]) << 8) | (uint32_t(p[2]) << 16) | (uint32_t(p[3]) << 24);
}
struct Choice {
    int mode, w;
    size_t size;
    uint8_t base;
};
static Choice choose(const uint8_t* b) {
    uint8_t mn = 255, mx = 0, zmax = 0;
    int nnz = 0;
    for (int i = 0; i < 64; ++i) {
        mn = std::min(mn, b[i]);
        mx = std::max(mx, b[i]);
        zmax = std::max(zmax, zigzag(b[i]));
        nnz += b[i] != 0;
    }
    Choice best{0, 0, 65, 0};
    auto consider = [&](int mode, int w, size_t size, uint8_t base) {
        if (size < best.size) best = Choice{mode, w, size, base};
    };
    if (mn == mx) consider(1, 0, 2, mn);
    const int wu = bitWidth(static_cast<uint8_t>(mx - mn));
    if (wu >= 1 && wu <= 7) consider(2, wu, 2 + 8 * static_cast<size_t>(wu), mn);
    const int ws = bitWidth(zmax);
    if (ws >= 1 && ws <= 7) consider(3, ws, 1 + 8 * static_cast<size_t>(ws), 0);
    consider(4, 0, 9 + static_cast<size_t>(nnz), 0);
    return best;
}
static void packGroup(const uint8_t* v8, int w, uint8_t* out) {
    uint64_t word = 0;
    for (int k = 0; k < 8; ++k) word |= static_cast<uint64_t>(v8[k]) << (k * w);
    for (int j = 0; j < w; ++j) out[j] = static_cast<uint8_t>(word >> (8 * j));
}
static void unpackGroup(const uint8_t* in, int w, uint8_t* v8) {
    uint64_t word = 0;
    for (int j = 0; j < w; ++j) word |= static_cast<uint64_t>(in[j]) << (8 * j);
    for (int k = 0; k < 8; ++k) v8[k] = static_cast<uint8_t>((word >> (k * w)) & ((1u << w) - 1u));
}
static size_t compress(const uint8_t* in, size_t n, uint8_t* out, size_t cap) {
    if (cap < bound(n)) throwf("codec: output capacity below the bound");
    const size_t blocks = (n + 63) / 64;
    const size_t supers = (blocks + SUPER - 1) / SUPER;
    std::memset(out, 0, HDR);
    out[0] = 'B';
    out[1] = '2';
    out[2] = 'B';
    out[3] = 'C';
    put32(out + 4, 1);
    put32(out + 8, static_cast<uint32_t>(n));
    put32(out + 12, static_cast<uint32_t>(static_cast<uint64_t>(n) >> 32));
    put32(out + 16, static_cast<uint32_t>(blocks));
    put32(out + 20, static_cast<uint32_t>(static_cast<uint64_t>(blocks) >> 32));
    put32(out + 24, static_cast<uint32_t>(supers));
    const size_t recordsAt = HDR + 4 * supers;
    size_t o = recordsAt;
    for (size_t bi = 0; bi < blocks; ++bi) {
        if (bi % SUPER == 0) put32(out + HDR + 4 * (bi / SUPER), static_cast<uint32_t>(o - recordsAt));
        uint8_t b[64] = {0};
        std::memcpy(b, in + bi * 64, std::min<size_t>(64, n - bi * 64));
        const Choice c = choose(b);
        out[o++] = static_cast<uint8_t>((c.mode << 5) | c.w);
        uint8_t t[8];
        switch (c.mode) {
        case 0:
            std::memcpy(out + o, b, 64);
            o += 64;
            break;
        case 1:
            out[o++] = c.base;
            break;
        case 2:
            out[o++] = c.base;
            for (int g = 0; g < 8; ++g) {
                for (int k = 0; k < 8; ++k) t[k] = static_cast<uint8_t>(b[g * 8 + k] - c.base);
                packGroup(t, c.w, out + o);
                o += c.w;
            }
            break;
        case 3:
            for (int g = 0; g < 8; ++g) {
                for (int k = 0; k < 8; ++k) t[k] = zigzag(b[g * 8 + k]);
                packGroup(t, c.w, out + o);
                o += c.w;
            }
            break;
        default:
            for (int g = 0; g < 8; ++g) {
                uint8_t m = 0;
                for (int k = 0; k < 8; ++k) m |= static_cast<uint8_t>((b[g * 8 + k] != 0) << k);
                out[o++] = m;
            }
            for (int i = 0; i < 64; ++i)
                if (b[i] != 0) out[o++] = b[i];
            break;
        }
    }
    const size_t padded = static_cast<size_t>(alignUp(static_cast<int64_t>(o), 32));
    std::memset(out + o, 0, padded - o);
    return padded;
}
static size_t decompress(const uint8_t* in, size_t n, uint8_t* out, size_t cap) {
    if (n < HDR || in[0] != 'B' || in[1] != '2' || in[2] != 'B' || in[3] != 'C' || get32(in + 4) != 1) {
        throwf("codec: bad stream header");
    }
    const uint64_t total = get32(in + 8) | (static_cast<uint64_t>(get32(in + 12)) << 32);
    if (total > cap) throwf("codec: output capacity too small");
    const size_t blocks = (total + 63) / 64;
    const size_t supers = (blocks + SUPER - 1) / SUPER;
    if (get32(in + 24) != supers) throwf("codec: inconsistent stream header");
    size_t i = HDR + 4 * supers;
    for (size_t bi = 0; bi < blocks; ++bi) {
        if (bi % SUPER == 0 && get32(in + HDR + 4 * (bi / SUPER)) != i - (HDR + 4 * supers)) {
            throwf("codec: index entry does not match the record position");
        }
        if (i >= n) throwf("codec: truncated stream");
        const int mode = in[i] >> 5, w = in[i] & 31;
        ++i;
        uint8_t b[64], t[8];
        switch (mode) {
        case 0:
            std::memcpy(b, in + i, 64);
            i += 64;
            break;
        case 1:
            std::memset(b, in[i++], 64);
            break;
        case 2: {
            const uint8_t base = in[i++];
            for (int g = 0; g < 8; ++g) {
                unpackGroup(in + i, w, t);
                i += w;
                for (int k = 0; k < 8; ++k) b[g * 8 + k] = static_cast<uint8_t>(t[k] + base);
            }
            break;
        }
        case 3:
            for (int g = 0; g < 8; ++g) {
                unpackGroup(in + i, w, t);
                i += w;
                for (int k = 0; k < 8; ++k) b[g * 8 + k] = unzigzag(t[k]);
            }
            break;
        case 4: {
            const uint8_t* mask = in + i;
            i += 8;
            for (int e = 0; e < 64; ++e) b[e] = ((mask[e / 8] >> (e % 8)) & 1) ? in[i++] : 0;
            break;
        }
        default:
            throwf("codec: bad block mode");
        }
        std::memcpy(out + bi * 64, b, std::min<size_t>(64, total - bi * 64));
    }
    return static_cast<size_t>(total);
}
}  // namespace codec

}  // namespace orc

// ---------------------------------------------------------------------------
// C surface used by the tests (ctypes) and by the benchmark's CPU leg
// ---------------------------------------------------------------------------
static thread_local std::string g_err;

template <class F>
static int guarded(F&& f) {
    try {
        f();
        return B200C_OK;
    } catch (const orc::Thrown& e) {
        g_err = e.what();
        return B200C_ERR_THROW;
    } catch (const orc::Unsupported& e) {
        g_err = e.what();
        return B200C_ERR_UNSUPPORTED;
    } catch (const std::bad_alloc&) {
        g_err = "out of memory";
        return B200C_ERR_NOMEM;
    } catch (const std::exception& e) {
        g_err = e.what();
        return B200C_ERR_INVALID;
    }
}

extern "C" {

const char* orc_last_error(void) {
    return g_err.c_str();
}

int orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

int orc_infer_type(const b200c_type* in, const b200c_xform* chain, int n, b200c_type* out) {
    return guarded([&] {
        orc::Type t = orc::fromC(*in);
        orc::validateQuant(t);
        for (int i = 0; i < n; ++i) t = orc::inferOutputType(orc::xformFromC(chain[i]), t);
        orc::toC(t, out);
    });
}

int orc_insert_position(const int32_t* kinds, int n, int32_t new_kind, int* pos) {
    return guarded([&] {
        std::vector<int> k(kinds, kinds + n);
        *pos = orc::insertionPosition(k, new_kind);
    });
}

int64_t orc_total_alloc_size(const b200c_type* t) {
    int64_t r = -1;
    guarded([&] { r = orc::fromC(*t).totalAllocSize(); });
    return r;
}

// fold + copyTo.  `out` is filled like the reference's callers do: they pre-zero a buffer of the
// type's total alloc size, then copyTo (export.cpp:471-473); only the copied bytes are written here.
int orc_fold(const b200c_type* base, const void* data, size_t nbytes, int is_splat, const b200c_xform* chain, int n,
             void* out, size_t out_cap, size_t* out_bytes, b200c_type* out_type) {
    return guarded([&] {
        const orc::Type bt = orc::fromC(*base);
        std::vector<orc::Xform> xs;
        for (int i = 0; i < n; ++i) xs.push_back(orc::xformFromC(chain[i]));
        orc::Content c = orc::fold(bt, static_cast<const char*>(data), nbytes, is_splat != 0, xs);
        const size_t need = static_cast<size_t>(c.type.totalAllocSize());
        if (out_cap < need) {
            g_err = "output capacity too small";
            throw orc::Unsupported(g_err);
        }
        const size_t wrote = orc::copyTo(c, static_cast<char*>(out), need);
        if (out_bytes) *out_bytes = wrote;
        if (out_type) orc::toC(c.type, out_type);
    });
}

int orc_count_nonsparse_per_oc(const b200c_type* base, const void* data, size_t nbytes, int is_splat,
                               const b200c_xform* chain, int n, int64_t* counts, int64_t ncounts) {
    return guarded([&] {
        const orc::Type bt = orc::fromC(*base);
        std::vector<orc::Xform> xs;
        for (int i = 0; i < n; ++i) xs.push_back(orc::xformFromC(chain[i]));
        orc::Content c = orc::fold(bt, static_cast<const char*>(data), nbytes, is_splat != 0, xs);
        const auto v = orc::countNonSparse(c);
        if (static_cast<int64_t>(v.size()) > ncounts) throw orc::Unsupported("counts capacity too small");
        std::copy(v.begin(), v.end(), counts);
    });
}

int orc_swizzle(const void* in, size_t n, void* out, uint32_t key) {
    return guarded([&] { orc::swizzleBuffer(static_cast<const char*>(in), n, static_cast<char*>(out), key); });
}
int orc_deswizzle(const void* in, size_t n, void* out, uint32_t key) {
    return guarded([&] { orc::deswizzleBuffer(static_cast<const char*>(in), n, static_cast<char*>(out), key); });
}

int orc_btc_bound(size_t n, size_t* bound) {
    *bound = orc::codec::bound(n);
    return B200C_OK;
}
int orc_btc_compress(const void* in, size_t n, void* out, size_t cap, size_t* out_n) {
    int notSmaller = 0;
    const int rc = guarded([&] {
        if (n == 0) orc::throwf("BitCompactorCodec::compress: Empty input data vector");
        const size_t sz = orc::codec::compress(static_cast<const uint8_t*>(in), n, static_cast<uint8_t*>(out), cap);
        *out_n = sz;
        notSmaller = (n <= sz);  // bit_compactor_codec.cpp:36-39
    });
    return rc != B200C_OK ? rc : (notSmaller ? B200C_NOT_SMALLER : B200C_OK);
}
int orc_btc_decompress(const void* in, size_t n, void* out, size_t cap, size_t* out_n) {
    return guarded([&] {
        *out_n = orc::codec::decompress(static_cast<const uint8_t*>(in), n, static_cast<uint8_t*>(out), cap);
    });
}

uint16_t orc_f32_to_f16(float f) {
    return orc::f16(f).bits;
}
float orc_f16_to_f32(uint16_t h) {
    orc::f16 x;
    x.bits = h;
    return static_cast<float>(x);
}
uint16_t orc_f32_to_bf16(float f) {
    return orc::bf16(f).bits;
}

}  // extern "C"
