// Device-side description of a fused fold pass and the per-element evaluator.
//
// A "view" says how every element of the current Content is obtained from a source buffer:
// an affine index map (one stride per output memory dim plus a base offset), a list of fill
// boxes left behind by PadWithZero, and a short value program (Dequantize / Rescale / Add /
// QuantizeSynth) that runs on the loaded element.  Index-only transformations (Reorder, SubView,
// PadWithZero) are composed into the map on the host, so a whole chain becomes one pass.
//
// The element-level semantics follow the reference's lazy conversion rules: values are read with
// checked_cast from the *storage* type (src/vpux_utils/include/vpux/utils/core/checked_cast.hpp:43-146,
// src/vpux_compiler/include/vpux/compiler/dialect/const/utils/content.hpp:162-174); a failed check
// sets an error word instead of throwing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace b200c {

#define B2_HD __host__ __device__ __forceinline__

// C type used to read/write an element type (Content::dispatchByElemType, content.hpp:253-299)
enum ElemTag : int {
    T_U8 = 0,
    T_U16,
    T_U32,
    T_U64,
    T_I8,
    T_I16,
    T_I32,
    T_I64,
    T_F16,
    T_BF16,
    T_F32,
    T_F64,
    T_NONE
};

B2_HD int tagBytes(int tag) {
    switch (tag) {
    case T_U8:
    case T_I8:
        return 1;
    case T_U16:
    case T_I16:
    case T_F16:
    case T_BF16:
        return 2;
    case T_U32:
    case T_I32:
    case T_F32:
        return 4;
    default:
        return 8;
    }
}

// error words written by kernels (first failure wins)
enum FoldErr : int {
    E_NONE = 0,
    E_CAST_RANGE = 1,    // "Can not safely cast ..." (checked_cast)
    E_CAST_INEXACT = 2,  // int -> float or double -> float does not round-trip
    E_OOB = 3,           // out-of-bound access checks of the reference
    E_SPARSE_OVERFLOW = 4,
    E_CODEC = 5
};

constexpr int kMaxDims = 8;
constexpr int kMaxBoxes = 3;
constexpr int kMaxOps = 6;

enum ValueOpKind : int { OP_DEQUANT = 1, OP_MUL, OP_ADD, OP_QSYM, OP_QASYM };

struct ValueOp {
    int kind;
    int dim;  // per-axis ops: output coordinate holding the axis, -1 for per-tensor
    long long off;
    float k;         // OP_MUL / OP_ADD constant
    double scale;    // OP_DEQUANT per-tensor
    long long zp;    // OP_DEQUANT per-tensor
    const double* scales;  // OP_DEQUANT per-axis (device)
    const long long* zps;
    const float* fscales;  // OP_QSYM / OP_QASYM per-row tables (device)
    const int* izps;
};

struct FillBox {
    long long lo[kMaxDims];
    long long hi[kMaxDims];
    unsigned long long bits;  // raw storage-typed fill value
    const void* table;        // per-channel fill values (raw, tagBytes(tag) each) or nullptr
    int tableDim;
    long long tableOff;
    int tag;  // storage tag of the fill value
    int pos;  // value-program position at which the fill enters
};

enum OutMode : int {
    OUT_RAW = 0,       // store the storage element unchanged
    OUT_CAST = 1,      // checked_cast to outTag, then store
    OUT_PACK_MSB = 2,  // copySubByteContent: packBits-wide fields, first element in the high bits
    OUT_BITPACK4 = 3   // BitPackAttr: two nibbles per byte, first element in the low nibble
};

struct GenParams {
    const void* src;
    void* dst;
    int* err;
    int srcTag;
    int rank;
    long long shape[kMaxDims];
    long long stride[kMaxDims];
    long long base;
    int nBoxes;
    FillBox box[kMaxBoxes];
    int nOps;
    ValueOp ops[kMaxOps];
    int outMode;
    int outTag;
    int packBits;
    int swizzleKey;       // < 0: none
    long long outElems;   // elements to produce
    long long outUnits;   // threads of work: elements, or packed output bytes
    long long dataBytes;  // bytes the elements occupy in dst
    long long totalBytes; // dataBytes + zero tail (swizzle size alignment)
};

struct Val {
    unsigned long long bits;
    int tag;
};

// ---------------------------------------------------------------------------- bit casts
B2_HD float bitsToFloat(unsigned int u) {
#ifdef __CUDA_ARCH__
    return __uint_as_float(u);
#else
    float f;
    memcpy(&f, &u, 4);
    return f;
#endif
}
B2_HD unsigned int floatToBits(float f) {
#ifdef __CUDA_ARCH__
    return __float_as_uint(f);
#else
    unsigned int u;
    memcpy(&u, &f, 4);
    return u;
#endif
}
B2_HD double bitsToDouble(unsigned long long u) {
#ifdef __CUDA_ARCH__
    return __longlong_as_double(static_cast<long long>(u));
#else
    double d;
    memcpy(&d, &u, 8);
    return d;
#endif
}
B2_HD unsigned long long doubleToBits(double d) {
#ifdef __CUDA_ARCH__
    return static_cast<unsigned long long>(__double_as_longlong(d));
#else
    unsigned long long u;
    memcpy(&u, &d, 8);
    return u;
#endif
}

// IEEE binary16 <-> binary32, round to nearest even (ov::float16)
B2_HD float halfBitsToFloat(unsigned short h) {
#ifdef __CUDA_ARCH__
    return __half2float(__ushort_as_half(h));
#else
    const unsigned int sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, mant = h & 0x3FFu;
    if (exp == 0) {
        if (mant == 0) return bitsToFloat(sign);
        const float v = static_cast<float>(mant) * 5.9604644775390625e-08f;
        return sign ? -v : v;
    }
    if (exp == 31) return bitsToFloat(sign | 0x7F800000u | (mant << 13));
    return bitsToFloat(sign | ((exp + 112u) << 23) | (mant << 13));
#endif
}
B2_HD unsigned short floatToHalfBits(float f) {
#ifdef __CUDA_ARCH__
    return __half_as_ushort(__float2half_rn(f));
#else
    const unsigned int x = floatToBits(f), sign = (x >> 16) & 0x8000u, a = x & 0x7FFFFFFFu;
    unsigned int out;
    if (a >= 0x7F800000u) {
        out = 0x7C00u | ((a > 0x7F800000u) ? (0x0200u | ((a >> 13) & 0x03FFu)) : 0u);
    } else if (a >= 0x477FF000u) {
        out = 0x7C00u;
    } else if (a >= 0x38800000u) {
        const unsigned int mant = a & 0x007FFFFFu;
        unsigned int h = (((a >> 23) - 112u) << 10) | (mant >> 13);
        const unsigned int rem = mant & 0x1FFFu;
        if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;
        out = h;
    } else if (a >= 0x33000000u) {
        const unsigned int shift = 126u - (a >> 23);
        const unsigned int mant = (a & 0x007FFFFFu) | 0x00800000u;
        unsigned int h = mant >> shift;
        const unsigned int rem = mant & ((1u << shift) - 1u), half = 1u << (shift - 1u);
        if (rem > half || (rem == half && (h & 1u))) ++h;
        out = h;
    } else {
        out = 0;
    }
    return static_cast<unsigned short>(sign | out);
#endif
}
// bfloat16: upper half of binary32, round to nearest even (ov::bfloat16)
B2_HD float bf16BitsToFloat(unsigned short b) {
    return bitsToFloat(static_cast<unsigned int>(b) << 16);
}
B2_HD unsigned short floatToBf16Bits(float f) {
    unsigned int x = floatToBits(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return static_cast<unsigned short>((x >> 16) | 0x0040u);
    x += 0x7FFFu + ((x >> 16) & 1u);
    return static_cast<unsigned short>(x >> 16);
}

// ---------------------------------------------------------------------------- element load/store
B2_HD unsigned long long loadRaw(const void* p, long long idx, int tag) {
    switch (tagBytes(tag)) {
    case 1:
        return static_cast<const unsigned char*>(p)[idx];
    case 2:
        return static_cast<const unsigned short*>(p)[idx];
    case 4:
        return static_cast<const unsigned int*>(p)[idx];
    default:
        return static_cast<const unsigned long long*>(p)[idx];
    }
}
B2_HD void storeRawAt(void* base, long long byteAddr, int bytes, unsigned long long bits) {
    char* p = static_cast<char*>(base) + byteAddr;
    switch (bytes) {
    case 1:
        *reinterpret_cast<unsigned char*>(p) = static_cast<unsigned char>(bits);
        break;
    case 2:
        *reinterpret_cast<unsigned short*>(p) = static_cast<unsigned short>(bits);
        break;
    case 4:
        *reinterpret_cast<unsigned int*>(p) = static_cast<unsigned int>(bits);
        break;
    default:
        *reinterpret_cast<unsigned long long*>(p) = bits;
        break;
    }
}

// ---------------------------------------------------------------------------- checked conversions
// The value is widened to one of four classes first; every reference check is a predicate on the
// value, so it can be evaluated on the widened form.
enum WideClass : int { W_I64, W_U64, W_F32, W_F64 };
struct Wide {
    int cls;
    long long i;
    unsigned long long u;
    float f;
    double d;
};

B2_HD Wide widen(Val v) {
    Wide w;
    w.cls = W_I64;
    w.i = 0;
    w.u = 0;
    w.f = 0.f;
    w.d = 0.0;
    switch (v.tag) {
    case T_U8:
        w.cls = W_U64;
        w.u = v.bits & 0xFFull;
        break;
    case T_U16:
        w.cls = W_U64;
        w.u = v.bits & 0xFFFFull;
        break;
    case T_U32:
        w.cls = W_U64;
        w.u = v.bits & 0xFFFFFFFFull;
        break;
    case T_U64:
        w.cls = W_U64;
        w.u = v.bits;
        break;
    case T_I8:
        w.i = static_cast<signed char>(v.bits);
        break;
    case T_I16:
        w.i = static_cast<short>(v.bits);
        break;
    case T_I32:
        w.i = static_cast<int>(v.bits);
        break;
    case T_I64:
        w.i = static_cast<long long>(v.bits);
        break;
    case T_F16:
        w.cls = W_F32;
        w.f = halfBitsToFloat(static_cast<unsigned short>(v.bits));
        break;
    case T_BF16:
        w.cls = W_F32;
        w.f = bf16BitsToFloat(static_cast<unsigned short>(v.bits));
        break;
    case T_F32:
        w.cls = W_F32;
        w.f = bitsToFloat(static_cast<unsigned int>(v.bits));
        break;
    default:
        w.cls = W_F64;
        w.d = bitsToDouble(v.bits);
        break;
    }
    return w;
}

// checked_cast<float>(x)
B2_HD float toFloatChecked(Val v, int& err) {
    const Wide w = widen(v);
    switch (w.cls) {
    case W_F32:
        return w.f;
    case W_F64: {
        const float f = static_cast<float>(w.d);
        if (!(static_cast<double>(f) == w.d)) err = E_CAST_INEXACT;
        return f;
    }
    case W_I64: {
        const float f = static_cast<float>(w.i);
        // round trip; |f| == 2^63 cannot convert back and cannot equal an int64 that differs from it
        if (!(f < 9.2233720368547758e18f && f >= -9.2233720368547758e18f && static_cast<long long>(f) == w.i)) {
            if (!(f == -9.2233720368547758e18f && w.i == (-9223372036854775807LL - 1))) err = E_CAST_INEXACT;
        }
        return f;
    }
    default: {
        const float f = static_cast<float>(w.u);
        if (!(f < 1.8446744073709552e19f && static_cast<unsigned long long>(f) == w.u)) err = E_CAST_INEXACT;
        return f;
    }
    }
}

// checked_cast<int64_t>(x)
B2_HD long long toI64Checked(Val v, int& err) {
    const Wide w = widen(v);
    switch (w.cls) {
    case W_I64:
        return w.i;
    case W_U64:
        if (w.u > 0x7FFFFFFFFFFFFFFFull) err = E_CAST_RANGE;
        return static_cast<long long>(w.u);
    case W_F32:
        // value <= float(INT64_MAX) == 2^63 and value >= -2^63; NaN fails both.  2^63 itself is
        // undefined behaviour in the reference and reported as a range error here.
        if (!(w.f < 9.2233720368547758e18f && w.f >= -9.2233720368547758e18f)) {
            err = E_CAST_RANGE;
            return 0;
        }
        return static_cast<long long>(w.f);
    default:
        if (!(w.d < 9.2233720368547758e18 && w.d >= -9.2233720368547758e18)) {
            err = E_CAST_RANGE;
            return 0;
        }
        return static_cast<long long>(w.d);
    }
}

// limits of the integer tags
B2_HD void intLimits(int tag, long long& lo, unsigned long long& hi) {
    switch (tag) {
    case T_U8:
        lo = 0;
        hi = 0xFFull;
        break;
    case T_U16:
        lo = 0;
        hi = 0xFFFFull;
        break;
    case T_U32:
        lo = 0;
        hi = 0xFFFFFFFFull;
        break;
    case T_U64:
        lo = 0;
        hi = 0xFFFFFFFFFFFFFFFFull;
        break;
    case T_I8:
        lo = -128;
        hi = 127;
        break;
    case T_I16:
        lo = -32768;
        hi = 32767;
        break;
    case T_I32:
        lo = -2147483647LL - 1;
        hi = 2147483647ull;
        break;
    default:
        lo = -9223372036854775807LL - 1;
        hi = 0x7FFFFFFFFFFFFFFFull;
        break;
    }
}

// checked_cast<Out>(x) for every Out tag; returns the raw bits of the result
B2_HD unsigned long long castChecked(Val v, int outTag, int& err) {
    if (v.tag == outTag) return v.bits;
    switch (outTag) {
    case T_F32:
        return floatToBits(toFloatChecked(v, err));
    case T_F16:
        return floatToHalfBits(toFloatChecked(v, err));
    case T_BF16:
        return floatToBf16Bits(toFloatChecked(v, err));
    case T_F64: {
        const Wide w = widen(v);
        double d;
        if (w.cls == W_F32) {
            d = static_cast<double>(w.f);
        } else if (w.cls == W_F64) {
            d = w.d;
        } else if (w.cls == W_I64) {
            d = static_cast<double>(w.i);
            if (!(d < 9.2233720368547758e18 && static_cast<long long>(d) == w.i)) {
                if (!(w.i == (-9223372036854775807LL - 1))) err = E_CAST_INEXACT;
            }
        } else {
            d = static_cast<double>(w.u);
            if (!(d < 1.8446744073709552e19 && static_cast<unsigned long long>(d) == w.u)) err = E_CAST_INEXACT;
        }
        return doubleToBits(d);
    }
    default:
        break;
    }
    // integer targets
    long long lo;
    unsigned long long hi;
    intLimits(outTag, lo, hi);
    const bool outSigned = outTag >= T_I8 && outTag <= T_I64;
    const Wide w = widen(v);
    switch (w.cls) {
    case W_I64:
        if (w.i < lo || (w.i >= 0 && static_cast<unsigned long long>(w.i) > hi)) err = E_CAST_RANGE;
        return static_cast<unsigned long long>(w.i);
    case W_U64:
        if (w.u > hi) err = E_CAST_RANGE;
        return w.u;
    case W_F32: {
        // value <= In(max(Out)) && value >= In(lowest(Out)), then truncation toward zero
        const float fhi = static_cast<float>(hi), flo = static_cast<float>(lo);
        if (!(w.f <= fhi && w.f >= flo)) {
            err = E_CAST_RANGE;
            return 0;
        }
        // max(Out) rounded up to a power of two passes the reference's test but cannot be
        // represented (undefined behaviour there); reported as a range error
        if (outSigned) {
            if (!(w.f < 9.2233720368547758e18f)) {
                err = E_CAST_RANGE;
                return 0;
            }
            const long long r = static_cast<long long>(w.f);
            if (r > static_cast<long long>(hi)) err = E_CAST_RANGE;
            return static_cast<unsigned long long>(r);
        }
        if (!(w.f < 1.8446744073709552e19f)) {
            err = E_CAST_RANGE;
            return 0;
        }
        const unsigned long long r = static_cast<unsigned long long>(w.f);
        if (r > hi) err = E_CAST_RANGE;
        return r;
    }
    default: {
        const double dhi = static_cast<double>(hi), dlo = static_cast<double>(lo);
        if (!(w.d <= dhi && w.d >= dlo)) {
            err = E_CAST_RANGE;
            return 0;
        }
        if (outSigned) {
            if (!(w.d < 9.2233720368547758e18)) {
                err = E_CAST_RANGE;
                return 0;
            }
            const long long r = static_cast<long long>(w.d);
            if (r > static_cast<long long>(hi)) err = E_CAST_RANGE;
            return static_cast<unsigned long long>(r);
        }
        if (!(w.d < 1.8446744073709552e19)) {
            err = E_CAST_RANGE;
            return 0;
        }
        const unsigned long long r = static_cast<unsigned long long>(w.d);
        if (r > hi) err = E_CAST_RANGE;
        return r;
    }
    }
}

// ---------------------------------------------------------------------------- value program
B2_HD float rintHalfEven(float x) {
#ifdef __CUDA_ARCH__
    return rintf(x);
#else
    return nearbyintf(x);
#endif
}
B2_HD float divRn(float a, float b) {
#ifdef __CUDA_ARCH__
    return __fdiv_rn(a, b);
#else
    return a / b;
#endif
}

// One step of the value program; the result is always f32 storage.
B2_HD Val applyOp(const ValueOp& op, Val v, const long long* coord, int& err) {
    float r;
    switch (op.kind) {
    case OP_DEQUANT: {  // dequantize(): float((q - zp) * double scale), quantization.cpp:633-635
        const long long q = toI64Checked(v, err);
        double s = op.scale;
        long long zp = op.zp;
        if (op.dim >= 0) {
            const long long a = coord[op.dim] + op.off;
            s = op.scales[a];
            zp = op.zps[a];
        }
        r = static_cast<float>(static_cast<double>(q - zp) * s);
        break;
    }
    case OP_MUL:
        r = toFloatChecked(v, err) * op.k;  // rescale.cpp:73-75
        break;
    case OP_ADD:
        r = toFloatChecked(v, err) + op.k;  // add.cpp:69-71
        break;
    case OP_QSYM: {
        const float s = op.fscales[coord[op.dim] + op.off];
        r = rintHalfEven(divRn(toFloatChecked(v, err), s));
        r = fminf(fmaxf(r, -127.0f), 127.0f);
        break;
    }
    default: {  // OP_QASYM
        const long long a = coord[op.dim] + op.off;
        r = rintHalfEven(divRn(toFloatChecked(v, err), op.fscales[a])) + static_cast<float>(op.izps[a]);
        r = fminf(fmaxf(r, 0.0f), 15.0f);
        break;
    }
    }
    Val out;
    out.bits = floatToBits(r);
    out.tag = T_F32;
    return out;
}

// Storage-typed value of the Content at output memory coordinates `coord`.
B2_HD Val evalAt(const GenParams& p, const long long* coord, int& err) {
    int start = 0;
    Val v;
    int hit = -1;
    for (int b = p.nBoxes - 1; b >= 0 && hit < 0; --b) {
        bool inside = true;
        for (int k = 0; k < p.rank; ++k) inside = inside && coord[k] >= p.box[b].lo[k] && coord[k] < p.box[b].hi[k];
        if (!inside) hit = b;
    }
    if (hit >= 0) {
        const FillBox& fb = p.box[hit];
        v.tag = fb.tag;
        v.bits = fb.table ? loadRaw(fb.table, coord[fb.tableDim] + fb.tableOff, fb.tag) : fb.bits;
        start = fb.pos;
    } else {
        long long off = p.base;
        for (int k = 0; k < p.rank; ++k) off += coord[k] * p.stride[k];
        v.tag = p.srcTag;
        v.bits = loadRaw(p.src, off, p.srcTag);
    }
    for (int i = start; i < p.nOps; ++i) v = applyOp(p.ops[i], v, coord, err);
    return v;
}

B2_HD void coordsOf(const GenParams& p, long long idx, long long* coord) {
    for (int k = p.rank - 1; k >= 0; --k) {
        const long long s = p.shape[k];
        const long long q = idx / s;
        coord[k] = idx - q * s;
        idx = q;
    }
}

// 16-byte-chunk rotation inside each 512-byte block (AddressTransform::getPhysicalAddress,
// src/vpux_compiler/src/dialect/const/attributes/swizzle_transform.cpp:64-79).
B2_HD long long swizzleAddr(long long a, int key) {
    if (key <= 0) return a;
    const long long block = (a >> 9) & 63;
    const long long stagger = (block & ((1ll << key) - 1)) << (9 - key);
    return (a & ~511ll) + ((a + stagger) & 511ll);
}

// One unit of work of the generic pass: one element, or one packed output byte, or one tail byte.
B2_HD void genericUnit(const GenParams& p, long long unit) {
    int err = E_NONE;
    long long coord[kMaxDims];
    if (unit >= p.outUnits) {  // zero tail up to the swizzle size alignment
        const long long a = p.dataBytes + (unit - p.outUnits);
        if (a < p.totalBytes) static_cast<unsigned char*>(p.dst)[swizzleAddr(a, p.swizzleKey)] = 0;
        return;
    }
    if (p.outMode == OUT_RAW || p.outMode == OUT_CAST) {
        coordsOf(p, unit, coord);
        Val v = evalAt(p, coord, err);
        int bytes = tagBytes(v.tag);
        unsigned long long bits = v.bits;
        if (p.outMode == OUT_CAST) {
            bits = castChecked(v, p.outTag, err);
            bytes = tagBytes(p.outTag);
        }
        storeRawAt(p.dst, swizzleAddr(unit * bytes, p.swizzleKey), bytes, bits);
    } else {
        const int perByte = 8 / p.packBits;
        const unsigned int mask = (1u << p.packBits) - 1u;
        unsigned int byte = 0;
        for (int e = 0; e < perByte; ++e) {
            const long long idx = unit * perByte + e;
            if (idx >= p.outElems) break;
            coordsOf(p, idx, coord);
            const Val v = evalAt(p, coord, err);
            if (p.outMode == OUT_PACK_MSB) {
                // getValues<int8_t>() & mask, element idx+0 in the most significant field (content.cpp:166-177)
                const unsigned int field = static_cast<unsigned int>(castChecked(v, T_I8, err)) & mask;
                byte |= field << (p.packBits * (perByte - 1 - e));
            } else {
                // getValues<uint8_t>() & 0xF, element idx+0 in the low nibble (bit_pack.cpp:122-127)
                const unsigned int field = static_cast<unsigned int>(castChecked(v, T_U8, err)) & mask;
                byte |= field << (p.packBits * e);
            }
        }
        static_cast<unsigned char*>(p.dst)[swizzleAddr(unit, p.swizzleKey)] = static_cast<unsigned char>(byte);
    }
    if (err != E_NONE) {
#ifdef __CUDA_ARCH__
        atomicCAS(p.err, E_NONE, err);
#else
        if (*p.err == E_NONE) *p.err = err;
#endif
    }
}

}  // namespace b200c
