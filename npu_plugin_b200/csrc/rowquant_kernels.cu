// Fused per-output-channel quantiser: the synthetic producer step (scale from max|w| or min/max),
// the quantisation, an optional within-row permutation (e.g. [I][Y*X] -> [Y*X][I] of an OIYX->OYXI
// reorder), nibble packing (BitPack) and the swizzled store, in one pass over the tensor.
//
// One CTA (or one warp for short rows) owns a row.  Rows that fit are kept in registers between
// the reduction and the quantisation (128-bit loads, 128-bit stores, nothing staged); longer or
// permuted rows are staged in shared memory.  The input is read from HBM exactly once.
//
// Arithmetic is bit-identical to the CPU definition q = clamp(rint(w / scale) [+ zp]):
//  * w / scale is the correctly rounded quotient, obtained without a per-element reciprocal from
//    r = RN(1/scale) once per row and one residual correction q = fma(fma(-q0, s, w), r, q0),
//    q0 = RN(w * r) (Markstein's correction step; exact for normal-range operands, the rest takes
//    the IEEE division),
//  * rint is the add-magic-constant trick (|quotient| <= 127 here), whose low mantissa bits are the
//    two's complement integer, so no float->int conversion instruction is needed.
// This keeps the per-element work on the FMA/ALU pipes; the conversion/special-function pipe was the
// limiter of the straightforward version.  Whether a row may take this path is decided once per
// row from its statistics (scale in range, no NaN, no magnitudes below 1e-30), so the inner loop
// carries no per-element guards; it runs on packed f32x2 instructions (sm_100) and packs the result
// bytes with byte-permute instructions.
#include "runtime.h"

#include <algorithm>
#include <atomic>

namespace b200c {

namespace {

struct Stats {
    float mx, mn, amax;
    float odd;  // > 0 when the row holds a NaN or a non-zero magnitude below 1e-30 (slow path)
};

__device__ __forceinline__ Stats warpReduce(Stats s) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s.mx = fmaxf(s.mx, __shfl_xor_sync(0xFFFFFFFFu, s.mx, o));
        s.mn = fminf(s.mn, __shfl_xor_sync(0xFFFFFFFFu, s.mn, o));
        s.amax = fmaxf(s.amax, __shfl_xor_sync(0xFFFFFFFFu, s.amax, o));
        s.odd = fmaxf(s.odd, __shfl_xor_sync(0xFFFFFFFFu, s.odd, o));
    }
    return s;
}

// the symmetric scheme takes its scale from max|w| alone: the signed extremes are not tracked for it
template <int SCHEME>
__device__ __forceinline__ void accum(Stats& s, float w) {
    if (SCHEME != B200C_QSYNTH_SYM_I8) {
        s.mx = fmaxf(s.mx, w);
        s.mn = fminf(s.mn, w);
    }
    const float aw = fabsf(w);
    s.amax = fmaxf(s.amax, aw);
    if (!(w == w) || (aw != 0.0f && aw < 1e-30f)) s.odd = 1.0f;
}

// statistics of 8 halves held in a uint4, on the packed-half pipe
template <int SCHEME>
__device__ __forceinline__ void accumHalf8(__half2& mx2, __half2& mn2, __half2& am2, __half2& nan2, uint4 v) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (SCHEME != B200C_QSYNTH_SYM_I8) {
            mx2 = __hmax2(mx2, h[i]);
            mn2 = __hmin2(mn2, h[i]);
        }
        const __half2 a = __habs2(h[i]);
        am2 = __hmax2(am2, a);
        nan2 = __hmax2_nan(nan2, a);  // becomes NaN as soon as one element is
    }
}

__device__ __forceinline__ void scaleOf(int scheme, Stats s, float& scale, int& zp) {
    zp = 0;
    if (scheme == B200C_QSYNTH_SYM_I8) {
        scale = __fdiv_rn(s.amax, 127.0f);
        if (!(scale > 0.0f)) scale = 1.0f;
    } else {
        scale = __fdiv_rn(__fsub_rn(s.mx, s.mn), 15.0f);
        if (!(scale > 0.0f)) scale = 1.0f;
        float z = rintf(__fdiv_rn(-s.mn, scale));
        z = fminf(fmaxf(z, 0.0f), 15.0f);
        zp = static_cast<int>(z);
    }
}

// per-row constants of the quantisation
struct RowQ {
    float scale, recip;
    int zp;
    bool fast;  // scale is in the range where the corrected-reciprocal quotient is exact
};

__device__ __forceinline__ RowQ makeRowQ(float scale, int zp, const Stats& s) {
    RowQ q;
    q.scale = scale;
    q.zp = zp;
    // every |w| of the row is 0 or in [1e-30, amax], the scale is in range: the corrected-reciprocal
    // quotient is the IEEE quotient and stays within +-127.01, so no per-element guard is needed
    q.fast = scale > 1e-30f && scale < 1e30f && s.amax < 1e30f && !(s.odd > 0.0f);
    q.recip = q.fast ? __frcp_rn(scale) : 0.0f;
    return q;
}

template <int SCHEME>
__device__ __forceinline__ int quantOne(float w, const RowQ& rq) {
    float x;
    const float aw = fabsf(w);
    if (rq.recip != 0.0f && (aw == 0.0f || (aw > 1e-30f && aw < 1e30f))) {
        const float q0 = __fmul_rn(w, rq.recip);
        const float e = __fmaf_rn(-q0, rq.scale, w);
        x = __fmaf_rn(e, rq.recip, q0);
    } else {
        x = __fdiv_rn(w, rq.scale);
    }
    int n;
    if (fabsf(x) < 4194304.0f) {
        n = __float_as_int(__fadd_rn(x, 12582912.0f)) - 0x4B400000;  // rint to even
    } else {
        n = x > 0.0f ? 0x7FFFFF : -0x7FFFFF;  // far outside any clamp range (also NaN -> negative side)
    }
    if (SCHEME == B200C_QSYNTH_SYM_I8) return min(max(n, -127), 127);
    return min(max(n + rq.zp, 0), 15);
}

template <typename T>
__device__ __forceinline__ float elemToFloat(T v);
template <>
__device__ __forceinline__ float elemToFloat<__half>(__half v) {
    return __half2float(v);
}
template <>
__device__ __forceinline__ float elemToFloat<float>(float v) {
    return v;
}

// source index inside the row of output element j (rank <= 3 mixed-radix map); irank == 0: identity
__device__ __forceinline__ long long rowMap(const RowQuantParams& p, long long j) {
    if (p.irank == 0) return j;
    long long off = 0;
#pragma unroll
    for (int k = 2; k >= 0; --k) {
        if (k < p.irank) {
            const long long s = p.ishape[k];
            const long long q = j / s;
            off += (j - q * s) * p.istride[k];
            j = q;
        }
    }
    return off;
}

__device__ __forceinline__ Stats blockReduce256(Stats s, float* redMx, float* redMn, float* redAm, float* redOdd) {
    s = warpReduce(s);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        redMx[warp] = s.mx;
        redMn[warp] = s.mn;
        redAm[warp] = s.amax;
        redOdd[warp] = s.odd;
    }
    __syncthreads();
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        s.mx = fmaxf(s.mx, redMx[w]);
        s.mn = fminf(s.mn, redMn[w]);
        s.amax = fmaxf(s.amax, redAm[w]);
        s.odd = fmaxf(s.odd, redOdd[w]);
    }
    return s;
}

// reduction over the TPR threads that share a row (TPR = 32, 64, 128 or 256; 256 / TPR rows per CTA)
template <int TPR>
__device__ __forceinline__ Stats rowReduce(Stats s, float* redMx, float* redMn, float* redAm, float* redOdd) {
    s = warpReduce(s);
    if (TPR > 32) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (lane == 0) {
            redMx[warp] = s.mx;
            redMn[warp] = s.mn;
            redAm[warp] = s.amax;
            redOdd[warp] = s.odd;
        }
        // only the TPR threads of a row wait for one another: rows of a CTA proceed independently
        if (TPR == 256) {
            __syncthreads();
        } else {
            asm volatile("bar.sync %0, %1;" ::"r"(1 + static_cast<int>(threadIdx.x) / TPR), "n"(TPR) : "memory");
        }
        constexpr int WPR = TPR / 32;
        const int first = (warp / WPR) * WPR;
#pragma unroll
        for (int w = 0; w < WPR; ++w) {
            s.mx = fmaxf(s.mx, redMx[first + w]);
            s.mn = fminf(s.mn, redMn[first + w]);
            s.amax = fmaxf(s.amax, redAm[first + w]);
            s.odd = fmaxf(s.odd, redOdd[first + w]);
        }
    }
    return s;
}

// float bits of (x + 1.5 * 2^23) for the correctly rounded x = w / scale, two elements at a time
__device__ __forceinline__ float2 quotMagic2(float2 w, float2 negS2, float2 r2) {
    const float2 q0 = __fmul2_rn(w, r2);
    const float2 e = __ffma2_rn(q0, negS2, w);  // w - q0 * s, exact
    const float2 x = __ffma2_rn(e, r2, q0);
    return __fadd2_rn(x, make_float2(12582912.0f, 12582912.0f));
}

template <typename T>
__device__ __forceinline__ float2 pairToFloat2(const T* e);
template <>
__device__ __forceinline__ float2 pairToFloat2<__half>(const __half* e) {
    return __half22float2(*reinterpret_cast<const __half2*>(e));
}
template <>
__device__ __forceinline__ float2 pairToFloat2<float>(const float* e) {
    return make_float2(e[0], e[1]);
}

// fast rows: 16 elements -> 16 bytes / 8 packed bytes without per-element guards or clamps
template <typename T, int SCHEME>
__device__ __forceinline__ void emitUnitFast(const RowQuantParams& p, const T* e, const RowQ& rq, long long row,
                                             long long unit) {
    unsigned char* dst = static_cast<unsigned char*>(p.dst);
    const float2 s2 = make_float2(-rq.scale, -rq.scale), r2 = make_float2(rq.recip, rq.recip);
    unsigned int bits[16];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float2 t = quotMagic2(pairToFloat2<T>(e + 2 * k), s2, r2);
        bits[2 * k] = __float_as_uint(t.x);
        bits[2 * k + 1] = __float_as_uint(t.y);
    }
    if (SCHEME == B200C_QSYNTH_SYM_I8) {
        // |quotient| <= 127: the low byte of the magic sum is the two's complement result
        unsigned int w4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const unsigned int lo = __byte_perm(bits[4 * i], bits[4 * i + 1], 0x0040);
            const unsigned int hi = __byte_perm(bits[4 * i + 2], bits[4 * i + 3], 0x0040);
            w4[i] = __byte_perm(lo, hi, 0x5410);
        }
        const long long a = row * p.rowElems + unit * 16;
        *reinterpret_cast<uint4*>(dst + swizzleAddr(a, p.swizzleKey)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
    } else {
        int n[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) n[k] = min(max(static_cast<int>(bits[k]) - 0x4B400000 + rq.zp, 0), 15);
        if (p.outMode == 0) {
            unsigned int w4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) w4[i] = n[4 * i] | (n[4 * i + 1] << 8) | (n[4 * i + 2] << 16) | (n[4 * i + 3] << 24);
            const long long a = row * p.rowElems + unit * 16;
            *reinterpret_cast<uint4*>(dst + swizzleAddr(a, p.swizzleKey)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
        } else {
            unsigned int w2[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                unsigned int word = 0;
#pragma unroll
                for (int b = 0; b < 8; ++b) word |= static_cast<unsigned int>(n[i * 8 + b]) << (4 * b);
                w2[i] = word;
            }
            *reinterpret_cast<uint2*>(dst + row * (p.rowElems / 2) + unit * 8) = make_uint2(w2[0], w2[1]);
        }
    }
}

// quantise 16 consecutive elements held in registers and emit them (16 bytes, or 8 packed bytes)
template <typename T, int SCHEME>
__device__ __forceinline__ void emitUnit(const RowQuantParams& p, const T* e, const RowQ& rq, long long row,
                                         long long unit) {
    if (rq.fast && (SCHEME != B200C_QSYNTH_SYM_I8 || p.outMode == 0)) {
        emitUnitFast<T, SCHEME>(p, e, rq, row, unit);
        return;
    }
    unsigned char* dst = static_cast<unsigned char*>(p.dst);
    if (p.outMode == 0) {
        unsigned int w4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            unsigned int word = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                word |= (static_cast<unsigned int>(quantOne<SCHEME>(elemToFloat<T>(e[i * 4 + b]), rq)) & 0xFFu) << (8 * b);
            }
            w4[i] = word;
        }
        const long long a = row * p.rowElems + unit * 16;
        *reinterpret_cast<uint4*>(dst + swizzleAddr(a, p.swizzleKey)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
    } else {
        unsigned int w2[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            unsigned int word = 0;
#pragma unroll
            for (int b = 0; b < 8; ++b) {
                word |= (static_cast<unsigned int>(quantOne<SCHEME>(elemToFloat<T>(e[i * 8 + b]), rq)) & 0xFu) << (4 * b);
            }
            w2[i] = word;
        }
        *reinterpret_cast<uint2*>(dst + row * (p.rowElems / 2) + unit * 8) = make_uint2(w2[0], w2[1]);
    }
}

__device__ __forceinline__ void zeroTail(const RowQuantParams& p) {
    if (blockIdx.x == 0) {
        for (long long a = p.dataBytes + threadIdx.x; a < p.totalBytes; a += blockDim.x) {
            static_cast<unsigned char*>(p.dst)[swizzleAddr(a, p.swizzleKey)] = 0;
        }
    }
}

// ---- register-resident rows: identity map, 16-element units, 128-bit loads and stores -------------
// TPR threads per row, each holding up to MAXU units; `g` is the index of the CTA's row group.
template <typename T, int TPR, int MAXU, int SCHEME>
__device__ __forceinline__ void rowQuantRegBody(const RowQuantParams& p, long long g, float* redMx, float* redMn,
                                                float* redAm, float* redOdd) {
    constexpr int ROWS_PER_CTA = 256 / TPR;
    constexpr int VPU = 16 * sizeof(T) / 16;  // 128-bit vectors per unit
    const int sub = threadIdx.x / TPR, t = threadIdx.x % TPR;
    const int units = static_cast<int>(p.rowElems / 16);
    const long long row = g * ROWS_PER_CTA + sub;
    const bool live = row < p.rows;
    const uint4* src4 = reinterpret_cast<const uint4*>(static_cast<const T*>(p.src) + row * p.rowElems);
    uint4 x[MAXU][VPU];
#pragma unroll
    for (int i = 0; i < MAXU; ++i) {
        const int u = t + i * TPR;
        if (live && u < units) {
#pragma unroll
            for (int v = 0; v < VPU; ++v) x[i][v] = __ldg(src4 + u * VPU + v);
        }
    }
    Stats s;
    s.mx = -INFINITY;
    s.mn = INFINITY;
    s.amax = 0.0f;
    s.odd = 0.0f;
    if (sizeof(T) == 2) {
        __half2 mx2 = __float2half2_rn(-INFINITY), mn2 = __float2half2_rn(INFINITY), am2 = __float2half2_rn(0.0f);
        __half2 nan2 = am2;
#pragma unroll
        for (int i = 0; i < MAXU; ++i) {
            const int u = t + i * TPR;
            if (live && u < units) {
#pragma unroll
                for (int v = 0; v < VPU; ++v) accumHalf8<SCHEME>(mx2, mn2, am2, nan2, x[i][v]);
            }
        }
        s.mx = fmaxf(__low2float(mx2), __high2float(mx2));
        s.mn = fminf(__low2float(mn2), __high2float(mn2));
        s.amax = fmaxf(__low2float(am2), __high2float(am2));
        const float nl = __low2float(nan2), nh = __high2float(nan2);
        s.odd = (nl == nl && nh == nh) ? 0.0f : 1.0f;  // halves have no magnitude below 1e-30 other than 0
    } else {
#pragma unroll
        for (int i = 0; i < MAXU; ++i) {
            const int u = t + i * TPR;
            if (live && u < units) {
                const float* f = reinterpret_cast<const float*>(&x[i][0]);
#pragma unroll
                for (int k = 0; k < 16; ++k) accum<SCHEME>(s, f[k]);
            }
        }
    }
    s = rowReduce<TPR>(s, redMx, redMn, redAm, redOdd);
    float scale;
    int zp;
    scaleOf(SCHEME, s, scale, zp);
    const RowQ rq = makeRowQ(scale, zp, s);
    if (live && t == 0) {
        p.scales[row] = scale;
        p.zps[row] = zp;
    }
#pragma unroll
    for (int i = 0; i < MAXU; ++i) {
        const int u = t + i * TPR;
        if (live && u < units) emitUnit<T, SCHEME>(p, reinterpret_cast<const T*>(&x[i][0]), rq, row, u);
    }
    if (g == 0) {  // zero tail of the swizzle size alignment
        for (long long a = p.dataBytes + threadIdx.x; a < p.totalBytes; a += blockDim.x) {
            static_cast<unsigned char*>(p.dst)[swizzleAddr(a, p.swizzleKey)] = 0;
        }
    }
}

template <typename T, int TPR, int MAXU, int SCHEME>
__global__ void __launch_bounds__(256) rowQuantRegKernel(const __grid_constant__ RowQuantParams p) {
    __shared__ float redMx[8], redMn[8], redAm[8], redOdd[8];
    constexpr int ROWS_PER_CTA = 256 / TPR;
    const long long rowGroups = (p.rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA;
    for (long long g = blockIdx.x; g < rowGroups; g += gridDim.x) {
        rowQuantRegBody<T, TPR, MAXU, SCHEME>(p, g, redMx, redMn, redAm, redOdd);
        if (TPR > 32) __syncthreads();  // reduction slots are reused by the next row group
    }
}

// Many tensors in one launch: CTA b works on row group (b - groupStart[i]) of tensor i, found by a
// binary search over the prefix sums.  Removes the launch gaps and tail effects of per-tensor launches.
template <typename T, int TPR, int MAXU, int SCHEME>
__global__ void __launch_bounds__(256) rowQuantRegBatchKernel(const RowQuantParams* __restrict__ items,
                                                              const long long* __restrict__ groupStart, int nitems) {
    __shared__ float redMx[8], redMn[8], redAm[8], redOdd[8];
    __shared__ RowQuantParams p;
    const long long b = blockIdx.x;
    const int lo = findBatchItem(groupStart, nitems, b);
    // stage the tensor's parameters in shared memory (one copy per CTA)
    {
        const int words = sizeof(RowQuantParams) / 4;
        const unsigned int* srcw = reinterpret_cast<const unsigned int*>(items + lo);
        unsigned int* dstw = reinterpret_cast<unsigned int*>(&p);
        for (int i = threadIdx.x; i < words; i += blockDim.x) dstw[i] = srcw[i];
    }
    __syncthreads();
    rowQuantRegBody<T, TPR, MAXU, SCHEME>(p, b - groupStart[lo], redMx, redMn, redAm, redOdd);
}

// ---- shared-memory staged rows: any length up to the shared-memory capacity, optional permutation ---
template <typename T, int TPR, int SCHEME>
__device__ __forceinline__ void rowQuantSmemBody(const RowQuantParams& p, long long g, unsigned char* smemRaw, float* redMx,
                                                 float* redMn, float* redAm, float* redOdd) {
    constexpr int ROWS_PER_CTA = 256 / TPR;
    const int sub = threadIdx.x / TPR, t = threadIdx.x % TPR;
    const int L = static_cast<int>(p.rowElems);
    T* rowSm = reinterpret_cast<T*>(smemRaw) + static_cast<long long>(sub) * p.smemRowElems;
    const long long row = g * ROWS_PER_CTA + sub;
    const bool live = row < p.rows;
    const T* src = static_cast<const T*>(p.src) + row * p.rowElems;
    Stats s;
    s.mx = -INFINITY;
    s.mn = INFINITY;
    s.amax = 0.0f;
    s.odd = 0.0f;
    if (live) {
        if (p.vecIn) {
            constexpr int PER = 16 / sizeof(T);
            const int nvec = L / PER;
            const uint4* src4 = reinterpret_cast<const uint4*>(src);
            uint4* sm4 = reinterpret_cast<uint4*>(rowSm);
            // four independent 128-bit loads per thread and round
            for (int v0 = t; v0 < nvec; v0 += 4 * TPR) {
                uint4 xv[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int v = v0 + r * TPR;
                    if (v < nvec) xv[r] = __ldg(src4 + v);
                }
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int v = v0 + r * TPR;
                    if (v >= nvec) continue;
                    sm4[v + ((v * PER) >> p.padLog2)] = xv[r];  // padLog2 is 31 when the row is not padded
                    const T* e = reinterpret_cast<const T*>(&xv[r]);
#pragma unroll
                    for (int i = 0; i < PER; ++i) accum<SCHEME>(s, elemToFloat<T>(e[i]));
                }
            }
        } else {
            for (int j = t; j < L; j += TPR) {
                const T xv = src[j];
                rowSm[j] = xv;
                accum<SCHEME>(s, elemToFloat<T>(xv));
            }
        }
    }
    s = rowReduce<TPR>(s, redMx, redMn, redAm, redOdd);  // its barrier also publishes the staged row
    if (TPR == 32) __syncwarp();
    float scale;
    int zp;
    scaleOf(SCHEME, s, scale, zp);
    const RowQ rq = makeRowQ(scale, zp, s);
    if (live && t == 0) {
        p.scales[row] = scale;
        p.zps[row] = zp;
    }
    if (live) {
        unsigned char* dst = static_cast<unsigned char*>(p.dst);
        if (p.vecOut) {
            // two-level permutation whose inner extent is a multiple of 16 (e.g. [I][Y*X] -> [Y*X][I]
            // with I % 16 == 0): the 16 outputs of a unit share the outer index, one division per unit
            const bool twoLevel = p.irank == 2 && (p.ishape[1] % 16) == 0;
            const int inner = static_cast<int>(p.ishape[1]), st0 = static_cast<int>(p.istride[0]),
                      st1 = static_cast<int>(p.istride[1]);
            for (int u = t; u < L / 16; u += TPR) {
                T e[16];
                if (p.irank == 0) {
                    const uint4* sm4 = reinterpret_cast<const uint4*>(rowSm + u * 16);
                    uint4* e4 = reinterpret_cast<uint4*>(e);
#pragma unroll
                    for (int v = 0; v < static_cast<int>(16 * sizeof(T) / 16); ++v) e4[v] = sm4[v];
                } else if (twoLevel) {
                    // the staged row carries 16 bytes of padding per 2^padLog2 elements, chosen so that
                    // the lanes of a warp (16 * st1 elements apart) fall into different banks
                    constexpr int PADSH = sizeof(T) == 4 ? 2 : 3;
                    const int j = u * 16;
                    const int outer = j / inner, in0 = j - outer * inner;
                    const int s0 = outer * st0 + in0 * st1;
#pragma unroll
                    for (int k = 0; k < 16; ++k) {
                        const int si = s0 + k * st1;
                        e[k] = rowSm[si + ((si >> p.padLog2) << PADSH)];
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < 16; ++k) e[k] = rowSm[rowMap(p, u * 16 + k)];
                }
                emitUnit<T, SCHEME>(p, e, rq, row, u);
            }
        } else if (p.outMode == 0) {
            for (int j = t; j < L; j += TPR) {
                const int q = quantOne<SCHEME>(elemToFloat<T>(rowSm[rowMap(p, j)]), rq);
                dst[swizzleAddr(row * p.rowElems + j, p.swizzleKey)] = static_cast<unsigned char>(q);
            }
        } else {
            for (int j = t; j < L / 2; j += TPR) {
                const unsigned int lo = static_cast<unsigned int>(quantOne<SCHEME>(elemToFloat<T>(rowSm[rowMap(p, 2 * j)]), rq)) & 0xFu;
                const unsigned int hi = static_cast<unsigned int>(quantOne<SCHEME>(elemToFloat<T>(rowSm[rowMap(p, 2 * j + 1)]), rq)) & 0xFu;
                dst[row * (p.rowElems / 2) + j] = static_cast<unsigned char>(lo | (hi << 4));
            }
        }
    }
    if (g == 0) {  // zero tail of the swizzle size alignment
        for (long long a = p.dataBytes + threadIdx.x; a < p.totalBytes; a += blockDim.x) {
            static_cast<unsigned char*>(p.dst)[swizzleAddr(a, p.swizzleKey)] = 0;
        }
    }
}

template <typename T, int TPR, int SCHEME>
__global__ void __launch_bounds__(256, 4) rowQuantSmemKernel(const __grid_constant__ RowQuantParams p) {
    extern __shared__ __align__(16) unsigned char smemRaw[];
    __shared__ float redMx[8], redMn[8], redAm[8], redOdd[8];
    constexpr int ROWS_PER_CTA = 256 / TPR;
    const long long rowGroups = (p.rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA;
    for (long long g = blockIdx.x; g < rowGroups; g += gridDim.x) {
        rowQuantSmemBody<T, TPR, SCHEME>(p, g, smemRaw, redMx, redMn, redAm, redOdd);
        __syncthreads();  // the row buffer and the reduction slots are reused by the next row group
    }
}

template <typename T, int TPR, int SCHEME>
__global__ void __launch_bounds__(256, 4) rowQuantSmemBatchKernel(const RowQuantParams* __restrict__ items,
                                                               const long long* __restrict__ groupStart, int nitems) {
    extern __shared__ __align__(16) unsigned char smemRaw[];
    __shared__ float redMx[8], redMn[8], redAm[8], redOdd[8];
    __shared__ RowQuantParams p;
    const long long b = blockIdx.x;
    const int lo = findBatchItem(groupStart, nitems, b);
    {
        const int words = sizeof(RowQuantParams) / 4;
        const unsigned int* srcw = reinterpret_cast<const unsigned int*>(items + lo);
        unsigned int* dstw = reinterpret_cast<unsigned int*>(&p);
        for (int i = threadIdx.x; i < words; i += blockDim.x) dstw[i] = srcw[i];
    }
    __syncthreads();
    rowQuantSmemBody<T, TPR, SCHEME>(p, b - groupStart[lo], smemRaw, redMx, redMn, redAm, redOdd);
}

// ---- launch configuration -----------------------------------------------------------------------
// A register-path configuration is (element type, threads per row, units per thread, scheme).
struct RegConfig {
    int srcTag, tpr, maxu, scheme;
    bool operator==(const RegConfig& o) const {
        return srcTag == o.srcTag && tpr == o.tpr && maxu == o.maxu && scheme == o.scheme;
    }
};

// threads per row: the smallest group that holds the row with at most MAXU units per thread, so
// every thread keeps several 128-bit loads in flight.  Returns false when the row needs staging.
bool pickRegConfig(const RowQuantParams& p, RegConfig* c) {
    const long long units = p.rowElems / 16;
    const bool regOk = p.irank == 0 && p.vecIn && p.vecOut && p.rowElems % 16 == 0;
    const int maxu = p.srcTag == T_F16 ? 4 : 2;
    if (!regOk || units > 256LL * maxu) return false;
    c->srcTag = p.srcTag;
    c->scheme = p.scheme;
    if (units <= 32LL * maxu) {
        c->tpr = 32;
        c->maxu = units <= 32 ? 1 : (units <= 64 ? 2 : maxu);
    } else if (units <= 64LL * maxu) {
        c->tpr = 64;
        c->maxu = maxu;
    } else if (units <= 128LL * maxu) {
        c->tpr = 128;
        c->maxu = maxu;
    } else {
        c->tpr = 256;
        c->maxu = units <= 512 ? 2 : ((p.srcTag == T_F16 && units <= 768) ? 3 : maxu);
    }
    return true;
}

template <typename T, int TPR, int MAXU, int SCHEME>
void launchRegT(Context* ctx, const RowQuantParams* one, const RowQuantParams* itemsDev, const long long* startDev,
                int nitems, long long totalGroups) {
    if (one) {
        constexpr int ROWS_PER_CTA = 256 / TPR;
        const long long groups = (one->rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA;
        // one row group per CTA: the block scheduler staggers the load / reduce / store phases of the
        // CTAs resident on an SM, which keeps more loads in flight than a persistent lock-step loop
        const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>(groups, 1LL << 30)));
        rowQuantRegKernel<T, TPR, MAXU, SCHEME><<<grid, 256, 0, ctx->stream>>>(*one);
    } else {
        rowQuantRegBatchKernel<T, TPR, MAXU, SCHEME>
                <<<static_cast<unsigned int>(totalGroups), 256, 0, ctx->stream>>>(itemsDev, startDev, nitems);
    }
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
}

template <typename T, int SCHEME>
void launchRegTS(Context* ctx, const RegConfig& c, const RowQuantParams* one, const RowQuantParams* itemsDev,
                 const long long* startDev, int nitems, long long totalGroups) {
#define B2_RQ_CASE(TPR_, MAXU_)                                                                                   \
    if (c.tpr == TPR_ && c.maxu == MAXU_) {                                                                       \
        launchRegT<T, TPR_, MAXU_, SCHEME>(ctx, one, itemsDev, startDev, nitems, totalGroups);                    \
        return;                                                                                                   \
    }
    B2_RQ_CASE(32, 1)
    B2_RQ_CASE(32, 2)
    B2_RQ_CASE(64, 2)
    B2_RQ_CASE(128, 2)
    B2_RQ_CASE(256, 2)
    if (sizeof(T) == 2) {
        B2_RQ_CASE(32, 4)
        B2_RQ_CASE(64, 4)
        B2_RQ_CASE(128, 4)
        B2_RQ_CASE(256, 3)
        B2_RQ_CASE(256, 4)
    }
#undef B2_RQ_CASE
    throw BadArg("row quantiser: no kernel for this configuration");
}

void launchRegConfig(Context* ctx, const RegConfig& c, const RowQuantParams* one, const RowQuantParams* itemsDev,
                     const long long* startDev, int nitems, long long totalGroups) {
    const bool sym = c.scheme == B200C_QSYNTH_SYM_I8;
    if (c.srcTag == T_F16) {
        sym ? launchRegTS<__half, B200C_QSYNTH_SYM_I8>(ctx, c, one, itemsDev, startDev, nitems, totalGroups)
            : launchRegTS<__half, B200C_QSYNTH_ASYM_U4>(ctx, c, one, itemsDev, startDev, nitems, totalGroups);
    } else {
        sym ? launchRegTS<float, B200C_QSYNTH_SYM_I8>(ctx, c, one, itemsDev, startDev, nitems, totalGroups)
            : launchRegTS<float, B200C_QSYNTH_ASYM_U4>(ctx, c, one, itemsDev, startDev, nitems, totalGroups);
    }
}

template <typename T, int TPR, int SCHEME>
void launchSmemT(Context* ctx, const RowQuantParams* one, const RowQuantParams* itemsDev, const long long* startDev,
                 int nitems, long long totalGroups, size_t smem) {
    constexpr int ROWS_PER_CTA = 256 / TPR;
    {
        // as much shared memory per SM as the part offers: the staged rows, not the L1, bound the residency.
        // Function attributes belong to a device: one bit per device, set once by whichever thread gets there
        // first (a second thread setting the same attribute again is harmless).
        static std::atomic<unsigned long long> carved{0};
        const unsigned long long bit = 1ull << (ctx->device & 63);
        if (!(carved.fetch_or(bit) & bit)) {
            cudaFuncSetAttribute(rowQuantSmemKernel<T, TPR, SCHEME>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
            cudaFuncSetAttribute(rowQuantSmemBatchKernel<T, TPR, SCHEME>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
        }
    }
    if (smem > 48 * 1024) {
        B2_CUDA(cudaFuncSetAttribute(rowQuantSmemKernel<T, TPR, SCHEME>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem)));
        B2_CUDA(cudaFuncSetAttribute(rowQuantSmemBatchKernel<T, TPR, SCHEME>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem)));
    }
    if (one) {
        const long long groups = (one->rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA;
        const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>(groups, 1LL << 30)));
        rowQuantSmemKernel<T, TPR, SCHEME><<<grid, 256, smem, ctx->stream>>>(*one);
    } else {
        rowQuantSmemBatchKernel<T, TPR, SCHEME>
                <<<static_cast<unsigned int>(totalGroups), 256, smem, ctx->stream>>>(itemsDev, startDev, nitems);
    }
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
}

// staged configuration: (element type, threads per row, scheme); maxu is 0
void launchSmemConfig(Context* ctx, const RegConfig& c, const RowQuantParams* one, const RowQuantParams* itemsDev,
                      const long long* startDev, int nitems, long long totalGroups, size_t smem) {
    const bool sym = c.scheme == B200C_QSYNTH_SYM_I8;
#define B2_SM_CASE(T_, TPR_)                                                                                              \
    if (sym) {                                                                                                            \
        launchSmemT<T_, TPR_, B200C_QSYNTH_SYM_I8>(ctx, one, itemsDev, startDev, nitems, totalGroups, smem);              \
    } else {                                                                                                              \
        launchSmemT<T_, TPR_, B200C_QSYNTH_ASYM_U4>(ctx, one, itemsDev, startDev, nitems, totalGroups, smem);             \
    }
#define B2_SM_TPR(T_)               \
    switch (c.tpr) {                \
    case 32:                        \
        B2_SM_CASE(T_, 32) break;   \
    case 64:                        \
        B2_SM_CASE(T_, 64) break;   \
    case 128:                       \
        B2_SM_CASE(T_, 128) break;  \
    default:                        \
        B2_SM_CASE(T_, 256) break;  \
    }
    if (c.srcTag == T_F16) {
        B2_SM_TPR(__half)
    } else {
        B2_SM_TPR(float)
    }
#undef B2_SM_TPR
#undef B2_SM_CASE
}

size_t smemBytesOf(const RowQuantParams& p, int tpr) {
    return static_cast<size_t>(256 / tpr) * p.smemRowElems * (p.srcTag == T_F16 ? 2 : 4);
}

// configuration of any item: register path when it fits, staged path otherwise (maxu == 0)
void pickConfig(const RowQuantParams& p, RegConfig* c) {
    if (pickRegConfig(p, c)) return;
    c->srcTag = p.srcTag;
    c->scheme = p.scheme;
    c->maxu = 0;
    // threads per row by the staged row's size: several short rows share a CTA, so the per-CTA start-up
    // (item lookup, parameter copy) is spread over more bytes and more loads are in flight per SM
    const long long rowBytes = p.rowElems * (p.srcTag == T_F16 ? 2 : 4);
    c->tpr = rowBytes <= 4096 ? 32 : rowBytes <= 16384 ? 64 : rowBytes <= 49152 ? 128 : 256;
}

}  // namespace

size_t rowQuantMaxRowBytes() {
    return 96 * 1024;
}

void launchRowQuantFused(Context* ctx, RowQuantParams p) {
    if (p.rows <= 0 || p.rowElems <= 0) return;
    const int es = p.srcTag == T_F16 ? 2 : 4;
    p.vecIn = ((reinterpret_cast<uintptr_t>(p.src) & 15) == 0 && (p.rowElems * es) % 16 == 0) ? 1 : 0;
    p.vecOut = ((reinterpret_cast<uintptr_t>(p.dst) & 15) == 0 && p.rowElems % 16 == 0) ? 1 : 0;
    // rows padded to 16 bytes in shared memory so every row slot stays 128-bit aligned
    p.smemRowElems = (p.rowElems * es + 15) / 16 * 16 / es;
    p.padLog2 = 31;  // no padding
    if (p.vecIn && p.vecOut && p.irank == 2 && p.ishape[1] % 16 == 0 && p.istride[1] > 1) {
        // two-level permutation read back with a stride: pad the staged row (see rowQuantSmemBody)
        int tz = 0;
        while (((p.istride[1] >> tz) & 1) == 0) ++tz;
        p.padLog2 = 6 + tz;
        p.smemRowElems += ((p.rowElems >> p.padLog2) + 1) * (16 / es);
    }
    if (ctx->batching) {
        ctx->rqBatch.push_back(p);  // launched by flushRowQuantBatch with its peers
        ctx->queuedBytes += p.rows * p.rowElems * es;
        return;
    }
    RegConfig c;
    pickConfig(p, &c);
    if (c.maxu > 0) {
        launchRegConfig(ctx, c, &p, nullptr, nullptr, 0, 0);
    } else {
        launchSmemConfig(ctx, c, &p, nullptr, nullptr, 0, 0, smemBytesOf(p, c.tpr));
    }
}

// Launch everything queued during a batched fold: one launch per kernel configuration.
void flushRowQuantBatch(Context* ctx) {
    std::vector<RowQuantParams> pending;
    pending.swap(ctx->rqBatch);
    std::vector<bool> done(pending.size(), false);
    for (size_t i = 0; i < pending.size(); ++i) {
        if (done[i]) continue;
        RegConfig c;
        pickConfig(pending[i], &c);
        std::vector<RowQuantParams> group;
        std::vector<long long> start;
        long long total = 0;
        size_t smem = 0;
        for (size_t j = i; j < pending.size(); ++j) {
            RegConfig cj;
            if (done[j]) continue;
            pickConfig(pending[j], &cj);
            if (!(cj == c)) continue;
            const int rowsPerCta = 256 / c.tpr;
            const long long groups = (pending[j].rows + rowsPerCta - 1) / rowsPerCta;
            if (total + groups > 0x7FFFFFFFLL) continue;  // next flush round
            done[j] = true;
            group.push_back(pending[j]);
            start.push_back(total);
            total += groups;
            if (c.maxu == 0) smem = std::max(smem, smemBytesOf(pending[j], c.tpr));
        }
        const bool one = group.size() == 1;
        RowQuantParams* itemsDev = nullptr;
        long long* startDev = nullptr;
        if (!one) {
            itemsDev = static_cast<RowQuantParams*>(ctx->arena.alloc(sizeof(RowQuantParams) * group.size()));
            appendCoarseIndex(start, total);
            startDev = static_cast<long long*>(ctx->arena.alloc(sizeof(long long) * start.size()));
            uploadSmall(ctx, itemsDev, group.data(), sizeof(RowQuantParams) * group.size());
            uploadSmall(ctx, startDev, start.data(), sizeof(long long) * start.size());
        }
        if (c.maxu > 0) {
            launchRegConfig(ctx, c, one ? &group[0] : nullptr, itemsDev, startDev, static_cast<int>(group.size()), total);
        } else {
            launchSmemConfig(ctx, c, one ? &group[0] : nullptr, itemsDev, startDev, static_cast<int>(group.size()), total,
                             smem);
        }
    }
}

}  // namespace b200c
