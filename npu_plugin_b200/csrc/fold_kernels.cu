// Fold kernels: the generic fused gather/convert/scatter pass, per-row statistics for the
// synthetic quantiser, the standalone swizzle copy and the bit-addressed SubView.
// All are HBM-bound byte/integer work; no tensor cores are involved.
#include "runtime.h"

#include <algorithm>
#include <cmath>

namespace b200c {

static inline int gridFor(const Context* ctx, long long units, int threads, int ctasPerSm) {
    const long long want = (units + threads - 1) / threads;
    const long long cap = static_cast<long long>(ctx->smCount) * ctasPerSm;
    return static_cast<int>(std::max<long long>(1, std::min(want, cap)));
}

// ---------------------------------------------------------------------------- generic pass
__global__ void __launch_bounds__(256) foldGenericKernel(const __grid_constant__ GenParams p, long long units) {
    const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long u = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; u < units; u += step) {
        genericUnit(p, u);
    }
}

void launchGeneric(Context* ctx, const GenParams& p) {
    const long long units = p.outUnits + std::max<long long>(0, p.totalBytes - p.dataBytes);
    if (units <= 0) return;
    foldGenericKernel<<<gridFor(ctx, units, 256, 8), 256, 0, ctx->stream>>>(p, units);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
}

// ---------------------------------------------------------------------------- ExpandDilated
// One output element per thread: positions whose kernel coordinates are multiples of the dilations
// take the source element, all others the fill value (expand_dilated.cpp:88-122).
B2_HD void expandDilatedUnit(const unsigned char* src, unsigned char* dst, int es, long long ky, long long kx, long long dky,
                             long long dkx, long long d0, long long d1, unsigned long long fill, long long o) {
    const long long x = o % dkx;
    const long long y = (o / dkx) % dky;
    const long long plane = o / (dkx * dky);
    unsigned long long bits = fill;
    if (y % d0 == 0 && x % d1 == 0) {
        const unsigned char* s = src + ((plane * ky + y / d0) * kx + x / d1) * es;
        bits = 0;
        for (int b = 0; b < es; ++b) bits |= static_cast<unsigned long long>(s[b]) << (8 * b);
    }
    for (int b = 0; b < es; ++b) dst[o * es + b] = static_cast<unsigned char>(bits >> (8 * b));
}

__global__ void __launch_bounds__(256) expandDilatedKernel(const unsigned char* __restrict__ src, unsigned char* __restrict__ dst,
                                                           int es, long long ky, long long kx, long long dky, long long dkx,
                                                           long long d0, long long d1, unsigned long long fill, long long n) {
    const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long o = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; o < n; o += step) {
        expandDilatedUnit(src, dst, es, ky, kx, dky, dkx, d0, d1, fill, o);
    }
}

void launchExpandDilated(Context* ctx, const void* src, void* dst, int es, long long planes, long long ky, long long kx,
                         long long dky, long long dkx, long long d0, long long d1, unsigned long long fill) {
    const long long n = planes * dky * dkx;
    if (n <= 0) return;
    const unsigned char* s = static_cast<const unsigned char*>(src);
    unsigned char* d = static_cast<unsigned char*>(dst);
    expandDilatedKernel<<<gridFor(ctx, n, 256, 8), 256, 0, ctx->stream>>>(s, d, es, ky, kx, dky, dkx, d0, d1, fill, n);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
}

// ---------------------------------------------------------------------------- RelocateWeightsTable
B2_HD void relocateUnit(const RelocateParams& p, long long oc) {
    int weightStep = 0, sparsityStep = 0;
    if (p.oc >= 2) {
        weightStep = p.values[4] - p.values[0];
        sparsityStep = p.values[5] - p.values[1];
    }
    const int c = p.clusterOf[oc];
    const long long rel = oc - p.offsets[c];
    const long long step = p.steps ? p.steps[oc] : static_cast<long long>(weightStep) * rel;
    const long long at = oc * 4;
    int err = E_NONE;
    const long long w = p.weightsPtr[c] + step;
    if (w < -2147483648ll || w > 2147483647ll) err = E_CAST_RANGE;
    p.patched[at] = static_cast<int>(w);
    int sp = p.values[at + 1];
    if (sp != 0xFFFFFF) {  // SPARSITY_PTR_WHEN_NO_SPARSITY
        const long long v = p.sparsityPtr + rel * static_cast<long long>(sparsityStep);
        if (v < -2147483648ll || v > 2147483647ll) err = E_CAST_RANGE;
        sp = static_cast<int>(v);
    }
    p.patched[at + 1] = sp;
    p.patched[at + 2] = p.values[at + 2];
    p.patched[at + 3] = p.values[at + 3];
    if (err != E_NONE) {
#ifdef __CUDA_ARCH__
        atomicCAS(p.err, E_NONE, err);
#else
        if (*p.err == E_NONE) *p.err = err;
#endif
    }
}

__global__ void __launch_bounds__(256) relocateWeightsTableKernel(const __grid_constant__ RelocateParams p) {
    const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long oc = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; oc < p.oc; oc += step) relocateUnit(p, oc);
}

void launchRelocateWeightsTable(Context* ctx, const RelocateParams& p) {
    if (p.oc <= 0) return;
    relocateWeightsTableKernel<<<gridFor(ctx, p.oc, 256, 8), 256, 0, ctx->stream>>>(p);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
}

// ---------------------------------------------------------------------------- row statistics
struct RowAcc {
    float mx, mn, amax;
};

B2_HD void rowCoords(const RowStatsParams& rp, long long row, long long j, long long* coord) {
    const GenParams& p = rp.view;
    for (int k = p.rank - 1; k >= 0; --k) {
        if (k == rp.rowDim) {
            coord[k] = row;
            continue;
        }
        const long long s = p.shape[k];
        const long long q = j / s;
        coord[k] = j - q * s;
        j = q;
    }
}

B2_HD void rowFinish(const RowStatsParams& rp, long long row, RowAcc a) {
    float scale;
    int zp = 0;
    if (rp.scheme == B200C_QSYNTH_SYM_I8) {
        scale = divRn(a.amax, 127.0f);
        if (!(scale > 0.0f)) scale = 1.0f;
    } else {
        scale = divRn(a.mx - a.mn, 15.0f);
        if (!(scale > 0.0f)) scale = 1.0f;
        float z = rintHalfEven(divRn(-a.mn, scale));
        z = fminf(fmaxf(z, 0.0f), 15.0f);
        zp = static_cast<int>(z);
    }
    rp.scales[row] = scale;
    rp.zps[row] = zp;
}

__global__ void __launch_bounds__(256) rowStatsKernel(const __grid_constant__ RowStatsParams rp) {
    __shared__ float smx[8], smn[8], sam[8];
    for (long long row = blockIdx.x; row < rp.rows; row += gridDim.x) {
        RowAcc a;
        a.mx = -INFINITY;
        a.mn = INFINITY;
        a.amax = 0.0f;
        int err = E_NONE;
        long long coord[kMaxDims];
        for (long long j = threadIdx.x; j < rp.rowElems; j += blockDim.x) {
            rowCoords(rp, row, j, coord);
            const float w = toFloatChecked(evalAt(rp.view, coord, err), err);
            a.mx = fmaxf(a.mx, w);
            a.mn = fminf(a.mn, w);
            a.amax = fmaxf(a.amax, fabsf(w));
        }
        for (int o = 16; o > 0; o >>= 1) {
            a.mx = fmaxf(a.mx, __shfl_xor_sync(0xFFFFFFFFu, a.mx, o));
            a.mn = fminf(a.mn, __shfl_xor_sync(0xFFFFFFFFu, a.mn, o));
            a.amax = fmaxf(a.amax, __shfl_xor_sync(0xFFFFFFFFu, a.amax, o));
        }
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (lane == 0) {
            smx[warp] = a.mx;
            smn[warp] = a.mn;
            sam[warp] = a.amax;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < 8; ++w) {
                a.mx = fmaxf(a.mx, smx[w]);
                a.mn = fminf(a.mn, smn[w]);
                a.amax = fmaxf(a.amax, sam[w]);
            }
            rowFinish(rp, row, a);
        }
        if (err != E_NONE) atomicCAS(rp.view.err, E_NONE, err);
        __syncthreads();
    }
}

void launchRowStats(Context* ctx, const RowStatsParams& rp) {
    const int grid = static_cast<int>(std::min<long long>(rp.rows, static_cast<long long>(ctx->smCount) * 8));
    rowStatsKernel<<<grid, 256, 0, ctx->stream>>>(rp);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
}

// ---------------------------------------------------------------------------- swizzle copy
// dst[swizzle(a)] = src[a] for every 16-byte chunk a of [0, totalBytes); bytes beyond srcBytes
// read as tailByte (SwizzleConstant's size alignment padding).
B2_HD void swizzleChunk(const unsigned char* src, long long srcBytes, unsigned char* dst, long long chunk, int key,
                        int tailByte) {
    const long long a = chunk << 4;
    const long long d = swizzleAddr(a, key);
    for (int i = 0; i < 16; ++i) {
        dst[d + i] = (a + i < srcBytes) ? src[a + i] : static_cast<unsigned char>(tailByte);
    }
}

__global__ void __launch_bounds__(256) swizzleCopyKernel(const unsigned char* __restrict__ src, long long srcBytes,
                                                         unsigned char* __restrict__ dst, long long chunks, int key,
                                                         int tailByte, int aligned) {
    const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long c = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; c < chunks; c += step) {
        const long long a = c << 4;
        if (aligned && a + 16 <= srcBytes) {
            const uint4 v = *reinterpret_cast<const uint4*>(src + a);
            *reinterpret_cast<uint4*>(dst + swizzleAddr(a, key)) = v;
        } else {
            swizzleChunk(src, srcBytes, dst, c, key, tailByte);
        }
    }
}

void launchSwizzleCopy(Context* ctx, const void* src, long long srcBytes, void* dst, long long totalBytes, int key,
                       int tailByte) {
    const long long chunks = (totalBytes + 15) >> 4;
    if (chunks <= 0) return;
    const unsigned char* s = static_cast<const unsigned char*>(src);
    unsigned char* d = static_cast<unsigned char*>(dst);
    const int aligned = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
    swizzleCopyKernel<<<gridFor(ctx, chunks, 256, 8), 256, 0, ctx->stream>>>(s, srcBytes, d, chunks, key, tailByte,
                                                                              aligned);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
}

// ---------------------------------------------------------------------------- SubView on packed i1
struct BitViewParams {
    const unsigned char* src;
    unsigned char* dst;
    int rank;
    long long outShape[kMaxDims];
    long long inStride[kMaxDims];
    long long base;
    long long outBits;
};

// bit k of a byte is element k (subview.cpp:158-169)
B2_HD void subViewByte(const BitViewParams& p, long long byteIdx) {
    unsigned int byte = 0;
    for (int b = 0; b < 8; ++b) {
        long long o = byteIdx * 8 + b;
        if (o >= p.outBits) break;
        long long in = p.base;
        for (int k = p.rank - 1; k >= 0; --k) {
            const long long s = p.outShape[k];
            const long long q = o / s;
            in += (o - q * s) * p.inStride[k];
            o = q;
        }
        byte |= ((p.src[in >> 3] >> (in & 7)) & 1u) << b;
    }
    p.dst[byteIdx] = static_cast<unsigned char>(byte);
}

__global__ void __launch_bounds__(256) subViewBitsKernel(const __grid_constant__ BitViewParams p, long long bytes) {
    const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < bytes; i += step) {
        subViewByte(p, i);
    }
}

void launchSubViewBits(Context* ctx, const void* src, void* dst, int rank, const long long* outShape,
                       const long long* inStride, long long base, long long outBits) {
    BitViewParams p;
    p.src = static_cast<const unsigned char*>(src);
    p.dst = static_cast<unsigned char*>(dst);
    p.rank = rank;
    for (int k = 0; k < rank; ++k) {
        p.outShape[k] = outShape[k];
        p.inStride[k] = inStride[k];
    }
    p.base = base;
    p.outBits = outBits;
    const long long bytes = (outBits + 7) / 8;
    subViewBitsKernel<<<gridFor(ctx, bytes, 256, 8), 256, 0, ctx->stream>>>(p, bytes);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
}

}  // namespace b200c
