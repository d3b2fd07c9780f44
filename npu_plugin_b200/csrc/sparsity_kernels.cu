// Sparsity kernels: GetSparsityMap (1 bit per element, LSB first, per-channel rows padded to
// 128 bits) and Sparsify (per-channel compaction with 16-byte aligned channel starts), restating
// src/vpux_compiler/src/dialect/const/attributes/get_sparsity_map.cpp:23-107,
// sparsify.cpp:115-186 and src/vpux_compiler/src/utils/sparsity.cpp:28-72 as count -> scan -> scatter.
// Inputs are dense [OC][work] buffers of si8/ui8/f16/bf16/f32 elements.
#include "runtime.h"

#include <algorithm>
#include <unordered_map>
#include <vector>

namespace b200c {

// element != sparse value, with float semantics for the float types (ov::float16 compares as float)
B2_HD bool differs(const void* src, long long idx, int tag, unsigned long long sparseBits) {
    switch (tag) {
    case T_I8:
    case T_U8:
        return static_cast<const unsigned char*>(src)[idx] != static_cast<unsigned char>(sparseBits);
    case T_F16:
        return halfBitsToFloat(static_cast<const unsigned short*>(src)[idx]) !=
               halfBitsToFloat(static_cast<unsigned short>(sparseBits));
    case T_BF16:
        return bf16BitsToFloat(static_cast<const unsigned short*>(src)[idx]) !=
               bf16BitsToFloat(static_cast<unsigned short>(sparseBits));
    default:
        return bitsToFloat(static_cast<const unsigned int*>(src)[idx]) !=
               bitsToFloat(static_cast<unsigned int>(sparseBits));
    }
}

// ---------------------------------------------------------------------------- GetSparsityMap
struct MapParams {
    const void* src;
    unsigned char* dst;
    int tag;
    long long oc, work, outBytesPerOC;
    unsigned long long sparseBits;
    int swizzleKey;
};

// one output byte: 8 consecutive elements of one channel, element k -> bit k; bytes past the
// channel's data are the zero fill of the 128-bit alignment
B2_HD void mapByte(const MapParams& p, long long byteIdx) {
    const long long oc = byteIdx / p.outBytesPerOC;
    const long long j = byteIdx - oc * p.outBytesPerOC;
    unsigned int byte = 0;
    if (j * 8 < p.work) {
        const long long first = oc * p.work + j * 8;
        for (int b = 0; b < 8; ++b) byte |= static_cast<unsigned int>(differs(p.src, first + b, p.tag, p.sparseBits)) << b;
    }
    p.dst[swizzleAddr(byteIdx, p.swizzleKey)] = static_cast<unsigned char>(byte);
}

__global__ void __launch_bounds__(256) sparsityMapKernel(const __grid_constant__ MapParams p, long long bytes) {
    const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < bytes; i += step) mapByte(p, i);
}

// 8-bit elements, work % 16 == 0 and 16-byte aligned rows: one 128-bit load -> 16 mask bits per thread.
// The per-byte "not equal" flags are gathered into a nibble with one multiply.
__global__ void __launch_bounds__(256) sparsityMapBytesKernel(const __grid_constant__ MapParams p, long long units,
                                                              long long unitsPerOC, long long dataUnitsPerOC) {
    const unsigned int sv = static_cast<unsigned int>(p.sparseBits & 0xFF) * 0x01010101u;
    const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long u = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; u < units; u += step) {
        const long long oc = u / unitsPerOC;
        const long long j = u - oc * unitsPerOC;
        unsigned int mask16 = 0;
        if (j < dataUnitsPerOC) {
            const uint4 v = *reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(p.src) + oc * p.work + j * 16);
            const unsigned int w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const unsigned int ne = (__vcmpne4(w[i], sv) >> 7) & 0x01010101u;
                mask16 |= ((ne * 0x01020408u) >> 24 & 0xFu) << (4 * i);
            }
        }
        const long long a = u * 2;  // two output bytes; a 16-byte swizzle chunk is never split
        *reinterpret_cast<unsigned short*>(p.dst + swizzleAddr(a, p.swizzleKey)) = static_cast<unsigned short>(mask16);
    }
}

void launchSparsityMap(Context* ctx, const void* src, int tag, long long oc, long long work, long long outBitsPerOC,
                       unsigned long long sparseBits, void* dstBits, int swizzleKey) {
    MapParams p;
    p.src = src;
    p.dst = static_cast<unsigned char*>(dstBits);
    p.tag = tag;
    p.oc = oc;
    p.work = work;
    p.outBytesPerOC = outBitsPerOC / 8;
    p.sparseBits = sparseBits;
    p.swizzleKey = swizzleKey;
    const long long bytes = oc * p.outBytesPerOC;
    if (bytes <= 0) return;
    const bool fast = tagBytes(tag) == 1 && work % 16 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(dstBits) & 1) == 0;
    if (fast) {
        const long long unitsPerOC = p.outBytesPerOC / 2, units = oc * unitsPerOC;
        const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>((units + 255) / 256, ctx->smCount * 8LL)));
        sparsityMapBytesKernel<<<grid, 256, 0, ctx->stream>>>(p, units, unitsPerOC, work / 16);
    } else {
        const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>((bytes + 255) / 256, ctx->smCount * 8LL)));
        sparsityMapKernel<<<grid, 256, 0, ctx->stream>>>(p, bytes);
    }
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
}

// ---------------------------------------------------------------------------- count per channel
__global__ void __launch_bounds__(256) countNonSparseKernel(const void* __restrict__ src, int tag, long long oc,
                                                            long long work, unsigned long long sparseBits,
                                                            long long* __restrict__ counts) {
    __shared__ long long part[8];
    for (long long c = blockIdx.x; c < oc; c += gridDim.x) {
        long long n = 0;
        const long long first = c * work;
        if (tagBytes(tag) == 1 && ((reinterpret_cast<uintptr_t>(src) + first) & 15) == 0) {
            const unsigned int sv = static_cast<unsigned int>(sparseBits & 0xFF) * 0x01010101u;
            const unsigned char* row = static_cast<const unsigned char*>(src) + first;
            const long long vec = work / 16;
            for (long long j = threadIdx.x; j < vec; j += blockDim.x) {
                const uint4 v = *reinterpret_cast<const uint4*>(row + j * 16);
                n += (__popc(__vcmpne4(v.x, sv)) + __popc(__vcmpne4(v.y, sv)) + __popc(__vcmpne4(v.z, sv)) +
                      __popc(__vcmpne4(v.w, sv))) >> 3;
            }
            for (long long j = vec * 16 + threadIdx.x; j < work; j += blockDim.x) n += row[j] != (sparseBits & 0xFF);
        } else {
            for (long long j = threadIdx.x; j < work; j += blockDim.x) n += differs(src, first + j, tag, sparseBits);
        }
        for (int o = 16; o > 0; o >>= 1) n += __shfl_xor_sync(0xFFFFFFFFu, n, o);
        if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = n;
        __syncthreads();
        if (threadIdx.x == 0) {
            long long t = 0;
            for (int w = 0; w < 8; ++w) t += part[w];
            counts[c] = t;
        }
        __syncthreads();
    }
}

void launchCountNonSparse(Context* ctx, const void* src, int tag, long long oc, long long work,
                          unsigned long long sparseBits, long long* counts) {
    if (oc <= 0) return;
    const int grid = static_cast<int>(std::min<long long>(oc, ctx->smCount * 8LL));
    countNonSparseKernel<<<grid, 256, 0, ctx->stream>>>(src, tag, oc, work, sparseBits, counts);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
}

// ---------------------------------------------------------------------------- channel offsets
// offsets[c] = sum over earlier channels of align16(count * elemBytes); *total = the full sum.
// One CTA walks the channels in tiles of 1024 with a shuffle-based block scan (no inter-CTA waits).
__global__ void __launch_bounds__(1024) sparsifyOffsetsKernel(const long long* __restrict__ counts, long long oc,
                                                              int elemBytes, long long* __restrict__ offsets,
                                                              long long* __restrict__ total) {
    __shared__ long long warpSum[32];
    __shared__ long long carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (long long tile = 0; tile < oc; tile += blockDim.x) {
        const long long c = tile + threadIdx.x;
        const long long mine = c < oc ? ((counts[c] * elemBytes + 15) & ~15ll) : 0;
        long long incl = mine;
        for (int o = 1; o < 32; o <<= 1) {
            const long long t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warpSum[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            long long w = warpSum[lane];
            for (int o = 1; o < 32; o <<= 1) {
                const long long t = __shfl_up_sync(0xFFFFFFFFu, w, o);
                if (lane >= o) w += t;
            }
            warpSum[lane] = w;
        }
        __syncthreads();
        const long long before = carry + (warp ? warpSum[warp - 1] : 0) + incl - mine;
        if (c < oc) offsets[c] = before;
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = before + mine;
        __syncthreads();
    }
    if (threadIdx.x == 0) *total = carry;
}

void launchSparsifyOffsets(Context* ctx, const long long* counts, long long oc, int elemBytes, long long* offsets,
                           long long* total) {
    sparsifyOffsetsKernel<<<1, 1024, 0, ctx->stream>>>(counts, oc, elemBytes, offsets, total);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
}

// ---------------------------------------------------------------------------- compaction
// One CTA per channel keeps the element order: every round takes blockDim consecutive elements,
// ranks the survivors with ballot/popc inside each warp and a small shared-memory scan across warps.
__global__ void __launch_bounds__(256) sparsifyScatterKernel(const void* __restrict__ src, int tag, long long oc,
                                                             long long work, unsigned long long sparseBits,
                                                             const long long* __restrict__ offsets,
                                                             unsigned char* __restrict__ dst, long long dstBytes,
                                                             int swizzleKey, int* err) {
    __shared__ int warpCount[8];
    __shared__ long long running;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int eb = tagBytes(tag);
    for (long long c = blockIdx.x; c < oc; c += gridDim.x) {
        if (threadIdx.x == 0) running = offsets[c];
        __syncthreads();
        for (long long tile = 0; tile < work; tile += blockDim.x) {
            const long long j = tile + threadIdx.x;
            const long long idx = c * work + j;
            const bool keep = j < work && differs(src, idx, tag, sparseBits);
            const unsigned int votes = __ballot_sync(0xFFFFFFFFu, keep);
            if (lane == 0) warpCount[warp] = __popc(votes);
            __syncthreads();
            int before = __popc(votes & ((1u << lane) - 1u));
            for (int w = 0; w < warp; ++w) before += warpCount[w];
            if (keep) {
                const long long at = running + static_cast<long long>(before) * eb;
                if (at + eb > dstBytes) {
                    atomicCAS(err, E_NONE, E_SPARSE_OVERFLOW);
                } else {
                    storeRawAt(dst, swizzleAddr(at, swizzleKey), eb, loadRaw(src, idx, tag));
                }
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                int all = 0;
                for (int w = 0; w < 8; ++w) all += warpCount[w];
                running += static_cast<long long>(all) * eb;
            }
            __syncthreads();
        }
    }
}

void launchSparsifyScatter(Context* ctx, const void* src, int tag, long long oc, long long work,
                           unsigned long long sparseBits, const long long* offsets, void* dst, long long dstBytes,
                           int swizzleKey, int* err) {
    if (oc <= 0 || work <= 0) return;
    const int grid = static_cast<int>(std::min<long long>(oc, ctx->smCount * 8LL));
    sparsifyScatterKernel<<<grid, 256, 0, ctx->stream>>>(src, tag, oc, work, sparseBits, offsets,
                                                         static_cast<unsigned char*>(dst), dstBytes, swizzleKey, err);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
}

// ---------------------------------------------------------------------------- batched 8-bit paths
// Many tensors per launch; a CTA (or warp) finds its item with a binary search over prefix sums.
namespace {

// 0x80 in every byte of w that differs from the matching byte of sv4
__device__ __forceinline__ unsigned int neBytes(unsigned int w, unsigned int sv4) {
    const unsigned int y = w ^ sv4;
    return (((y & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | y) & 0x80808080u;
}

// bit k set when byte k of the 16-byte vector differs from the sparse value
__device__ __forceinline__ unsigned int neMask16(const uint4& v, unsigned int sv4) {
    const unsigned int w[4] = {v.x, v.y, v.z, v.w};
    unsigned int m = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const unsigned int ne = neBytes(w[i], sv4) >> 7;  // 0x01 per differing byte
        m |= (((ne * 0x01020408u) >> 24) & 0xFu) << (4 * i);
    }
    return m;
}

constexpr int kMapUnitsPerCta = 2048;  // 16 input bytes -> 2 map bytes per unit, 8 units per thread
constexpr int kMapMaxChanPerCta = 256;  // map rows are at least 16 bytes (8 units)

// A CTA covers 2048 units (32 KB of elements -> 4 KB of map); in every round a warp loads 32 consecutive
// units (512 coalesced bytes), the 16-bit masks of 8 neighbouring lanes are joined with shuffles and every
// eighth lane stores one whole 16-byte chunk through the swizzle rotation.  Index arithmetic is 32-bit
// relative to the CTA's first channel (a shift when the units per channel are a power of two).
//
// When a Sparsify of the same batch reads the same source (it.counts), the per-channel counts it needs
// fall out of this pass: every unit adds the population count of its mask to a shared-memory counter
// of its channel, and the CTA writes the counters of the channels it covers.  The host only asks for
// this when CTAs cover whole channels (kMapUnitsPerCta is a multiple of the units per channel).
__global__ void __launch_bounds__(256) sparsityMapBatchKernel(const MapItem* __restrict__ items,
                                                              const long long* __restrict__ ctaStart, int nitems) {
    __shared__ int chanCount[kMapMaxChanPerCta];
    const int k = findBatchItem(ctaStart, nitems, blockIdx.x);
    const MapItem it = items[k];
    const unsigned int sv4 = it.sparseByte * 0x01010101u;
    const long long unitsPerOC = it.outBytesPerOC / 2;
    const long long units = (it.totalBytes + 1) / 2, mapUnits = it.oc * unitsPerOC;  // both multiples of 8
    const long long first = (blockIdx.x - ctaStart[k]) * kMapUnitsPerCta;
    const bool counting = it.counts != nullptr;
    const long long oc0 = first / unitsPerOC;  // first channel of this CTA (counting: CTAs start on channel boundaries)
    const unsigned int rem0 = static_cast<unsigned int>(first - oc0 * unitsPerOC);
    const unsigned int upo = static_cast<unsigned int>(unitsPerOC);
    const int upoShift = (upo & (upo - 1)) == 0 ? 31 - __clz(upo) : -1;
    const unsigned int dataUnits = static_cast<unsigned int>(it.work / 16);
    const unsigned int work = static_cast<unsigned int>(it.work);
    // units of this CTA that belong to the map / that are written at all
    const unsigned int liveMap = static_cast<unsigned int>(min(static_cast<long long>(kMapUnitsPerCta), max(0ll, mapUnits - first)));
    const unsigned int liveAll = static_cast<unsigned int>(min(static_cast<long long>(kMapUnitsPerCta), max(0ll, units - first)));
    const unsigned char* src0 = it.src + oc0 * it.work;
    const int lane = threadIdx.x & 31;
    if (counting) {
        chanCount[threadIdx.x] = 0;
        __syncthreads();
    }
    constexpr int R = kMapUnitsPerCta / 256;
    uint4 x[R];
    unsigned int chan[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {  // all loads of the thread are issued before the first is used
        const unsigned int local = r * 256 + threadIdx.x;
        const unsigned int at = rem0 + local;
        const unsigned int dc = upoShift >= 0 ? (at >> upoShift) : (at / upo);
        const unsigned int j = at - dc * upo;
        chan[r] = dc;
        x[r] = make_uint4(sv4, sv4, sv4, sv4);  // padding units compare equal everywhere: mask 0
        if (local < liveMap && j < dataUnits) {
            x[r] = __ldg(reinterpret_cast<const uint4*>(src0 + static_cast<unsigned long long>(dc) * work) + j);
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const unsigned int local = r * 256 + threadIdx.x;
        const unsigned int mask16 = neMask16(x[r], sv4);
        if (counting) {
            const int n = __popc(mask16);
            if (upo >= 32) {
                // the 32 units of a warp lie in one channel (the units per channel are a multiple of 32)
                const int total = __reduce_add_sync(0xFFFFFFFFu, n);
                if (lane == 0 && total) atomicAdd(&chanCount[chan[r]], total);
            } else if (n) {
                atomicAdd(&chanCount[chan[r]], n);
            }
        }
        // eight neighbouring lanes -> one 16-byte chunk in the first of them
        const unsigned int m32 = mask16 | (__shfl_down_sync(0xFFFFFFFFu, mask16, 1) << 16);
        const unsigned int b = __shfl_down_sync(0xFFFFFFFFu, m32, 2);
        const unsigned int c = __shfl_down_sync(0xFFFFFFFFu, m32, 4);
        const unsigned int d = __shfl_down_sync(0xFFFFFFFFu, b, 4);
        if ((lane & 7) == 0 && local < liveAll) {
            const long long a = (first + local) * 2;  // a 16-byte swizzle chunk is never split
            *reinterpret_cast<uint4*>(it.dst + swizzleAddr(a, it.swizzleKey)) = make_uint4(m32, b, c, d);
        }
    }
    if (counting) {
        __syncthreads();
        const long long oc = oc0 + threadIdx.x;
        if (threadIdx.x < kMapUnitsPerCta / unitsPerOC && oc < it.oc) it.counts[oc] = chanCount[threadIdx.x];
    }
}

// one warp per kChanPerWarp consecutive channels (the item lookup is paid once per warp)
constexpr int kChanPerWarp = 4;

__device__ __forceinline__ int nextItem(const long long* __restrict__ chanStart, int nitems, int k, long long ch) {
    while (k + 1 < nitems && chanStart[k + 1] <= ch) ++k;
    return k;
}

__global__ void __launch_bounds__(256) sparseCountBatchKernel(const SparseItem* __restrict__ items,
                                                              const long long* __restrict__ chanStart, int nitems,
                                                              long long nchan) {
    const long long ch0 = (static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5)) * kChanPerWarp;
    if (ch0 >= nchan) return;
    const int lane = threadIdx.x & 31;
    int k = findBatchItem(chanStart, nitems, ch0);
    for (int q = 0; q < kChanPerWarp; ++q) {
        const long long ch = ch0 + q;
        if (ch >= nchan) break;
        k = nextItem(chanStart, nitems, k, ch);
        const SparseItem& it = items[k];
        if (it.countsReady) continue;  // counted by the sparsity-map kernel of the same source
        const long long c = ch - chanStart[k];
        const unsigned int sv4 = it.sparseByte * 0x01010101u;
        const uint4* row = reinterpret_cast<const uint4*>(it.src + c * it.work);
        const long long nvec = it.work / 16;
        int n = 0;
        for (long long v = lane; v < nvec; v += 32) {
            const uint4 x = __ldg(row + v);
            n += __popc(neBytes(x.x, sv4)) + __popc(neBytes(x.y, sv4)) + __popc(neBytes(x.z, sv4)) + __popc(neBytes(x.w, sv4));
        }
        for (int o = 16; o > 0; o >>= 1) n += __shfl_xor_sync(0xFFFFFFFFu, n, o);
        if (lane == 0) it.counts[c] = n;
    }
}

// one CTA per item: channel offsets (16-byte aligned channel starts) and the size of the result
__global__ void __launch_bounds__(1024) sparseOffsetsBatchKernel(const SparseItem* __restrict__ items) {
    __shared__ long long warpSum[32];
    __shared__ long long carry;
    const SparseItem& it = items[blockIdx.x];
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (long long tile = 0; tile < it.oc; tile += blockDim.x) {
        const long long c = tile + threadIdx.x;
        const long long mine = c < it.oc ? ((it.counts[c] + 15) & ~15ll) : 0;
        long long incl = mine;
        for (int o = 1; o < 32; o <<= 1) {
            const long long t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warpSum[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            long long w = warpSum[lane];
            for (int o = 1; o < 32; o <<= 1) {
                const long long t = __shfl_up_sync(0xFFFFFFFFu, w, o);
                if (lane >= o) w += t;
            }
            warpSum[lane] = w;
        }
        __syncthreads();
        const long long before = carry + (warp ? warpSum[warp - 1] : 0) + incl - mine;
        if (c < it.oc) it.offsets[c] = before;
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = before + mine;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        it.offsets[it.oc] = carry;
        const long long buffer = it.fixedBytes >= 0 ? it.fixedBytes : carry;
        *it.bytesOut = it.swizzleKey >= 0 ? ((buffer + 511) & ~511ll) : buffer;
    }
}

// One warp per channel keeps the element order: every round takes 32 x 16 elements, ranks the
// survivors with popc and a warp scan, compacts them into a shared-memory staging line and writes
// whole 16-byte chunks (channel starts are 16-byte aligned, so chunks never straddle channels and
// the swizzle rotation applies to them directly).  The last chunk of a channel is padded with
// zeros; the warp of the last channel also zeroes the rest of the buffer.
__global__ void __launch_bounds__(256) sparseScatterBatchKernel(const SparseItem* __restrict__ items,
                                                                const long long* __restrict__ chanStart, int nitems,
                                                                long long nchan) {
    __shared__ __align__(16) unsigned char stage[8][544];
    const long long ch0 = (static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5)) * kChanPerWarp;
    if (ch0 >= nchan) return;
    const int lane = threadIdx.x & 31;
    unsigned char* st = stage[threadIdx.x >> 5];
    int k = findBatchItem(chanStart, nitems, ch0);
    for (int q = 0; q < kChanPerWarp; ++q) {
    const long long ch = ch0 + q;
    if (ch >= nchan) break;
    k = nextItem(chanStart, nitems, k, ch);
    const SparseItem& it = items[k];
    const long long c = ch - chanStart[k];
    const unsigned int sv4 = it.sparseByte * 0x01010101u;
    const uint4* row = reinterpret_cast<const uint4*>(it.src + c * it.work);
    const long long nvec = it.work / 16;
    const long long written = *it.bytesOut;                                    // size of the result
    const long long dataEnd = it.fixedBytes >= 0 ? it.fixedBytes : written;   // values must end here
    const long long cap = min(written, it.dstCap);
    long long outPos = it.offsets[c];
    int fill = 0;
    bool overflow = false;
    uint4 ahead = lane < nvec ? __ldg(row + lane) : make_uint4(0, 0, 0, 0);  // the next round's vector is always in flight
    for (long long base = 0; base < nvec; base += 32) {
        const long long v = base + lane;
        const uint4 x = ahead;
        if (v + 32 < nvec) ahead = __ldg(row + v + 32);
        const unsigned int m = v < nvec ? neMask16(x, sv4) : 0u;
        const int cnt = __popc(m);
        int incl = cnt;
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += t;
        }
        int pos = fill + incl - cnt;
        const unsigned int w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if ((m >> i) & 1u) st[pos++] = static_cast<unsigned char>(w[i >> 2] >> (8 * (i & 3)));
        }
        fill += __shfl_sync(0xFFFFFFFFu, incl, 31);
        __syncwarp();
        const int nch = fill >> 4, rem = fill & 15;
        if (lane < nch) {
            const long long a = outPos + lane * 16;
            if (a + 16 > dataEnd) {
                overflow = true;
            } else if (a + 16 <= cap) {
                *reinterpret_cast<uint4*>(it.dst + swizzleAddr(a, it.swizzleKey)) = *reinterpret_cast<const uint4*>(st + lane * 16);
            }
        }
        const unsigned char keep = lane < rem ? st[nch * 16 + lane] : 0;
        __syncwarp();
        if (lane < rem) st[lane] = keep;
        __syncwarp();
        outPos += static_cast<long long>(nch) * 16;
        fill = rem;
    }
    if (fill > 0) {
        if (lane >= fill && lane < 16) st[lane] = 0;
        __syncwarp();
        if (lane == 0) {
            if (outPos + 16 > dataEnd) {
                overflow = true;
            } else if (outPos + 16 <= cap) {
                *reinterpret_cast<uint4*>(it.dst + swizzleAddr(outPos, it.swizzleKey)) = *reinterpret_cast<const uint4*>(st);
            }
        }
        outPos += 16;
    }
    if (overflow) atomicCAS(it.err, E_NONE, E_SPARSE_OVERFLOW);
    if (c == it.oc - 1) {  // zero fill behind the last channel (16-byte chunks, then bytes)
        long long a = outPos + lane * 16ll;
        for (; a + 16 <= cap; a += 512) *reinterpret_cast<uint4*>(it.dst + swizzleAddr(a, it.swizzleKey)) = make_uint4(0, 0, 0, 0);
        const long long tailAt = outPos + ((cap > outPos ? cap - outPos : 0) / 16) * 16;
        for (long long b = tailAt + lane; b < cap; b += 32) it.dst[swizzleAddr(b, it.swizzleKey)] = 0;
    }
    __syncwarp();  // the staging line is reused by the next channel
    }
}

__global__ void gatherWordsKernel(const long long* const* __restrict__ ptrs, long long* __restrict__ out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = *ptrs[i];
}

template <typename T>
T* uploadItems(Context* ctx, const std::vector<T>& v) {
    T* d = static_cast<T*>(ctx->arena.alloc(sizeof(T) * v.size()));
    uploadSmall(ctx, d, v.data(), sizeof(T) * v.size());
    return d;
}

void runMapItems(Context* ctx, const std::vector<MapItem>& items) {
    if (items.empty()) return;
    std::vector<long long> start;
    long long ctas = 0;
    for (const MapItem& it : items) {
        start.push_back(ctas);
        ctas += ((it.totalBytes + 1) / 2 + kMapUnitsPerCta - 1) / kMapUnitsPerCta;
    }
    if (ctas <= 0 || ctas > 0x7FFFFFFFLL) throw NotBuilt("sparsity map batch too large for one launch");
    appendCoarseIndex(start, ctas);
    sparsityMapBatchKernel<<<static_cast<unsigned int>(ctas), 256, 0, ctx->stream>>>(uploadItems(ctx, items), uploadItems(ctx, start),
                                                                                      static_cast<int>(items.size()));
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
}

void runSparseItems(Context* ctx, const std::vector<SparseItem>& items) {
    if (items.empty()) return;
    std::vector<long long> start;
    long long nchan = 0;
    for (const SparseItem& it : items) {
        start.push_back(nchan);
        nchan += it.oc;
    }
    const long long ctas = (nchan + 8 * kChanPerWarp - 1) / (8 * kChanPerWarp);
    if (ctas <= 0 || ctas > 0x7FFFFFFFLL) throw NotBuilt("sparsify batch too large for one launch");
    appendCoarseIndex(start, nchan);
    const SparseItem* d = uploadItems(ctx, items);
    const long long* ds = uploadItems(ctx, start);
    const int n = static_cast<int>(items.size());
    sparseCountBatchKernel<<<static_cast<unsigned int>(ctas), 256, 0, ctx->stream>>>(d, ds, n, nchan);
    B2_CUDA(cudaGetLastError());
    sparseOffsetsBatchKernel<<<n, 1024, 0, ctx->stream>>>(d);
    B2_CUDA(cudaGetLastError());
    sparseScatterBatchKernel<<<static_cast<unsigned int>(ctas), 256, 0, ctx->stream>>>(d, ds, n, nchan);
    B2_CUDA(cudaGetLastError());
    ctx->launches += 3;
}

}  // namespace

void launchMapItem(Context* ctx, const MapItem& it) {
    if (it.totalBytes <= 0) return;
    if (ctx->batching) {
        ctx->mapBatch.push_back(it);
        ctx->queuedBytes += it.oc * it.work;
        return;
    }
    runMapItems(ctx, std::vector<MapItem>(1, it));
}

void launchSparseItem(Context* ctx, const SparseItem& it) {
    if (ctx->batching) {
        ctx->sparseBatch.push_back(it);
        ctx->queuedBytes += it.oc * it.work;
        return;
    }
    runSparseItems(ctx, std::vector<SparseItem>(1, it));
}

// out[i] = *ptrs[i] for n device words scattered over scratch memory: one launch and one copy
// instead of n small copies
void gatherDeviceWords(Context* ctx, const std::vector<const long long*>& ptrs, long long* hostOut) {
    if (ptrs.empty()) return;
    const int n = static_cast<int>(ptrs.size());
    const long long* const* d = uploadItems(ctx, ptrs);
    long long* out = static_cast<long long*>(ctx->arena.alloc(sizeof(long long) * ptrs.size()));
    gatherWordsKernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>(d, out, n);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
    copyD2H(ctx, hostOut, out, sizeof(long long) * ptrs.size());
}

void flushSparsityBatch(Context* ctx) {
    std::vector<MapItem> maps;
    std::vector<SparseItem> sparse;
    maps.swap(ctx->mapBatch);
    sparse.swap(ctx->sparseBatch);
    // A sparsity map and a Sparsify of the same source (the two constants of one sparse weight) need the
    // same comparison of every element: the map kernel then leaves the per-channel counts behind and the
    // Sparsify skips its counting pass, so the source is read twice instead of three times.
    if (!maps.empty() && !sparse.empty()) {
        std::unordered_map<const void*, size_t> bySrc;
        for (size_t i = 0; i < sparse.size(); ++i) bySrc.emplace(sparse[i].src, i);
        for (MapItem& m : maps) {
            const auto hit = bySrc.find(m.src);
            if (hit == bySrc.end()) continue;
            SparseItem& sp = sparse[hit->second];
            const long long unitsPerOC = m.outBytesPerOC / 2;
            if (sp.countsReady || sp.oc != m.oc || sp.work != m.work || sp.sparseByte != m.sparseByte || unitsPerOC <= 0 ||
                kMapUnitsPerCta % unitsPerOC != 0) {
                continue;
            }
            m.counts = sp.counts;
            sp.countsReady = 1;
        }
    }
    runMapItems(ctx, maps);
    runSparseItems(ctx, sparse);
}

}  // namespace b200c
