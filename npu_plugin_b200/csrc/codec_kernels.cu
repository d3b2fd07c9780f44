// Block codec kernels: per-block mode selection (analyze), device exclusive prefix sum of the
// record sizes (reduce -> scan -> scatter over tiles, no inter-CTA waits), stream emission and a
// group-parallel decoder.  Format and contract: codec.h.
#include "codec.h"
#include "runtime.h"

#include <algorithm>
#include <cstring>
#include <mutex>
#include <string>

namespace b200c {

size_t codecBound(size_t n) {
    const size_t blocks = (n + kCodecBlock - 1) / kCodecBlock;
    const size_t supers = (blocks + kCodecSuper - 1) / kCodecSuper;
    return static_cast<size_t>(roundUp(static_cast<int64_t>(kCodecHeaderBytes + 4 * supers + 65 * blocks), 32));
}

// Blocks are indexed in a padded space in which every buffer starts on a tile boundary
// (kTileBlocks blocks), so one tile never straddles two buffers.
constexpr int kTileBlocks = 4096;

B2_HD void loadBlock(const CodecJobDev& job, unsigned long long blk, unsigned char* b) {
    const unsigned long long first = blk * kCodecBlock;
    const unsigned char* src = job.in + first;
    for (int i = 0; i < kCodecBlock; ++i) b[i] = (first + i < job.n) ? src[i] : 0;
}

// ---------------------------------------------------------------------------- analyze
// One thread per 64-byte block: four 128-bit loads, min / max / zigzag-or / non-zero count with
// byte-SIMD instructions, mode choice, and one packed 32-bit summary per block
// (header | base << 8 | record size << 16), so consecutive threads store consecutive words.
// Per-block statistics.  Byte min/max run on 16-bit lanes (bytes widened with one byte-permute per
// half, then the native three-input u16x2 min/max); the packed-byte min/max intrinsics are emulated
// with long instruction sequences on this architecture and made the kernel ALU-bound.
struct BlockStats {
    unsigned int mn, mx;  // u16x2 lanes holding byte values
    unsigned int mag;     // OR of (b ^ signmask(b)) over the bytes: magnitude bits of the zigzag code
    unsigned int any;     // OR of the bytes (a set bit 7 anywhere: some byte is negative)
    unsigned int nz128;   // 128 x number of non-zero bytes
};

// 0xFF in every byte whose top bit is set: prmt's selector nibbles 8..11 replicate the sign of
// bytes 0..3 (the generic prmt form; written as PTX because the C intrinsic documents 3-bit selectors)
__device__ __forceinline__ unsigned int signMask4(unsigned int x) {
    unsigned int m;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(m) : "r"(x), "r"(0u), "r"(0xBA98u));
    return m;
}

// zigzag code of four int8 values at once: (b << 1) ^ (b >> 7, arithmetic), per byte
__device__ __forceinline__ unsigned int zigzag4(unsigned int x) {
    return ((x << 1) & 0xFEFEFEFEu) ^ signMask4(x);
}

__device__ __forceinline__ void statsAddPair(BlockStats& s, unsigned int a, unsigned int b) {
    const unsigned int a0 = __byte_perm(a, 0, 0x4240), a1 = __byte_perm(a, 0, 0x4341);
    const unsigned int b0 = __byte_perm(b, 0, 0x4240), b1 = __byte_perm(b, 0, 0x4341);
    s.mn = __vimin3_u16x2(s.mn, a0, a1);
    s.mn = __vimin3_u16x2(s.mn, b0, b1);
    s.mx = __vimax3_u16x2(s.mx, a0, a1);
    s.mx = __vimax3_u16x2(s.mx, b0, b1);
    // byte-permute with the sign-replicate selector gives 0xFF for negative bytes, 0x00 otherwise
    s.mag |= (a ^ signMask4(a)) | (b ^ signMask4(b));
    s.any |= a | b;
    // bit 7 of every non-zero byte: (((x & 0x7F..) + 0x7F..) | x) & 0x80..; summed by a byte dot product
    const unsigned int na = (((a & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | a) & 0x80808080u;
    const unsigned int nb = (((b & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | b) & 0x80808080u;
    s.nz128 = __dp4a(na, 0x01010101u, s.nz128);
    s.nz128 = __dp4a(nb, 0x01010101u, s.nz128);
}

__device__ __forceinline__ void statsAdd(BlockStats& s, uint4 v) {
    statsAddPair(s, v.x, v.y);
    statsAddPair(s, v.z, v.w);
}

// same decision as codecChoose(), from the folded statistics
__device__ __forceinline__ unsigned int summaryOf(BlockStats s) {
    const unsigned int mn = min(s.mn & 0xFFFFu, s.mn >> 16);
    const unsigned int mx = max(s.mx & 0xFFFFu, s.mx >> 16);
    // OR of zigzag(b) = (OR of (b ^ sign)) << 1 | (any negative), folded over the four byte lanes
    unsigned int o = s.mag | (s.mag >> 16);
    o = (o | (o >> 8)) & 0x7Fu;
    const unsigned int zor = (o << 1) | ((s.any & 0x80808080u) ? 1u : 0u);
    const int nnz = static_cast<int>(s.nz128 >> 7);
    int mode = 0, w = 0, size = 65;
    if (mn == mx) {
        mode = 1;
        size = 2;
    }
    const int wu = 32 - __clz(mx - mn);
    if (wu >= 1 && wu <= 7 && 2 + 8 * wu < size) {
        mode = 2;
        w = wu;
        size = 2 + 8 * wu;
    }
    const int ws = 32 - __clz(zor);
    if (ws >= 1 && ws <= 7 && 1 + 8 * ws < size) {
        mode = 3;
        w = ws;
        size = 1 + 8 * ws;
    }
    if (9 + nnz < size) {
        mode = 4;
        w = 0;
        size = 9 + nnz;
    }
    return static_cast<unsigned int>((mode << 5) | w) | (mn << 8) | (static_cast<unsigned int>(size) << 16);
}

__device__ __forceinline__ uint4 loadLane16(const unsigned char* in, unsigned long long n, unsigned long long blk,
                                            int lane4, bool vec) {
    const unsigned long long first = blk * kCodecBlock + static_cast<unsigned long long>(lane4) * 16;
    if (vec && first + 16 <= n) return __ldg(reinterpret_cast<const uint4*>(in + first));
    unsigned int w[4] = {0, 0, 0, 0};
    for (int i = 0; i < 16; ++i) {
        if (first + i < n) w[i >> 2] |= static_cast<unsigned int>(in[first + i]) << (8 * (i & 3));
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

__global__ void __launch_bounds__(256) codecAnalyzeKernel(const CodecJobDev* __restrict__ jobs,
                                                          const unsigned int* __restrict__ tileJob,
                                                          unsigned long long ntiles, unsigned int* __restrict__ summary,
                                                          unsigned int* __restrict__ tileSums) {
    __shared__ unsigned int red[8];
    for (unsigned long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const CodecJobDev* job = jobs + tileJob[tile];
        const unsigned char* in = job->in;
        const unsigned long long n = job->n, nblocks = job->nblocks;
        const bool vec = (reinterpret_cast<uintptr_t>(in) & 15) == 0;
        const unsigned long long tileFirst = (tile - job->firstBlock / kTileBlocks) * kTileBlocks;
        const unsigned long long gBase = tile * kTileBlocks;
        unsigned int sum = 0;
        constexpr int UNROLL = 2;  // blocks per thread in flight (8 independent 128-bit loads)
#pragma unroll 1
        for (int it0 = 0; it0 < kTileBlocks / 256; it0 += UNROLL) {
            uint4 v[UNROLL][4];
            bool valid[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const unsigned long long blk = tileFirst + static_cast<unsigned long long>(it0 + u) * 256 + threadIdx.x;
                valid[u] = blk < nblocks;
                if (valid[u]) {
                    if (vec && (blk + 1) * kCodecBlock <= n) {
                        const uint4* p4 = reinterpret_cast<const uint4*>(in + blk * kCodecBlock);
#pragma unroll
                        for (int k = 0; k < 4; ++k) v[u][k] = __ldg(p4 + k);
                    } else {
#pragma unroll
                        for (int k = 0; k < 4; ++k) v[u][k] = loadLane16(in, n, blk, k, false);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                unsigned int word = 0;  // padding slot: size 0
                if (valid[u]) {
                    BlockStats st;
                    st.mn = 0x00FF00FFu;
                    st.mx = 0;
                    st.mag = 0;
                    st.any = 0;
                    st.nz128 = 0;
#pragma unroll
                    for (int k = 0; k < 4; ++k) statsAdd(st, v[u][k]);
                    word = summaryOf(st);
                }
                summary[gBase + static_cast<unsigned long long>(it0 + u) * 256 + threadIdx.x] = word;
                sum += word >> 16;
            }
        }
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned int t = 0;
            for (int w = 0; w < 8; ++w) t += red[w];
            tileSums[tile] = t;
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------- layout
// Per-buffer record bytes, stream size, "not smaller" flag and output placement (each segment
// starts on a 32-byte boundary).  tileOffsets is the exclusive prefix sum of the per-tile sums.
B2_HD void layoutJobs(CodecJobDev* jobs, int njobs, const unsigned long long* tileOffsets, unsigned long long outCap,
                      int rawFallback, int* err) {
    unsigned long long run = 0;
    for (int j = 0; j < njobs; ++j) {
        CodecJobDev& job = jobs[j];
        const unsigned long long t0 = job.firstBlock / kTileBlocks;
        const unsigned long long t1 = t0 + (job.nblocks + kTileBlocks - 1) / kTileBlocks;
        job.recordsBytes = tileOffsets[t1] - tileOffsets[t0];
        const unsigned long long raw = kCodecHeaderBytes + 4 * job.nsuper + job.recordsBytes;
        job.streamBytes = (raw + 31) & ~31ull;
        job.notSmaller = job.n <= job.streamBytes;  // bit_compactor_codec.cpp:36-39
        job.failed = 0;
        // rawFallback 0: always the stream; 1: buffers that do not shrink are stored unchanged;
        // 2: buffers that do not shrink take no output at all (the caller keeps them where they are)
        if (rawFallback == 2 && job.notSmaller) {
            job.outBytes = 0;
            job.outBase = run;
            continue;
        }
        job.outBytes = (rawFallback == 1 && job.notSmaller) ? job.n : job.streamBytes;
        job.outBase = run;
        run = (run + job.outBytes + 31) & ~31ull;
        if (job.outBase + job.outBytes > outCap) {
            if (*err == E_NONE) *err = E_CODEC;
            job.outBytes = 0;
            job.failed = 1;
        }
    }
}

// single CTA: exclusive scan of the tile sums (the device prefix sum behind every record offset),
// grand total at tileOffsets[ntiles], then the per-buffer layout, then the list of tiles whose buffer
// gets a stream (emitTiles[0 .. *emitCount), in tile order), so that the emit launch can follow without
// the host looking at the sizes first
__global__ void __launch_bounds__(1024) codecScanKernel(const unsigned int* __restrict__ tileSums,
                                                        unsigned long long ntiles, unsigned long long* tileOffsets,
                                                        CodecJobDev* jobs, int njobs, unsigned long long outCap,
                                                        int rawFallback, int* err, const unsigned int* __restrict__ tileJob,
                                                        unsigned int* emitTiles, unsigned int* emitCount) {
    __shared__ unsigned long long warpSum[32];
    __shared__ unsigned long long carry;
    __shared__ int anyFailed;
    if (threadIdx.x == 0) {
        carry = 0;
        anyFailed = 0;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (unsigned long long base = 0; base < ntiles; base += blockDim.x) {
        const unsigned long long i = base + threadIdx.x;
        const unsigned long long mine = i < ntiles ? tileSums[i] : 0;
        unsigned long long incl = mine;
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warpSum[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            unsigned long long w = warpSum[lane];
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long t = __shfl_up_sync(0xFFFFFFFFu, w, o);
                if (lane >= o) w += t;
            }
            warpSum[lane] = w;
        }
        __syncthreads();
        const unsigned long long before = carry + (warp ? warpSum[warp - 1] : 0) + incl - mine;
        if (i < ntiles) tileOffsets[i] = before;
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = before + mine;
        __syncthreads();
    }
    if (threadIdx.x == 0) tileOffsets[ntiles] = carry;
    __syncthreads();  // tileOffsets (written by this CTA) is read back below
    // per-buffer layout, the parallel form of layoutJobs: sizes per buffer, then an exclusive scan of
    // the 32-byte aligned output sizes for the placement
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < njobs; base += blockDim.x) {
        const int j = base + threadIdx.x;
        unsigned long long mine = 0, outBytes = 0;
        bool skip = false;
        if (j < njobs) {
            CodecJobDev& job = jobs[j];
            const unsigned long long t0 = job.firstBlock / kTileBlocks;
            const unsigned long long t1 = t0 + (job.nblocks + kTileBlocks - 1) / kTileBlocks;
            job.recordsBytes = tileOffsets[t1] - tileOffsets[t0];
            const unsigned long long raw = kCodecHeaderBytes + 4 * job.nsuper + job.recordsBytes;
            job.streamBytes = (raw + 31) & ~31ull;
            job.notSmaller = job.n <= job.streamBytes;
            job.failed = 0;
            skip = rawFallback == 2 && job.notSmaller;
            outBytes = skip ? 0 : ((rawFallback == 1 && job.notSmaller) ? job.n : job.streamBytes);
            mine = (outBytes + 31) & ~31ull;
        }
        unsigned long long incl = mine;
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warpSum[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            unsigned long long w = warpSum[lane];
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long t = __shfl_up_sync(0xFFFFFFFFu, w, o);
                if (lane >= o) w += t;
            }
            warpSum[lane] = w;
        }
        __syncthreads();
        const unsigned long long before = carry + (warp ? warpSum[warp - 1] : 0) + incl - mine;
        if (j < njobs) {
            CodecJobDev& job = jobs[j];
            job.outBase = before;
            job.outBytes = outBytes;
            if (!skip && before + outBytes > outCap) {
                // in place the "output" is the library's own capped scratch: the host lays the batch out again
                if (rawFallback != 2) atomicCAS(err, E_NONE, E_CODEC);
                job.outBytes = 0;
                job.failed = 1;
                anyFailed = 1;
            }
        }
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = before + mine;
        __syncthreads();
    }
    // tiles of the buffers that are emitted, compacted in order
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (unsigned long long base = 0; base < ntiles; base += blockDim.x) {
        const unsigned long long t = base + threadIdx.x;
        bool emits = false;
        if (t < ntiles) {
            const CodecJobDev& job = jobs[tileJob[t]];
            emits = job.outBytes > 0 && !job.failed && !(rawFallback == 1 && job.notSmaller);
        }
        const unsigned int m = __ballot_sync(0xFFFFFFFFu, emits);
        if (lane == 0) warpSum[warp] = __popc(m);
        __syncthreads();
        if (warp == 0) {
            unsigned long long w = warpSum[lane];
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long x = __shfl_up_sync(0xFFFFFFFFu, w, o);
                if (lane >= o) w += x;
            }
            warpSum[lane] = w;
        }
        __syncthreads();
        const unsigned long long pos = carry + (warp ? warpSum[warp - 1] : 0) + __popc(m & ((1u << lane) - 1u));
        if (emits) emitTiles[pos] = static_cast<unsigned int>(t);
        const unsigned long long total = warpSum[31];
        __syncthreads();
        if (threadIdx.x == 0) carry += total;
        __syncthreads();
    }
    // in place, a batch with a buffer that found no room is emitted as a whole on the second attempt
    if (threadIdx.x == 0) *emitCount = (rawFallback == 2 && anyFailed) ? 0u : static_cast<unsigned int>(carry);
}

// In-place mode: every stream built in scratch memory goes over the head of its own input buffer.
// One CTA per tile of a compressed buffer copies the tile's share (256 KB) of the stream.
__global__ void __launch_bounds__(256) codecCopyBackKernel(const CodecJobDev* __restrict__ jobs,
                                                           const unsigned int* __restrict__ tileJob,
                                                           const unsigned int* __restrict__ emitTiles,
                                                           const unsigned int* __restrict__ emitCount,
                                                           const unsigned char* __restrict__ scratch) {
    const unsigned long long nEmitTiles = *emitCount;
    for (unsigned long long e = blockIdx.x; e < nEmitTiles; e += gridDim.x) {
        const unsigned long long tile = emitTiles[e];
        const CodecJobDev& job = jobs[tileJob[tile]];
        const unsigned long long rel = tile - job.firstBlock / kTileBlocks;
        const unsigned long long span = static_cast<unsigned long long>(kTileBlocks) * kCodecBlock;
        const unsigned long long lo = rel * span;
        if (lo >= job.outBytes) continue;
        const unsigned long long len = min(span, job.outBytes - lo);
        const unsigned char* src = scratch + job.outBase + lo;
        unsigned char* dst = const_cast<unsigned char*>(job.in) + lo;
        if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
            const unsigned long long nvec = len / 16;
            for (unsigned long long v = threadIdx.x; v < nvec; v += blockDim.x) {
                reinterpret_cast<uint4*>(dst)[v] = reinterpret_cast<const uint4*>(src)[v];
            }
            for (unsigned long long b = nvec * 16 + threadIdx.x; b < len; b += blockDim.x) dst[b] = src[b];
        } else {
            for (unsigned long long b = threadIdx.x; b < len; b += blockDim.x) dst[b] = src[b];
        }
    }
}

// ---------------------------------------------------------------------------- emit
B2_HD void putU32(unsigned char* p, unsigned int v) {
    p[0] = static_cast<unsigned char>(v);
    p[1] = static_cast<unsigned char>(v >> 8);
    p[2] = static_cast<unsigned char>(v >> 16);
    p[3] = static_cast<unsigned char>(v >> 24);
}
B2_HD void putU64(unsigned char* p, unsigned long long v) {
    putU32(p, static_cast<unsigned int>(v));
    putU32(p + 4, static_cast<unsigned int>(v >> 32));
}

B2_HD void writeStreamHeader(const CodecJobDev& job, unsigned char* dst) {
    dst[0] = 'B';
    dst[1] = '2';
    dst[2] = 'B';
    dst[3] = 'C';
    putU32(dst + 4, 1);
    putU64(dst + 8, job.n);
    putU64(dst + 16, job.nblocks);
    putU32(dst + 24, static_cast<unsigned int>(job.nsuper));
    putU32(dst + 28, 0);
}

// One CTA per tile of a buffer that is being compressed.  Record offsets inside the tile come from
// a block-wide exclusive scan of the tile's record sizes added to the tile's global offset.  An
// iteration covers 256 consecutive blocks, one per thread, whose records are built in a
// shared-memory window laid out like the output (same 16-byte phase) and then copied out with
// 128-bit stores.
//
// The lanes of a warp must not hold blocks of different modes, or the warp runs every encoder one
// after the other.  So the blocks of an iteration are handed out in class order -- RAW, then CONST
// and PACKU, then PACKS, then SPARSE -- through an index list built with warp ballots: only indices
// are sorted, every thread loads its 64 bytes straight from global memory, and at most three warps
// of an iteration straddle a class boundary.
constexpr int kEmitClasses = 4;
// A CTA of 128 threads takes a quarter of a tile (1024 blocks) in iterations of 128 blocks: small CTAs
// mean many independent barrier domains per SM, which is what hides the chain summary -> order ->
// load -> encode -> copy-out of one iteration.
constexpr int kEmitThreads = 128;
constexpr int kEmitSub = 1024;                          // blocks per CTA
constexpr int kEmitSubsPerTile = kTileBlocks / kEmitSub;
constexpr int kEmitWarps = kEmitThreads / 32;

__device__ __forceinline__ int emitClass(unsigned int header) {
    const unsigned int mode = header >> 5;
    return mode == 0 ? 0 : (mode <= 2 ? 1 : (mode == 3 ? 2 : 3));
}

// the 64-bit word holding the eight w-bit fields of one group of eight bytes (a: bytes 0..3, b: 4..7)
__device__ __forceinline__ unsigned long long packGroup(unsigned int a, unsigned int b, int w) {
    const int sh = 8 - w;
    const unsigned int pa = (a & 0x00FF00FFu) | ((a & 0xFF00FF00u) >> sh);
    const unsigned int pb = (b & 0x00FF00FFu) | ((b & 0xFF00FF00u) >> sh);
    const unsigned int qa = (pa & 0xFFFFu) | ((pa >> 16) << (2 * w));
    const unsigned int qb = (pb & 0xFFFFu) | ((pb >> 16) << (2 * w));
    return static_cast<unsigned long long>(qa) | (static_cast<unsigned long long>(qb) << (4 * w));
}

// NW words (4 * NW bytes, byte 0 first) written to shared memory at a byte address of any alignment:
// the words are shifted to the address's phase and stored as whole words; only the bytes of the first
// and of the last, partly covered word are stored one by one (the neighbouring records own the rest of
// those words).
template <int NW>
__device__ __forceinline__ void storeWords(unsigned char* at, const unsigned int (&w)[NW]) {
    const unsigned int a = static_cast<unsigned int>(reinterpret_cast<uintptr_t>(at) & 3u);
    unsigned int* base = reinterpret_cast<unsigned int*>(at - a);
    const unsigned int sh = 8u * a;
#pragma unroll
    for (int k = 1; k < NW; ++k) base[k] = __funnelshift_l(w[k - 1], w[k], sh);
    if (a == 0) {
        base[0] = w[0];
    } else {
        // bytes a .. 3 of the first word: the low 4 - a bytes of w[0]
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            if (i < static_cast<int>(4u - a)) at[i] = static_cast<unsigned char>(w[0] >> (8 * i));
        }
        // bytes 0 .. a - 1 of the word behind the last whole one: the top a bytes of w[NW - 1]
        const unsigned int top = w[NW - 1] >> (32u - sh);
        unsigned char* tail = reinterpret_cast<unsigned char*>(base + NW);
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            if (i < static_cast<int>(a)) tail[i] = static_cast<unsigned char>(top >> (8 * i));
        }
    }
}

// payload of a PACKU / PACKS record with fields of W bits: eight groups of 8 * W bits, 2 * W words in all.
// Field widths are compile-time constants here, so every shift below is an immediate.
template <int W, bool SIGNED>
__device__ __forceinline__ void packPayload(const unsigned int (&words)[16], unsigned int base, unsigned int (&p)[2 * W]) {
    const unsigned int base4 = base * 0x01010101u, lowBase = base4 & 0x7F7F7F7Fu, notBase = ~base4;
#pragma unroll
    for (int i = 0; i < 2 * W; ++i) p[i] = 0;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const unsigned int lo = words[g * 2], hi = words[g * 2 + 1];
        unsigned int flo, fhi;
        if (SIGNED) {
            flo = zigzag4(lo);
            fhi = zigzag4(hi);
        } else {
            // (b - base) & 0xFF per byte without borrows across bytes
            flo = ((lo | 0x80808080u) - lowBase) ^ ((lo ^ notBase) & 0x80808080u);
            fhi = ((hi | 0x80808080u) - lowBase) ^ ((hi ^ notBase) & 0x80808080u);
        }
        const unsigned long long v = packGroup(flo, fhi, W);  // 8 * W bits
        const unsigned int vlo = static_cast<unsigned int>(v), vhi = static_cast<unsigned int>(v >> 32);
        const int bit = 8 * W * g, idx = bit >> 5, off = bit & 31;
        if (off == 0) {
            p[idx] |= vlo;
            if (idx + 1 < 2 * W) p[idx + 1] |= vhi;
        } else {
            p[idx] |= vlo << off;
            if (idx + 1 < 2 * W) p[idx + 1] |= __funnelshift_l(vlo, vhi, off);
            if (idx + 2 < 2 * W) p[idx + 2] |= vhi >> (32 - off);
        }
    }
}

template <int W>
__device__ __forceinline__ void emitPack(const unsigned int (&words)[16], int mode, unsigned int header, unsigned int base,
                                         unsigned char* rec) {
    unsigned int p[2 * W];
    rec[0] = static_cast<unsigned char>(header);
    if (mode == 2) {
        rec[1] = static_cast<unsigned char>(base);
        packPayload<W, false>(words, base, p);
        storeWords<2 * W>(rec + 2, p);
    } else {
        packPayload<W, true>(words, 0u, p);
        storeWords<2 * W>(rec + 1, p);
    }
}

__global__ void __launch_bounds__(kEmitThreads) codecEmitKernel(const CodecJobDev* __restrict__ jobs,
                                                       const unsigned int* __restrict__ tileJob,
                                                       const unsigned int* __restrict__ emitTiles,
                                                       const unsigned int* __restrict__ emitCount,
                                                       const unsigned int* __restrict__ summary,
                                                       const unsigned long long* __restrict__ tileOffsets,
                                                       unsigned char* __restrict__ out) {
    __shared__ unsigned int relOff[kEmitSub + 1];                           // record offsets inside the tile
    __shared__ __align__(16) unsigned char window[kEmitThreads * 65 + 48];  // one iteration's records
    __shared__ unsigned int warpTot[kEmitWarps];
    __shared__ unsigned int sumW[kEmitThreads];      // summary words of the iteration's blocks
    __shared__ unsigned char order[kEmitThreads];    // block indices of the iteration in class order
    __shared__ unsigned int warpCnt[kEmitWarps][kEmitClasses];
    __shared__ unsigned int compactSel[16];          // byte-permute selector that moves the kept bytes of a word down
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x < 16) {
        unsigned int sel = 0, k = 0;
        for (unsigned int b = 0; b < 4; ++b) {
            if (threadIdx.x & (1u << b)) sel |= b << (4 * k++);
        }
        for (; k < 4; ++k) sel |= 4u << (4 * k);  // byte 0 of the second operand: zero
        compactSel[threadIdx.x] = sel;
    }

    const unsigned long long nEmitTiles = *emitCount;
    for (unsigned long long e = blockIdx.x; e < nEmitTiles * kEmitSubsPerTile; e += gridDim.x) {
        const unsigned long long tile = emitTiles[e / kEmitSubsPerTile];
        const int sub = static_cast<int>(e % kEmitSubsPerTile);
        const CodecJobDev& job = jobs[tileJob[tile]];
        const bool vec = (reinterpret_cast<uintptr_t>(job.in) & 15) == 0;
        const unsigned long long jobFirstTile = job.firstBlock / kTileBlocks;
        // first block of this CTA's share in the job
        const unsigned long long tileFirst = (tile - jobFirstTile) * kTileBlocks + static_cast<unsigned long long>(sub) * kEmitSub;
        if (tileFirst >= job.nblocks) continue;  // uniform over the CTA
        unsigned char* dst = out + job.outBase;
        unsigned char* records = dst + kCodecHeaderBytes + 4 * job.nsuper;
        const unsigned int* tileSummary = summary + tile * kTileBlocks;

        // record bytes of the tile's blocks in front of this share, then the exclusive scan of the share's
        // 1024 record sizes (8 per thread)
        unsigned int lead = 0;
        {
            const uint4* pre4 = reinterpret_cast<const uint4*>(tileSummary);
            for (int q = threadIdx.x; q < sub * (kEmitSub / 4); q += kEmitThreads) {
                const uint4 v = pre4[q];
                lead += (v.x >> 16) + (v.y >> 16) + (v.z >> 16) + (v.w >> 16);
            }
            const uint4* sm4 = reinterpret_cast<const uint4*>(tileSummary + sub * kEmitSub + threadIdx.x * 8);
            unsigned int local[8], s = 0;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const uint4 v = sm4[q];
                const unsigned int w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    local[q * 4 + i] = s;
                    s += w[i] >> 16;
                }
            }
            unsigned int incl = s;
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned int x = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if (lane >= o) incl += x;
            }
            for (int o = 16; o > 0; o >>= 1) lead += __shfl_xor_sync(0xFFFFFFFFu, lead, o);
            __syncthreads();  // the previous share's readers of warpTot and relOff are done
            if (lane == 31) warpTot[warp] = incl;
            if (lane == 0) warpCnt[warp][0] = lead;
            __syncthreads();
            unsigned int before = incl - s;
            for (int wv = 0; wv < warp; ++wv) before += warpTot[wv];
            lead = 0;
            for (int wv = 0; wv < kEmitWarps; ++wv) lead += warpCnt[wv][0];
#pragma unroll
            for (int i = 0; i < 8; ++i) relOff[threadIdx.x * 8 + i] = before + local[i];
            if (threadIdx.x == kEmitThreads - 1) relOff[kEmitSub] = before + s;
            __syncthreads();
        }
        const unsigned long long tileRel = tileOffsets[tile] - tileOffsets[jobFirstTile] + lead;

        if (tileFirst == 0 && threadIdx.x == 0) writeStreamHeader(job, dst);

        for (int it = 0; it < kEmitSub / kEmitThreads; ++it) {
            const unsigned long long blk0 = tileFirst + static_cast<unsigned long long>(it) * kEmitThreads;
            if (blk0 >= job.nblocks) break;
            const unsigned int winStart = relOff[it * kEmitThreads];
            const unsigned int winEnd = relOff[(it + 1) * kEmitThreads];
            const unsigned long long outStart = tileRel + winStart;  // offset inside the records area
            const unsigned int phase = static_cast<unsigned int>(reinterpret_cast<uintptr_t>(records + outStart) & 15);

            // ---- the iteration's blocks in class order
            unsigned int nvalid;
            {
                const int bi = threadIdx.x;
                const unsigned long long blk = blk0 + bi;
                const bool valid = blk < job.nblocks;
                unsigned int word = 0;
                if (valid) {
                    word = tileSummary[sub * kEmitSub + it * kEmitThreads + bi];
                    if ((bi & (kCodecSuper - 1)) == 0) {  // first block of an index group of 64
                        putU32(dst + kCodecHeaderBytes + 4 * (blk / kCodecSuper),
                               static_cast<unsigned int>(tileRel + relOff[it * kEmitThreads + bi]));
                    }
                }
                sumW[bi] = word;
                const int cls = valid ? emitClass(word & 0xFFu) : -1;
                unsigned int mine = 0;
#pragma unroll
                for (int c = 0; c < kEmitClasses; ++c) {
                    const unsigned int m = __ballot_sync(0xFFFFFFFFu, cls == c);
                    if (lane == 0) warpCnt[warp][c] = __popc(m);
                    if (cls == c) mine = m;
                }
                __syncthreads();
                unsigned int pos = __popc(mine & ((1u << lane) - 1u)), total = 0;
#pragma unroll
                for (int c = 0; c < kEmitClasses; ++c) {
#pragma unroll
                    for (int wv = 0; wv < kEmitWarps; ++wv) {
                        const unsigned int n = warpCnt[wv][c];
                        total += n;
                        if (c < cls || (c == cls && wv < warp)) pos += n;
                    }
                }
                nvalid = total;
                if (valid) order[pos] = static_cast<unsigned char>(bi);
                __syncthreads();
            }

            if (threadIdx.x < nvalid) {
                const int bi = order[threadIdx.x];
                const unsigned long long blk = blk0 + bi;
                unsigned int words[16];
                if (vec && (blk + 1) * kCodecBlock <= job.n) {
                    const uint4* p4 = reinterpret_cast<const uint4*>(job.in + blk * kCodecBlock);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint4 q = __ldg(p4 + k);
                        words[4 * k] = q.x;
                        words[4 * k + 1] = q.y;
                        words[4 * k + 2] = q.z;
                        words[4 * k + 3] = q.w;
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint4 q = loadLane16(job.in, job.n, blk, k, false);
                        words[4 * k] = q.x;
                        words[4 * k + 1] = q.y;
                        words[4 * k + 2] = q.z;
                        words[4 * k + 3] = q.w;
                    }
                }
                const unsigned int word = sumW[bi];
                const unsigned int header = word & 0xFFu, base = (word >> 8) & 0xFFu;
                const int mode = header >> 5, w = header & 31;
                unsigned char* rec = window + phase + (relOff[it * kEmitThreads + bi] - winStart);
                if (mode == 0) {
                    rec[0] = static_cast<unsigned char>(header);
                    storeWords<16>(rec + 1, words);
                } else if (mode == 1) {
                    rec[0] = static_cast<unsigned char>(header);
                    rec[1] = static_cast<unsigned char>(base);
                } else if (mode <= 3) {
                    switch (w) {
                    case 1: emitPack<1>(words, mode, header, base, rec); break;
                    case 2: emitPack<2>(words, mode, header, base, rec); break;
                    case 3: emitPack<3>(words, mode, header, base, rec); break;
                    case 4: emitPack<4>(words, mode, header, base, rec); break;
                    case 5: emitPack<5>(words, mode, header, base, rec); break;
                    case 6: emitPack<6>(words, mode, header, base, rec); break;
                    default: emitPack<7>(words, mode, header, base, rec); break;
                    }
                } else {  // sparse: 8 mask bytes, then the non-zero bytes in order
                    rec[0] = static_cast<unsigned char>(header);
                    unsigned char* nz = rec + 9;
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        unsigned int m8 = 0;
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const unsigned int v = words[q * 2 + h];
                            const unsigned int t = (((v & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | v) & 0x80808080u;
                            const unsigned int m = ((t >> 7) * 0x01020408u) >> 24;  // bit k: byte k of the word is non-zero
                            const unsigned int kept = __byte_perm(v, 0u, compactSel[m]);
                            const int n = __popc(m);
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                if (k < n) nz[k] = static_cast<unsigned char>(kept >> (8 * k));
                            }
                            nz += n;
                            m8 |= m << (4 * h);
                        }
                        rec[1 + q] = static_cast<unsigned char>(m8);
                    }
                }
            }
            __syncthreads();
            // copy the window out: [outStart, outStart + len) of the records area
            {
                const unsigned int len = winEnd - winStart;
                unsigned char* gdst = records + outStart;
                const unsigned int head = (16 - phase) & 15;  // bytes up to the first 16-byte boundary
                for (unsigned int i = threadIdx.x; i < len && i < head; i += blockDim.x) gdst[i] = window[phase + i];
                const unsigned int bodyStart = head < len ? head : len;
                const unsigned int nvec = (len - bodyStart) / 16;
                for (unsigned int q = threadIdx.x; q < nvec; q += blockDim.x) {
                    *reinterpret_cast<uint4*>(gdst + bodyStart + q * 16) =
                            *reinterpret_cast<const uint4*>(window + phase + bodyStart + q * 16);
                }
                for (unsigned int i = bodyStart + nvec * 16 + threadIdx.x; i < len; i += blockDim.x) gdst[i] = window[phase + i];
            }
            __syncthreads();
        }
        // trailing zero bytes of the stream (32-byte alignment), written by the CTA that holds the buffer's last block
        if (tileFirst + kEmitSub >= job.nblocks) {
            for (unsigned long long a = kCodecHeaderBytes + 4 * job.nsuper + job.recordsBytes + threadIdx.x; a < job.streamBytes;
                 a += blockDim.x) {
                dst[a] = 0;
            }
        }
        __syncthreads();
    }
}

static void fillResults(const CodecJobDev* jobs, int count, bool inPlace, CodecResult* results) {
    for (int j = 0; j < count; ++j) {
        results[j].offset = inPlace ? 0 : jobs[j].outBase;
        results[j].size = (inPlace && jobs[j].notSmaller) ? jobs[j].n : jobs[j].outBytes;
        results[j].notSmaller = jobs[j].notSmaller != 0;
    }
}

void codecCollect(Context* ctx, CodecPending* pending, CodecResult* results) {
    B2_CUDA(cudaEventSynchronize(pending->done));
    pending->open = false;
    pending->errCode = *reinterpret_cast<const int*>(pending->jobsHost + pending->capacity);
    if (pending->errCode != E_NONE) {
        B2_CUDA(cudaMemsetAsync(ctx->errWord, 0, sizeof(int), ctx->stream));
        return;  // the caller reports it; the buffers of this batch are not to be trusted
    }
    bool failed = false;
    for (int j = 0; j < pending->count; ++j) failed = failed || pending->jobsHost[j].failed;
    if (failed) {
        // the capped scratch was too small and nothing was emitted: compress again, waiting for the result
        codecCompressBatch(ctx, pending->count, pending->bufs.data(), nullptr, 0, /*rawFallback=*/2, results);
        return;
    }
    fillResults(pending->jobsHost, pending->count, true, results);
}

void codecCompressBatch(Context* ctx, int count, const CodecBuf* bufs, unsigned char* outDev, size_t outCap,
                        int rawFallback, CodecResult* results, CodecPending* pending) {
    TraceRange range("codec: compress batch");
    const bool inPlace = rawFallback == 2;  // streams replace the head of their own input buffer
    if (pending && !inPlace) throw BadArg("only the in-place batch compression can be left pending");
    if (inPlace) outCap = ~static_cast<size_t>(0) >> 1;
    if (count <= 0) return;
    std::vector<CodecJobDev> jobs(count);
    std::vector<unsigned int> tileJob;
    unsigned long long ntiles = 0;
    for (int j = 0; j < count; ++j) {
        if (bufs[j].n == 0) refThrow("BitCompactorCodec::compress: Empty input data vector");
        if (bufs[j].n >= (1ull << 32)) throw NotBuilt("codec input of 4 GiB or more");
        std::memset(&jobs[j], 0, sizeof(CodecJobDev));
        jobs[j].in = bufs[j].in;
        jobs[j].n = bufs[j].n;
        jobs[j].nblocks = (bufs[j].n + kCodecBlock - 1) / kCodecBlock;
        jobs[j].nsuper = (jobs[j].nblocks + kCodecSuper - 1) / kCodecSuper;
        jobs[j].firstBlock = ntiles * kTileBlocks;
        const unsigned long long t = (jobs[j].nblocks + kTileBlocks - 1) / kTileBlocks;
        tileJob.insert(tileJob.end(), t, static_cast<unsigned int>(j));
        ntiles += t;
    }
    const unsigned long long padded = ntiles * kTileBlocks;
    CodecJobDev* jobsDev = static_cast<CodecJobDev*>(ctx->arena.alloc(sizeof(CodecJobDev) * count));
    unsigned int* tileJobDev = static_cast<unsigned int*>(ctx->arena.alloc(sizeof(unsigned int) * ntiles));
    unsigned int* summary = static_cast<unsigned int*>(ctx->arena.alloc(padded * sizeof(unsigned int)));
    unsigned int* tileSums = static_cast<unsigned int*>(ctx->arena.alloc(sizeof(unsigned int) * (ntiles + 1)));
    unsigned long long* tileOffsets =
            static_cast<unsigned long long*>(ctx->arena.alloc(sizeof(unsigned long long) * (ntiles + 1)));
    unsigned int* emitDev = static_cast<unsigned int*>(ctx->arena.alloc(sizeof(unsigned int) * (ntiles + 1)));
    unsigned int* emitCount = emitDev + ntiles;
    uploadSmall(ctx, jobsDev, jobs.data(), sizeof(CodecJobDev) * count);
    uploadSmall(ctx, tileJobDev, tileJob.data(), sizeof(unsigned int) * ntiles);

    // In-place mode builds the streams in scratch memory and copies them over the head of their inputs.
    // A stream is only kept when it is shorter than its buffer, so the buffers' total size bounds the
    // scratch; it is capped, and a batch whose streams outgrow the cap is laid out again with the exact need.
    size_t scratchCap = 0;
    if (inPlace) {
        size_t total = 64;
        for (int j = 0; j < count; ++j) total += (bufs[j].n + 31) / 32 * 32;
        scratchCap = std::min<size_t>(total, 1ull << 30);
        outDev = static_cast<unsigned char*>(ctx->arena.alloc(scratchCap));
        outCap = scratchCap;
    }
    // One pass of launches with a single wait at the end: analysis, the device prefix sum with the
    // per-buffer layout and the list of tiles to emit, emission, (in place) the copy back.
    const unsigned long long subs = ntiles * kEmitSubsPerTile;
    const int agrid = static_cast<int>(std::max<unsigned long long>(1, std::min<unsigned long long>(ntiles, ctx->smCount * 8ULL)));
    const int egrid = static_cast<int>(std::max<unsigned long long>(1, std::min<unsigned long long>(subs, ctx->smCount * 16ULL)));
    const int cgrid = static_cast<int>(std::max<unsigned long long>(1, std::min<unsigned long long>(ntiles, ctx->smCount * 4ULL)));
    codecAnalyzeKernel<<<agrid, 256, 0, ctx->stream>>>(jobsDev, tileJobDev, ntiles, summary, tileSums);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
    auto layoutAndEmit = [&](bool wait) {
        codecScanKernel<<<1, 1024, 0, ctx->stream>>>(tileSums, ntiles, tileOffsets, jobsDev, count, outCap, rawFallback,
                                                     ctx->errWord, tileJobDev, emitDev, emitCount);
        B2_CUDA(cudaGetLastError());
        codecEmitKernel<<<egrid, kEmitThreads, 0, ctx->stream>>>(jobsDev, tileJobDev, emitDev, emitCount, summary, tileOffsets, outDev);
        B2_CUDA(cudaGetLastError());
        ctx->launches += 2;
        if (inPlace) {
            codecCopyBackKernel<<<cgrid, 256, 0, ctx->stream>>>(jobsDev, tileJobDev, emitDev, emitCount, outDev);
            B2_CUDA(cudaGetLastError());
            ++ctx->launches;
        }
        if (!wait) {
            copyD2H(ctx, pending->jobsHost, jobsDev, sizeof(CodecJobDev) * count);
            copyD2H(ctx, pending->jobsHost + pending->capacity, ctx->errWord, sizeof(int));
            B2_CUDA(cudaEventRecord(pending->done, ctx->stream));
            return;
        }
        copyD2H(ctx, jobs.data(), jobsDev, sizeof(CodecJobDev) * count);
        checkDeviceError(ctx);  // waits for the stream: the call hands finished buffers back
    };
    if (pending) {
        if (pending->capacity < static_cast<size_t>(count)) {
            if (pending->jobsHost) cudaFreeHost(pending->jobsHost);
            pending->jobsHost = nullptr;
            pending->capacity = 0;
            B2_CUDA(cudaMallocHost(&pending->jobsHost, sizeof(CodecJobDev) * (static_cast<size_t>(count) * 2 + 1)));
            pending->capacity = static_cast<size_t>(count) * 2;
        }
        if (!pending->done) B2_CUDA(cudaEventCreateWithFlags(&pending->done, cudaEventDisableTiming));
        pending->count = count;
        pending->bufs.assign(bufs, bufs + count);
        layoutAndEmit(false);
        pending->open = true;
        return;
    }
    layoutAndEmit(true);
    bool failed = false;
    for (int j = 0; j < count; ++j) failed = failed || jobs[j].failed;
    if (failed && inPlace) {
        // the capped scratch was too small and nothing was emitted: lay the batch out again with room for
        // every stream
        size_t need = 64;
        for (int j = 0; j < count; ++j) need += (std::min<size_t>(jobs[j].streamBytes, jobs[j].n) + 31) / 32 * 32;
        outDev = static_cast<unsigned char*>(ctx->arena.alloc(need));
        outCap = need;
        layoutAndEmit(true);
        failed = false;
        for (int j = 0; j < count; ++j) failed = failed || jobs[j].failed;
    }
    if (failed) throw Capacity("codec: output capacity exceeded");
    if (rawFallback == 1) {
        // buffers that do not shrink are stored as they are
        bool copied = false;
        for (int j = 0; j < count; ++j) {
            if (jobs[j].notSmaller && jobs[j].outBytes) {
                copyD2D(ctx, outDev + jobs[j].outBase, jobs[j].in, jobs[j].n);
                copied = true;
            }
        }
        if (copied) syncStream(ctx);
    }
    fillResults(jobs.data(), count, inPlace, results);
}

// ---------------------------------------------------------------------------- allocation-free compress
// Some hosts cannot let a library allocate device memory: a process whose whole GPU is claimed up
// front by its own memory pool (a further cudaMalloc fails or fragments the pool), or one that must
// not take the device-wide synchronisation an allocation implies while its other streams are busy.
// For them the same analyse -> scan -> emit sequence runs with its working arrays carved out of a
// fixed buffer that is part of the loaded library image.
//
// The buffer is a file-scope device array.  In host code its name is only a handle of the host-side
// shadow symbol, never a device address, so the real address is fetched once per device with
// cudaGetSymbolAddress (that device being current) and kept; kernels only ever receive that address.
constexpr size_t kNoAllocMaxInput = 16u << 20;                                // bytes per call
constexpr size_t kNoAllocMaxTiles = kNoAllocMaxInput / kCodecBlock / kTileBlocks;  // 64
constexpr size_t kNoAllocPadded = kNoAllocMaxTiles * kTileBlocks;             // block slots
constexpr size_t kNoAllocSmall = 4096;                                        // job, tile tables, error word
constexpr size_t kNoAllocScratchBytes = kNoAllocSmall + 4 * kNoAllocPadded;  // one 32-bit summary per block slot
static __device__ __align__(256) unsigned char g_noAllocScratch[kNoAllocScratchBytes];

constexpr int kNoAllocMaxDevices = 64;
static std::mutex g_noAllocMutex;
static unsigned char* g_noAllocPtr[kNoAllocMaxDevices] = {nullptr};

size_t codecNoAllocMaxInput() {
    return kNoAllocMaxInput;
}

// Returns the stream length through *outN; notSmaller as in codecCompressBatch.  Nothing here calls
// cudaMalloc/cudaFree or any allocating routine; host-side temporaries live on the stack.
void codecCompressNoAlloc(int device, const unsigned char* inDev, size_t n, unsigned char* outDev, size_t cap,
                          cudaStream_t stream, size_t* outN, bool* notSmaller) {
    if (n == 0) refThrow("BitCompactorCodec::compress: Empty input data vector");
    if (n > kNoAllocMaxInput) {
        throw Capacity("b200c_btc_compress_noalloc handles at most " + std::to_string(kNoAllocMaxInput) +
                       " input bytes per call (got " + std::to_string(n) + ")");
    }
    if (cap < codecBound(n)) throw Capacity("output capacity below b200c_btc_bound(n)");
    if (device < 0 || device >= kNoAllocMaxDevices) throw BadArg("device index out of range");
    // the caller's current device is put back when the call returns, whichever way it returns
    struct DeviceScope {
        int previous = -1;
        explicit DeviceScope(int d) {
            B2_CUDA(cudaGetDevice(&previous));
            if (previous != d) B2_CUDA(cudaSetDevice(d));
        }
        ~DeviceScope() {
            int now = -1;
            if (previous >= 0 && cudaGetDevice(&now) == cudaSuccess && now != previous) cudaSetDevice(previous);
        }
    } deviceScope(device);

    unsigned char* scratch = nullptr;
    {
        // one-time set-up per device: resolve the device address of the static array
        std::lock_guard<std::mutex> lock(g_noAllocMutex);
        if (g_noAllocPtr[device] == nullptr) {
            void* p = nullptr;
            B2_CUDA(cudaGetSymbolAddress(&p, g_noAllocScratch));
            g_noAllocPtr[device] = static_cast<unsigned char*>(p);
        }
        scratch = g_noAllocPtr[device];
    }

    // carve the working arrays out of the fixed buffer
    CodecJobDev* jobDev = reinterpret_cast<CodecJobDev*>(scratch);
    unsigned int* tileJobDev = reinterpret_cast<unsigned int*>(scratch + 256);
    unsigned int* tileSums = reinterpret_cast<unsigned int*>(scratch + 1024);
    unsigned long long* tileOffsets = reinterpret_cast<unsigned long long*>(scratch + 2048);
    int* errDev = reinterpret_cast<int*>(scratch + 3072);
    unsigned int* emitCountDev = reinterpret_cast<unsigned int*>(scratch + 3072 + 64);
    unsigned int* summary = reinterpret_cast<unsigned int*>(scratch + kNoAllocSmall);
    // slots: job record [0, 256), tile table and emit list [256, 1024), tile sums [1024, 2048),
    // tile offsets [2048, 3072), error word at 3072, length of the emit list at 3136, summaries from kNoAllocSmall
    static_assert(sizeof(CodecJobDev) <= 256 && 2 * kNoAllocMaxTiles * 4 <= 768 && (kNoAllocMaxTiles + 1) * 4 <= 1024 &&
                          (kNoAllocMaxTiles + 1) * 8 <= 1024 && kNoAllocSmall >= 3072 + 64 + sizeof(int) &&
                          kNoAllocMaxTiles * kTileBlocks * kCodecBlock >= kNoAllocMaxInput,
                  "layout of the fixed scratch buffer");

    CodecJobDev job;
    std::memset(&job, 0, sizeof(job));
    job.in = inDev;
    job.n = n;
    job.nblocks = (n + kCodecBlock - 1) / kCodecBlock;
    job.nsuper = (job.nblocks + kCodecSuper - 1) / kCodecSuper;
    job.firstBlock = 0;
    const unsigned long long ntiles = (job.nblocks + kTileBlocks - 1) / kTileBlocks;
    unsigned int tileJob[kNoAllocMaxTiles] = {0};  // one buffer: every tile belongs to job 0

    // The array keeps whatever the previous call left: everything read below is rewritten first --
    // the job record and tile table here, the error word by the memset, the per-block summaries and
    // tile sums by the analysis kernel (including the zero sizes of the padding slots), the emit list
    // and its length by the scan kernel.
    B2_CUDA(cudaMemcpyAsync(jobDev, &job, sizeof(job), cudaMemcpyHostToDevice, stream));
    B2_CUDA(cudaMemcpyAsync(tileJobDev, tileJob, sizeof(unsigned int) * ntiles, cudaMemcpyHostToDevice, stream));
    B2_CUDA(cudaMemsetAsync(errDev, 0, sizeof(int), stream));
    const int grid = static_cast<int>(ntiles);
    codecAnalyzeKernel<<<grid, 256, 0, stream>>>(jobDev, tileJobDev, ntiles, summary, tileSums);
    B2_CUDA(cudaGetLastError());
    // the scan also writes the list of tiles to emit (second half of the table slot) and its length
    codecScanKernel<<<1, 1024, 0, stream>>>(tileSums, ntiles, tileOffsets, jobDev, 1, cap, /*rawFallback=*/0, errDev, tileJobDev,
                                            tileJobDev + kNoAllocMaxTiles, emitCountDev);
    B2_CUDA(cudaGetLastError());
    codecEmitKernel<<<grid * kEmitSubsPerTile, kEmitThreads, 0, stream>>>(jobDev, tileJobDev, tileJobDev + kNoAllocMaxTiles, emitCountDev,
                                                                          summary, tileOffsets, outDev);
    B2_CUDA(cudaGetLastError());
    int err = 0;
    B2_CUDA(cudaMemcpyAsync(&job, jobDev, sizeof(job), cudaMemcpyDeviceToHost, stream));
    B2_CUDA(cudaMemcpyAsync(&err, errDev, sizeof(int), cudaMemcpyDeviceToHost, stream));
    B2_CUDA(cudaStreamSynchronize(stream));
    if (err != E_NONE || job.outBytes == 0) throw Capacity("codec: output capacity exceeded");
    *outN = static_cast<size_t>(job.streamBytes);
    *notSmaller = job.notSmaller != 0;
}

// ---------------------------------------------------------------------------- decode
struct DecodeParams {
    const unsigned char* in;
    unsigned long long inBytes;
    unsigned char* out;
    unsigned long long n, nblocks, nsuper;
    int* err;
};

B2_HD unsigned int getU32(const unsigned char* p) {
    return static_cast<unsigned int>(p[0]) | (static_cast<unsigned int>(p[1]) << 8) |
           (static_cast<unsigned int>(p[2]) << 16) | (static_cast<unsigned int>(p[3]) << 24);
}

// one 64-block group: walk its records in order
B2_HD void decodeGroup(const DecodeParams& p, unsigned long long s) {
    const unsigned char* records = p.in + kCodecHeaderBytes + 4 * p.nsuper;
    unsigned long long at = getU32(p.in + kCodecHeaderBytes + 4 * s);
    const unsigned long long limit = p.inBytes - (kCodecHeaderBytes + 4 * p.nsuper);
    int bad = 0;
    for (unsigned long long blk = s * kCodecSuper; blk < p.nblocks && blk < (s + 1) * kCodecSuper; ++blk) {
        unsigned char b[kCodecBlock];
        if (at + 2 > limit) {
            bad = 1;
            break;
        }
        // a SPARSE record's size is read from its 8 mask bytes: they must lie inside the stream before
        // they are looked at; modes above SPARSE do not exist
        const int headerMode = records[at] >> 5;
        if (headerMode > 4 || (headerMode == 4 && at + 9 > limit)) {
            bad = 1;
            break;
        }
        const int need = codecRecordSize(records[at], records + at + 1);
        if (at + need > limit) {
            bad = 1;
            break;
        }
        if (codecReadRecord(records + at, b) < 0) {
            bad = 1;
            break;
        }
        at += need;
        const unsigned long long first = blk * kCodecBlock;
        for (int i = 0; i < kCodecBlock && first + i < p.n; ++i) p.out[first + i] = b[i];
    }
    if (bad) {
#ifdef __CUDA_ARCH__
        atomicCAS(p.err, E_NONE, E_CODEC);
#else
        if (*p.err == E_NONE) *p.err = E_CODEC;
#endif
    }
}

__global__ void __launch_bounds__(64) codecDecodeKernel(const __grid_constant__ DecodeParams p) {
    const unsigned long long step = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
    for (unsigned long long s = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x; s < p.nsuper;
         s += step) {
        decodeGroup(p, s);
    }
}

size_t codecDecompress(Context* ctx, const unsigned char* inDev, size_t n, unsigned char* outDev, size_t cap) {
    unsigned char hdr[kCodecHeaderBytes];
    if (n < static_cast<size_t>(kCodecHeaderBytes)) refThrow("codec: truncated stream");
    copyD2H(ctx, hdr, inDev, kCodecHeaderBytes);
    syncStream(ctx);
    if (!(hdr[0] == 'B' && hdr[1] == '2' && hdr[2] == 'B' && hdr[3] == 'C' && getU32(hdr + 4) == 1)) {
        refThrow("codec: bad stream header");
    }
    DecodeParams p;
    p.in = inDev;
    p.inBytes = n;
    p.out = outDev;
    p.n = getU32(hdr + 8) | (static_cast<unsigned long long>(getU32(hdr + 12)) << 32);
    p.nblocks = getU32(hdr + 16) | (static_cast<unsigned long long>(getU32(hdr + 20)) << 32);
    p.nsuper = getU32(hdr + 24);
    p.err = ctx->errWord;
    if (p.nblocks != (p.n + kCodecBlock - 1) / kCodecBlock || p.nsuper != (p.nblocks + kCodecSuper - 1) / kCodecSuper ||
        n < kCodecHeaderBytes + 4 * p.nsuper) {
        refThrow("codec: inconsistent stream header");
    }
    if (p.n > cap) throw Capacity("codec: output capacity too small");
    {
        const int grid = static_cast<int>(std::max<unsigned long long>(1, std::min<unsigned long long>((p.nsuper + 63) / 64, ctx->smCount * 16ULL)));
        codecDecodeKernel<<<grid, 64, 0, ctx->stream>>>(p);
        B2_CUDA(cudaGetLastError());
        ++ctx->launches;
    }
    syncStream(ctx);
    checkDeviceError(ctx);
    return static_cast<size_t>(p.n);
}

}  // namespace b200c
