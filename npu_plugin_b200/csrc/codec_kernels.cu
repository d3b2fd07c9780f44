// Block codec kernels: per-block mode selection (analyze), device exclusive prefix sum of the
// record sizes (reduce -> scan -> scatter over tiles, no inter-CTA waits), stream emission and a
// group-parallel decoder.  Format and contract: codec.h.
#include "codec.h"
#include "runtime.h"

#include <algorithm>
#include <cstring>

namespace b200c {

size_t codecBound(size_t n) {
    const size_t blocks = (n + kCodecBlock - 1) / kCodecBlock;
    const size_t supers = (blocks + kCodecSuper - 1) / kCodecSuper;
    return static_cast<size_t>(roundUp(static_cast<int64_t>(kCodecHeaderBytes + 4 * supers + 65 * blocks), 32));
}

B2_HD int jobOfBlock(const CodecJobDev* jobs, int njobs, unsigned long long g) {
    int lo = 0, hi = njobs - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (jobs[mid].firstBlock <= g) {
            lo = mid;
        } else {
            hi = mid - 1;
        }
    }
    return lo;
}

B2_HD void loadBlock(const CodecJobDev& job, unsigned long long blk, unsigned char* b) {
    const unsigned long long first = blk * kCodecBlock;
    const unsigned char* src = job.in + first;
#ifdef __CUDA_ARCH__
    if (first + kCodecBlock <= job.n && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        uint4* d = reinterpret_cast<uint4*>(b);
        const uint4* s = reinterpret_cast<const uint4*>(src);
        d[0] = s[0];
        d[1] = s[1];
        d[2] = s[2];
        d[3] = s[3];
        return;
    }
#endif
    for (int i = 0; i < kCodecBlock; ++i) b[i] = (first + i < job.n) ? src[i] : 0;
}

// ---------------------------------------------------------------------------- analyze
B2_HD void analyzeOne(const CodecJobDev* jobs, int njobs, unsigned long long g, unsigned char* headers,
                      unsigned char* bases, unsigned char* sizes) {
    const CodecJobDev& job = jobs[jobOfBlock(jobs, njobs, g)];
    const unsigned long long blk = g - job.firstBlock;
    if (blk >= job.nblocks) {
        sizes[g] = 0;
        headers[g] = 0;
        bases[g] = 0;
        return;
    }
    alignas(16) unsigned char b[kCodecBlock];
    loadBlock(job, blk, b);
    unsigned char h, base;
    sizes[g] = static_cast<unsigned char>(codecChoose(b, &h, &base));
    headers[g] = h;
    bases[g] = base;
}

__global__ void __launch_bounds__(128) codecAnalyzeKernel(const CodecJobDev* __restrict__ jobs, int njobs,
                                                          unsigned long long totalBlocks, unsigned char* headers,
                                                          unsigned char* bases, unsigned char* sizes) {
    const unsigned long long step = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
    for (unsigned long long g = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x; g < totalBlocks;
         g += step) {
        analyzeOne(jobs, njobs, g, headers, bases, sizes);
    }
}

// ---------------------------------------------------------------------------- exclusive scan (u8 -> u64)
constexpr int kScanThreads = 256;
constexpr int kScanPerThread = 16;
constexpr int kScanTile = kScanThreads * kScanPerThread;

__device__ __forceinline__ unsigned int blockReduceSum(unsigned int v, unsigned int* smem) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    unsigned int t = 0;
    for (int w = 0; w < kScanThreads / 32; ++w) t += smem[w];
    __syncthreads();
    return t;
}

__global__ void __launch_bounds__(kScanThreads) scanTileSumsKernel(const unsigned char* __restrict__ in,
                                                                   unsigned long long n, unsigned int* tileSums,
                                                                   unsigned long long ntiles) {
    __shared__ unsigned int smem[kScanThreads / 32];
    for (unsigned long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const unsigned long long first = t * kScanTile + static_cast<unsigned long long>(threadIdx.x) * kScanPerThread;
        unsigned int s = 0;
        if (first + kScanPerThread <= n) {
            const uint4 v = *reinterpret_cast<const uint4*>(in + first);
            s = __vsadu4(v.x, 0) + __vsadu4(v.y, 0) + __vsadu4(v.z, 0) + __vsadu4(v.w, 0);
        } else {
            for (int i = 0; i < kScanPerThread; ++i)
                if (first + i < n) s += in[first + i];
        }
        const unsigned int total = blockReduceSum(s, smem);
        if (threadIdx.x == 0) tileSums[t] = total;
    }
}

// single CTA: exclusive scan of the tile sums; also stores the grand total at tileOffsets[ntiles]
__global__ void __launch_bounds__(1024) scanTilesKernel(const unsigned int* __restrict__ tileSums,
                                                        unsigned long long ntiles, unsigned long long* tileOffsets) {
    __shared__ unsigned long long warpSum[32];
    __shared__ unsigned long long carry;
    if (threadIdx.x == 0) carry = 0;
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
}

__global__ void __launch_bounds__(kScanThreads) scanScatterKernel(const unsigned char* __restrict__ in,
                                                                  unsigned long long n,
                                                                  const unsigned long long* __restrict__ tileOffsets,
                                                                  unsigned long long* __restrict__ out,
                                                                  unsigned long long ntiles) {
    __shared__ unsigned int warpSum[kScanThreads / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (unsigned long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const unsigned long long first = t * kScanTile + static_cast<unsigned long long>(threadIdx.x) * kScanPerThread;
        unsigned char v[kScanPerThread];
        unsigned int s = 0;
        for (int i = 0; i < kScanPerThread; ++i) {
            v[i] = (first + i < n) ? in[first + i] : 0;
            s += v[i];
        }
        unsigned int incl = s;
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned int x = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += x;
        }
        if (lane == 31) warpSum[warp] = incl;
        __syncthreads();
        unsigned int before = incl - s;
        for (int w = 0; w < warp; ++w) before += warpSum[w];
        unsigned long long run = tileOffsets[t] + before;
        for (int i = 0; i < kScanPerThread; ++i) {
            if (first + i < n) out[first + i] = run;
            run += v[i];
        }
        __syncthreads();
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) out[n] = tileOffsets[ntiles];
}

// Exclusive prefix sum of n byte-sized values into out[0..n]; out[n] is the total.
static void exclusiveScanU8(Context* ctx, const unsigned char* in, unsigned long long n, unsigned long long* out) {
#ifdef B200C_HOST_EMULATION
    if (B2_EMU(ctx)) {
        unsigned long long run = 0;
        for (unsigned long long i = 0; i < n; ++i) {
            out[i] = run;
            run += in[i];
        }
        out[n] = run;
        ctx->launches += 3;
        return;
    }
#endif
    const unsigned long long ntiles = (n + kScanTile - 1) / kScanTile;
    unsigned int* tileSums = static_cast<unsigned int*>(ctx->arena.alloc((ntiles + 1) * sizeof(unsigned int)));
    unsigned long long* tileOffsets =
            static_cast<unsigned long long*>(ctx->arena.alloc((ntiles + 1) * sizeof(unsigned long long)));
    const int grid = static_cast<int>(std::max<unsigned long long>(1, std::min<unsigned long long>(ntiles, ctx->smCount * 8ULL)));
    scanTileSumsKernel<<<grid, kScanThreads, 0, ctx->stream>>>(in, n, tileSums, ntiles);
    scanTilesKernel<<<1, 1024, 0, ctx->stream>>>(tileSums, ntiles, tileOffsets);
    scanScatterKernel<<<grid, kScanThreads, 0, ctx->stream>>>(in, n, tileOffsets, out, ntiles);
    B2_CUDA(cudaGetLastError());
    ctx->launches += 3;
}

// ---------------------------------------------------------------------------- layout
// Single thread: per-buffer record bytes, stream size, "not smaller" flag and output placement
// (each segment starts on a 32-byte boundary).
B2_HD void layoutJobs(CodecJobDev* jobs, int njobs, const unsigned long long* offsets, unsigned long long outCap,
                      int rawFallback, int* err) {
    unsigned long long run = 0;
    for (int j = 0; j < njobs; ++j) {
        CodecJobDev& job = jobs[j];
        job.recordsBytes = offsets[job.firstBlock + job.nblocks] - offsets[job.firstBlock];
        const unsigned long long raw = kCodecHeaderBytes + 4 * job.nsuper + job.recordsBytes;
        job.streamBytes = (raw + 31) & ~31ull;
        job.notSmaller = job.n <= job.streamBytes;  // bit_compactor_codec.cpp:36-39
        job.outBytes = (rawFallback && job.notSmaller) ? job.n : job.streamBytes;
        job.outBase = run;
        run = (run + job.outBytes + 31) & ~31ull;
        if (job.outBase + job.outBytes > outCap) {
            if (*err == E_NONE) *err = E_CODEC;
            job.outBytes = 0;
        }
    }
}

__global__ void codecLayoutKernel(CodecJobDev* jobs, int njobs, const unsigned long long* offsets,
                                  unsigned long long outCap, int rawFallback, int* err) {
    if (blockIdx.x == 0 && threadIdx.x == 0) layoutJobs(jobs, njobs, offsets, outCap, rawFallback, err);
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

B2_HD void emitOne(const CodecJobDev* jobs, int njobs, unsigned long long g, const unsigned char* headers,
                   const unsigned char* bases, const unsigned long long* offsets, unsigned char* out,
                   int rawFallback) {
    const CodecJobDev& job = jobs[jobOfBlock(jobs, njobs, g)];
    const unsigned long long blk = g - job.firstBlock;
    if (blk >= job.nblocks || job.outBytes == 0) return;
    unsigned char* dst = out + job.outBase;
    alignas(16) unsigned char b[kCodecBlock];
    loadBlock(job, blk, b);
    if (rawFallback && job.notSmaller) {  // segment keeps the input bytes
        const unsigned long long first = blk * kCodecBlock;
        for (int i = 0; i < kCodecBlock && first + i < job.n; ++i) dst[first + i] = b[i];
        return;
    }
    const unsigned long long rel = offsets[g] - offsets[job.firstBlock];
    unsigned char* records = dst + kCodecHeaderBytes + 4 * job.nsuper;
    codecWriteRecord(b, headers[g], bases[g], records + rel);
    if (blk % kCodecSuper == 0) putU32(dst + kCodecHeaderBytes + 4 * (blk / kCodecSuper), static_cast<unsigned int>(rel));
    if (blk == 0) {
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
    if (blk + 1 == job.nblocks) {
        for (unsigned long long a = kCodecHeaderBytes + 4 * job.nsuper + job.recordsBytes; a < job.streamBytes; ++a) dst[a] = 0;
    }
}

__global__ void __launch_bounds__(128) codecEmitKernel(const CodecJobDev* __restrict__ jobs, int njobs,
                                                       unsigned long long totalBlocks,
                                                       const unsigned char* __restrict__ headers,
                                                       const unsigned char* __restrict__ bases,
                                                       const unsigned long long* __restrict__ offsets,
                                                       unsigned char* out, int rawFallback) {
    const unsigned long long step = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
    for (unsigned long long g = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x; g < totalBlocks;
         g += step) {
        emitOne(jobs, njobs, g, headers, bases, offsets, out, rawFallback);
    }
}

void codecCompressBatch(Context* ctx, int count, const CodecBuf* bufs, unsigned char* outDev, size_t outCap,
                        bool rawFallback, CodecResult* results) {
    if (count <= 0) return;
    std::vector<CodecJobDev> jobs(count);
    unsigned long long totalBlocks = 0;
    for (int j = 0; j < count; ++j) {
        if (bufs[j].n == 0) refThrow("BitCompactorCodec::compress: Empty input data vector");
        if (bufs[j].n >= (1ull << 32)) throw NotBuilt("codec input of 4 GiB or more");
        std::memset(&jobs[j], 0, sizeof(CodecJobDev));
        jobs[j].in = bufs[j].in;
        jobs[j].n = bufs[j].n;
        jobs[j].nblocks = (bufs[j].n + kCodecBlock - 1) / kCodecBlock;
        jobs[j].nsuper = (jobs[j].nblocks + kCodecSuper - 1) / kCodecSuper;
        jobs[j].firstBlock = totalBlocks;
        totalBlocks += jobs[j].nblocks;
    }
    CodecJobDev* jobsDev = static_cast<CodecJobDev*>(ctx->arena.alloc(sizeof(CodecJobDev) * count));
    unsigned char* headers = static_cast<unsigned char*>(ctx->arena.alloc(totalBlocks + 16));
    unsigned char* bases = static_cast<unsigned char*>(ctx->arena.alloc(totalBlocks + 16));
    unsigned char* sizes = static_cast<unsigned char*>(ctx->arena.alloc(totalBlocks + 16));
    unsigned long long* offsets =
            static_cast<unsigned long long*>(ctx->arena.alloc((totalBlocks + 1) * sizeof(unsigned long long)));
    copyH2D(ctx, jobsDev, jobs.data(), sizeof(CodecJobDev) * count);

#ifdef B200C_HOST_EMULATION
    if (B2_EMU(ctx)) {
        for (unsigned long long g = 0; g < totalBlocks; ++g) analyzeOne(jobsDev, count, g, headers, bases, sizes);
        exclusiveScanU8(ctx, sizes, totalBlocks, offsets);
        layoutJobs(jobsDev, count, offsets, outCap, rawFallback, ctx->errWord);
        for (unsigned long long g = 0; g < totalBlocks; ++g)
            emitOne(jobsDev, count, g, headers, bases, offsets, outDev, rawFallback);
        ctx->launches += 3;
    } else
#endif
    {
        const int grid = static_cast<int>(
                std::max<unsigned long long>(1, std::min<unsigned long long>((totalBlocks + 127) / 128, ctx->smCount * 16ULL)));
        codecAnalyzeKernel<<<grid, 128, 0, ctx->stream>>>(jobsDev, count, totalBlocks, headers, bases, sizes);
        B2_CUDA(cudaGetLastError());
        exclusiveScanU8(ctx, sizes, totalBlocks, offsets);
        codecLayoutKernel<<<1, 32, 0, ctx->stream>>>(jobsDev, count, offsets, outCap, rawFallback ? 1 : 0, ctx->errWord);
        codecEmitKernel<<<grid, 128, 0, ctx->stream>>>(jobsDev, count, totalBlocks, headers, bases, offsets, outDev,
                                                       rawFallback ? 1 : 0);
        B2_CUDA(cudaGetLastError());
        ctx->launches += 3;
    }
    copyD2H(ctx, jobs.data(), jobsDev, sizeof(CodecJobDev) * count);
    syncStream(ctx);
    checkDeviceError(ctx);
    for (int j = 0; j < count; ++j) {
        results[j].offset = jobs[j].outBase;
        results[j].size = jobs[j].outBytes;
        results[j].notSmaller = jobs[j].notSmaller != 0;
    }
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
#ifdef B200C_HOST_EMULATION
    if (B2_EMU(ctx)) {
        for (unsigned long long s = 0; s < p.nsuper; ++s) decodeGroup(p, s);
        ++ctx->launches;
    } else
#endif
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
