// Whole-buffer reductions: the "all elements equal" probe behind splat detection of dense resources
// (detectSplatElementWise, src/vpux_compiler/src/dialect/const/attributes/content.cpp:103-137) and the
// 64-bit buffer digest used to compare blobs produced by different shardings.
#include "runtime.h"

#include <algorithm>
#include <vector>

namespace b200c {

// ---------------------------------------------------------------------------- splat probe
// Every element is compared with element 0.  The element pattern is replicated into 16 bytes, so the
// aligned body is one 128-bit load and one compare per 16 bytes; the unaligned head and tail are
// compared byte-wise against the pattern at the same phase.  A mismatch sets *differs; CTAs look at the
// word before each of their strides and stop early once it is set.
__global__ void __launch_bounds__(256) splatProbeKernel(const unsigned char* __restrict__ data, unsigned long long n,
                                                        int elemBytes, int* differs) {
    __shared__ unsigned char pat[16];
    if (threadIdx.x < 16) pat[threadIdx.x] = data[threadIdx.x % elemBytes];
    __syncthreads();
    const unsigned long long head = min(n, static_cast<unsigned long long>((16 - (reinterpret_cast<uintptr_t>(data) & 15)) & 15));
    const unsigned long long nvec = (n - head) / 16;
    const unsigned long long tailAt = head + nvec * 16;
    const unsigned long long tid = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const unsigned long long step = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
    bool bad = false;
    if (tid < head) bad = data[tid] != pat[tid % elemBytes];
    if (tailAt + tid < n) bad = bad || data[tailAt + tid] != pat[(tailAt + tid) % elemBytes];
    // the aligned body starts at byte `head`: its pattern is the element pattern rotated by head % elemBytes
    uint4 want;
    {
        unsigned int w[4];
        for (int k = 0; k < 4; ++k) {
            w[k] = 0;
            for (int b = 0; b < 4; ++b) w[k] |= static_cast<unsigned int>(pat[(head + 4 * k + b) % elemBytes]) << (8 * b);
        }
        want = make_uint4(w[0], w[1], w[2], w[3]);
    }
    const uint4* body = reinterpret_cast<const uint4*>(data + head);
    int round = 0;
    for (unsigned long long v = tid; v < nvec && !bad; v += step) {
        const uint4 x = __ldg(body + v);
        bad = (x.x != want.x) | (x.y != want.y) | (x.z != want.z) | (x.w != want.w);
        if ((++round & 63) == 0 && *reinterpret_cast<volatile int*>(differs)) break;  // someone else found a mismatch
    }
    if (bad) *differs = 1;
}

bool probeSplat(Context* ctx, const void* dataDev, size_t nbytes, int elemBytes) {
    int* flag = static_cast<int*>(ctx->arena.alloc(sizeof(int)));
    fillBytes(ctx, flag, 0, sizeof(int));
    const unsigned long long nvec = nbytes / 16 + 1;
    const int grid = static_cast<int>(std::max<unsigned long long>(1, std::min<unsigned long long>((nvec + 255) / 256, ctx->smCount * 8ULL)));
    splatProbeKernel<<<grid, 256, 0, ctx->stream>>>(static_cast<const unsigned char*>(dataDev), nbytes, elemBytes, flag);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
    int differs = 0;
    copyD2H(ctx, &differs, flag, sizeof(int));
    syncStream(ctx);
    return differs == 0;
}

// ---------------------------------------------------------------------------- digest
// digest64(bytes, n) = mix(C0 * (n + 1) + sum_j mix(word_j ^ (C1 * (j + 1)))) over the little-endian
// 64-bit words of the buffer (the last one zero-extended), all modulo 2^64; mix is the splitmix64
// finaliser.  The kernel accumulates the sum per buffer; the host adds the length term and the final mix.
__host__ __device__ __forceinline__ unsigned long long digestMix(unsigned long long x) {
    x ^= x >> 30;
    x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27;
    x *= 0x94D049BB133111EBull;
    x ^= x >> 31;
    return x;
}

struct DigestItem {
    const unsigned char* data;
    unsigned long long n;
    unsigned long long firstTile;  // index of the item's first tile in the launch
};
constexpr unsigned long long kDigestTileWords = 8192;  // 64 KB per CTA tile

__global__ void __launch_bounds__(256) digestKernel(const DigestItem* __restrict__ items, const unsigned int* __restrict__ tileItem,
                                                    unsigned long long ntiles, unsigned long long* __restrict__ sums) {
    __shared__ unsigned long long red[8];
    for (unsigned long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const unsigned int it = tileItem[tile];
        const DigestItem item = items[it];
        const unsigned long long words = (item.n + 7) / 8;
        const unsigned long long w0 = (tile - item.firstTile) * kDigestTileWords;
        const unsigned long long w1 = min(words, w0 + kDigestTileWords);
        const bool aligned = (reinterpret_cast<uintptr_t>(item.data) & 7) == 0;
        unsigned long long acc = 0;
        for (unsigned long long j = w0 + threadIdx.x; j < w1; j += blockDim.x) {
            unsigned long long w = 0;
            if (aligned && (j + 1) * 8 <= item.n) {
                w = __ldg(reinterpret_cast<const unsigned long long*>(item.data) + j);
            } else {
                for (int b = 0; b < 8; ++b) {
                    const unsigned long long at = j * 8 + b;
                    if (at < item.n) w |= static_cast<unsigned long long>(item.data[at]) << (8 * b);
                }
            }
            acc += digestMix(w ^ (0xD6E8FEB86659FD93ull * (j + 1)));
        }
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long t = 0;
            for (int w = 0; w < 8; ++w) t += red[w];
            atomicAdd(sums + it, t);
        }
        __syncthreads();
    }
}

void digestBatch(Context* ctx, int count, const void* const* bufs, const size_t* sizes, unsigned long long* out) {
    if (count <= 0) return;
    std::vector<DigestItem> items(count);
    std::vector<unsigned int> tileItem;
    unsigned long long ntiles = 0;
    for (int i = 0; i < count; ++i) {
        items[i].data = static_cast<const unsigned char*>(bufs[i]);
        items[i].n = sizes[i];
        items[i].firstTile = ntiles;
        const unsigned long long words = (sizes[i] + 7) / 8;
        const unsigned long long t = (words + kDigestTileWords - 1) / kDigestTileWords;
        tileItem.insert(tileItem.end(), t, static_cast<unsigned int>(i));
        ntiles += t;
    }
    DigestItem* itemsDev = static_cast<DigestItem*>(ctx->arena.alloc(sizeof(DigestItem) * count));
    unsigned long long* sums = static_cast<unsigned long long*>(ctx->arena.alloc(sizeof(unsigned long long) * count));
    uploadSmall(ctx, itemsDev, items.data(), sizeof(DigestItem) * count);
    fillBytes(ctx, sums, 0, sizeof(unsigned long long) * count);
    if (ntiles) {
        unsigned int* tileDev = static_cast<unsigned int*>(ctx->arena.alloc(sizeof(unsigned int) * ntiles));
        uploadSmall(ctx, tileDev, tileItem.data(), sizeof(unsigned int) * ntiles);
        const int grid = static_cast<int>(std::min<unsigned long long>(ntiles, ctx->smCount * 8ULL));
        digestKernel<<<grid, 256, 0, ctx->stream>>>(itemsDev, tileDev, ntiles, sums);
        B2_CUDA(cudaGetLastError());
        ++ctx->launches;
    }
    copyD2H(ctx, out, sums, sizeof(unsigned long long) * count);
    syncStream(ctx);
    for (int i = 0; i < count; ++i) out[i] = digestMix(0x9E3779B97F4A7C15ull * (static_cast<unsigned long long>(sizes[i]) + 1) + out[i]);
}

}  // namespace b200c
