// Per-context runtime state: stream, scratch arena, error word, launch accounting.
#pragma once

#include "../../include/b200const.h"
#include "ctype.h"
#include "view.h"

#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include <cstdint>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

namespace b200c {

#define B2_CUDA(call)                                                                              \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess) {                                                                   \
            throw ::b200c::CudaFail(std::string(#call) + ": " + cudaGetErrorString(e_));           \
        }                                                                                          \
    } while (0)

struct Context;

// Named range on the profiler's timeline (NVTX; a no-op when no tool is attached): the phases of a
// batched fold -- planning, flushing, compression, exchange -- show up next to the kernels they launch.
struct TraceRange {
    explicit TraceRange(const char* name) {
        nvtxRangePushA(name);
    }
    ~TraceRange() {
        nvtxRangePop();
    }
    TraceRange(const TraceRange&) = delete;
    TraceRange& operator=(const TraceRange&) = delete;
};

// Fused single-pass quantiser (rowquant_kernels.cu): rows are contiguous in the source; the output
// keeps the row order and may permute elements inside a row.
struct RowQuantParams {
    const void* src;
    int srcTag;  // T_F16 or T_F32
    long long rows, rowElems;
    int scheme;
    float* scales;
    int* zps;
    int irank;  // within-row output map: 0 = identity, else mixed radix ishape/istride (outermost first)
    long long ishape[3], istride[3];
    void* dst;
    int outMode;  // 0: one byte per element, 1: BitPack nibbles
    int swizzleKey;
    long long dataBytes, totalBytes;
    int vecIn, vecOut;  // filled by the launcher
    long long smemRowElems;
    int padLog2;  // staged rows: 16 bytes of padding after every 2^padLog2 elements (31: none), filled by the launcher
};


// Bump allocator over device memory.  Blocks are kept for the life of the context and reused by
// every call; reset() rewinds to the start.
class Arena {
public:
    explicit Arena(Context* ctx): _ctx(ctx) {
    }
    void setMinBlock(size_t bytes) {
        _minBlock = bytes;
    }
    ~Arena();
    void* alloc(size_t bytes, size_t align = 256);
    void reset();
    void releaseAll();
    size_t reserved() const;

private:
    struct Block {
        char* ptr;
        size_t size, used;
    };
    Context* _ctx;
    std::vector<Block> _blocks;
    size_t _minBlock = 64ull << 20;
};

// One tile-kernel work item (tile_kernels.cu): a view in canonical form plus its tiling.
struct TileItem {
    GenParams g;
    int py;          // output dim whose source stride is 1 (the transposed direction), or -1
    int tx, ty;      // tile extents along the innermost output dim and along py
    int esIn;        // bytes per source element
    int needCoords;  // a per-axis operation needs the full coordinates of every element
    int fast;        // 0: element-wise body; 1: raw contiguous copy; 2: raw transpose of source-contiguous blocks
    int tz;          // fast == 2: consecutive outer blocks (dim rank-3) per tile
    long long tilesX, tilesY, tilesZ, tiles;
    long long outStride[kMaxDims];
};
bool makeTileItem(const GenParams& p, TileItem* out);

// A queued tile-kernel item of a batched fold: the launch parameters live once in device memory (a
// "template": constants of the same type, chain and alignment share it), the item itself is only the
// template's address, its own buffers and its tile count.
struct TileRef {
    const TileItem* templ;  // device
    const void* src;
    void* dst;
    long long tiles;
};
// Templates are written into slabs of device memory reserved from the arena; the host copies wait in
// the slab until the next flush uploads them with one copy per slab.
struct TileSlab {
    static constexpr int kCapacity = 64;
    TileItem* dev = nullptr;
    std::vector<TileItem> host;
    size_t uploaded = 0;
};

// One GetSparsityMap of 8-bit elements written straight to its final place (sparsity_kernels.cu).
struct MapItem {
    const unsigned char* src;
    unsigned char* dst;
    long long oc, work;        // channels, elements per channel (a multiple of 16)
    long long outBytesPerOC;   // map bytes per channel (rows padded to 128 bits)
    long long totalBytes;      // bytes to write: the map, then zeros up to the swizzle size alignment
    unsigned int sparseByte;
    int swizzleKey;
    long long* counts;         // when a Sparsify of the same batch reads the same source: its per-channel counts,
                               // written here as a by-product of the one read (else nullptr)
};

// One Sparsify of 8-bit elements written straight to its final place.
struct SparseItem {
    const unsigned char* src;
    unsigned char* dst;
    long long oc, work;
    long long* counts;     // [oc] non-sparse elements per channel (device scratch)
    long long* offsets;    // [oc + 1] byte offset of every channel, total at [oc] (device scratch)
    long long* bytesOut;   // device word: size of the result in bytes
    long long dstCap;      // bytes available at dst
    long long fixedBytes;  // buffer size given by numActualElements, or -1 when the data decides
    unsigned int sparseByte;
    int swizzleKey;        // -1: not swizzled
    int* err;
    int countsReady;       // the sparsity-map kernel of the same batch has already counted this source
};

class PlanPool;

// block codec (codec.h, codec_kernels.cu)
struct CodecJobDev {
    const unsigned char* in;
    unsigned long long n, nblocks, nsuper, firstBlock;
    unsigned long long recordsBytes, streamBytes, outBase, outBytes;
    int notSmaller;
    int failed;
};
struct CodecBuf {
    const unsigned char* in;  // device
    size_t n;
};
struct CodecResult {
    size_t offset, size;
    bool notSmaller;
};
// An in-place batch compression whose launches are queued and whose sizes have not been read yet: the
// per-buffer records come back into pinned host memory behind `done`.
struct CodecPending {
    bool open = false;
    int count = 0;
    CodecJobDev* jobsHost = nullptr;  // pinned
    size_t capacity = 0;              // records jobsHost can hold; one more slot behind them holds the error word
    int errCode = 0;                  // device error word as it stood behind the queued work (set by codecCollect)
    cudaEvent_t done = nullptr;
    std::vector<CodecBuf> bufs;
};

// What planning one constant of a batched fold came to, when that was a single queued launch item and
// nothing else: kept under a key made of the constant's descriptors so that the next constant with the
// same base type, chain and buffer alignment (another layer of the same shape) reuses the item with its
// own pointers instead of being planned again.  Entries live for one b200c_fold_batch call.
struct PlanMemo {
    int queue;  // 0: fused quantiser, 1: tile kernel, 2: sparsity map, 3: sparsify
    RowQuantParams rq;
    TileRef tile;
    MapItem map;
    SparseItem sparse;
    size_t outBytes;
    long long queuedBytes;
};

struct Context {
    int device = 0;
    // device memory for the library's own scratch (arena blocks): the caller's allocator when one is
    // installed with b200c_set_allocator, else cudaMalloc / cudaFree
    b200c_alloc_fn allocFn = nullptr;
    b200c_free_fn freeFn = nullptr;
    void* allocUser = nullptr;
    cudaStream_t ownStream = nullptr;
    cudaStream_t stream = nullptr;
    std::mutex mu;
    Arena arena{this};
    int* errWord = nullptr;      // device
    int* errHost = nullptr;      // pinned host mirror
    int64_t launches = 0;
    int smCount = 148;
    size_t l2Bytes = 0;
    bool batching = false;                 // inside b200c_fold_batch: fused quantiser launches are queued
    std::vector<RowQuantParams> rqBatch;
    std::vector<TileRef> tileBatch;
    std::vector<TileSlab> tileSlabs;       // templates of this call's tile items (reset with the arena)
    std::vector<MapItem> mapBatch;
    std::vector<SparseItem> sparseBatch;
    long long queuedBytes = 0;             // input bytes of the queued launches (drives early flushes)
    static constexpr int kCodecTickets = 8;
    CodecPending codecTickets[kCodecTickets];  // asynchronous in-place compressions not collected yet
    long long directOps = 0;               // copies and fills issued straight to the stream (not queued items)
    std::unordered_map<std::string, PlanMemo> planMemo;
    std::string planKey;
    // planning threads of the batched entry point: each plans items into a context of its own
    // (same stream and error word, own scratch arena and launch queues)
    PlanPool* pool = nullptr;
    std::vector<Context*> workers;
    // pinned staging for the library's own small uploads (tables, launch parameter arrays): two sets of
    // chunks used by alternate calls; a set is refilled only after the uploads of the call that used it
    // last (two calls ago) have passed, so back-to-back asynchronous calls never wait for each other
    struct StageChunk {
        char* ptr;
        size_t size, used;
    };
    std::vector<StageChunk> stage[2];
    cudaEvent_t stageDone[2] = {nullptr, nullptr};
    bool stagePending[2] = {false, false};
    int stageSet = 0;
    // multi-GPU exchange (exchange_kernels.cu), created on first use: a second stream for pushes and
    // downloads, completion counters of the push kernels (each reset by its last CTA), the status word
    // of the bounded waits, and a ring of parameter buffers the arena's rewinding cannot touch
    static constexpr unsigned kXferCounters = 256, kXferParamSlots = 8;
    struct XferParams {
        void* dev = nullptr;
        void* host = nullptr;
        size_t bytes = 0;
        cudaEvent_t done = nullptr;
        bool pending = false;
    };
    cudaStream_t xferStream = nullptr;
    cudaEvent_t xferEvent = nullptr;
    unsigned int* xferCounters = nullptr;
    int* xferStatus = nullptr;
    unsigned xferCounterNext = 0, xferSlotNext = 0;
    XferParams xferParams[kXferParamSlots];
};


// ---- batched launches: which item does unit b belong to? ------------------------------------
// `start` holds the exclusive prefix sums of the items' unit counts (nitems entries) followed by a
// coarse index: entry g is the item that contains unit 64 * g, plus one closing entry.  A lookup
// reads two neighbouring coarse entries and then searches only between them (usually nothing).
inline void appendCoarseIndex(std::vector<long long>& start, long long total) {
    const size_t n = start.size();
    const long long groups = (total + 63) / 64;
    size_t k = 0;
    for (long long g = 0; g < groups; ++g) {
        while (k + 1 < n && start[k + 1] <= g * 64) ++k;
        start.push_back(static_cast<long long>(k));
    }
    start.push_back(static_cast<long long>(n ? n - 1 : 0));
}
#ifdef __CUDACC__
__device__ __forceinline__ int findBatchItem(const long long* __restrict__ start, int nitems, long long b) {
    const long long* coarse = start + nitems;
    int lo = static_cast<int>(coarse[b >> 6]), hi = static_cast<int>(coarse[(b >> 6) + 1]);
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (start[mid] <= b) {
            lo = mid;
        } else {
            hi = mid - 1;
        }
    }
    return lo;
}
#endif

// device memory through the context
void* devMalloc(Context* ctx, size_t bytes);
void devFree(Context* ctx, void* p);
void copyH2D(Context* ctx, void* dst, const void* src, size_t n);
// host -> device copy of internal data through pinned staging: returns at once, never waits for the
// stream (a copy from pageable memory may); `src` can be freed on return
void uploadSmall(Context* ctx, void* dst, const void* src, size_t n);
void resetStage(Context* ctx);
void releaseStage(Context* ctx);
void copyD2H(Context* ctx, void* dst, const void* src, size_t n);
void copyD2D(Context* ctx, void* dst, const void* src, size_t n);
void fillBytes(Context* ctx, void* dst, int value, size_t n);
void syncStream(Context* ctx);
// Reads and clears the device error word (synchronises); maps it to a RefThrow.
void checkDeviceError(Context* ctx);

// ---- kernel entry points (defined in the .cu files) ----------------------------------------
void launchGeneric(Context* ctx, const GenParams& p);
// RelocateWeightsTable (relocate_weights_table.cpp:122-203): one thread per output channel patches
// the weights pointer and, unless it holds the "no sparsity" marker, the sparsity pointer
struct RelocateParams {
    const int* values;  // dense weights table, 4 entries per output channel
    int* patched;
    long long oc;
    const int* clusterOf;            // cluster index of every output channel (the reference's running index)
    long long offsets[kMaxDims];     // first output channel of every cluster
    long long weightsPtr[kMaxDims];  // base weights pointer of every cluster
    int sparsityPtr;
    const long long* steps;  // per-channel weights pointer offsets of a compressed layout, or nullptr
    int* err;
};
void launchRelocateWeightsTable(Context* ctx, const RelocateParams& p);
// ExpandDilated: element (plane, ky, kx) of the dense source goes to (plane, ky * d0, kx * d1); the rest is `fill`
void launchExpandDilated(Context* ctx, const void* src, void* dst, int es, long long planes, long long ky, long long kx,
                         long long dky, long long dkx, long long d0, long long d1, unsigned long long fill);
// queued while ctx->batching is set, launched by flushTileBatch
void launchTile(Context* ctx, const TileItem& it);
// uploads the templates `from` has gathered since its last upload (through `ctx`'s staging) and launches
// what `ctx` has queued
void uploadTileTemplates(Context* ctx, Context* from);
void flushTileBatch(Context* ctx);
// contiguous rows of 8-bit storage with one Dequantize and f16/f32 output (dequant_kernels.cu)
bool tryLaunchDequantRows(Context* ctx, const GenParams& p);

struct RowStatsParams {
    GenParams view;       // evaluates the Content before quantisation (outMode unused)
    int rowDim;           // view dim holding logical dim 0
    long long rows;
    long long rowElems;   // elements per row
    int scheme;
    float* scales;        // [rows]
    int* zps;             // [rows]
};
void launchRowStats(Context* ctx, const RowStatsParams& p);

// Fused single-pass quantiser (rowquant_kernels.cu)
void launchRowQuantFused(Context* ctx, RowQuantParams p);
void flushRowQuantBatch(Context* ctx);
size_t rowQuantMaxRowBytes();

// 8-bit sparsity transforms whose result goes straight to the caller's buffer: queued while
// ctx->batching is set and launched by flushSparsityBatch (one launch per stage for all items)
void launchMapItem(Context* ctx, const MapItem& it);
void launchSparseItem(Context* ctx, const SparseItem& it);
void flushSparsityBatch(Context* ctx);
// hostOut[i] = *ptrs[i] (device words), valid after the stream has been synchronised
void gatherDeviceWords(Context* ctx, const std::vector<const long long*>& ptrs, long long* hostOut);
// sparsity (GetSparsityMap / Sparsify) on a dense buffer of `tag` elements laid out [OC][work]
void launchSparsityMap(Context* ctx, const void* src, int tag, long long oc, long long work, long long outBitsPerOC,
                       unsigned long long sparseBits, void* dstBits, int swizzleKey);
void launchCountNonSparse(Context* ctx, const void* src, int tag, long long oc, long long work,
                          unsigned long long sparseBits, long long* counts);
void launchSparsifyOffsets(Context* ctx, const long long* counts, long long oc, int elemBytes, long long* offsets,
                           long long* total);
void launchSparsifyScatter(Context* ctx, const void* src, int tag, long long oc, long long work,
                           unsigned long long sparseBits, const long long* offsets, void* dst, long long dstBytes,
                           int swizzleKey, int* err);

// swizzle of an existing byte buffer (16-byte chunks), zero or constant tail
void launchSwizzleCopy(Context* ctx, const void* src, long long srcBytes, void* dst, long long totalBytes, int key,
                       int tailByte);
// SubView on bit-packed i1 storage
void launchSubViewBits(Context* ctx, const void* src, void* dst, int rank, const long long* outShape,
                       const long long* inStride, long long base, long long outBits);

// block codec (codec.h, codec_kernels.cu)
size_t codecBound(size_t n);
// Compresses `count` device buffers into outDev; segment i starts at results[i].offset (32-byte
// aligned).  With rawFallback a buffer whose stream would not be smaller is stored unchanged.
// rawFallback 2: in place -- a buffer whose stream is smaller gets the stream written over its own
// head (results[i].size = stream length), every other buffer is left untouched; outDev is unused.
// With `pending` (in-place mode only) the call returns after queueing its launches; codecCollect waits for
// them and delivers the results.
void codecCompressBatch(Context* ctx, int count, const CodecBuf* bufs, unsigned char* outDev, size_t outCap,
                        int rawFallback, CodecResult* results, CodecPending* pending = nullptr);
void codecCollect(Context* ctx, CodecPending* pending, CodecResult* results);
// allocation-free single-buffer variant (fixed scratch inside the library image)
size_t codecNoAllocMaxInput();
void codecCompressNoAlloc(int device, const unsigned char* inDev, size_t n, unsigned char* outDev, size_t cap,
                          cudaStream_t stream, size_t* outN, bool* notSmaller);
size_t codecDecompress(Context* ctx, const unsigned char* inDev, size_t n, unsigned char* outDev, size_t cap);

// whole-buffer reductions (probe_kernels.cu)
bool probeSplat(Context* ctx, const void* dataDev, size_t nbytes, int elemBytes);
void digestBatch(Context* ctx, int count, const void* const* bufs, const size_t* sizes, unsigned long long* out);

// multi-GPU exchange (exchange_kernels.cu)
void registerAllocation(void* p, size_t n);
void unregisterAllocation(void* p);
void ipcExport(Context* ctx, void* devPtr, size_t size, unsigned char handle[64], unsigned long long* offset);
void* ipcOpen(Context* ctx, const unsigned char handle[64], unsigned long long offset);
void ipcClose(Context* ctx, void* mapped);
void pushSegments(Context* ctx, const b200c_copy_seg* segs, int count, const unsigned long long* waitFlag,
                  unsigned long long waitValue, unsigned long long* doneFlag, unsigned long long doneValue,
                  unsigned int timeoutMs, int mode, int ctas, cudaEvent_t after = nullptr);
void waitFlags(Context* ctx, const unsigned long long* flagsDev, int count, unsigned long long value, unsigned int timeoutMs,
               bool onTransferStream);
void signalFlags(Context* ctx, unsigned long long* const* targets, int count, unsigned long long value);
int exchangeStatus(Context* ctx);
void releaseExchange(Context* ctx);

// synthetic weights
void launchSynthFill(Context* ctx, void* dst, long long count, int dtype, int dist, double p0, double p1,
                     unsigned long long seed, unsigned long long stream);

}  // namespace b200c
