// The one exchange of a multi-GPU fold: every rank's finished blob slots travel into rank 0's blob
// buffer over NVLink.  The owner of the data pushes: its own SMs (or copy engine) store into rank 0's
// buffer, mapped into the pushing process through CUDA IPC, so neither an SM nor a copy engine of
// rank 0 is spent on the transfer.  Hand-shakes are 64-bit sequence words in device memory:
//   done flag    (in rank 0's memory, one per pushing rank and chunk): written by the pusher after
//                its stores, read by rank 0's wait kernel;
//   release flag (in the pusher's memory): written by rank 0 once the previous blob has been
//                consumed, read by the pusher before its first store of the next step.
// Every wait is bounded: after the time limit the kernel records the time-out in a status word and
// returns (a pusher that timed out stores nothing and raises no flag), so a missing peer becomes an
// error code on the host instead of a hang.
//
// Only plain loads and stores touch peer memory -- no TMA, no multicast, no library kernel.
#include "runtime.h"

#include <algorithm>
#include <atomic>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

namespace b200c {

// ---------------------------------------------------------------------------- allocation registry
// b200c_dev_alloc records (base, size) so that an interior pointer can be exported as handle + offset.
static std::mutex g_allocMutex;
static std::map<uintptr_t, size_t> g_allocs;

void registerAllocation(void* p, size_t n) {
    std::lock_guard<std::mutex> lock(g_allocMutex);
    g_allocs[reinterpret_cast<uintptr_t>(p)] = n;
}
void unregisterAllocation(void* p) {
    std::lock_guard<std::mutex> lock(g_allocMutex);
    g_allocs.erase(reinterpret_cast<uintptr_t>(p));
}
static bool findAllocation(const void* p, size_t n, uintptr_t* base, size_t* size) {
    std::lock_guard<std::mutex> lock(g_allocMutex);
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    auto it = g_allocs.upper_bound(a);
    if (it == g_allocs.begin()) return false;
    --it;
    if (a + n > it->first + it->second) return false;
    *base = it->first;
    *size = it->second;
    return true;
}

void ipcExport(Context* ctx, void* devPtr, size_t size, unsigned char handle[64], unsigned long long* offset) {
    (void)ctx;
    uintptr_t base = 0;
    size_t total = 0;
    if (!findAllocation(devPtr, size, &base, &total)) {
        throw BadArg("b200c_ipc_export: the range is not inside a b200c_dev_alloc allocation");
    }
    cudaIpcMemHandle_t h;
    B2_CUDA(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
    static_assert(sizeof(h) == 64, "CUDA IPC handle size");
    std::memcpy(handle, &h, 64);
    *offset = reinterpret_cast<uintptr_t>(devPtr) - base;
}

// mapped base pointers of this process: handle bytes -> (base, reference count)
struct OpenWindow {
    void* base;
    int refs;
};
static std::mutex g_ipcMutex;
static std::map<std::vector<unsigned char>, OpenWindow> g_windows;

void* ipcOpen(Context* ctx, const unsigned char handle[64], unsigned long long offset) {
    (void)ctx;
    std::lock_guard<std::mutex> lock(g_ipcMutex);
    std::vector<unsigned char> key(handle, handle + 64);
    auto it = g_windows.find(key);
    if (it == g_windows.end()) {
        cudaIpcMemHandle_t h;
        std::memcpy(&h, handle, 64);
        void* base = nullptr;
        B2_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
        it = g_windows.emplace(key, OpenWindow{base, 0}).first;
    }
    ++it->second.refs;
    return static_cast<char*>(it->second.base) + offset;
}

void ipcClose(Context* ctx, void* mapped) {
    (void)ctx;
    std::lock_guard<std::mutex> lock(g_ipcMutex);
    // the window whose base is the greatest one not above `mapped`
    auto best = g_windows.end();
    for (auto it = g_windows.begin(); it != g_windows.end(); ++it) {
        if (it->second.base <= mapped && (best == g_windows.end() || it->second.base > best->second.base)) best = it;
    }
    if (best == g_windows.end()) throw BadArg("b200c_ipc_close: not a mapped window");
    if (--best->second.refs == 0) {
        cudaIpcCloseMemHandle(best->second.base);
        g_windows.erase(best);
    }
}

// ---------------------------------------------------------------------------- kernels
__device__ __forceinline__ unsigned long long globalTimerNs() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// true when *flag >= value within the limit
__device__ bool boundedWait(const unsigned long long* flag, unsigned long long value, unsigned long long timeoutNs) {
    const volatile unsigned long long* f = flag;
    const unsigned long long t0 = globalTimerNs();
    // two bounds: wall time, and a number of polls (each sleeps at least 100 ns) in case the timer stalls
    const unsigned long long maxPolls = timeoutNs / 50 + 1000;
    for (unsigned long long polls = 0; polls < maxPolls; ++polls) {
        if (*f >= value) {
            __threadfence_system();
            return true;
        }
        if (globalTimerNs() - t0 > timeoutNs) return false;
        __nanosleep(100);
    }
    return false;
}

struct CopySeg {
    const unsigned char* src;
    unsigned char* dst;
    unsigned long long n;
    unsigned long long firstTile;
};
constexpr unsigned long long kPushTile = 128ull << 10;  // bytes per CTA tile

// status word: bit 0 = a release wait timed out (pusher), bit 1 = a done wait timed out (rank 0)
__global__ void __launch_bounds__(256) pushSegmentsKernel(const CopySeg* __restrict__ segs, const unsigned int* __restrict__ tileSeg,
                                                          unsigned long long ntiles, const unsigned long long* waitFlag,
                                                          unsigned long long waitValue, unsigned long long* doneFlag,
                                                          unsigned long long doneValue, unsigned long long timeoutNs,
                                                          unsigned int* counter, int* status) {
    __shared__ int go;
    if (threadIdx.x == 0) {
        go = 1;
        if (waitFlag && !boundedWait(waitFlag, waitValue, timeoutNs)) {
            go = 0;
            atomicOr(status, 1);
        }
    }
    __syncthreads();
    if (go) {
        for (unsigned long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
            const CopySeg s = segs[tileSeg[tile]];
            const unsigned long long lo = (tile - s.firstTile) * kPushTile;
            const unsigned long long len = min(kPushTile, s.n - lo);
            const unsigned char* src = s.src + lo;
            unsigned char* dst = s.dst + lo;
            if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
                const unsigned long long nvec = len / 16;
                const uint4* s4 = reinterpret_cast<const uint4*>(src);
                uint4* d4 = reinterpret_cast<uint4*>(dst);
                unsigned long long v = threadIdx.x;
                for (; v + 3 * 256 < nvec; v += 4 * 256) {  // four loads in flight per thread
                    const uint4 a = __ldcs(s4 + v), b = __ldcs(s4 + v + 256), c = __ldcs(s4 + v + 512), d = __ldcs(s4 + v + 768);
                    d4[v] = a;
                    d4[v + 256] = b;
                    d4[v + 512] = c;
                    d4[v + 768] = d;
                }
                for (; v < nvec; v += 256) d4[v] = __ldcs(s4 + v);
                for (unsigned long long b = nvec * 16 + threadIdx.x; b < len; b += 256) dst[b] = src[b];
            } else {
                for (unsigned long long b = threadIdx.x; b < len; b += 256) dst[b] = src[b];
            }
        }
    }
    // the last CTA to finish raises the done flag, after every thread's stores have been fenced
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(counter, 1u);
        if (prev == gridDim.x - 1) {
            *counter = 0;  // ready for the next launch that uses this slot
            __threadfence_system();
            if (doneFlag && go) *reinterpret_cast<volatile unsigned long long*>(doneFlag) = doneValue;
        }
    }
}

// ---- bulk-copy form of the push ---------------------------------------------------------------
// The same transfer with the copy done by the SM's bulk-copy (TMA) unit instead of its load/store
// pipeline: one thread per CTA streams 16 KB tiles local HBM -> shared memory -> peer memory through an
// 8-stage ring (cp.async.bulk with an mbarrier per stage on the way in, bulk groups on the way out).
// Plain stores that wait on NVLink fill the load/store queues of their SM and slow every other CTA
// resident there -- a pushing rank folds its next chunk at the same time -- while bulk copies queue
// in the copy unit and leave those queues alone.  No multicast, no tensor map: untiled bulk copies
// with 16-byte aligned addresses and sizes; everything else (tails, unaligned or host-resident
// segments) takes plain loads and stores from the CTA's other warps.
constexpr unsigned int kBulkTile = 16384;
constexpr int kBulkStages = 8;

__device__ __forceinline__ unsigned int smemAddr(const void* p) {
    return static_cast<unsigned int>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ bool barTryWait(unsigned int bar, unsigned int parity) {
    unsigned int ok;
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
    return ok != 0;
}
// bounded: gives up after the time limit (checked every 256 polls) or a fixed number of polls
__device__ bool barWaitBounded(unsigned int bar, unsigned int parity, unsigned long long timeoutNs) {
    const unsigned long long t0 = globalTimerNs();
    for (unsigned int polls = 0; polls < (1u << 26); ++polls) {
        if (barTryWait(bar, parity)) return true;
        if ((polls & 255u) == 255u && globalTimerNs() - t0 > timeoutNs) return false;
    }
    return false;
}

__device__ __forceinline__ int findSeg(const CopySeg* __restrict__ segs, int n, unsigned long long tile) {
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (segs[mid].firstTile <= tile) {
            lo = mid;
        } else {
            hi = mid - 1;
        }
    }
    return lo;
}

__global__ void __launch_bounds__(128) pushBulkKernel(const CopySeg* __restrict__ bulk, int nbulk, unsigned long long nbulkTiles,
                                                      const CopySeg* __restrict__ ragged, int nragged,
                                                      const unsigned long long* waitFlag, unsigned long long waitValue,
                                                      unsigned long long* doneFlag, unsigned long long doneValue,
                                                      unsigned long long timeoutNs, unsigned int* counter, int* status) {
    extern __shared__ __align__(128) unsigned char ring[];
    __shared__ __align__(8) unsigned long long bars[kBulkStages];
    __shared__ unsigned char* dstOf[kBulkStages];
    __shared__ unsigned int bytesOf[kBulkStages];
    __shared__ int go;
    if (threadIdx.x == 0) {
        go = 1;
        for (int s = 0; s < kBulkStages; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smemAddr(&bars[s])) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (waitFlag && !boundedWait(waitFlag, waitValue, timeoutNs)) {
            go = 0;
            atomicOr(status, 1);
        }
    }
    __syncthreads();
    if (go && threadIdx.x == 0) {
        // tiles blockIdx.x, blockIdx.x + gridDim.x, ... ; tile i of this CTA uses stage i % kBulkStages
        const unsigned long long nmine = nbulkTiles > blockIdx.x ? (nbulkTiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        auto issueLoad = [&](unsigned long long i) {
            const unsigned long long tile = blockIdx.x + i * gridDim.x;
            const CopySeg sg = bulk[findSeg(bulk, nbulk, tile)];
            const unsigned long long lo = (tile - sg.firstTile) * kBulkTile;
            const unsigned int bytes = static_cast<unsigned int>(min(static_cast<unsigned long long>(kBulkTile), sg.n - lo));
            const int st = static_cast<int>(i % kBulkStages);
            dstOf[st] = sg.dst + lo;
            bytesOf[st] = bytes;
            const unsigned int bar = smemAddr(&bars[st]);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 smemAddr(ring + static_cast<size_t>(st) * kBulkTile)),
                         "l"(sg.src + lo), "r"(bytes), "r"(bar)
                         : "memory");
        };
        unsigned long long issued = 0;
        for (; issued < nmine && issued < static_cast<unsigned long long>(kBulkStages - 1); ++issued) issueLoad(issued);
        bool ok = true;
        unsigned long long i = 0;
        for (; i < nmine; ++i) {
            const int st = static_cast<int>(i % kBulkStages);
            if (!barWaitBounded(smemAddr(&bars[st]), static_cast<unsigned int>((i / kBulkStages) & 1), timeoutNs)) {
                ok = false;
                break;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dstOf[st]),
                         "r"(smemAddr(ring + static_cast<size_t>(st) * kBulkTile)), "r"(bytesOf[st])
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            if (issued < nmine) {
                // the stage of tile i - 1 is refilled: its store must have read the shared memory (at most the
                // store just issued may still be pending)
                asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                issueLoad(issued);
                ++issued;
            }
        }
        if (!ok) {
            // a load never arrived: record it, give the loads still in flight a bounded chance to land (they
            // write this CTA's shared memory), raise no flag
            atomicOr(status, 4);
            for (unsigned long long j = i + 1; j < issued; ++j) {
                barWaitBounded(smemAddr(&bars[j % kBulkStages]), static_cast<unsigned int>((j / kBulkStages) & 1), timeoutNs);
            }
            go = 0;
        }
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        asm volatile("fence.proxy.async;" ::: "memory");
    } else if (go && threadIdx.x >= 32) {
        for (int r = blockIdx.x; r < nragged; r += gridDim.x) {
            const CopySeg sg = ragged[r];
            for (unsigned long long b = threadIdx.x - 32; b < sg.n; b += blockDim.x - 32) sg.dst[b] = sg.src[b];
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int fine = go;
        const unsigned int prev = atomicAdd(counter, fine ? 1u : 0x10000u);  // a failed CTA poisons the count
        if ((prev & 0xFFFFu) + (prev >> 16) == gridDim.x - 1) {
            *counter = 0;
            __threadfence_system();
            if (doneFlag && fine && (prev >> 16) == 0) *reinterpret_cast<volatile unsigned long long*>(doneFlag) = doneValue;
        }
    }
}

__global__ void __launch_bounds__(32) waitFlagsKernel(const unsigned long long* flags, int count, unsigned long long value,
                                                      unsigned long long timeoutNs, int* status) {
    for (int i = threadIdx.x; i < count; i += 32) {
        if (!boundedWait(flags + i, value, timeoutNs)) atomicOr(status, 2);
    }
}

// one 64-bit word per target (targets may be peer memory)
__global__ void __launch_bounds__(32) signalFlagsKernel(unsigned long long* const* targets, int count, unsigned long long value) {
    __threadfence_system();
    for (int i = threadIdx.x; i < count; i += 32) *reinterpret_cast<volatile unsigned long long*>(targets[i]) = value;
}

// ---------------------------------------------------------------------------- host side
static void ensureExchange(Context* ctx) {
    if (ctx->xferStream) return;
    int lo = 0, hi = 0;
    B2_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    B2_CUDA(cudaStreamCreateWithPriority(&ctx->xferStream, cudaStreamNonBlocking, hi));
    B2_CUDA(cudaEventCreateWithFlags(&ctx->xferEvent, cudaEventDisableTiming));
    B2_CUDA(cudaMalloc(&ctx->xferCounters, sizeof(unsigned int) * Context::kXferCounters + sizeof(int)));
    B2_CUDA(cudaMemset(ctx->xferCounters, 0, sizeof(unsigned int) * Context::kXferCounters + sizeof(int)));
    ctx->xferStatus = reinterpret_cast<int*>(ctx->xferCounters + Context::kXferCounters);
}

void releaseExchange(Context* ctx) {
    if (!ctx->xferStream) return;
    cudaStreamSynchronize(ctx->xferStream);
    cudaFree(ctx->xferCounters);
    for (auto& slot : ctx->xferParams) {
        if (slot.dev) cudaFree(slot.dev);
        if (slot.host) cudaFreeHost(slot.host);
        if (slot.done) cudaEventDestroy(slot.done);
        slot = Context::XferParams();
    }
    cudaEventDestroy(ctx->xferEvent);
    cudaStreamDestroy(ctx->xferStream);
    ctx->xferStream = nullptr;
    ctx->xferCounters = nullptr;
    ctx->xferStatus = nullptr;
}

// parameter ring of the exchange: a slot whose previous user has finished, grown to `bytes`
static Context::XferParams* takeParamSlot(Context* ctx, size_t bytes) {
    Context::XferParams* slot = &ctx->xferParams[ctx->xferSlotNext++ % Context::kXferParamSlots];
    if (!slot->done) B2_CUDA(cudaEventCreateWithFlags(&slot->done, cudaEventDisableTiming));
    if (slot->pending) {
        B2_CUDA(cudaEventSynchronize(slot->done));
        slot->pending = false;
    }
    if (slot->bytes < bytes) {
        if (slot->dev) cudaFree(slot->dev);
        if (slot->host) cudaFreeHost(slot->host);
        slot->dev = slot->host = nullptr;
        slot->bytes = std::max<size_t>(bytes * 2, 1 << 16);
        B2_CUDA(cudaMalloc(&slot->dev, slot->bytes));
        B2_CUDA(cudaMallocHost(&slot->host, slot->bytes));
    }
    return slot;
}

static void pushSegmentsBulk(Context* ctx, const b200c_copy_seg* segs, int count, const unsigned long long* waitFlag,
                             unsigned long long waitValue, unsigned long long* doneFlag, unsigned long long doneValue,
                             unsigned long long timeoutNs, int ctas, unsigned int* counter) {
    std::vector<CopySeg> bulk, ragged;
    unsigned long long ntiles = 0;
    for (int i = 0; i < count; ++i) {
        if (segs[i].n == 0) continue;
        const unsigned char* src = static_cast<const unsigned char*>(segs[i].src);
        unsigned char* dst = static_cast<unsigned char*>(segs[i].dst);
        unsigned long long body = 0;
        if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0 && segs[i].n >= 4096) {
            // the bulk unit reads device memory only: a host-resident source takes the plain path
            cudaPointerAttributes attr;
            if (cudaPointerGetAttributes(&attr, src) == cudaSuccess && attr.type == cudaMemoryTypeDevice) {
                body = segs[i].n & ~15ull;
            } else {
                cudaGetLastError();
            }
        }
        if (body) {
            CopySeg s{src, dst, body, ntiles};
            ntiles += (body + kBulkTile - 1) / kBulkTile;
            bulk.push_back(s);
        }
        if (segs[i].n > body) ragged.push_back(CopySeg{src + body, dst + body, segs[i].n - body, 0});
    }
    static std::atomic<unsigned long long> attrSet{0};
    const unsigned long long bit = 1ull << (ctx->device & 63);
    if (!(attrSet.fetch_or(bit) & bit)) {
        B2_CUDA(cudaFuncSetAttribute(pushBulkKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBulkStages * kBulkTile));
    }
    CopySeg *bulkDev = nullptr, *raggedDev = nullptr;
    Context::XferParams* slot = nullptr;
    if (!bulk.empty() || !ragged.empty()) {
        const size_t bytes = sizeof(CopySeg) * (bulk.size() + ragged.size());
        slot = takeParamSlot(ctx, bytes);
        CopySeg* h = static_cast<CopySeg*>(slot->host);
        std::copy(bulk.begin(), bulk.end(), h);
        std::copy(ragged.begin(), ragged.end(), h + bulk.size());
        B2_CUDA(cudaMemcpyAsync(slot->dev, slot->host, bytes, cudaMemcpyHostToDevice, ctx->xferStream));
        bulkDev = static_cast<CopySeg*>(slot->dev);
        raggedDev = bulkDev + bulk.size();
    }
    const unsigned long long want = std::max<unsigned long long>(ntiles / 4, ragged.empty() ? 1 : std::min<size_t>(ragged.size(), 8));
    const int grid = static_cast<int>(std::max<unsigned long long>(1, std::min<unsigned long long>(want, static_cast<unsigned long long>(std::max(1, ctas)))));
    pushBulkKernel<<<grid, 128, kBulkStages * kBulkTile, ctx->xferStream>>>(bulkDev, static_cast<int>(bulk.size()), ntiles, raggedDev,
                                                                          static_cast<int>(ragged.size()), waitFlag, waitValue, doneFlag,
                                                                          doneValue, timeoutNs, counter, ctx->xferStatus);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
    if (slot) {
        B2_CUDA(cudaEventRecord(slot->done, ctx->xferStream));
        slot->pending = true;
    }
}

void pushSegments(Context* ctx, const b200c_copy_seg* segs, int count, const unsigned long long* waitFlag,
                  unsigned long long waitValue, unsigned long long* doneFlag, unsigned long long doneValue,
                  unsigned int timeoutMs, int mode, int ctas, cudaEvent_t after) {
    TraceRange range("exchange: copy segments");
    ensureExchange(ctx);
    if (after) {
        // the pushed bytes were complete when `after` was recorded; work queued on the context's stream since
        // then (the next chunk's kernels) does not hold the transfer back
        B2_CUDA(cudaStreamWaitEvent(ctx->xferStream, after, 0));
    } else {
        // the pushed bytes are whatever the context's stream has produced so far
        B2_CUDA(cudaEventRecord(ctx->xferEvent, ctx->stream));
        B2_CUDA(cudaStreamWaitEvent(ctx->xferStream, ctx->xferEvent, 0));
    }
    const unsigned long long timeoutNs = static_cast<unsigned long long>(timeoutMs) * 1000000ull;
    auto nextCounter = [&] { return ctx->xferCounters + (ctx->xferCounterNext++ % Context::kXferCounters); };
    if (mode == 2) {
        pushSegmentsBulk(ctx, segs, count, waitFlag, waitValue, doneFlag, doneValue, timeoutNs, ctas, nextCounter());
        return;
    }
    std::vector<CopySeg> host;
    std::vector<unsigned int> tileSeg;
    unsigned long long ntiles = 0;
    if (mode == 0) {
        for (int i = 0; i < count; ++i) {
            if (segs[i].n == 0) continue;
            CopySeg s;
            s.src = static_cast<const unsigned char*>(segs[i].src);
            s.dst = static_cast<unsigned char*>(segs[i].dst);
            s.n = segs[i].n;
            s.firstTile = ntiles;
            const unsigned long long t = (s.n + kPushTile - 1) / kPushTile;
            tileSeg.insert(tileSeg.end(), t, static_cast<unsigned int>(host.size()));
            host.push_back(s);
            ntiles += t;
        }
    } else {
        // copy engine: the release wait first (a one-CTA launch of the same kernel with nothing to copy),
        // then one copy per segment; the flag is raised by the launch below.  Unlike the kernel form, a
        // wait that ran out cannot hold the queued copies back.
        if (waitFlag) {
            pushSegmentsKernel<<<1, 256, 0, ctx->xferStream>>>(nullptr, nullptr, 0, waitFlag, waitValue, nullptr, 0, timeoutNs,
                                                              nextCounter(), ctx->xferStatus);
            B2_CUDA(cudaGetLastError());
            ++ctx->launches;
            waitFlag = nullptr;
        }
        for (int i = 0; i < count; ++i) {
            if (segs[i].n) B2_CUDA(cudaMemcpyAsync(segs[i].dst, segs[i].src, segs[i].n, cudaMemcpyDefault, ctx->xferStream));
        }
        if (!doneFlag) return;  // plain copies (a download): no flag to raise
    }
    CopySeg* segDev = nullptr;
    unsigned int* tileDev = nullptr;
    Context::XferParams* slot = nullptr;
    if (ntiles) {
        // The parameter arrays live in a ring of the exchange's own buffers: the context's arena is rewound
        // by the next call while this kernel may still be queued on the other stream.
        const size_t tileAt = (sizeof(CopySeg) * host.size() + 15) / 16 * 16;
        const size_t bytes = tileAt + sizeof(unsigned int) * ntiles;
        slot = takeParamSlot(ctx, bytes);
        char* h = static_cast<char*>(slot->host);
        std::memcpy(h, host.data(), sizeof(CopySeg) * host.size());
        std::memcpy(h + tileAt, tileSeg.data(), sizeof(unsigned int) * ntiles);
        B2_CUDA(cudaMemcpyAsync(slot->dev, slot->host, bytes, cudaMemcpyHostToDevice, ctx->xferStream));
        segDev = static_cast<CopySeg*>(slot->dev);
        tileDev = reinterpret_cast<unsigned int*>(static_cast<char*>(slot->dev) + tileAt);
    }
    const int grid = static_cast<int>(std::max<unsigned long long>(1, std::min<unsigned long long>(ntiles, static_cast<unsigned long long>(std::max(1, ctas)))));
    pushSegmentsKernel<<<grid, 256, 0, ctx->xferStream>>>(segDev, tileDev, ntiles, waitFlag, waitValue, doneFlag, doneValue, timeoutNs,
                                                         nextCounter(), ctx->xferStatus);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
    if (slot) {
        B2_CUDA(cudaEventRecord(slot->done, ctx->xferStream));
        slot->pending = true;
    }
}

void waitFlags(Context* ctx, const unsigned long long* flagsDev, int count, unsigned long long value, unsigned int timeoutMs,
               bool onTransferStream) {
    ensureExchange(ctx);
    if (count <= 0) return;
    waitFlagsKernel<<<1, 32, 0, onTransferStream ? ctx->xferStream : ctx->stream>>>(flagsDev, count, value, static_cast<unsigned long long>(timeoutMs) * 1000000ull,
                                               ctx->xferStatus);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
}

void signalFlags(Context* ctx, unsigned long long* const* targets, int count, unsigned long long value) {
    ensureExchange(ctx);
    if (count <= 0) return;
    if (count > 64) throw BadArg("b200c_signal_flags: at most 64 targets per call");
    unsigned long long** dev = static_cast<unsigned long long**>(ctx->arena.alloc(sizeof(void*) * count));
    uploadSmall(ctx, dev, targets, sizeof(void*) * count);
    signalFlagsKernel<<<1, 32, 0, ctx->stream>>>(dev, count, value);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
}

int exchangeStatus(Context* ctx) {
    if (!ctx->xferStream) return 0;
    B2_CUDA(cudaStreamSynchronize(ctx->xferStream));
    B2_CUDA(cudaStreamSynchronize(ctx->stream));
    int st = 0;
    B2_CUDA(cudaMemcpy(&st, ctx->xferStatus, sizeof(int), cudaMemcpyDeviceToHost));
    if (st) B2_CUDA(cudaMemset(ctx->xferStatus, 0, sizeof(int)));
    return st;
}

}  // namespace b200c
