// C ABI of the library (include/b200const.h): context management, memory helpers and the entry
// points that drive the planner and the codec.  No exception crosses this file's boundary.
#include "../../include/b200const.h"
#include "plan.h"

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdio>
#include <condition_variable>
#include <cstdlib>
#include <exception>
#include <functional>
#include <thread>
#include <cstring>
#include <memory>
#include <string>

namespace b200c {

static thread_local std::string t_lastError;

// ---------------------------------------------------------------------------- memory
void* devMalloc(Context* ctx, size_t bytes) {
    if (bytes == 0) bytes = 1;
    if (ctx && ctx->allocFn) {
        void* q = ctx->allocFn(ctx->allocUser, bytes);
        if (!q) throw NoMem("the installed allocator returned no memory for " + std::to_string(bytes) + " bytes");
        return q;
    }
    void* p = nullptr;
    const cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        throw NoMem(std::string("cudaMalloc of ") + std::to_string(bytes) + " bytes: " + cudaGetErrorString(e));
    }
    return p;
}

void devFree(Context* ctx, void* p) {
    if (!p) return;
    if (ctx && ctx->freeFn) {
        ctx->freeFn(ctx->allocUser, p);
        return;
    }
    cudaFree(p);
}

void copyH2D(Context* ctx, void* dst, const void* src, size_t n) {
    if (n == 0) return;
    ++ctx->directOps;
    B2_CUDA(cudaMemcpyAsync(dst, src, n, cudaMemcpyHostToDevice, ctx->stream));
}
void uploadSmall(Context* ctx, void* dst, const void* src, size_t n) {
    if (n == 0) return;
    const int set = ctx->stageSet;
    const size_t need = (n + 63) / 64 * 64;
    Context::StageChunk* c = nullptr;
    for (auto& k : ctx->stage[set]) {
        if (k.used + need <= k.size) {
            c = &k;
            break;
        }
    }
    if (!c) {
        Context::StageChunk nk;
        nk.size = std::max<size_t>(need, 4ull << 20);
        nk.used = 0;
        void* p = nullptr;
        const cudaError_t e = cudaHostAlloc(&p, nk.size, cudaHostAllocDefault);
        if (e != cudaSuccess) {
            cudaGetLastError();
            throw NoMem(std::string("cudaHostAlloc of staging memory failed: ") + cudaGetErrorString(e));
        }
        nk.ptr = static_cast<char*>(p);
        ctx->stage[set].push_back(nk);
        c = &ctx->stage[set].back();
    }
    char* at = c->ptr + c->used;
    c->used += need;
    std::memcpy(at, src, n);
    B2_CUDA(cudaMemcpyAsync(dst, at, n, cudaMemcpyHostToDevice, ctx->stream));
    if (!ctx->stageDone[set]) B2_CUDA(cudaEventCreateWithFlags(&ctx->stageDone[set], cudaEventDisableTiming));
    B2_CUDA(cudaEventRecord(ctx->stageDone[set], ctx->stream));
    ctx->stagePending[set] = true;
}

// Start of a call: switch to the other set of staging chunks; its last user was the call before the
// previous one.
void resetStage(Context* ctx) {
    const int set = ctx->stageSet ^ 1;
    if (ctx->stagePending[set]) {
        B2_CUDA(cudaEventSynchronize(ctx->stageDone[set]));
        ctx->stagePending[set] = false;
    }
    for (auto& k : ctx->stage[set]) k.used = 0;
    ctx->stageSet = set;
}

void releaseStage(Context* ctx) {
    for (int set = 0; set < 2; ++set) {
        if (ctx->stagePending[set]) cudaEventSynchronize(ctx->stageDone[set]);
        ctx->stagePending[set] = false;
        for (auto& k : ctx->stage[set]) cudaFreeHost(k.ptr);
        ctx->stage[set].clear();
        if (ctx->stageDone[set]) cudaEventDestroy(ctx->stageDone[set]);
        ctx->stageDone[set] = nullptr;
    }
}

void copyD2H(Context* ctx, void* dst, const void* src, size_t n) {
    if (n == 0) return;
    ++ctx->directOps;
    B2_CUDA(cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToHost, ctx->stream));
}
void copyD2D(Context* ctx, void* dst, const void* src, size_t n) {
    if (n == 0) return;
    ++ctx->directOps;
    B2_CUDA(cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToDevice, ctx->stream));
}
void fillBytes(Context* ctx, void* dst, int value, size_t n) {
    if (n == 0) return;
    ++ctx->directOps;
    B2_CUDA(cudaMemsetAsync(dst, value, n, ctx->stream));
}
void syncStream(Context* ctx) {
    B2_CUDA(cudaStreamSynchronize(ctx->stream));
}

static const char* errText(int code) {
    switch (code) {
    case E_CAST_RANGE:
        return "Can not safely cast a value: it is outside the range of the target element type";
    case E_CAST_INEXACT:
        return "Can not safely cast a value: the conversion to the floating point type is not exact";
    case E_OOB:
        return "Out-of-bound access";
    case E_SPARSE_OVERFLOW:
        return "Sparsify: more non-sparse elements than numActualElements allows";
    case E_CODEC:
        return "codec: malformed stream or output capacity exceeded";
    default:
        return "unknown device-side error";
    }
}

void checkDeviceError(Context* ctx) {
    int code = E_NONE;
    B2_CUDA(cudaMemcpyAsync(ctx->errHost, ctx->errWord, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    B2_CUDA(cudaStreamSynchronize(ctx->stream));
    code = *ctx->errHost;
    if (code != E_NONE) {
        B2_CUDA(cudaMemsetAsync(ctx->errWord, 0, sizeof(int), ctx->stream));
    }
    if (code != E_NONE) throw RefThrow(errText(code));
}

// ---------------------------------------------------------------------------- arena
Arena::~Arena() {
    releaseAll();
}

void Arena::releaseAll() {
    for (auto& b : _blocks) devFree(_ctx, b.ptr);
    _blocks.clear();
}

void* Arena::alloc(size_t bytes, size_t align) {
    if (bytes == 0) bytes = 1;
    for (auto& b : _blocks) {
        const size_t at = (b.used + align - 1) / align * align;
        if (at + bytes <= b.size) {
            b.used = at + bytes;
            return b.ptr + at;
        }
    }
    const size_t minBlock = _minBlock;
    const size_t size = std::max(minBlock, (bytes + align + 4095) / 4096 * 4096);
    Block nb;
    nb.ptr = static_cast<char*>(devMalloc(_ctx, size));
    nb.size = size;
    nb.used = bytes;
    _blocks.push_back(nb);
    return nb.ptr;
}

void Arena::reset() {
    // keep the largest block only when fragmentation grew: several blocks are merged into one
    if (_blocks.size() > 4) {
        size_t total = 0;
        for (auto& b : _blocks) total += b.size;
        for (auto& b : _blocks) devFree(_ctx, b.ptr);
        _blocks.clear();
        Block nb;
        nb.ptr = static_cast<char*>(devMalloc(_ctx, total));
        nb.size = total;
        nb.used = 0;
        _blocks.push_back(nb);
    }
    for (auto& b : _blocks) b.used = 0;
}

size_t Arena::reserved() const {
    size_t t = 0;
    for (auto& b : _blocks) t += b.size;
    return t;
}

// ---------------------------------------------------------------------------- error mapping
template <class F>
static int guarded(F&& body) {
    try {
        body();
        return B200C_OK;
    } catch (const RefThrow& e) {
        t_lastError = e.what();
        return B200C_ERR_THROW;
    } catch (const NotBuilt& e) {
        t_lastError = e.what();
        return B200C_ERR_UNSUPPORTED;
    } catch (const BadArg& e) {
        t_lastError = e.what();
        return B200C_ERR_INVALID;
    } catch (const CudaFail& e) {
        t_lastError = e.what();
        return B200C_ERR_CUDA;
    } catch (const NoMem& e) {
        t_lastError = e.what();
        return B200C_ERR_NOMEM;
    } catch (const Capacity& e) {
        t_lastError = e.what();
        return B200C_ERR_CAPACITY;
    } catch (const std::bad_alloc&) {
        t_lastError = "host allocation failed";
        return B200C_ERR_NOMEM;
    } catch (const std::exception& e) {
        t_lastError = e.what();
        return B200C_ERR_INVALID;
    }
}

static std::vector<Transformation> chainFromC(const b200c_xform* chain, int n) {
    if (n < 0 || (n > 0 && chain == nullptr)) throw BadArg("bad transformation list");
    std::vector<Transformation> xs;
    xs.reserve(n);
    for (int i = 0; i < n; ++i) xs.push_back(xformFromC(chain[i]));
    return xs;
}

// After an asynchronous failure the arena and the error word must be left clean for the next call.
// ---------------------------------------------------------------------------- planning threads
// The reference folds constants in a parallel loop (export.cpp:465); here the host part of a fold --
// type inference, view composition, launch parameters -- is what runs in parallel, while every
// launch still goes to the context's one stream.
class PlanPool {
public:
    explicit PlanPool(int n) {
        for (int i = 0; i < n; ++i) _threads.emplace_back([this, i] { loop(i); });
    }
    ~PlanPool() {
        {
            std::lock_guard<std::mutex> lk(_m);
            _stop = true;
            ++_gen;
        }
        _cv.notify_all();
        for (auto& t : _threads) t.join();
    }
    int size() const {
        return static_cast<int>(_threads.size());
    }
    // runs fn(worker index) once on every thread and waits for all of them
    void run(const std::function<void(int)>& fn) {
        std::unique_lock<std::mutex> lk(_m);
        _job = &fn;
        _pending = size();
        ++_gen;
        _cv.notify_all();
        _done.wait(lk, [&] { return _pending == 0; });
        _job = nullptr;
    }

private:
    void loop(int id) {
        unsigned long long seen = 0;
        for (;;) {
            std::unique_lock<std::mutex> lk(_m);
            _cv.wait(lk, [&] { return _gen != seen; });
            seen = _gen;
            if (_stop) return;
            const std::function<void(int)>* fn = _job;
            lk.unlock();
            (*fn)(id);
            lk.lock();
            if (--_pending == 0) _done.notify_one();
        }
    }
    std::vector<std::thread> _threads;
    std::mutex _m;
    std::condition_variable _cv, _done;
    const std::function<void(int)>* _job = nullptr;
    unsigned long long _gen = 0;
    int _pending = 0;
    bool _stop = false;
};

static int planThreads() {
    if (const char* e = std::getenv("B200C_PLAN_THREADS")) return std::max(0, std::min(64, std::atoi(e)));
    const unsigned hw = std::thread::hardware_concurrency();
    return static_cast<int>(std::max(1u, std::min(8u, hw / 2)));
}

static void ensurePool(Context* ctx) {
    if (ctx->pool) return;
    const int n = planThreads();
    if (n < 2) return;
    for (int i = 0; i < n; ++i) {
        Context* w = new Context();
        w->device = ctx->device;
        w->allocFn = ctx->allocFn;
        w->freeFn = ctx->freeFn;
        w->allocUser = ctx->allocUser;
        w->errWord = ctx->errWord;
        w->errHost = ctx->errHost;
        w->smCount = ctx->smCount;
        w->l2Bytes = ctx->l2Bytes;
        w->arena.setMinBlock(4ull << 20);
        ctx->workers.push_back(w);
    }
    ctx->pool = new PlanPool(n);
}

static void destroyPool(Context* ctx) {
    delete ctx->pool;
    ctx->pool = nullptr;
    for (Context* w : ctx->workers) {
        w->arena.releaseAll();
        releaseStage(w);
        delete w;
    }
    ctx->workers.clear();
}

struct CallScope {
    Context* ctx;
    std::unique_lock<std::mutex> lock;
    explicit CallScope(Context* c): ctx(c), lock(c->mu) {
        const cudaError_t e = cudaSetDevice(ctx->device);
        if (e != cudaSuccess) throw CudaFail(std::string("cudaSetDevice: ") + cudaGetErrorString(e));
        ctx->arena.reset();
        ctx->tileSlabs.clear();  // their device memory was the arena's
        resetStage(ctx);
    }
};

}  // namespace b200c

using namespace b200c;

extern "C" {

const char* b200c_last_error(void) {
    return t_lastError.c_str();
}

const char* b200c_version(void) {
    return "b200const 0.1 (sm_100a)";
}

int b200c_create(int device, b200c_ctx** out) {
    return guarded([&] {
        if (!out) throw BadArg("null output pointer");
        auto ctx = std::make_unique<Context>();
        ctx->device = device;
        int count = 0;
        cudaError_t e = cudaGetDeviceCount(&count);
        if (e != cudaSuccess || count == 0) {
            cudaGetLastError();
            throw CudaFail(std::string("no usable CUDA device: ") + (e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0"));
        }
        if (device < 0 || device >= count) throw BadArg("device index out of range");
        B2_CUDA(cudaSetDevice(device));
        cudaDeviceProp prop;
        B2_CUDA(cudaGetDeviceProperties(&prop, device));
        ctx->smCount = prop.multiProcessorCount;
        ctx->l2Bytes = static_cast<size_t>(prop.l2CacheSize);
        B2_CUDA(cudaStreamCreateWithFlags(&ctx->ownStream, cudaStreamNonBlocking));
        ctx->stream = ctx->ownStream;
        B2_CUDA(cudaMalloc(&ctx->errWord, sizeof(int)));
        B2_CUDA(cudaMemset(ctx->errWord, 0, sizeof(int)));
        B2_CUDA(cudaMallocHost(&ctx->errHost, sizeof(int)));
        *ctx->errHost = 0;
        *out = reinterpret_cast<b200c_ctx*>(ctx.release());
    });
}

void b200c_destroy(b200c_ctx* h) {
    if (!h) return;
    Context* ctx = reinterpret_cast<Context*>(h);
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->errWord) cudaFree(ctx->errWord);
    if (ctx->errHost) cudaFreeHost(ctx->errHost);
    destroyPool(ctx);
    releaseExchange(ctx);
    releaseStage(ctx);
    for (CodecPending& t : ctx->codecTickets) {
        if (t.jobsHost) cudaFreeHost(t.jobsHost);
        if (t.done) cudaEventDestroy(t.done);
    }
    ctx->arena.releaseAll();  // frees the blocks while the device is still current
    if (ctx->ownStream) cudaStreamDestroy(ctx->ownStream);
    delete ctx;
}

int b200c_set_allocator(b200c_ctx* h, b200c_alloc_fn alloc_fn, b200c_free_fn free_fn, void* user) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        if ((alloc_fn == nullptr) != (free_fn == nullptr)) throw BadArg("give both functions, or neither");
        Context* ctx = reinterpret_cast<Context*>(h);
        std::lock_guard<std::mutex> lock(ctx->mu);
        B2_CUDA(cudaSetDevice(ctx->device));
        B2_CUDA(cudaStreamSynchronize(ctx->stream));
        // everything the old allocator handed out goes back to it first
        destroyPool(ctx);
        ctx->arena.releaseAll();
        ctx->allocFn = alloc_fn;
        ctx->freeFn = free_fn;
        ctx->allocUser = user;
    });
}

int b200c_set_stream(b200c_ctx* h, void* stream) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        Context* ctx = reinterpret_cast<Context*>(h);
        std::lock_guard<std::mutex> lock(ctx->mu);
        ctx->stream = stream ? static_cast<cudaStream_t>(stream) : ctx->ownStream;
    });
}

void* b200c_get_stream(b200c_ctx* h) {
    return h ? static_cast<void*>(reinterpret_cast<Context*>(h)->stream) : nullptr;
}

int b200c_synchronize(b200c_ctx* h) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        Context* ctx = reinterpret_cast<Context*>(h);
        std::lock_guard<std::mutex> lock(ctx->mu);
        B2_CUDA(cudaSetDevice(ctx->device));
        if (ctx->xferStream) B2_CUDA(cudaStreamSynchronize(ctx->xferStream));
        syncStream(ctx);
        checkDeviceError(ctx);
    });
}

int64_t b200c_launch_count(b200c_ctx* h) {
    return h ? reinterpret_cast<Context*>(h)->launches : 0;
}

int b200c_infer_type(const b200c_type* in, const b200c_xform* chain, int n, b200c_type* out) {
    return guarded([&] {
        if (!in || !out) throw BadArg("null type pointer");
        const TensorType t = inferChain(typeFromC(*in), chainFromC(chain, n));
        typeToC(t, out);
    });
}

int b200c_insert_position(const int32_t* kinds, int n, int32_t new_kind, int* pos) {
    return guarded([&] {
        if (n < 0 || (n > 0 && !kinds) || !pos) throw BadArg("bad arguments");
        *pos = insertPosition(std::vector<int>(kinds, kinds + n), new_kind);
    });
}

int64_t b200c_total_alloc_size(const b200c_type* t) {
    int64_t r = -1;
    guarded([&] {
        if (!t) throw BadArg("null type pointer");
        r = typeFromC(*t).allocBytes();
    });
    return r;
}

// Stage the base content on the device (or use it in place) and build the planner.
static std::unique_ptr<Planner> makePlanner(Context* ctx, const b200c_type* base, const void* data, size_t nbytes,
                                            int is_splat, int data_on_device) {
    if (!base) throw BadArg("null base type");
    const TensorType bt = typeFromC(*base);
    if (bt.quantized()) throw BadArg("the base content cannot have a quantised element type");
    if (nbytes > 0 && !data) throw BadArg("null data pointer");
    const void* dev = data;
    if (!data_on_device) {
        void* d = ctx->arena.alloc(nbytes ? nbytes : 1);
        copyH2D(ctx, d, data, nbytes);
        dev = d;
    }
    return std::make_unique<Planner>(ctx, bt, dev, nbytes, is_splat != 0);
}

int b200c_fold(b200c_ctx* h, const b200c_type* base, const void* data, size_t nbytes, int is_splat, int data_on_device,
               const b200c_xform* chain, int n, void* out, size_t out_cap, int out_on_device, size_t* out_bytes,
               b200c_type* out_type, int flags) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        Context* ctx = reinterpret_cast<Context*>(h);
        CallScope scope(ctx);
        TraceRange range("b200c_fold");
        if (!out && out_cap > 0) throw BadArg("null output pointer");
        const auto xs = chainFromC(chain, n);
        auto plan = makePlanner(ctx, base, data, nbytes, is_splat, data_on_device);
        plan->setSideOnDevice(out_on_device != 0);
        void* devOut = out;
        if (!out_on_device) devOut = ctx->arena.alloc(out_cap ? out_cap : 1);
        const size_t wrote = plan->run(xs, devOut, out_cap);
        if (!out_on_device) copyD2H(ctx, out, devOut, wrote);
        for (const auto& so : plan->sideOutputs()) {
            if (out_on_device) {
                copyD2D(ctx, so.user, so.dev, so.bytes);
            } else {
                copyD2H(ctx, so.user, so.dev, so.bytes);
            }
        }
        if (out_bytes) *out_bytes = wrote;
        if (out_type) typeToC(plan->state().type, out_type);
        const bool async = out_on_device && (flags & B200C_FOLD_ASYNC);
        if (!async) {
            syncStream(ctx);
            checkDeviceError(ctx);
        }
    });
}

// Key of a constant's plan: every byte of its descriptors the planner can see -- base type, size, the
// transformations with their types, quantisation tables and auxiliary arrays -- plus the low address
// bits of its buffers (the kernels pick vector widths by alignment).  Returns false for descriptors too
// large to be worth comparing.
static bool planKeyOf(const b200c_fold_item& it, std::string& key) {
    constexpr int64_t kMaxTable = 2048;
    key.clear();
    auto add = [&](const void* p, size_t n) { key.append(static_cast<const char*>(p), n); };
    auto addType = [&](const b200c_type& t) {
        add(&t, offsetof(b200c_type, scales));
        if (t.qkind == B200C_Q_NONE) return true;
        if (t.nq < 1 || t.nq > kMaxTable || !t.scales || !t.zps) return false;
        add(t.scales, sizeof(double) * static_cast<size_t>(t.nq));
        add(t.zps, sizeof(int64_t) * static_cast<size_t>(t.nq));
        return true;
    };
    if (!it.base || it.n < 0 || (it.n > 0 && !it.chain)) return false;
    if (!addType(*it.base)) return false;
    const uint64_t head[4] = {static_cast<uint64_t>(it.nbytes), static_cast<uint64_t>(it.out_cap),
                              (static_cast<uint64_t>(it.is_splat != 0) << 32) | static_cast<uint32_t>(it.n),
                              ((reinterpret_cast<uintptr_t>(it.data) & 255u) << 16) | (reinterpret_cast<uintptr_t>(it.out) & 511u)};
    add(head, sizeof(head));
    for (int k = 0; k < it.n; ++k) {
        const b200c_xform& x = it.chain[k];
        add(&x, offsetof(b200c_xform, type));
        if (!addType(x.type)) return false;
        const int64_t naux = x.aux ? x.naux : -1;
        if (naux > kMaxTable) return false;
        add(&naux, sizeof(naux));
        if (naux > 0) add(x.aux, sizeof(int64_t) * static_cast<size_t>(naux));
        const unsigned char sides = static_cast<unsigned char>((x.side0 != nullptr) | ((x.side1 != nullptr) << 1));
        add(&sides, 1);
    }
    return true;
}

int b200c_fold_batch(b200c_ctx* h, b200c_fold_item* items, int count, int data_on_device, int out_on_device, int flags) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        if (count < 0 || (count > 0 && !items)) throw BadArg("bad item list");
        Context* ctx = reinterpret_cast<Context*>(h);
        CallScope scope(ctx);
        TraceRange range("b200c_fold_batch");
        struct BatchGuard {
            Context* c;
            ~BatchGuard() {
                for (Context* q : c->workers) clear(q);
                clear(c);
            }
            static void clear(Context* q) {
                q->batching = false;
                q->rqBatch.clear();
                q->tileBatch.clear();
                q->mapBatch.clear();
                q->sparseBatch.clear();
                q->queuedBytes = 0;
                q->planMemo.clear();
            }
        } guard{ctx};
        BatchGuard::clear(ctx);
        for (Context* q : ctx->workers) q->planMemo.clear();
        ctx->batching = out_on_device != 0;
        ctx->queuedBytes = 0;
        typedef std::vector<std::pair<int, const long long*>> Deferred;  // items whose size is read back at the end
        Deferred deferred;

        // one item: plan it, launch or queue its kernels on `c`, note a size that is still on the device
        auto foldItem = [&](Context* c, int i, Deferred& later) {
            b200c_fold_item& it = items[i];
            if (!it.out && it.out_cap > 0) throw BadArg("null output pointer");
            // the quantiser's per-row tables, when the caller keeps them on the device
            void *side0 = nullptr, *side1 = nullptr;
            int nsynth = 0;
            for (int k = 0; k < it.n && it.chain; ++k) {
                if (it.chain[k].kind == B200C_X_QUANTIZE_SYNTH) {
                    side0 = it.chain[k].side0;
                    side1 = it.chain[k].side1;
                    ++nsynth;
                }
            }
            const bool memoOk = c->batching && data_on_device && out_on_device && it.data && it.out && nsynth <= 1 &&
                                (nsynth == 0 || (side0 && side1)) && planKeyOf(it, c->planKey);
            if (memoOk) {
                const auto hit = c->planMemo.find(c->planKey);
                if (hit != c->planMemo.end()) {
                    const PlanMemo& m = hit->second;
                    if (m.queue == 0) {
                        c->rqBatch.push_back(m.rq);
                        RowQuantParams& p = c->rqBatch.back();
                        p.src = it.data;
                        p.dst = it.out;
                        p.scales = static_cast<float*>(side0);
                        p.zps = static_cast<int*>(side1);
                    } else if (m.queue == 1) {
                        c->tileBatch.push_back(m.tile);  // the same template, this constant's buffers
                        c->tileBatch.back().src = it.data;
                        c->tileBatch.back().dst = it.out;
                    } else if (m.queue == 2) {
                        c->mapBatch.push_back(m.map);
                        c->mapBatch.back().src = static_cast<const unsigned char*>(it.data);
                        c->mapBatch.back().dst = static_cast<unsigned char*>(it.out);
                    } else {
                        // the per-channel counts, offsets and the size word are scratch of the constant itself
                        c->sparseBatch.push_back(m.sparse);
                        SparseItem& sp = c->sparseBatch.back();
                        sp.src = static_cast<const unsigned char*>(it.data);
                        sp.dst = static_cast<unsigned char*>(it.out);
                        sp.counts = static_cast<long long*>(c->arena.alloc(static_cast<size_t>(sp.oc) * sizeof(long long)));
                        sp.offsets = static_cast<long long*>(c->arena.alloc(static_cast<size_t>(sp.oc + 1) * sizeof(long long)));
                        sp.bytesOut = static_cast<long long*>(c->arena.alloc(sizeof(long long)));
                        if (sp.fixedBytes < 0) later.push_back({i, sp.bytesOut});
                    }
                    c->queuedBytes += m.queuedBytes;
                    it.out_bytes = m.outBytes;
                    return;
                }
            }
            const size_t rq0 = c->rqBatch.size(), tile0 = c->tileBatch.size(), map0 = c->mapBatch.size(),
                         sparse0 = c->sparseBatch.size();
            const int64_t launches0 = c->launches;
            const long long direct0 = c->directOps, queued0 = c->queuedBytes;
            const auto xs = chainFromC(it.chain, it.n);
            auto plan = makePlanner(c, it.base, it.data, it.nbytes, it.is_splat, data_on_device);
            plan->setSideOnDevice(out_on_device != 0);
            void* devOut = it.out;
            if (!out_on_device) devOut = c->arena.alloc(it.out_cap ? it.out_cap : 1);
            it.out_bytes = plan->run(xs, devOut, it.out_cap);
            if (!out_on_device) copyD2H(c, it.out, devOut, it.out_bytes);
            for (const auto& so : plan->sideOutputs()) {
                if (out_on_device) {
                    copyD2D(c, so.user, so.dev, so.bytes);
                } else {
                    copyD2H(c, so.user, so.dev, so.bytes);
                }
            }
            if (plan->deferredBytes()) later.push_back({i, plan->deferredBytes()});
            // Remember the plan when it came to exactly one queued item that reads the constant's own data and
            // writes its own output, and nothing was launched, copied or kept aside for it.
            if (memoOk && c->launches == launches0 && c->directOps == direct0 && plan->sideOutputs().empty() &&
                c->planMemo.size() < 4096) {
                const size_t dr = c->rqBatch.size() - rq0, dt = c->tileBatch.size() - tile0, dm = c->mapBatch.size() - map0,
                             ds = c->sparseBatch.size() - sparse0;
                if (dr + dt + dm + ds == 1 && (ds == 1 || !plan->deferredBytes())) {
                    PlanMemo m;
                    std::memset(static_cast<void*>(&m), 0, sizeof(m));
                    m.outBytes = it.out_bytes;
                    m.queuedBytes = c->queuedBytes - queued0;
                    bool keep = false;
                    if (dr) {
                        m.queue = 0;
                        m.rq = c->rqBatch.back();
                        keep = m.rq.src == it.data && m.rq.dst == it.out && nsynth == 1 && m.rq.scales == side0 && m.rq.zps == side1;
                    } else if (dt) {
                        m.queue = 1;
                        m.tile = c->tileBatch.back();
                        keep = m.tile.src == it.data && m.tile.dst == it.out && nsynth == 0;
                    } else if (dm) {
                        m.queue = 2;
                        m.map = c->mapBatch.back();
                        keep = m.map.src == it.data && m.map.dst == it.out && nsynth == 0;
                    } else {
                        m.queue = 3;
                        m.sparse = c->sparseBatch.back();
                        keep = m.sparse.src == it.data && m.sparse.dst == it.out && nsynth == 0 &&
                               ((m.sparse.fixedBytes < 0) == (plan->deferredBytes() != nullptr)) &&
                               (!plan->deferredBytes() || plan->deferredBytes() == m.sparse.bytesOut);
                    }
                    if (keep) c->planMemo.emplace(c->planKey, m);
                }
            }
        };
        auto flushAll = [&] {
            flushRowQuantBatch(ctx);
            flushTileBatch(ctx);
            flushSparsityBatch(ctx);
            ctx->queuedBytes = 0;
        };

        // Items are taken in waves of growing input size (256 MB, then twice as much each time): the
        // queued launches of a wave go out when it has been planned, so the device starts early and
        // works while the host plans the rest.  A wave with enough items is planned by the pool.
        const bool parallelOk = ctx->batching && data_on_device;
        if (parallelOk) ensurePool(ctx);
        long long waveBytes = 256LL << 20;
        int first = 0;
        bool workersReset = false;
        // B200C_TRACE=1: host time of planning, flushing and the final wait, on stderr
        static const bool trace = std::getenv("B200C_TRACE") != nullptr;
        double tPlan = 0, tFlush = 0, tSync = 0;
        int waves = 0, parallelWaves = 0;
        auto now = [] { return std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now().time_since_epoch()).count(); };
        while (first < count) {
            const double t0 = now();
            TraceRange waveRange("fold_batch: plan and flush one wave");
            ++waves;
            int last = first;
            long long bytes = 0;
            while (last < count && (last == first || bytes < waveBytes)) bytes += static_cast<long long>(items[last++].nbytes);
            const int n = last - first;
            if (parallelOk && ctx->pool && n >= 4 * ctx->pool->size()) {
                ++parallelWaves;
                const int nw = ctx->pool->size();
                std::atomic<int> next(first);
                std::vector<std::exception_ptr> failure(nw);
                std::vector<int> failedAt(nw, count);
                std::vector<Deferred> later(nw);
                for (Context* w : ctx->workers) {
                    w->stream = ctx->stream;
                    w->batching = true;
                    w->launches = 0;
                    if (!workersReset) {  // first parallel wave of this call
                        w->arena.reset();
                        w->tileSlabs.clear();
                        resetStage(w);
                    }
                }
                workersReset = true;
                ctx->pool->run([&](int id) {
                    Context* w = ctx->workers[id];
                    if (cudaSetDevice(w->device) != cudaSuccess) {
                        failure[id] = std::make_exception_ptr(CudaFail("cudaSetDevice failed on a planning thread"));
                        failedAt[id] = first;
                        return;
                    }
                    // runs of 16 consecutive items per grab: neighbours share cache lines of the item array
                    for (bool stop = false; !stop;) {
                        const int i0 = next.fetch_add(16);
                        if (i0 >= last) break;
                        for (int i = i0; i < std::min(i0 + 16, last); ++i) {
                            try {
                                foldItem(w, i, later[id]);
                            } catch (...) {
                                failure[id] = std::current_exception();
                                failedAt[id] = i;
                                stop = true;
                                break;
                            }
                        }
                    }
                });
                int bad = -1;
                for (int k = 0; k < nw; ++k)
                    if (failure[k] && (bad < 0 || failedAt[k] < failedAt[bad])) bad = k;
                if (bad >= 0) std::rethrow_exception(failure[bad]);  // the error of the earliest failing item
                for (int k = 0; k < nw; ++k) {
                    Context* w = ctx->workers[k];
                    ctx->rqBatch.insert(ctx->rqBatch.end(), w->rqBatch.begin(), w->rqBatch.end());
                    uploadTileTemplates(ctx, w);
                    ctx->tileBatch.insert(ctx->tileBatch.end(), w->tileBatch.begin(), w->tileBatch.end());
                    ctx->mapBatch.insert(ctx->mapBatch.end(), w->mapBatch.begin(), w->mapBatch.end());
                    ctx->sparseBatch.insert(ctx->sparseBatch.end(), w->sparseBatch.begin(), w->sparseBatch.end());
                    w->rqBatch.clear();
                    w->tileBatch.clear();
                    w->mapBatch.clear();
                    w->sparseBatch.clear();
                    ctx->launches += w->launches;
                    w->launches = 0;
                    deferred.insert(deferred.end(), later[k].begin(), later[k].end());
                }
            } else {
                for (int i = first; i < last; ++i) foldItem(ctx, i, deferred);
            }
            const double t1 = now();
            flushAll();
            tPlan += t1 - t0;
            tFlush += now() - t1;
            waveBytes = std::min(waveBytes * 2, 4LL << 30);
            first = last;
        }
        const double tEnd = now();
        const bool async = out_on_device && (flags & B200C_FOLD_ASYNC) && deferred.empty();
        if (!async) {
            // results whose size only the data decides: one read-back for all of them
            std::vector<long long> sizes(deferred.size(), 0);
            std::vector<const long long*> words;
            for (const auto& d : deferred) words.push_back(d.second);
            gatherDeviceWords(ctx, words, sizes.data());
            syncStream(ctx);
            checkDeviceError(ctx);
            for (size_t k = 0; k < deferred.size(); ++k) {
                b200c_fold_item& it = items[deferred[k].first];
                if (static_cast<size_t>(sizes[k]) > it.out_cap) throw Capacity("output buffer too small");
                it.out_bytes = static_cast<size_t>(sizes[k]);
            }
        }
        tSync = now() - tEnd;
        if (trace) {
            std::fprintf(stderr, "[b200c] fold_batch: %d items, %d waves (%d parallel), plan %.0f us, flush %.0f us, wait %.0f us\n", count,
                         waves, parallelWaves, tPlan, tFlush, tSync);
        }
    });
}

int b200c_count_nonsparse_per_oc(b200c_ctx* h, const b200c_type* base, const void* data, size_t nbytes, int is_splat,
                                 int data_on_device, const b200c_xform* chain, int n, int64_t* counts,
                                 int64_t ncounts) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        Context* ctx = reinterpret_cast<Context*>(h);
        CallScope scope(ctx);
        const auto xs = chainFromC(chain, n);
        auto plan = makePlanner(ctx, base, data, nbytes, is_splat, data_on_device);
        plan->runNoCopy(xs);
        const auto v = plan->countNonSparse();
        if (static_cast<int64_t>(v.size()) > ncounts || (!counts && !v.empty())) throw Capacity("counts array too small");
        std::copy(v.begin(), v.end(), counts);
    });
}

// ---------------------------------------------------------------------------- codec
int b200c_btc_bound(size_t n, size_t* bound) {
    if (!bound) return B200C_ERR_INVALID;
    *bound = codecBound(n);
    return B200C_OK;
}

int b200c_btc_compress(b200c_ctx* h, const void* in, size_t n, int in_on_device, void* out, size_t cap,
                       int out_on_device, size_t* out_n) {
    bool notSmaller = false;
    const int rc = guarded([&] {
        if (!h) throw BadArg("null context");
        Context* ctx = reinterpret_cast<Context*>(h);
        CallScope scope(ctx);
        if (n == 0) refThrow("BitCompactorCodec::compress: Empty input data vector");
        if (!in || !out || !out_n) throw BadArg("null pointer");
        if (cap < codecBound(n)) throw Capacity("output capacity below b200c_btc_bound(n)");
        const unsigned char* devIn = static_cast<const unsigned char*>(in);
        if (!in_on_device) {
            void* d = ctx->arena.alloc(n);
            copyH2D(ctx, d, in, n);
            devIn = static_cast<const unsigned char*>(d);
        }
        unsigned char* devOut = static_cast<unsigned char*>(out);
        if (!out_on_device) devOut = static_cast<unsigned char*>(ctx->arena.alloc(cap));
        CodecBuf buf{devIn, n};
        CodecResult res{};
        codecCompressBatch(ctx, 1, &buf, devOut, cap, /*rawFallback=*/0, &res);
        if (!out_on_device) {
            copyD2H(ctx, out, devOut + res.offset, res.size);
            syncStream(ctx);
        }
        *out_n = res.size;
        notSmaller = res.notSmaller;
    });
    return rc != B200C_OK ? rc : (notSmaller ? B200C_NOT_SMALLER : B200C_OK);
}

int b200c_btc_compress_noalloc(int device, const void* in_dev, size_t n, void* out_dev, size_t cap, void* stream,
                               size_t* out_n) {
    bool notSmaller = false;
    const int rc = guarded([&] {
        if (!in_dev || !out_dev || !out_n) throw BadArg("null pointer");
        codecCompressNoAlloc(device, static_cast<const unsigned char*>(in_dev), n, static_cast<unsigned char*>(out_dev), cap,
                             static_cast<cudaStream_t>(stream), out_n, &notSmaller);
    });
    return rc != B200C_OK ? rc : (notSmaller ? B200C_NOT_SMALLER : B200C_OK);
}

int b200c_btc_decompress(b200c_ctx* h, const void* in, size_t n, int in_on_device, void* out, size_t cap,
                         int out_on_device, size_t* out_n) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        Context* ctx = reinterpret_cast<Context*>(h);
        CallScope scope(ctx);
        if (!in || !out_n || (!out && cap)) throw BadArg("null pointer");
        const unsigned char* devIn = static_cast<const unsigned char*>(in);
        if (!in_on_device) {
            void* d = ctx->arena.alloc(n ? n : 1);
            copyH2D(ctx, d, in, n);
            devIn = static_cast<const unsigned char*>(d);
        }
        unsigned char* devOut = static_cast<unsigned char*>(out);
        if (!out_on_device) devOut = static_cast<unsigned char*>(ctx->arena.alloc(cap ? cap : 1));
        const size_t total = codecDecompress(ctx, devIn, n, devOut, cap);
        if (!out_on_device) {
            copyD2H(ctx, out, devOut, total);
            syncStream(ctx);
        }
        *out_n = total;
    });
}

int b200c_btc_compress_batch(b200c_ctx* h, int count, const void* const* in_dev, const size_t* sizes, void* out_dev,
                             size_t out_cap, size_t* out_offsets, size_t* out_sizes, int32_t* not_smaller) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        Context* ctx = reinterpret_cast<Context*>(h);
        CallScope scope(ctx);
        if (count < 0 || (count > 0 && (!in_dev || !sizes || !out_dev || !out_offsets || !out_sizes))) {
            throw BadArg("bad batch arguments");
        }
        std::vector<CodecBuf> bufs(count);
        for (int i = 0; i < count; ++i) bufs[i] = CodecBuf{static_cast<const unsigned char*>(in_dev[i]), sizes[i]};
        std::vector<CodecResult> res(count);
        codecCompressBatch(ctx, count, bufs.data(), static_cast<unsigned char*>(out_dev), out_cap, /*rawFallback=*/1,
                           res.data());
        for (int i = 0; i < count; ++i) {
            out_offsets[i] = res[i].offset;
            out_sizes[i] = res[i].size;
            if (not_smaller) not_smaller[i] = res[i].notSmaller ? 1 : 0;
        }
    });
}

int b200c_btc_compress_inplace_batch(b200c_ctx* h, int count, void* const* bufs_dev, const size_t* sizes, size_t* out_sizes,
                                     int32_t* compressed) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        Context* ctx = reinterpret_cast<Context*>(h);
        CallScope scope(ctx);
        if (count < 0 || (count > 0 && (!bufs_dev || !sizes || !out_sizes))) throw BadArg("bad batch arguments");
        std::vector<CodecBuf> bufs(count);
        for (int i = 0; i < count; ++i) bufs[i] = CodecBuf{static_cast<const unsigned char*>(bufs_dev[i]), sizes[i]};
        std::vector<CodecResult> res(count);
        codecCompressBatch(ctx, count, bufs.data(), nullptr, 0, /*rawFallback=*/2, res.data());
        for (int i = 0; i < count; ++i) {
            out_sizes[i] = res[i].size;
            if (compressed) compressed[i] = res[i].notSmaller ? 0 : 1;
        }
    });
}

int b200c_btc_compress_inplace_begin(b200c_ctx* h, int count, void* const* bufs_dev, const size_t* sizes, int* ticket) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        if (!ticket) throw BadArg("null ticket pointer");
        if (count <= 0 || !bufs_dev || !sizes) throw BadArg("bad batch arguments");
        Context* ctx = reinterpret_cast<Context*>(h);
        CallScope scope(ctx);
        int slot = -1;
        for (int k = 0; k < Context::kCodecTickets && slot < 0; ++k)
            if (!ctx->codecTickets[k].open) slot = k;
        if (slot < 0) throw BadArg("too many compressions are pending: collect one with b200c_btc_compress_inplace_end first");
        std::vector<CodecBuf> bufs(count);
        for (int i = 0; i < count; ++i) bufs[i] = CodecBuf{static_cast<const unsigned char*>(bufs_dev[i]), sizes[i]};
        codecCompressBatch(ctx, count, bufs.data(), nullptr, 0, /*rawFallback=*/2, nullptr, &ctx->codecTickets[slot]);
        *ticket = slot;
    });
}

int b200c_btc_compress_inplace_end(b200c_ctx* h, int ticket, size_t* out_sizes, int32_t* compressed) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        Context* ctx = reinterpret_cast<Context*>(h);
        if (ticket < 0 || ticket >= Context::kCodecTickets || !ctx->codecTickets[ticket].open) throw BadArg("not a pending compression");
        if (!out_sizes) throw BadArg("null result pointer");
        std::unique_lock<std::mutex> lock(ctx->mu);
        B2_CUDA(cudaSetDevice(ctx->device));
        CodecPending& pend = ctx->codecTickets[ticket];
        std::vector<CodecResult> res(pend.count);
        const int count = pend.count;
        codecCollect(ctx, &pend, res.data());
        if (pend.errCode != E_NONE) throw RefThrow(errText(pend.errCode));
        for (int i = 0; i < count; ++i) {
            out_sizes[i] = res[i].size;
            if (compressed) compressed[i] = res[i].notSmaller ? 0 : 1;
        }
    });
}

// ---------------------------------------------------------------------------- splat detection, digest
int b200c_detect_splat(b200c_ctx* h, const void* data, size_t nbytes, int elem_bytes, int data_on_device, int* is_splat) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        if (!is_splat) throw BadArg("null result pointer");
        if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 8) throw BadArg("element size must be 1, 2, 4 or 8 bytes");
        *is_splat = 0;
        if (nbytes == 0) return;  // detectSplatManually: empty data is not a splat
        if (!data) throw BadArg("null data pointer");
        if (nbytes < static_cast<size_t>(elem_bytes)) refThrow("The data must contain at least one element");
        if (nbytes % elem_bytes) refThrow("The data array has unexpected length");
        if (nbytes == static_cast<size_t>(elem_bytes)) {
            *is_splat = 1;
            return;
        }
        Context* ctx = reinterpret_cast<Context*>(h);
        CallScope scope(ctx);
        const void* dev = data;
        if (!data_on_device) {
            void* d = ctx->arena.alloc(nbytes);
            copyH2D(ctx, d, data, nbytes);
            dev = d;
        }
        *is_splat = probeSplat(ctx, dev, nbytes, elem_bytes) ? 1 : 0;
    });
}

int b200c_digest64_batch(b200c_ctx* h, int count, const void* const* bufs_dev, const size_t* sizes, uint64_t* out) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        if (count < 0 || (count > 0 && (!bufs_dev || !sizes || !out))) throw BadArg("bad digest arguments");
        Context* ctx = reinterpret_cast<Context*>(h);
        CallScope scope(ctx);
        static_assert(sizeof(uint64_t) == sizeof(unsigned long long), "64-bit words");
        digestBatch(ctx, count, bufs_dev, sizes, reinterpret_cast<unsigned long long*>(out));
    });
}

// ---------------------------------------------------------------------------- multi-GPU exchange
int b200c_ipc_export(b200c_ctx* h, void* dev_ptr, size_t size, b200c_ipc_handle* out) {
    return guarded([&] {
        if (!h || !dev_ptr || !out) throw BadArg("null pointer");
        Context* ctx = reinterpret_cast<Context*>(h);
        B2_CUDA(cudaSetDevice(ctx->device));
        unsigned long long off = 0;
        ipcExport(ctx, dev_ptr, size, out->handle, &off);
        out->offset = off;
        out->size = size;
    });
}
int b200c_ipc_open(b200c_ctx* h, const b200c_ipc_handle* in, void** mapped) {
    return guarded([&] {
        if (!h || !in || !mapped) throw BadArg("null pointer");
        Context* ctx = reinterpret_cast<Context*>(h);
        B2_CUDA(cudaSetDevice(ctx->device));
        *mapped = ipcOpen(ctx, in->handle, in->offset);
    });
}
int b200c_ipc_close(b200c_ctx* h, void* mapped) {
    return guarded([&] {
        if (!h || !mapped) throw BadArg("null pointer");
        Context* ctx = reinterpret_cast<Context*>(h);
        B2_CUDA(cudaSetDevice(ctx->device));
        ipcClose(ctx, mapped);
    });
}
int b200c_copy_segments_async(b200c_ctx* h, const b200c_copy_seg* segs, int count, const uint64_t* wait_flag, uint64_t wait_value,
                              uint64_t* done_flag, uint64_t done_value, unsigned timeout_ms, int mode, int ctas) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        if (count < 0 || (count > 0 && !segs)) throw BadArg("bad segment list");
        if (mode < 0 || mode > 2) throw BadArg("mode must be 0 (copy kernel), 1 (copy engine) or 2 (bulk-copy kernel)");
        for (int i = 0; i < count; ++i)
            if (segs[i].n && (!segs[i].src || !segs[i].dst)) throw BadArg("null segment pointer");
        Context* ctx = reinterpret_cast<Context*>(h);
        std::lock_guard<std::mutex> lock(ctx->mu);
        B2_CUDA(cudaSetDevice(ctx->device));
        pushSegments(ctx, segs, count, reinterpret_cast<const unsigned long long*>(wait_flag), wait_value,
                     reinterpret_cast<unsigned long long*>(done_flag), done_value, timeout_ms, mode, ctas > 0 ? ctas : 64);
    });
}
int b200c_copy_segments_after(b200c_ctx* h, int ticket, const b200c_copy_seg* segs, int count, const uint64_t* wait_flag,
                              uint64_t wait_value, uint64_t* done_flag, uint64_t done_value, unsigned timeout_ms, int mode,
                              int ctas) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        if (count < 0 || (count > 0 && !segs)) throw BadArg("bad segment list");
        if (mode < 0 || mode > 2) throw BadArg("mode must be 0 (copy kernel), 1 (copy engine) or 2 (bulk-copy kernel)");
        for (int i = 0; i < count; ++i)
            if (segs[i].n && (!segs[i].src || !segs[i].dst)) throw BadArg("null segment pointer");
        Context* ctx = reinterpret_cast<Context*>(h);
        if (ticket < 0 || ticket >= Context::kCodecTickets || !ctx->codecTickets[ticket].done) throw BadArg("not a compression ticket");
        std::lock_guard<std::mutex> lock(ctx->mu);
        B2_CUDA(cudaSetDevice(ctx->device));
        pushSegments(ctx, segs, count, reinterpret_cast<const unsigned long long*>(wait_flag), wait_value,
                     reinterpret_cast<unsigned long long*>(done_flag), done_value, timeout_ms, mode, ctas > 0 ? ctas : 64,
                     ctx->codecTickets[ticket].done);
    });
}
int b200c_wait_flags(b200c_ctx* h, const uint64_t* flags_dev, int count, uint64_t value, unsigned timeout_ms,
                     int on_transfer_stream) {
    return guarded([&] {
        if (!h || (count > 0 && !flags_dev)) throw BadArg("null pointer");
        Context* ctx = reinterpret_cast<Context*>(h);
        std::lock_guard<std::mutex> lock(ctx->mu);
        B2_CUDA(cudaSetDevice(ctx->device));
        waitFlags(ctx, reinterpret_cast<const unsigned long long*>(flags_dev), count, value, timeout_ms, on_transfer_stream != 0);
    });
}
int b200c_signal_flags(b200c_ctx* h, uint64_t* const* targets, int count, uint64_t value) {
    return guarded([&] {
        if (!h || (count > 0 && !targets)) throw BadArg("null pointer");
        Context* ctx = reinterpret_cast<Context*>(h);
        CallScope scope(ctx);
        signalFlags(ctx, reinterpret_cast<unsigned long long* const*>(targets), count, value);
    });
}
int b200c_stream_join(b200c_ctx* h) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        Context* ctx = reinterpret_cast<Context*>(h);
        std::lock_guard<std::mutex> lock(ctx->mu);
        if (!ctx->xferStream) return;
        B2_CUDA(cudaSetDevice(ctx->device));
        B2_CUDA(cudaEventRecord(ctx->xferEvent, ctx->xferStream));
        B2_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->xferEvent, 0));
    });
}
int b200c_exchange_status(b200c_ctx* h, int* timed_out) {
    return guarded([&] {
        if (!h || !timed_out) throw BadArg("null pointer");
        Context* ctx = reinterpret_cast<Context*>(h);
        std::lock_guard<std::mutex> lock(ctx->mu);
        B2_CUDA(cudaSetDevice(ctx->device));
        *timed_out = exchangeStatus(ctx);
    });
}

// ---------------------------------------------------------------------------- synthetic weights
int b200c_synth_fill(b200c_ctx* h, void* dst_dev, int64_t count, int32_t dtype, int32_t dist, double p0, double p1,
                     uint64_t seed, uint64_t stream_id) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        Context* ctx = reinterpret_cast<Context*>(h);
        std::lock_guard<std::mutex> lock(ctx->mu);
        B2_CUDA(cudaSetDevice(ctx->device));
        if (count > 0 && !dst_dev) throw BadArg("null destination");
        if (dist < 0 || dist > 2) throw BadArg("unknown distribution");
        launchSynthFill(ctx, dst_dev, count, dtype, dist, p0, p1, seed, stream_id);
    });
}

// ---------------------------------------------------------------------------- memory helpers
int b200c_dev_alloc(b200c_ctx* h, size_t n, void** out) {
    return guarded([&] {
        if (!h || !out) throw BadArg("null pointer");
        Context* ctx = reinterpret_cast<Context*>(h);
        B2_CUDA(cudaSetDevice(ctx->device));
        *out = devMalloc(nullptr, n);  // always the CUDA allocator: the range may be exported over IPC
        registerAllocation(*out, n ? n : 1);
    });
}
int b200c_dev_free(b200c_ctx* h, void* p) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        Context* ctx = reinterpret_cast<Context*>(h);
        B2_CUDA(cudaSetDevice(ctx->device));
        unregisterAllocation(p);
        devFree(nullptr, p);
    });
}
int b200c_host_alloc_pinned(size_t n, void** out) {
    return guarded([&] {
        if (!out) throw BadArg("null pointer");
        void* p = nullptr;
        const cudaError_t e = cudaMallocHost(&p, n ? n : 1);
        if (e != cudaSuccess) {
            cudaGetLastError();
            throw NoMem(std::string("cudaMallocHost: ") + cudaGetErrorString(e));
        }
        *out = p;
    });
}
int b200c_host_free_pinned(void* p) {
    return guarded([&] {
        if (p) B2_CUDA(cudaFreeHost(p));
    });
}
int b200c_dev_memset(b200c_ctx* h, void* dst_dev, int value, size_t n) {
    return guarded([&] {
        if (!h || (n && !dst_dev)) throw BadArg("null pointer");
        Context* ctx = reinterpret_cast<Context*>(h);
        std::lock_guard<std::mutex> lock(ctx->mu);
        B2_CUDA(cudaSetDevice(ctx->device));
        fillBytes(ctx, dst_dev, value, n);
    });
}
int b200c_memcpy_h2d(b200c_ctx* h, void* dst_dev, const void* src, size_t n) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        Context* ctx = reinterpret_cast<Context*>(h);
        std::lock_guard<std::mutex> lock(ctx->mu);
        B2_CUDA(cudaSetDevice(ctx->device));
        copyH2D(ctx, dst_dev, src, n);
        syncStream(ctx);
    });
}
int b200c_memcpy_d2h(b200c_ctx* h, void* dst, const void* src_dev, size_t n) {
    return guarded([&] {
        if (!h) throw BadArg("null context");
        Context* ctx = reinterpret_cast<Context*>(h);
        std::lock_guard<std::mutex> lock(ctx->mu);
        B2_CUDA(cudaSetDevice(ctx->device));
        copyD2H(ctx, dst, src_dev, n);
        syncStream(ctx);
    });
}

}  // extern "C"
