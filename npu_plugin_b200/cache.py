"""Folding cache and background folding requests, with the cached contents resident on the device.

Mirrors the reference's ConstantFoldingCache / ConstantFoldingCacheManager
(src/vpux_compiler/src/dialect/const/utils/constant_folding_cache.cpp:10-198) and its background folding threads
(src/vpux_compiler/src/dialect/const/utils/constant_folding_in_background.cpp:12-147): every new ContentAttr
built through addTransformation is enqueued as a folding request (content.cpp:320-328); worker threads fold
the requests ahead of time; ContentAttr.fold() first asks the cache and waits for a request that is still
PENDING.  When a request only appends a transformation to an attribute whose folded content is already cached,
the worker folds just the new tail on top of the cached content and drops the shorter entry
(tryFoldingPartially :12-49).

What is different on a GPU: a cached content is the folded bytes held in DEVICE memory, so the partial fold
reads its input where it already lies and nothing crosses PCIe until somebody asks for the bytes.  The
reference keeps the storage-typed Content of the prefix, whose pending lazy conversion still sees the original
values; the bytes kept here are the converted ones, so a prefix is reused only where both coincide -- its
storage element type equals its logical one, it is not a splat and not sub-byte -- and any other request is
folded from the base content.  Results are therefore always those of a direct fold.

A "context" (the reference's MLIRContext) is any hashable object the caller compiles under; here the backend.
"""
import queue
import threading

from . import _cabi as A


class FoldingRequestState:
    PENDING = "PENDING"
    COMPLETED = "COMPLETED"


class FoldingRequest:
    def __init__(self, attr, newTransformation=None):
        self.attr, self.newTransformation = attr, newTransformation


TERMINATE = object()  # Const::TerminateRequestAttr


class CacheStatistics:
    def __init__(self):
        self._mtx = threading.Lock()
        self.numCacheHits = self.numCacheMisses = self.numDuplicatedRequests = 0
        self.numElementsAddedToCache = self.numElementsErasedFromCache = 0
        self.numPartialFolds = 0
        self.memoryUsedCache = 0
        self._maxNumRequestsInQueue = self._maxCacheSize = self._maxMemoryUsedCache = 0

    def bump(self, name, by=1):
        with self._mtx:
            setattr(self, name, getattr(self, name) + by)

    def update_max(self, name, value):
        with self._mtx:
            setattr(self, name, max(getattr(self, name), value))

    def getMaxNumRequestsInQueue(self):
        return self._maxNumRequestsInQueue

    def getMaxCacheSize(self):
        return self._maxCacheSize

    def getMaxMemoryUsedCache(self):
        return self._maxMemoryUsedCache


class _Entry:
    def __init__(self):
        self.state, self.content = None, None


class ConstantFoldingCache:
    """Per-context cache: request queue + map ContentAttr key -> (state, resident content)."""

    def __init__(self):
        self._requests = queue.Queue()
        self._map = {}
        self._mtx = threading.Lock()
        self._cv = threading.Condition(self._mtx)
        self._collect = False
        self._stats = CacheStatistics()

    # ---- request queue
    def enqueueRequest(self, request):
        self._requests.put(request)
        if self._collect:
            self._stats.update_max("_maxNumRequestsInQueue", self._requests.qsize())

    def getRequest(self):
        return self._requests.get()

    # ---- states
    def setRequestState(self, attr, state):
        with self._cv:
            self._map.setdefault(attr.key(), _Entry()).state = state
            self._cv.notify_all()

    def getRequestState(self, attr):
        with self._mtx:
            e = self._map.get(attr.key())
            return e.state if e is not None else None

    # ---- contents
    def addContent(self, attr, content):
        with self._cv:
            self._map.setdefault(attr.key(), _Entry()).content = content
            size = len(self._map)
        if self._collect:
            self._stats.bump("numElementsAddedToCache")
            self._stats.bump("memoryUsedCache", content.nbytes)
            self._stats.update_max("_maxMemoryUsedCache", self._stats.memoryUsedCache)
            self._stats.update_max("_maxCacheSize", size)

    def removeContent(self, attr):
        with self._cv:
            e = self._map.pop(attr.key(), None)
        if e is not None and e.content is not None:
            if self._collect:
                self._stats.bump("numElementsErasedFromCache")
                self._stats.bump("memoryUsedCache", -e.content.nbytes)
            e.content.release()

    def getContent(self, attr):
        """The cached resident content of `attr`, waiting for a request that is still being folded; None on a miss."""
        key = attr.key()
        with self._cv:
            e = self._map.get(key)
            if e is None or e.state is None:
                if self._collect:
                    self._stats.bump("numCacheMisses")
                return None
            while e.state != FoldingRequestState.COMPLETED:
                self._cv.wait()
                e = self._map.get(key)
                if e is None:
                    break
            content = e.content if e is not None else None
        if self._collect:
            self._stats.bump("numCacheHits" if content is not None else "numCacheMisses")
        return content

    def clear(self):
        with self._cv:
            entries, self._map = list(self._map.values()), {}
        for e in entries:
            if e.content is not None:
                e.content.release()

    def enableStatisticsCollection(self):
        self._collect = True

    def disableStatisticsCollection(self):
        self._collect = False

    def isStatisticsCollectionEnabled(self):
        return self._collect

    def getStatistics(self):
        return self._stats


class ConstantFoldingCacheManager:
    """Singleton: one cache per compilation context."""

    _instance = None
    _lock = threading.Lock()

    def __init__(self):
        self._caches, self._mtx = {}, threading.Lock()

    @classmethod
    def getInstance(cls):
        with cls._lock:
            if cls._instance is None:
                cls._instance = ConstantFoldingCacheManager()
            return cls._instance

    def addCache(self, ctx):
        with self._mtx:
            if id(ctx) in self._caches:
                return False
            self._caches[id(ctx)] = ConstantFoldingCache()
            return True

    def removeCache(self, ctx):
        with self._mtx:
            c = self._caches.pop(id(ctx), None)
        if c is None:
            return False
        c.clear()
        return True

    def contains(self, ctx):
        return id(ctx) in self._caches

    def get(self, ctx):
        c = self._caches.get(id(ctx))
        if c is None:
            raise RuntimeError(f"Unable to find cache for {ctx}")
        return c


# --------------------------------------------------------------------------- storage type bookkeeping
def storage_dtype_after(base_dtype, transforms, infer):
    """Storage element type of the folded Content after `transforms` (the reference's Content keeps two types:
    the logical one changes at ConvertElemType / QuantCast, the storage one only when a transformation allocates).
    infer(k) gives the logical type after the first k transformations."""
    storage = base_dtype
    for k, t in enumerate(transforms):
        if t.kind in (A.X_DEQUANTIZE, A.X_RESCALE, A.X_ADD, A.X_QUANTIZE_SYNTH):
            storage = A.F32
        elif t.kind == A.X_BIT_PACK:
            storage = A.UI8
        elif t.kind == A.X_GET_SPARSITY_MAP:
            storage = A.I1
        elif t.kind in (A.X_SPARSIFY, A.X_SWIZZLE_CONSTANT):
            storage = infer(k + 1).dtype
        elif t.kind == A.X_RELOCATE_WEIGHTS_TABLE:
            storage = A.SI32
    return storage


def prefix_is_reusable(attr):
    """True when the cached bytes of `attr` (its copyTo bytes) are also what the reference's cached Content would
    hand to a further transformation: no pending lazy conversion, not a splat, byte-sized elements."""
    if attr._isSplat:
        return False
    ts = attr.getTransformations()
    logical = attr.getType()
    if logical.getElemTypeSize() < 8:
        return False
    storage = storage_dtype_after(attr._baseType.dtype, ts, lambda k: attr._backend.infer_type(attr._baseType, ts[:k]))

    def norm(dt):  # signless and unsigned integers are read the same way
        return (A.CLS_UINT << 8 | A.dtype_bits(dt)) if A.dtype_class(dt) == A.CLS_INT else dt
    return norm(storage) == norm(logical.dtype)


# --------------------------------------------------------------------------- background folding
def tryFoldingPartially(cache, request, newTransformation):
    if newTransformation is None:
        return False
    partial_attr = request.stripTransformationsFrom(newTransformation)
    if partial_attr is None:
        return False
    partial = cache.getContent(partial_attr)
    if partial is None:
        return False
    last = request.getLastTransformationsFrom(newTransformation)
    if not last:
        return False
    if not prefix_is_reusable(partial_attr):
        return False
    cache.setRequestState(request, FoldingRequestState.PENDING)
    # the remaining transformations are folded over the cached bytes, which stay where they are (device memory)
    content = request._backend.fold_resident(partial.type_as_base(), partial, False, last)
    cache.addContent(request, content)
    cache.removeContent(partial_attr)
    cache.setRequestState(request, FoldingRequestState.COMPLETED)
    if cache.isStatisticsCollectionEnabled():
        cache.getStatistics().bump("numPartialFolds")
    return True


def _folding_thread(ctx):
    cache = ConstantFoldingCacheManager.getInstance().get(ctx)
    while True:
        req = cache.getRequest()
        if req is TERMINATE or req.attr is TERMINATE:
            break
        request = req.attr
        # requests received before have a state already
        if cache.getRequestState(request) is not None:
            if cache.isStatisticsCollectionEnabled():
                cache.getStatistics().bump("numDuplicatedRequests")
            continue
        try:
            if tryFoldingPartially(cache, request, req.newTransformation):
                continue
            cache.setRequestState(request, FoldingRequestState.PENDING)
            content = request._backend.fold_resident(request._baseType, request._base, request._isSplat,
                                                     request.getTransformations())
            cache.addContent(request, content)
        except Exception as e:  # a request that cannot be folded (the foreground fold raises the same error)
            cache.addContent(request, FailedContent(e))
        cache.setRequestState(request, FoldingRequestState.COMPLETED)


class FailedContent:
    """Cache entry of a request whose fold raised: fold() re-raises it."""
    nbytes = 0

    def __init__(self, error):
        self.error = error

    def release(self):
        pass


def initBackgroundConstantFoldingThreads(ctx, numThreads, collectStatistics=False):
    mgr = ConstantFoldingCacheManager.getInstance()
    mgr.addCache(ctx)
    if collectStatistics:
        mgr.get(ctx).enableStatisticsCollection()
    threads = []
    for _ in range(numThreads):
        t = threading.Thread(target=_folding_thread, args=(ctx,), daemon=True)
        t.start()
        threads.append(t)
    return threads


def stopBackgroundConstantFoldingThreads(ctx, foldingThreads, collectStatistics=False):
    mgr = ConstantFoldingCacheManager.getInstance()
    cache = mgr.get(ctx)
    for _ in foldingThreads:
        cache.enqueueRequest(FoldingRequest(TERMINATE, None))
    for t in foldingThreads:
        t.join()
    stats = None
    if collectStatistics:
        s = cache.getStatistics()
        stats = {"cache hits": s.numCacheHits, "cache misses": s.numCacheMisses,
                 "max requests in queue": s.getMaxNumRequestsInQueue(), "max elements in cache": s.getMaxCacheSize(),
                 "memory used by cache": s.memoryUsedCache, "max memory used by cache": s.getMaxMemoryUsedCache(),
                 "duplicated requests": s.numDuplicatedRequests, "elements added": s.numElementsAddedToCache,
                 "elements erased": s.numElementsErasedFromCache, "partial folds": s.numPartialFolds}
    mgr.removeCache(ctx)
    return stats
