// Fold planner: walks a transformation chain the way ContentAttr::fold does
// (src/vpux_compiler/src/dialect/const/attributes/content.cpp:167-193), but instead of running one
// pass per transformation it composes index-only transformations (Reorder, SubView, PadWithZero)
// and elementwise ones (Dequantize, Rescale, Add, the synthetic quantiser) into a single view and
// only launches a kernel when it has to: at the end (Content::copyTo), or in front of a
// transformation that needs dense input (GetSparsityMap, Sparsify, Reshape of a permuted view ...).
#include "plan.h"

#include <algorithm>
#include <cstring>

namespace b200c {

// ---------------------------------------------------------------------------- tags
int tagOfStorage(int dtype) {
    const int c = dtClass(dtype), b = dtBits(dtype);
    if (c == B200C_CLS_UINT || c == B200C_CLS_INT) {
        switch (b) {
        case 4:
        case 8:
            return T_U8;
        case 16:
            return T_U16;
        case 32:
            return T_U32;
        case 64:
            return T_U64;
        }
    } else if (c == B200C_CLS_SINT) {
        switch (b) {
        case 4:
        case 8:
            return T_I8;
        case 16:
            return T_I16;
        case 32:
            return T_I32;
        case 64:
            return T_I64;
        }
    } else if (c == B200C_CLS_FLOAT) {
        if (b == 16) return T_F16;
        if (b == 32) return T_F32;
        if (b == 64) return T_F64;
    } else if (c == B200C_CLS_BFLOAT) {
        return T_BF16;
    }
    refThrow("Unsupported element type");
}

// C type for a logical element type: quantised types go by their storage integer and only
// 8/4-bit ones are accepted (content.hpp:283-296)
static int tagOfLogical(const TensorType& t) {
    if (t.quantized()) {
        const int b = t.bits();
        if (b != 8 && b != 4) refThrow("Unsupported quantized storage type");
    }
    return tagOfStorage(t.dtype);
}

// checked_cast<StorageT>(integer) on the host, for fill values and the sparsify value
static unsigned long long castIntToTag(long long v, int tag) {
    int err = E_NONE;
    Val in;
    in.bits = static_cast<unsigned long long>(v);
    in.tag = T_I64;
    const unsigned long long bits = castChecked(in, tag, err);
    if (err != E_NONE) refThrow("Can not safely cast %lld to the storage element type", v);
    return bits;
}

// ---------------------------------------------------------------------------- view helpers
static void contiguousStrides(View& v) {
    long long s = 1;
    for (int k = v.rank - 1; k >= 0; --k) {
        v.stride[k] = s;
        s *= v.shape[k];
    }
}

static void setShape(View& v, const Dims& memShape) {
    v.rank = static_cast<int>(memShape.size());
    for (int k = 0; k < v.rank; ++k) v.shape[k] = memShape[k];
}

static bool isPlain(const View& v) {
    if (!v.boxes.empty() || !v.ops.empty() || v.base != 0) return false;
    long long s = 1;
    for (int k = v.rank - 1; k >= 0; --k) {
        if (v.shape[k] != 1 && v.stride[k] != s) return false;
        s *= v.shape[k];
    }
    return true;
}

Planner::Planner(Context* ctx, const TensorType& baseType, const void* devData, size_t nbytes, bool splat)
        : _ctx(ctx) {
    _s.type = baseType;
    _s.storage = baseType.dtype;
    _s.splat = splat;
    const int sbits = dtBits(baseType.dtype);
    const int64_t expect = splat ? (sbits + 7) / 8 : (static_cast<int64_t>(sbits) * baseType.count() + 7) / 8;
    if (static_cast<int64_t>(nbytes) < expect) throw BadArg("base data is smaller than its type says");
    _s.view.src = devData;
    _s.view.srcBytes = nbytes;
    _s.view.srcTag = sbits >= 8 ? tagOfStorage(baseType.dtype) : T_NONE;
    setShape(_s.view, baseType.memShape());
    if (splat) {
        for (int k = 0; k < _s.view.rank; ++k) _s.view.stride[k] = 0;
    } else {
        contiguousStrides(_s.view);
    }
    _s.view.base = 0;
}

int Planner::curTag() const {
    return _s.view.ops.empty() ? _s.view.srcTag : static_cast<int>(T_F32);
}

void* Planner::uploadTable(const void* host, size_t bytes) {
    void* d = _ctx->arena.alloc(bytes);
    uploadSmall(_ctx, d, host, bytes);
    return d;
}

// ---------------------------------------------------------------------------- emission
GenParams Planner::paramsFor(const View& v) const {
    GenParams p;
    std::memset(&p, 0, sizeof(p));
    p.src = v.src;
    p.srcTag = v.srcTag;
    p.rank = v.rank;
    for (int k = 0; k < v.rank; ++k) {
        p.shape[k] = v.shape[k];
        p.stride[k] = v.stride[k];
    }
    p.base = v.base;
    p.nBoxes = static_cast<int>(v.boxes.size());
    for (int b = 0; b < p.nBoxes; ++b) p.box[b] = v.boxes[b];
    p.nOps = static_cast<int>(v.ops.size());
    for (int i = 0; i < p.nOps; ++i) p.ops[i] = v.ops[i];
    p.err = _ctx->errWord;
    p.swizzleKey = -1;
    return p;
}

// Materialise the current Content into a dense device buffer of storage-typed elements; the view
// becomes the identity over that buffer.  This is what a materialising transformation of the
// reference leaves behind (Content::allocTempBuffer, CU/content.cpp:32-47).
void Planner::materialize() {
    if (dtBits(_s.storage) < 8) return;  // packed sub-byte storage is always dense here
    if (isPlain(_s.view) && !_s.splat) return;
    const int tag = curTag();
    const int64_t n = _s.splat ? 1 : _s.type.count();
    const size_t bytes = static_cast<size_t>(n) * tagBytes(tag);
    void* dst = _ctx->arena.alloc(bytes ? bytes : 1);
    if (n > 0) {
        GenParams p = paramsFor(_s.view);
        if (_s.splat) {  // one element: evaluate at the origin
            p.rank = 0;
        }
        p.dst = dst;
        p.outMode = OUT_RAW;
        p.outTag = tag;
        p.outElems = p.outUnits = n;
        p.dataBytes = p.totalBytes = static_cast<long long>(bytes);
        runGeneric(p);
    }
    View nv;
    nv.src = dst;
    nv.srcBytes = bytes;
    nv.srcTag = tag;
    setShape(nv, _s.type.memShape());
    if (_s.splat) {
        for (int k = 0; k < nv.rank; ++k) nv.stride[k] = 0;
    } else {
        contiguousStrides(nv);
    }
    nv.base = 0;
    _s.view = nv;
}

// Dense buffer of the Content's values read as C type `tag` (getValues<T>() of every element).
const void* Planner::denseAs(int tag) {
    if (dtBits(_s.storage) < 8) refThrow("Unsupported storage type of size '%d' bits.", dtBits(_s.storage));
    if (isPlain(_s.view) && !_s.splat && _s.view.srcTag == tag) return _s.view.src;
    const int64_t n = _s.type.count();
    const size_t bytes = static_cast<size_t>(n) * tagBytes(tag);
    void* dst = _ctx->arena.alloc(bytes ? bytes : 1);
    if (n > 0) {
        GenParams p = paramsFor(_s.view);
        p.dst = dst;
        p.outMode = OUT_CAST;
        p.outTag = tag;
        p.outElems = p.outUnits = n;
        p.dataBytes = p.totalBytes = static_cast<long long>(bytes);
        runGeneric(p);
    }
    return dst;
}


void Planner::flushPendingStats() {
    if (!_pending.active) return;
    _pending.active = false;
    launchRowStats(_ctx, _pending.stats);
}

// Queued (batched) launches are only safe for the kernel that writes an item's final output:
// anything an item's later kernels read must have been launched in stream order.
struct ImmediateLaunches {
    Context* ctx;
    bool saved;
    ImmediateLaunches(Context* c, bool immediate): ctx(c), saved(c->batching) {
        if (immediate) ctx->batching = false;
    }
    ~ImmediateLaunches() {
        ctx->batching = saved;
    }
};

void Planner::runGeneric(const GenParams& p) {
    flushPendingStats();
    ImmediateLaunches scope(_ctx, !_emittingFinal);
    TileItem item;
    if (tryLaunchDequantRows(_ctx, p)) return;
    if (makeTileItem(p, &item)) {
        launchTile(_ctx, item);
    } else {
        launchGeneric(_ctx, p);
    }
}

// The whole remaining chain is "quantise every row, permute inside rows, store bytes/nibbles
// (swizzled)": hand it to the single-pass kernel.
bool Planner::tryFusedRowQuant(void* dst, int outMode, int outTag, int swizzleKey, int64_t dataBytes,
                               int64_t totalBytes) {
    if (!_pending.active) return false;
    const View& v = _s.view;
    const RowStatsParams& st = _pending.stats;
    if (_s.splat || v.ops.size() != 1 || !v.boxes.empty() || v.src != _pending.src || v.base != 0) return false;
    const ValueOp& op = v.ops[0];
    if (op.fscales != st.scales || op.off != 0 || op.dim < 0) return false;
    const bool sym = st.scheme == B200C_QSYNTH_SYM_I8;
    if (outMode == 0) {
        if (!(outTag == T_I8 || (outTag == T_U8 && !sym))) return false;
    } else if (sym) {
        return false;  // negative values fail BitPack's unsigned read; the generic pass reports that
    }
    if (v.shape[op.dim] != st.rows) return false;
    // the row dim must be the outermost dim that matters, with rows laid out back to back
    for (int k = 0; k < op.dim; ++k)
        if (v.shape[k] != 1) return false;
    if (st.rows > 1 && v.stride[op.dim] != st.rowElems) return false;
    // the remaining dims must enumerate the row exactly once (a mixed-radix permutation)
    std::vector<std::pair<long long, long long>> dims;  // (shape, stride), outermost first
    for (int k = op.dim + 1; k < v.rank; ++k)
        if (v.shape[k] != 1) dims.push_back({v.shape[k], v.stride[k]});
    {
        auto sorted = dims;
        std::sort(sorted.begin(), sorted.end(), [](const auto& a, const auto& b) { return a.second < b.second; });
        long long expect = 1;
        for (const auto& d : sorted) {
            if (d.second != expect) return false;
            expect *= d.first;
        }
        if (expect != st.rowElems) return false;
    }
    for (size_t k = 0; k + 1 < dims.size();) {  // merge dims that are contiguous in the source
        if (dims[k].second == dims[k + 1].second * dims[k + 1].first) {
            dims[k + 1].first *= dims[k].first;
            dims.erase(dims.begin() + k);
        } else {
            ++k;
        }
    }
    if (dims.size() > 3) return false;
    RowQuantParams rq;
    std::memset(&rq, 0, sizeof(rq));
    rq.src = _pending.src;
    rq.srcTag = _pending.srcTag;
    rq.rows = st.rows;
    rq.rowElems = st.rowElems;
    rq.scheme = st.scheme;
    rq.scales = st.scales;
    rq.zps = st.zps;
    if (dims.size() == 1 || dims.empty()) {
        rq.irank = 0;
    } else {
        rq.irank = static_cast<int>(dims.size());
        for (size_t k = 0; k < dims.size(); ++k) {
            rq.ishape[k] = dims[k].first;
            rq.istride[k] = dims[k].second;
        }
    }
    rq.dst = dst;
    rq.outMode = outMode;
    rq.swizzleKey = swizzleKey;
    rq.dataBytes = dataBytes;
    rq.totalBytes = totalBytes;
    _pending.active = false;
    ImmediateLaunches scope(_ctx, !_emittingFinal);
    launchRowQuantFused(_ctx, rq);
    return true;
}

// ---------------------------------------------------------------------------- transformations
void Planner::needByteStorage(const char* what) {
    if (dtBits(_s.storage) < 8) throw NotBuilt(std::string(what) + " on bit-packed storage is not built");
}

void Planner::apply(const Transformation& x) {
    // sub-byte storage guard of the fold loop (content.cpp:185-187)
    if (dtBits(_s.storage) < 8 && !acceptsSubByteStorage(x.kind)) {
        refThrow("Unsupported storage type of size '%d' bits.", dtBits(_s.storage));
    }
    if (_afterBitPack) throw NotBuilt("transformations after BitPack are not built");
    const TensorType outType = inferOne(x, _s.type);
    View& v = _s.view;
    // only the metadata-only transformations below carry a deviating storage size on
    const long long keepRaw = _s.rawBytes;
    _s.rawBytes = -1;

    switch (x.kind) {
    case B200C_X_CONVERT_ELEM_TYPE:
    case B200C_X_QUANT_CAST:
        _s.type = outType;  // metadata only (convert_elem_type.cpp:79-81, quant_cast.cpp:81-83)
        _s.rawBytes = keepRaw;
        return;

    case B200C_X_RESHAPE:
    case B200C_X_CHANGE_SHAPE_AND_ELEM_TYPE: {
        // metadata only in the reference (reshape.cpp:82-84); the linear storage order is kept, so a
        // permuted view has to be made dense before its shape can be reinterpreted
        if (!_s.splat) materialize();
        const int sbits = dtBits(_s.storage);
        if (!_s.splat && sbits >= 8) {
            const long long held = keepRaw >= 0 ? keepRaw : static_cast<long long>(_s.type.count()) * (sbits / 8);
            if (held != static_cast<long long>(outType.count()) * (sbits / 8)) _s.rawBytes = held;
        }
        _s.type = outType;
        setShape(v, outType.memShape());
        if (_s.splat) {
            for (int k = 0; k < v.rank; ++k) v.stride[k] = 0;
        } else if (sbits >= 8) {
            contiguousStrides(v);
        }
        return;
    }

    case B200C_X_REORDER: {  // reorder.cpp:75-95 -> memPermuteTransformation (CU/transformations.cpp:23-70)
        needByteStorage("Reorder");
        const int r = _s.type.rank();
        std::vector<int> from(r);  // output memory position k reads input memory position from[k]
        for (int k = 0; k < r; ++k) from[k] = _s.type.memPosOf(outType.order[k]);
        View nv = v;
        for (int k = 0; k < r; ++k) {
            nv.shape[k] = v.shape[from[k]];
            nv.stride[k] = v.stride[from[k]];
            for (size_t b = 0; b < v.boxes.size(); ++b) {
                nv.boxes[b].lo[k] = v.boxes[b].lo[from[k]];
                nv.boxes[b].hi[k] = v.boxes[b].hi[from[k]];
            }
        }
        auto moved = [&](int dim) {
            for (int k = 0; k < r; ++k)
                if (from[k] == dim) return k;
            return dim;
        };
        for (auto& op : nv.ops)
            if (op.dim >= 0) op.dim = moved(op.dim);
        for (auto& b : nv.boxes)
            if (b.table) b.tableDim = moved(b.tableDim);
        v = nv;
        _s.type = outType;
        return;
    }

    case B200C_X_SUBVIEW: {  // subview.cpp:123-301
        if (dtBits(_s.storage) == 1) {
            subviewBits(x, outType);
            return;
        }
        needByteStorage("SubView");
        const auto off = _s.type.memOrder(x.a);
        const auto shape = outType.memShape();
        for (int k = 0; k < v.rank; ++k) {
            v.base += off[k] * v.stride[k];
            v.shape[k] = shape[k];
            for (auto& b : v.boxes) {
                b.lo[k] -= off[k];
                b.hi[k] -= off[k];
            }
        }
        for (auto& op : v.ops)
            if (op.dim >= 0) op.off += off[op.dim];
        for (auto& b : v.boxes)
            if (b.table) b.tableOff += off[b.tableDim];
        _s.type = outType;
        return;
    }

    case B200C_X_PAD_WITH_ZERO: {  // pad_with_zero.cpp:108-262, fill value: Content::fillWithZero (CU/content.cpp:213-261)
        needByteStorage("PadWithZero");
        if (static_cast<int>(v.boxes.size()) >= kMaxBoxes) materialize();
        const int tag = curTag();
        const auto before = _s.type.memOrder(x.a);
        const auto inShape = _s.type.memShape();
        const auto shape = outType.memShape();
        FillBox fb;
        std::memset(&fb, 0, sizeof(fb));
        fb.tag = tag;
        fb.pos = static_cast<int>(v.ops.size());
        bool widens = false;
        for (int k = 0; k < v.rank; ++k) widens = widens || shape[k] != inShape[k];
        if (outType.q.kind == B200C_Q_PER_AXIS) {
            if (outType.rank() != 4) refThrow("Unsupported shape size %d", outType.rank());
            if (outType.q.axis != 0) refThrow("Only per-channel quantization is supported");
        }
        if (outType.q.kind == B200C_Q_PER_AXIS && (!widens || outType.q.zpsAllEqual())) {
            // nothing to fill, or one value for every channel: no table
            fb.bits = outType.q.n ? castIntToTag(outType.q.zps[0], tag) : 0;
        } else if (outType.q.kind == B200C_Q_PER_AXIS) {
            const size_t es = tagBytes(tag);
            std::vector<char> table(outType.q.n * es);
            for (size_t i = 0; i < outType.q.n; ++i) {
                const unsigned long long bits = castIntToTag(outType.q.zps[i], tag);
                std::memcpy(table.data() + i * es, &bits, es);  // little endian
            }
            fb.table = uploadTable(table.data(), table.size());
            fb.tableDim = outType.memPosOf(0);
            fb.tableOff = 0;
        } else if (outType.q.kind == B200C_Q_PER_TENSOR) {
            fb.bits = castIntToTag(outType.q.zps[0], tag);
        } else {
            fb.bits = 0;
        }
        for (int k = 0; k < v.rank; ++k) {
            v.base -= before[k] * v.stride[k];
            v.shape[k] = shape[k];
            for (auto& b : v.boxes) {
                b.lo[k] += before[k];
                b.hi[k] += before[k];
            }
            fb.lo[k] = before[k];
            fb.hi[k] = before[k] + inShape[k];
        }
        for (auto& op : v.ops)
            if (op.dim >= 0) op.off -= before[op.dim];
        for (auto& b : v.boxes)
            if (b.table) b.tableOff -= before[b.tableDim];
        if (widens) v.boxes.push_back(fb);  // a zero-width pad fills nothing
        _s.type = outType;
        _s.splat = false;
        return;
    }

    case B200C_X_DEQUANTIZE: {  // dequantize.cpp:47-94
        needByteStorage("Dequantize");
        if (static_cast<int>(v.ops.size()) >= kMaxOps) materialize();
        ValueOp op;
        std::memset(&op, 0, sizeof(op));
        op.kind = OP_DEQUANT;
        op.dim = -1;
        if (_s.type.q.kind == B200C_Q_PER_AXIS) {
            const auto& q = _s.type.q;
            const int memAxis = _s.type.memPosOf(q.axis);
            if (static_cast<int64_t>(q.n) != v.shape[memAxis]) refThrow("Wrong scales size");
            if (_s.type.count() == 0) refThrow("Inner size is zero");
            op.scales = static_cast<const double*>(uploadTable(q.scales, q.n * sizeof(double)));
            static_assert(sizeof(long long) == sizeof(int64_t), "");
            op.zps = static_cast<const long long*>(uploadTable(q.zps, q.n * sizeof(int64_t)));
            op.dim = memAxis;
            op.off = 0;
            _s.splat = false;  // dequantize.cpp:31-40
        } else {
            op.scale = _s.type.q.scales[0];
            op.zp = _s.type.q.zps[0];
        }
        v.ops.push_back(op);
        _s.type = outType;
        _s.storage = B200C_F32;
        return;
    }

    case B200C_X_RESCALE:
    case B200C_X_ADD: {  // rescale.cpp:64-78, add.cpp:60-74
        needByteStorage("Rescale/Add");
        if (static_cast<int>(v.ops.size()) >= kMaxOps) materialize();
        ValueOp op;
        std::memset(&op, 0, sizeof(op));
        op.kind = x.kind == B200C_X_RESCALE ? OP_MUL : OP_ADD;
        op.dim = -1;
        op.k = static_cast<float>(x.f);
        v.ops.push_back(op);
        _s.type = outType;
        _s.storage = B200C_F32;
        return;
    }

    case B200C_X_QUANTIZE_SYNTH:
        quantizeSynth(x, outType);
        return;

    case B200C_X_BIT_PACK: {  // bit_pack.cpp:108-130
        if (_s.splat) refThrow("Bit pack does not support splat inputs.");
        if (x.i0 != 4) refThrow("Bit pack does not support any bitwidth except for 4 at this point.");
        if (_s.type.count() % 2 != 0) refThrow("Storage buffer size is odd, which is unexpected for 4 bit packing.");
        _s.type = outType;
        _afterBitPack = true;
        return;
    }

    case B200C_X_GET_SPARSITY_MAP:
        getSparsityMap(outType, /*swizzleKey=*/-1);
        return;

    case B200C_X_SPARSIFY:
        sparsify(x);
        return;

    case B200C_X_SWIZZLE_CONSTANT:
        swizzle(x, outType);
        return;

    case B200C_X_TRANSPOSE: {  // transpose.cpp:92-100: a reorder followed by a reshape
        needByteStorage("Transpose");
        const int r = _s.type.rank();
        View nv = v;
        if (!_s.splat) {
            if (!v.boxes.empty() || !v.ops.empty()) materialize();
            nv = v;
            for (int k = 0; k < r; ++k) {
                const int from = static_cast<int>(x.a[_s.type.order[k]]);
                nv.shape[k] = v.shape[from];
                nv.stride[k] = v.stride[from];
            }
        } else {
            setShape(nv, outType.memShape());
        }
        v = nv;
        _s.type = outType;
        return;
    }

    case B200C_X_BROADCAST: {  // broadcast.cpp:84-116: the memory dim of `axis` is tiled value / extent times
        needByteStorage("Broadcast");
        if (_s.splat) {  // the single stored element is copied
            _s.type = outType;
            setShape(v, outType.memShape());
            return;
        }
        materialize();
        const int r = _s.type.rank();
        const int pos = _s.type.memPosOf(static_cast<int>(x.i0));
        const auto mem = _s.type.memShape();
        const int64_t extent = mem[pos];
        if (extent == 0 || x.i1 % extent) {
            refThrow("Can't broadcast from %lld to %lld", static_cast<long long>(extent), static_cast<long long>(x.i1));
        }
        if (r + 1 > kMaxDims) throw NotBuilt("Broadcast of a rank-8 tensor");
        // dense source read through a view with one more dim: [.., factor (stride 0), extent, ..]
        GenParams p = paramsFor(v);
        p.rank = r + 1;
        long long st = 1;
        std::vector<long long> dense(r);
        for (int k = r - 1; k >= 0; --k) {
            dense[k] = st;
            st *= mem[k];
        }
        for (int k = 0, j = 0; k < r; ++k) {
            if (k == pos) {
                p.shape[j] = x.i1 / extent;
                p.stride[j++] = 0;
            }
            p.shape[j] = mem[k];
            p.stride[j++] = dense[k];
        }
        p.base = 0;
        remapDense(p, curTag(), outType, _s.storage);
        return;
    }

    case B200C_X_REVERSE: {  // reverse.cpp:55-117: runs of `spatialDims` consecutive values are reversed
        needByteStorage("Reverse");
        const int dt = _s.type.dtype;
        if (!(dt == B200C_SI8 || dt == B200C_UI8 || dt == B200C_F16 || dt == B200C_BF16 || dt == B200C_F32)) {
            refThrow("Unexpected data type");
        }
        const int r = _s.type.rank();
        if (!(x.i0 >= 0 && x.i0 < r - 1)) {
            refThrow("Const::Content::reverse: got unexpected content dimension %lld", static_cast<long long>(x.i0));
        }
        int64_t spatial = 1;
        for (int k = r - 1; k > x.i0; --k) spatial *= _s.type.shape[k];
        const int tag = tagOfLogical(_s.type);
        const int64_t n = _s.type.count();
        const void* dense = denseAs(tag);  // getValues<StorageType>() of every element, splat included
        GenParams p;
        std::memset(&p, 0, sizeof(p));
        p.src = dense;
        p.srcTag = tag;
        p.err = _ctx->errWord;
        p.swizzleKey = -1;
        p.rank = 2;
        p.shape[0] = spatial ? n / spatial : 0;
        p.shape[1] = spatial;
        p.stride[0] = spatial;
        p.stride[1] = -1;
        p.base = spatial - 1;
        remapDense(p, tag, outType, dt);
        return;
    }

    case B200C_X_RELOCATE_WEIGHTS_TABLE: {  // relocate_weights_table.cpp:122-203
        needByteStorage("RelocateWeightsTable");
        const int64_t n = _s.type.count();
        const int64_t oc = n / 4;  // WEIGHT_TABLE_NUM_ELEMENTS_PER_OC entries per output channel
        const void* dense = denseAs(T_I32);  // getValues<int32_t>()
        int* dst = static_cast<int*>(_ctx->arena.alloc(n ? static_cast<size_t>(n) * 4 : 1));
        if (n > oc * 4) fillBytes(_ctx, dst + oc * 4, 0, static_cast<size_t>(n - oc * 4) * 4);
        RelocateParams rp;
        std::memset(&rp, 0, sizeof(rp));
        rp.values = static_cast<const int*>(dense);
        rp.patched = dst;
        rp.oc = oc;
        const int clusters = static_cast<int>(x.a.size());
        bool segmented = false;  // all clusters at the same channel offset: the weights are not segmented
        for (size_t k = 0; k < x.a.size(); ++k) {
            rp.offsets[k] = x.a[k];
            rp.weightsPtr[k] = static_cast<int32_t>(x.b[k]);
            if (k > 0 && x.a[k] != x.a[k - 1]) segmented = true;
        }
        // the reference advances its cluster index by at most one per channel (:141-143, :186-189)
        std::vector<int> clusterOf(static_cast<size_t>(std::max<int64_t>(oc, 1)), 0);
        for (int64_t c = 0, ch = 0; ch < oc; ++ch) {
            if (segmented && c + 1 < clusters && ch >= x.a[static_cast<size_t>(c + 1)]) ++c;
            clusterOf[static_cast<size_t>(ch)] = static_cast<int>(c);
        }
        rp.clusterOf = static_cast<const int*>(uploadTable(clusterOf.data(), clusterOf.size() * sizeof(int)));
        rp.sparsityPtr = static_cast<int32_t>(x.i0);
        rp.err = _ctx->errWord;
        if (x.hasAux) {
            if (static_cast<int64_t>(x.aux.size()) != oc) {
                refThrow("Invalid weights compression with %zu elements for %lld channels", x.aux.size(), static_cast<long long>(oc));
            }
            if (x.i1 == 0) refThrow("Missing weights element type attribute");
            const int64_t alignment = x.f > 0 ? static_cast<int64_t>(x.f) : kWeightSetAlign;
            std::vector<long long> steps(static_cast<size_t>(oc));
            int64_t off = 0;
            for (int64_t ch = 0; ch < oc; ++ch) {
                if (ch > 0 && clusterOf[static_cast<size_t>(ch)] != clusterOf[static_cast<size_t>(ch - 1)]) off = 0;
                steps[static_cast<size_t>(ch)] = off;
                off += roundUp((x.aux[static_cast<size_t>(ch)] * x.i1 + 7) / 8, alignment);
            }
            rp.steps = static_cast<const long long*>(uploadTable(steps.data(), steps.size() * sizeof(long long)));
        }
        launchRelocateWeightsTable(_ctx, rp);
        View nv;
        nv.src = dst;
        nv.srcBytes = static_cast<size_t>(n) * 4;
        nv.srcTag = T_I32;
        setShape(nv, outType.memShape());
        contiguousStrides(nv);
        v = nv;
        _s.type = outType;
        _s.storage = B200C_SI32;
        _s.splat = false;
        return;
    }

    case B200C_X_EXPAND_DILATED: {  // expand_dilated.cpp:88-122: raw storage elements scattered into a zero-filled buffer
        needByteStorage("ExpandDilated");
        if (_s.splat) throw NotBuilt("ExpandDilated of a splat (the reference reads past its single stored element)");
        if (outType.q.kind == B200C_Q_PER_AXIS) throw NotBuilt("ExpandDilated of a per-axis quantised constant");
        materialize();
        const int tag = curTag();
        const int es = tagBytes(tag);
        const int64_t n = outType.count();
        void* dst = _ctx->arena.alloc(n ? static_cast<size_t>(n) * es : 1);
        const unsigned long long fill = outType.q.kind == B200C_Q_PER_TENSOR ? castIntToTag(outType.q.zps[0], tag) : 0ull;
        if (n > 0) {
            launchExpandDilated(_ctx, v.src, dst, es, _s.type.shape[0] * _s.type.shape[1], _s.type.shape[2], _s.type.shape[3],
                                outType.shape[2], outType.shape[3], x.a[0], x.a[1], fill);
        }
        View nv;
        nv.src = dst;
        nv.srcBytes = static_cast<size_t>(n) * es;
        nv.srcTag = tag;
        setShape(nv, outType.memShape());
        contiguousStrides(nv);
        v = nv;
        _s.type = outType;
        return;
    }

    default:
        throw NotBuilt("transformation kind " + std::to_string(x.kind) + " is not built");
    }
}

// Runs the element kernel over a hand-built view of a dense buffer and makes the result the new
// (dense) content: what a materialising transformation of the reference leaves behind.
void Planner::remapDense(GenParams p, int tag, const TensorType& outType, int storage) {
    const int64_t n = outType.count();
    const size_t bytes = static_cast<size_t>(n) * tagBytes(tag);
    void* dst = _ctx->arena.alloc(bytes ? bytes : 1);
    if (n > 0) {
        p.dst = dst;
        p.outMode = OUT_RAW;
        p.outTag = tag;
        p.outElems = p.outUnits = n;
        p.dataBytes = p.totalBytes = static_cast<long long>(bytes);
        runGeneric(p);
    }
    View nv;
    nv.src = dst;
    nv.srcBytes = bytes;
    nv.srcTag = tag;
    setShape(nv, outType.memShape());
    contiguousStrides(nv);
    _s.view = nv;
    _s.type = outType;
    _s.storage = storage;
    _s.splat = false;
}

// ---------------------------------------------------------------------------- QuantizeSynth
// Synthetic per-output-channel quantiser (no reference counterpart).  Pass 1 reduces every row
// (slice along logical dim 0) to a scale / zero point; the quantisation itself becomes a value op
// so it fuses with whatever follows.
void Planner::quantizeSynth(const Transformation& x, const TensorType& outType) {
    needByteStorage("QuantizeSynth");
    if (_s.splat) refThrow("QuantizeSynth does not support splat inputs");
    if (_s.type.rank() < 1) refThrow("QuantizeSynth expects rank >= 1");
    View& v = _s.view;
    if (static_cast<int>(v.ops.size()) >= kMaxOps) materialize();
    const int64_t rows = _s.type.shape[0];
    const int rowDim = _s.type.memPosOf(0);
    const bool s0Direct = _sideOnDevice && x.side0 != nullptr, s1Direct = _sideOnDevice && x.side1 != nullptr;
    float* scales = s0Direct ? static_cast<float*>(x.side0)
                             : static_cast<float*>(_ctx->arena.alloc(std::max<int64_t>(rows, 1) * sizeof(float)));
    int* zps = s1Direct ? static_cast<int*>(x.side1)
                        : static_cast<int*>(_ctx->arena.alloc(std::max<int64_t>(rows, 1) * sizeof(int)));
    flushPendingStats();
    if (rows > 0 && _s.type.count() > 0) {
        RowStatsParams rp;
        rp.view = paramsFor(v);
        rp.rowDim = rowDim;
        rp.rows = rows;
        rp.rowElems = _s.type.count() / rows;
        rp.scheme = static_cast<int>(x.i0);
        rp.scales = scales;
        rp.zps = zps;
        const bool rowsContiguous = isPlain(v) && !_s.splat && rowDim == 0 &&
                                    (v.srcTag == T_F16 || v.srcTag == T_F32) &&
                                    static_cast<size_t>(rp.rowElems) * tagBytes(v.srcTag) <= rowQuantMaxRowBytes();
        if (rowsContiguous) {
            _pending.active = true;
            _pending.stats = rp;
            _pending.src = v.src;
            _pending.srcTag = v.srcTag;
            _pending.rowDim = rowDim;
        } else {
            launchRowStats(_ctx, rp);
        }
    }
    ValueOp op;
    std::memset(&op, 0, sizeof(op));
    op.kind = x.i0 == B200C_QSYNTH_SYM_I8 ? OP_QSYM : OP_QASYM;
    op.dim = rowDim;
    op.off = 0;
    op.fscales = scales;
    op.izps = zps;
    v.ops.push_back(op);
    _s.type = outType;
    _s.storage = B200C_F32;
    SideOutput so;
    so.dev = scales;
    so.user = x.side0;
    so.bytes = static_cast<size_t>(rows) * sizeof(float);
    if (so.user && !s0Direct) _sides.push_back(so);
    so.dev = zps;
    so.user = x.side1;
    so.bytes = static_cast<size_t>(rows) * sizeof(int);
    if (so.user && !s1Direct) _sides.push_back(so);
}

// ---------------------------------------------------------------------------- sparsity
static int sparsityTag(const TensorType& t) {
    // GetSparsityMap / Sparsify accept si8, ui8, f16, bf16, f32 after normalising quantised types
    // (get_sparsity_map.cpp:94-106, sparsify.cpp:172-183)
    switch (t.dtype) {
    case B200C_SI8:
        return T_I8;
    case B200C_UI8:
        return T_U8;
    case B200C_F16:
        return T_F16;
    case B200C_BF16:
        return T_BF16;
    case B200C_F32:
        return T_F32;
    default:
        refThrow("Unexpected weights data type");
    }
}

// raw bits of StorageType(sparsifyValue)
static unsigned long long sparseBitsFor(int64_t value, int tag, bool checked) {
    if (checked) return castIntToTag(value, tag);  // checked_cast<StorageType> (sparsify.cpp:134, sparsity.cpp:40)
    switch (tag) {                                 // plain StorageType(value) (get_sparsity_map.cpp:49)
    case T_I8:
    case T_U8:
        return static_cast<unsigned long long>(value) & 0xFF;
    case T_F16:
        return floatToHalfBits(static_cast<float>(value));
    case T_BF16:
        return floatToBf16Bits(static_cast<float>(value));
    default:
        return floatToBits(static_cast<float>(value));
    }
}

// the transformation being applied is followed by exactly one more, a SwizzleConstant that writes
// the caller's buffer
bool Planner::finalSwizzleFollows() const {
    return _next != nullptr && _nextIsLast && _next->kind == B200C_X_SWIZZLE_CONSTANT && _finalDst != nullptr;
}

void Planner::getSparsityMap(const TensorType& outType, int swizzleKey) {
    const int64_t sv = sparsifyValue(_s.type);
    const int tag = sparsityTag(_s.type);
    const int64_t oc = _s.type.shape[0];
    const int64_t work = _s.type.shape[1] * _s.type.shape[2] * _s.type.shape[3];
    const int64_t outBits = outType.shape[3];
    if (work % 8 != 0) {
        // the reference reads whole groups of 8 elements and runs past the last channel
        // (get_sparsity_map.cpp:43-52 with the bounds check of content.hpp:95-96)
        if (!_s.splat) refThrow("Out-of-bound access in ContentRangeBase");
        throw NotBuilt("GetSparsityMap of a splat with a workload that is not a multiple of 8");
    }
    const void* dense = denseAs(tag);
    const size_t bytes = static_cast<size_t>(oc * outBits / 8);
    void* dst = nullptr;
    const bool swzNext = finalSwizzleFollows();
    if (bytes > 0 && tagBytes(tag) == 1 && work % 16 == 0 && _finalDst && (_isLast || swzNext) &&
        ((reinterpret_cast<uintptr_t>(dense) | reinterpret_cast<uintptr_t>(_finalDst)) & 15) == 0) {
        // 8-bit elements and the result is the caller's output: one (batched) launch writes the map
        // where it belongs, through the swizzle rotation when the chain ends in SwizzleConstant
        MapItem it;
        it.src = static_cast<const unsigned char*>(dense);
        it.dst = static_cast<unsigned char*>(_finalDst);
        it.oc = oc;
        it.work = work;
        it.outBytesPerOC = outBits / 8;
        it.sparseByte = static_cast<unsigned int>(sparseBitsFor(sv, tag, false) & 0xFF);
        it.swizzleKey = swzNext ? static_cast<int>(static_cast<uint32_t>(_next->i0) % 6u) : -1;
        it.totalBytes = swzNext ? roundUp(static_cast<int64_t>(bytes), kSwizzleSizeAlign) : static_cast<int64_t>(bytes);
        it.counts = nullptr;
        if (static_cast<size_t>(it.totalBytes) > _finalCap) throw Capacity("output buffer too small");
        launchMapItem(_ctx, it);
        dst = _finalDst;
        if (swzNext) {
            _fusedSwizzle = true;
            _fusedTotal = it.totalBytes;
        } else {
            _wroteFinal = true;
            _finalBytes = bytes;
        }
    } else {
        dst = _ctx->arena.alloc(bytes ? bytes : 1);
        if (bytes) {
            launchSparsityMap(_ctx, dense, tag, oc, work, outBits, sparseBitsFor(sv, tag, false), dst, swizzleKey);
        }
    }
    View nv;
    nv.src = dst;
    nv.srcBytes = bytes;
    nv.srcTag = T_NONE;
    setShape(nv, outType.memShape());
    contiguousStrides(nv);
    _s.view = nv;
    _s.type = outType;
    _s.storage = B200C_UI1;
    _s.splat = false;
}

std::vector<int64_t> Planner::countNonSparse() {
    if (dtBits(_s.storage) < 8) refThrow("Unsupported storage type of size '%d' bits.", dtBits(_s.storage));
    const int64_t sv = sparsifyValue(_s.type);
    const int tag = sparsityTag(_s.type);
    if (_s.type.rank() != 4) refThrow("Const::Content::sparsify: got unxpected content shape %d", _s.type.rank());
    const int64_t oc = _s.type.shape[0];
    const int64_t work = _s.type.shape[1] * _s.type.shape[2] * _s.type.shape[3];
    const unsigned long long sbits = sparseBitsFor(sv, tag, true);
    std::vector<int64_t> counts(static_cast<size_t>(oc), 0);
    if (oc == 0) return counts;
    const void* dense = denseAs(tag);
    long long* dcounts = static_cast<long long*>(_ctx->arena.alloc(static_cast<size_t>(oc) * sizeof(long long)));
    launchCountNonSparse(_ctx, dense, tag, oc, work, sbits, dcounts);
    copyD2H(_ctx, counts.data(), dcounts, static_cast<size_t>(oc) * sizeof(long long));
    syncStream(_ctx);
    checkDeviceError(_ctx);
    return counts;
}

void Planner::sparsify(const Transformation& x) {  // sparsify.cpp:115-186
    const int64_t sv = sparsifyValue(_s.type);
    const int tag = sparsityTag(_s.type);
    if (_s.type.rank() != 4) refThrow("Expected 4D input shape.");
    const int64_t oc = _s.type.shape[0];
    const int64_t work = _s.type.shape[1] * _s.type.shape[2] * _s.type.shape[3];
    const int eb = tagBytes(tag);
    const unsigned long long sbits = sparseBitsFor(sv, tag, true);
    const void* dense = denseAs(tag);

    const bool swzNext = finalSwizzleFollows();
    if (eb == 1 && oc > 0 && work > 0 && work % 16 == 0 && _finalDst && (_isLast || swzNext) &&
        ((reinterpret_cast<uintptr_t>(dense) | reinterpret_cast<uintptr_t>(_finalDst)) & 15) == 0 &&
        (x.hasAux || _ctx->batching)) {
        // 8-bit elements and the result is the caller's output: count, channel offsets and the
        // compaction run as three (batched) launches that write the values where they belong.  Without
        // numActualElements the size of the result is only known on the device; the batched entry
        // point reads it back once for all items.
        SparseItem it;
        it.src = static_cast<const unsigned char*>(dense);
        it.dst = static_cast<unsigned char*>(_finalDst);
        it.oc = oc;
        it.work = work;
        it.counts = static_cast<long long*>(_ctx->arena.alloc(static_cast<size_t>(oc) * sizeof(long long)));
        it.offsets = static_cast<long long*>(_ctx->arena.alloc(static_cast<size_t>(oc + 1) * sizeof(long long)));
        it.bytesOut = static_cast<long long*>(_ctx->arena.alloc(sizeof(long long)));
        it.dstCap = static_cast<long long>(_finalCap);
        it.fixedBytes = -1;
        it.sparseByte = static_cast<unsigned int>(sbits & 0xFF);
        it.swizzleKey = swzNext ? static_cast<int>(static_cast<uint32_t>(_next->i0) % 6u) : -1;
        it.err = _ctx->errWord;
        it.countsReady = 0;
        int64_t total = 0;
        if (x.hasAux) {
            for (int64_t n : x.aux) total += roundUp(n * eb, kWeightSetAlign);
            it.fixedBytes = total;
            const int64_t written = swzNext ? roundUp(total, kSwizzleSizeAlign) : total;
            if (static_cast<size_t>(written) > _finalCap) throw Capacity("output buffer too small");
            _finalBytes = static_cast<size_t>(written);
        } else {
            _deferredBytes = it.bytesOut;
            _finalBytes = 0;
        }
        launchSparseItem(_ctx, it);
        const TensorType outType = withShapeAndElem(_s.type, {total, 1, 1, 1}, B200C_UI8, QuantInfo());
        View nv;
        nv.src = _finalDst;
        nv.srcBytes = static_cast<size_t>(total);
        nv.srcTag = T_U8;
        setShape(nv, outType.memShape());
        contiguousStrides(nv);
        _s.view = nv;
        _s.type = outType;
        _s.storage = B200C_UI8;
        _s.splat = false;
        if (swzNext) {
            _fusedSwizzle = true;
            _fusedTotal = static_cast<int64_t>(_finalBytes);
        } else {
            _wroteFinal = true;
        }
        return;
    }

    // actual per-channel counts always drive the layout (the running index of sparsify.cpp:137-154);
    // numActualElements only sizes the buffer
    long long* dcounts = static_cast<long long*>(_ctx->arena.alloc(std::max<int64_t>(oc, 1) * sizeof(long long)));
    long long* doffsets = static_cast<long long*>(_ctx->arena.alloc((std::max<int64_t>(oc, 1) + 1) * sizeof(long long)));
    if (oc > 0) {
        launchCountNonSparse(_ctx, dense, tag, oc, work, sbits, dcounts);
        launchSparsifyOffsets(_ctx, dcounts, oc, eb, doffsets, doffsets + oc);
    }
    int64_t total = 0;
    if (x.hasAux) {
        for (int64_t n : x.aux) total += roundUp(n * eb, kWeightSetAlign);
    } else if (oc > 0) {
        long long t = 0;
        copyD2H(_ctx, &t, doffsets + oc, sizeof(long long));
        syncStream(_ctx);
        checkDeviceError(_ctx);
        total = t;
    }
    const TensorType outType = withShapeAndElem(_s.type, {total, 1, 1, 1}, B200C_UI8, QuantInfo());
    void* dst = _ctx->arena.alloc(total ? static_cast<size_t>(total) : 1);
    if (total) fillBytes(_ctx, dst, 0, static_cast<size_t>(total));
    if (oc > 0 && work > 0) {
        launchSparsifyScatter(_ctx, dense, tag, oc, work, sbits, doffsets, dst, total, -1, _ctx->errWord);
    }
    View nv;
    nv.src = dst;
    nv.srcBytes = static_cast<size_t>(total);
    nv.srcTag = T_U8;
    setShape(nv, outType.memShape());
    contiguousStrides(nv);
    _s.view = nv;
    _s.type = outType;
    _s.storage = B200C_UI8;
    _s.splat = false;
}

// ---------------------------------------------------------------------------- SubView on i1
void Planner::subviewBits(const Transformation& x, const TensorType& outType) {  // subview.cpp:145-174
    View& v = _s.view;
    if (_s.splat) {  // splat: the single stored byte is copied (subview.cpp:130-131)
        _s.type = outType;
        setShape(v, outType.memShape());
        return;
    }
    const auto off = _s.type.memOrder(x.a);
    const auto inShape = _s.type.memShape();
    const auto shape = outType.memShape();
    long long inStride[kMaxDims], outShape[kMaxDims];
    long long s = 1, base = 0;
    const int r = _s.type.rank();
    for (int k = r - 1; k >= 0; --k) {
        inStride[k] = s;
        s *= inShape[k];
    }
    for (int k = 0; k < r; ++k) {
        base += off[k] * inStride[k];
        outShape[k] = shape[k];
    }
    const int64_t outBits = outType.count();
    const size_t bytes = static_cast<size_t>((outBits + 7) / 8);
    void* dst = _ctx->arena.alloc(bytes ? bytes : 1);
    if (outBits > 0) launchSubViewBits(_ctx, v.src, dst, r, outShape, inStride, base, outBits);
    View nv;
    nv.src = dst;
    nv.srcBytes = bytes;
    nv.srcTag = T_NONE;
    setShape(nv, shape);
    contiguousStrides(nv);
    _s.view = nv;
    _s.type = outType;
}

// ---------------------------------------------------------------------------- copy-out
// Content::copyTo into `dst` (device) of `cap` bytes, optionally through the swizzle address map
// with the buffer grown to `totalBytes` (SwizzleConstant, swizzle_transform.cpp:154-196).
// Returns the number of bytes written.
size_t Planner::emitCopyTo(void* dst, size_t cap, int swizzleKey, int64_t totalBytes) {
    const TensorType& t = _s.type;
    const int lbits = t.bits();
    const int64_t n = t.count();
    const int64_t alloc = t.allocBytes();
    const int64_t target = totalBytes > 0 ? totalBytes : alloc;
    View& v = _s.view;

    auto tail = [&](int64_t dataBytes, int tailByte) {
        if (target > dataBytes) {
            // the tail is zero (or the splat byte); swizzling only moves chunks inside 512-byte
            // blocks, so the tail bytes land inside [align_down(dataBytes, 512), target)
            (void)tailByte;
        }
    };
    (void)tail;

    if (lbits < 8) {  // copySubByteContent (CU/content.cpp:129-182)
        if (static_cast<size_t>(target) > cap) throw Capacity("output buffer too small");
        if (_s.splat) {
            // byte = the first storage byte replicated into every field
            unsigned char first = 0;
            materialize();
            copyD2H(_ctx, &first, v.src, 1);
            syncStream(_ctx);
            checkDeviceError(_ctx);
            char sub = static_cast<char>(first);
            if (dtBits(_s.storage) == 1) sub &= 1;
            unsigned char byte = 0;
            for (int i = 0; i < 8 / lbits; ++i) byte = static_cast<unsigned char>((byte << lbits) + sub);
            if (swizzleKey >= 0) {
                // SwizzleConstant on a sub-byte splat is handled by swizzle(); not reached
                throw NotBuilt("swizzled copy of a sub-byte splat");
            }
            fillBytes(_ctx, dst, byte, static_cast<size_t>(alloc));
            return static_cast<size_t>(alloc);
        }
        const int64_t storageBytes =
                _afterBitPack      ? n / 2
                : _s.rawBytes >= 0 ? static_cast<int64_t>(_s.rawBytes)
                                   : (static_cast<int64_t>(dtBits(_s.storage)) * n + 7) / 8;
        if (_afterBitPack) {
            // BitPack output: u8 storage of n/2 bytes, same size as the logical type -> memcpy branch
            if (tryFusedRowQuant(dst, 1, T_U8, -1, n / 2, n / 2)) return static_cast<size_t>(n / 2);
            GenParams p = paramsFor(v);
            p.dst = dst;
            p.outMode = OUT_BITPACK4;
            p.packBits = 4;
            p.outElems = n;
            p.outUnits = n / 2;
            p.dataBytes = p.totalBytes = n / 2;
            if (p.outUnits) runGeneric(p);
            return static_cast<size_t>(n / 2);
        }
        if (alloc < storageBytes) {
            if (alloc == 0 || storageBytes % alloc != 0) {
                refThrow("Cannot pack sub-byte elements into buffer: source data size '%lld', target data size '%lld'",
                         static_cast<long long>(storageBytes), static_cast<long long>(alloc));
            }
            const int64_t perByte = n / alloc;
            if (!(perByte >= 1 && perByte <= 8 && (perByte & (perByte - 1)) == 0)) {
                refThrow("Invalid number of elements per byte '%lld'", static_cast<long long>(perByte));
            }
            if (dtBits(_s.storage) < 8) refThrow("Unsupported storage type of size '%d' bits.", dtBits(_s.storage));
            GenParams p = paramsFor(v);
            p.dst = dst;
            p.outMode = OUT_PACK_MSB;
            p.packBits = static_cast<int>(8 / perByte);
            p.outElems = n;
            p.outUnits = alloc;
            p.dataBytes = p.totalBytes = alloc;
            runGeneric(p);
            return static_cast<size_t>(alloc);
        }
        // same size (or bit-packed storage): plain memcpy of the storage bytes
        if (storageBytes) copyD2D(_ctx, dst, v.src, static_cast<size_t>(storageBytes));
        return static_cast<size_t>(storageBytes);
    }

    // byte-sized logical types
    const bool trivial = !t.quantized() && t.dtype == _s.storage;
    GenParams p = paramsFor(v);
    p.dst = dst;
    p.swizzleKey = _s.splat ? -1 : swizzleKey;
    if (!_s.splat && trivial) {
        p.outMode = OUT_RAW;
        p.outTag = curTag();
    } else {
        p.outMode = OUT_CAST;
        p.outTag = tagOfLogical(t);
    }
    const int64_t dataBytes = n * tagBytes(p.outTag);
    if (static_cast<size_t>(std::max(target, dataBytes)) > cap) throw Capacity("output buffer too small");
    p.outElems = p.outUnits = n;
    p.dataBytes = dataBytes;
    p.totalBytes = std::max(target, dataBytes);
    if (_s.splat && totalBytes > 0) {
        // swizzled splat: no swizzle, tail padded with the first output byte (swizzle_transform.cpp:170-188)
        p.totalBytes = dataBytes;
        if (n > 0) runGeneric(p);
        if (target > dataBytes) {
            unsigned char first = 0;
            if (n > 0) {
                copyD2H(_ctx, &first, dst, 1);
                syncStream(_ctx);
                checkDeviceError(_ctx);
            }
            fillBytes(_ctx, static_cast<char*>(dst) + dataBytes, first, static_cast<size_t>(target - dataBytes));
        }
        return static_cast<size_t>(target);
    }
    if (p.totalBytes > 0 && p.outMode == OUT_RAW && isPlain(v)) {
        // nothing to compute: a device copy, or the chunk-rotating copy when swizzled.  Inside a batched
        // fold, small pass-through constants and swizzle-only chains join the one tile launch instead of
        // paying a copy call each.
        if (_ctx->batching && _emittingFinal && dataBytes <= (16ll << 20) && n > 0) {
            runGeneric(p);
        } else if (p.swizzleKey < 0) {
            copyD2D(_ctx, dst, v.src, static_cast<size_t>(dataBytes));
            if (p.totalBytes > dataBytes) {
                fillBytes(_ctx, static_cast<char*>(dst) + dataBytes, 0, static_cast<size_t>(p.totalBytes - dataBytes));
            }
        } else {
            launchSwizzleCopy(_ctx, v.src, dataBytes, dst, p.totalBytes, p.swizzleKey, 0);
        }
        return static_cast<size_t>(p.totalBytes);
    }
    if (p.totalBytes > 0) {
        if (p.outMode == OUT_CAST && n > 0 &&
            tryFusedRowQuant(dst, 0, p.outTag, p.swizzleKey, p.dataBytes, p.totalBytes)) {
            return static_cast<size_t>(p.totalBytes);
        }
        runGeneric(p);
    }
    return static_cast<size_t>(p.totalBytes);
}

// ---------------------------------------------------------------------------- SwizzleConstant
void Planner::swizzle(const Transformation& x, const TensorType& outType) {  // swizzle_transform.cpp:202-239
    const int key = static_cast<int>(static_cast<uint32_t>(x.i0) % 6u);  // setStaggerBits: bits % (MAX_SWIZZLE_KEY + 1)
    if (_fusedSwizzle) {  // the producing kernel already wrote the rotated bytes into the caller's buffer
        _fusedSwizzle = false;
        const int keep = _s.type.bits() == 1 ? _s.storage : outType.dtype;
        View nv;
        nv.src = _finalDst;
        nv.srcBytes = static_cast<size_t>(_fusedTotal);
        nv.srcTag = dtBits(keep) >= 8 ? tagOfStorage(keep) : static_cast<int>(T_NONE);
        setShape(nv, outType.memShape());
        contiguousStrides(nv);
        _s.view = nv;
        _s.type = outType;
        _s.storage = keep;
        _s.splat = false;
        _wroteFinal = true;
        _finalBytes = static_cast<size_t>(_fusedTotal);
        return;
    }
    const int64_t total = roundUp(_s.type.allocBytes(), kSwizzleSizeAlign);
    void* dst = nullptr;
    const bool direct = _finalDst != nullptr && _isLast;
    if (direct) {
        if (static_cast<size_t>(total) > _finalCap) throw Capacity("output buffer too small");
        dst = _finalDst;
    } else {
        dst = _ctx->arena.alloc(total ? static_cast<size_t>(total) : 1);
    }

    if (_s.type.bits() == 1) {
        // i1: the packed bits are swizzled as bytes; a splat `true` becomes 0xFF (:212-238)
        if (_s.type.count() % 8 != 0) refThrow("Elements cannot be packed in bytes");
        const int64_t packed = _s.type.count() / 8;
        if (_s.splat) {
            unsigned char first = 0;
            copyD2H(_ctx, &first, _s.view.src, 1);
            syncStream(_ctx);
            const unsigned char byte = first == 1 ? 0xFF : first;
            if (total) fillBytes(_ctx, dst, byte, static_cast<size_t>(total));
        } else {
            if (dtBits(_s.storage) != 1) throw NotBuilt("SwizzleConstant of i1 content held one element per byte");
            if (total) launchSwizzleCopy(_ctx, _s.view.src, packed, dst, total, key, 0);
        }
    } else {
        _emittingFinal = direct;
        emitCopyTo(dst, static_cast<size_t>(total), key, total);
        _emittingFinal = false;
    }
    const int keepStorage = _s.type.bits() == 1 ? _s.storage : outType.dtype;
    View nv;
    nv.src = dst;
    nv.srcBytes = static_cast<size_t>(total);
    nv.srcTag = dtBits(keepStorage) >= 8 ? tagOfStorage(keepStorage) : static_cast<int>(T_NONE);
    setShape(nv, outType.memShape());
    contiguousStrides(nv);
    _s.view = nv;
    _s.type = outType;
    _s.storage = keepStorage;
    _s.splat = false;
    _wroteFinal = direct;
    _finalBytes = static_cast<size_t>(total);
}

// ---------------------------------------------------------------------------- driver
size_t Planner::run(const std::vector<Transformation>& chain, void* dst, size_t cap) {
    _finalDst = dst;
    _finalCap = cap;
    for (size_t i = 0; i < chain.size(); ++i) {
        _isLast = (i + 1 == chain.size());
        _next = _isLast ? nullptr : &chain[i + 1];
        _nextIsLast = (i + 2 == chain.size());
        _wroteFinal = false;
        apply(chain[i]);
    }
    _next = nullptr;
    if (_wroteFinal) return _finalBytes;
    const size_t need = static_cast<size_t>(_s.type.allocBytes());
    if (need > cap) throw Capacity("output buffer too small: need " + std::to_string(need) + " bytes");
    _emittingFinal = true;
    const size_t wrote = emitCopyTo(dst, cap, -1, 0);
    _emittingFinal = false;
    return wrote;
}

void Planner::runNoCopy(const std::vector<Transformation>& chain) {
    _finalDst = nullptr;
    _finalCap = 0;
    for (size_t i = 0; i < chain.size(); ++i) {
        _isLast = false;
        apply(chain[i]);
    }
}

}  // namespace b200c
