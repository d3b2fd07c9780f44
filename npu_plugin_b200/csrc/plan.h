// Fold planner interface; see plan.cu.
#pragma once

#include "runtime.h"

#include <vector>

namespace b200c {

// Host-side form of a view (GenParams with growable lists).
struct View {
    const void* src = nullptr;  // device pointer
    size_t srcBytes = 0;
    int srcTag = T_NONE;  // C type of the source elements; T_NONE for bit-packed storage
    int rank = 0;
    long long shape[kMaxDims] = {0};
    long long stride[kMaxDims] = {0};
    long long base = 0;
    std::vector<FillBox> boxes;
    std::vector<ValueOp> ops;
};

// What Const::Content carries: logical type, storage element type, splat flag, and here the lazy view.
struct ContentState {
    TensorType type;
    int storage = 0;
    bool splat = false;
    View view;
    // Bytes the storage really holds when a shape-and-element-type change left fewer storage elements
    // than the logical type counts (packed sub-byte bytes kept as ui8); -1: count * storage element size.
    // Content::copySubByteContent compares this size, not the element count, with the target's.
    long long rawBytes = -1;
};

struct SideOutput {
    const void* dev;
    void* user;
    size_t bytes;
};

int tagOfStorage(int dtype);

class Planner {
public:
    Planner(Context* ctx, const TensorType& baseType, const void* devData, size_t nbytes, bool splat);

    // fold + copyTo into dst (device); returns bytes written
    size_t run(const std::vector<Transformation>& chain, void* dst, size_t cap);
    // fold only (for count queries)
    void runNoCopy(const std::vector<Transformation>& chain);
    std::vector<int64_t> countNonSparse();

    // QuantizeSynth side outputs that live on the device are written by the kernels directly
    void setSideOnDevice(bool v) {
        _sideOnDevice = v;
    }
    const ContentState& state() const {
        return _s;
    }
    const std::vector<SideOutput>& sideOutputs() const {
        return _sides;
    }
    // device word holding the size of the final result when only the data decides it (Sparsify
    // without numActualElements written straight to the output); nullptr otherwise
    const long long* deferredBytes() const {
        return _deferredBytes;
    }

private:
    void apply(const Transformation& x);
    void materialize();
    const void* denseAs(int tag);
    GenParams paramsFor(const View& v) const;
    int curTag() const;
    void* uploadTable(const void* host, size_t bytes);
    void needByteStorage(const char* what);
    void quantizeSynth(const Transformation& x, const TensorType& outType);
    void getSparsityMap(const TensorType& outType, int swizzleKey);
    void sparsify(const Transformation& x);
    void subviewBits(const Transformation& x, const TensorType& outType);
    void swizzle(const Transformation& x, const TensorType& outType);
    size_t emitCopyTo(void* dst, size_t cap, int swizzleKey, int64_t totalBytes);
    void runGeneric(const GenParams& p);
    void remapDense(GenParams p, int tag, const TensorType& outType, int storage);
    void flushPendingStats();
    bool tryFusedRowQuant(void* dst, int outMode, int outTag, int swizzleKey, int64_t dataBytes, int64_t totalBytes);

    // QuantizeSynth whose statistics pass has not run yet: if the chain ends in a shape the fused
    // kernel handles, statistics and quantisation happen in one pass over the tensor
    struct PendingStats {
        bool active = false;
        RowStatsParams stats;
        const void* src = nullptr;
        int srcTag = T_NONE;
        int rowDim = 0;
    } _pending;

    Context* _ctx;
    ContentState _s;
    std::vector<SideOutput> _sides;
    bool _afterBitPack = false;
    bool _sideOnDevice = false;
    bool _emittingFinal = false;  // the kernel being issued writes the caller's output and nothing reads it later
    void* _finalDst = nullptr;
    size_t _finalCap = 0;
    bool _isLast = false;
    bool _wroteFinal = false;
    size_t _finalBytes = 0;
    const Transformation* _next = nullptr;  // the transformation after the one being applied
    bool _nextIsLast = false;
    bool _fusedSwizzle = false;  // the producer already wrote the swizzled bytes of the final SwizzleConstant
    int64_t _fusedTotal = 0;
    const long long* _deferredBytes = nullptr;
    bool finalSwizzleFollows() const;
};

}  // namespace b200c
