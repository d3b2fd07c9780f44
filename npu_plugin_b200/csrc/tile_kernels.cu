// Tiled form of the fused fold pass, used for every view the generic element kernel would serve
// with byte-sized outputs.  The view is first put into a canonical form (unit dims dropped, dims
// that are contiguous in both source and output merged).  A tile spans the innermost output dim
// (x) and, when the view is a transpose, the output dim whose source stride is 1 (y): the tile is
// read along y with coalesced loads into shared memory and written along x with coalesced stores,
// so reorders such as OIYX -> OYXI move through HBM at full sector efficiency in both directions.
// Fill boxes (PadWithZero), the value program, the final checked cast and the swizzle address
// rotation are applied on the way out, exactly as in the generic kernel (view.h).
//
// Many tensors share one launch: in batch mode tiles of all queued items form one grid, and a CTA
// finds its item with a binary search over the prefix sums of the tile counts.
#include "runtime.h"

#include <algorithm>
#include <cstring>

namespace b200c {

constexpr int kTileSmemBytes = 20480;
constexpr int kTileThreads = 256;

B2_HD bool insideBoxes(const GenParams& g, const long long* coord, int* hit) {
    for (int b = g.nBoxes - 1; b >= 0; --b) {
        bool inside = true;
        for (int k = 0; k < g.rank; ++k) inside = inside && coord[k] >= g.box[b].lo[k] && coord[k] < g.box[b].hi[k];
        if (!inside) {
            *hit = b;
            return false;
        }
    }
    return true;
}

__device__ __forceinline__ void tileBody(const TileItem& it, long long tile, unsigned char* smem) {
    const GenParams& g = it.g;
    const int px = g.rank - 1, py = it.py;
    const long long shapeX = g.shape[px], sx = g.stride[px];
    const long long shapeY = py >= 0 ? g.shape[py] : 1;
    const long long tX = tile % it.tilesX;
    long long rest = tile / it.tilesX;
    const long long tY = rest % it.tilesY;
    rest /= it.tilesY;
    // outer coordinates (all dims but x and y), source and output offsets of the tile origin
    long long coord[kMaxDims];
    long long srcBase = g.base, outBase = 0;
    for (int k = g.rank - 2; k >= 0; --k) {
        if (k == py) continue;
        const long long s = g.shape[k];
        const long long q = rest / s;
        const long long c = rest - q * s;
        rest = q;
        coord[k] = c;
        srcBase += c * g.stride[k];
        outBase += c * it.outStride[k];
    }
    const long long x0 = tX * it.tx, y0 = tY * it.ty;
    const int nx = static_cast<int>(min(static_cast<long long>(it.tx), shapeX - x0));
    const int ny = static_cast<int>(min(static_cast<long long>(it.ty), shapeY - y0));
    const int es = it.esIn;
    const int pitch = it.ty * es + 4;
    const bool simple = g.nBoxes == 0 && !it.needCoords;
    int err = E_NONE;

    if (py >= 0) {  // stage the tile: consecutive threads walk the source-contiguous direction
        const long long tileSrc = srcBase + y0 + x0 * sx;
        for (int t = threadIdx.x; t < nx * ny; t += kTileThreads) {
            const int yi = t % ny, xi = t / ny;
            bool load = true;
            if (!simple && g.nBoxes) {
                coord[px] = x0 + xi;
                coord[py] = y0 + yi;
                int hit;
                load = insideBoxes(g, coord, &hit);
            }
            if (load) {
                const long long off = tileSrc + yi + xi * sx;
                unsigned char* d = smem + xi * pitch + yi * es;
                switch (es) {
                case 1:
                    *d = static_cast<const unsigned char*>(g.src)[off];
                    break;
                case 2:
                    *reinterpret_cast<unsigned short*>(d) = static_cast<const unsigned short*>(g.src)[off];
                    break;
                case 4:
                    *reinterpret_cast<unsigned int*>(d) = static_cast<const unsigned int*>(g.src)[off];
                    break;
                default: {
                    const unsigned long long v = static_cast<const unsigned long long*>(g.src)[off];
                    reinterpret_cast<unsigned int*>(d)[0] = static_cast<unsigned int>(v);
                    reinterpret_cast<unsigned int*>(d)[1] = static_cast<unsigned int>(v >> 32);
                    break;
                }
                }
            }
        }
        __syncthreads();
    }

    const int outBytes = tagBytes(g.outTag);
    for (int t = threadIdx.x; t < nx * ny; t += kTileThreads) {
        const int xi = t % nx, yi = t / nx;
        Val v;
        int start = 0;
        bool fromSource = true;
        if (!simple) {
            coord[px] = x0 + xi;
            if (py >= 0) coord[py] = y0 + yi;
            int hit = -1;
            if (g.nBoxes && !insideBoxes(g, coord, &hit)) {
                const FillBox& fb = g.box[hit];
                v.tag = fb.tag;
                v.bits = fb.table ? loadRaw(fb.table, coord[fb.tableDim] + fb.tableOff, fb.tag) : fb.bits;
                start = fb.pos;
                fromSource = false;
            }
        }
        if (fromSource) {
            v.tag = g.srcTag;
            if (py >= 0) {
                const unsigned char* s = smem + xi * pitch + yi * es;
                switch (es) {
                case 1:
                    v.bits = *s;
                    break;
                case 2:
                    v.bits = *reinterpret_cast<const unsigned short*>(s);
                    break;
                case 4:
                    v.bits = *reinterpret_cast<const unsigned int*>(s);
                    break;
                default:
                    v.bits = reinterpret_cast<const unsigned int*>(s)[0] |
                             (static_cast<unsigned long long>(reinterpret_cast<const unsigned int*>(s)[1]) << 32);
                    break;
                }
            } else {
                v.bits = loadRaw(g.src, srcBase + (x0 + xi) * sx, g.srcTag);
            }
        }
        for (int i = start; i < g.nOps; ++i) v = applyOp(g.ops[i], v, coord, err);
        unsigned long long bits = v.bits;
        if (g.outMode == OUT_CAST) bits = castChecked(v, g.outTag, err);
        const long long outIdx = outBase + (py >= 0 ? (y0 + yi) * it.outStride[py] : 0) + x0 + xi;
        storeRawAt(g.dst, swizzleAddr(outIdx * outBytes, g.swizzleKey), outBytes, bits);
    }
    if (err != E_NONE) atomicCAS(g.err, E_NONE, err);
    // zero tail up to the swizzle size alignment, by the item's first tile
    if (tile == 0) {
        for (long long a = g.dataBytes + threadIdx.x; a < g.totalBytes; a += kTileThreads) {
            static_cast<unsigned char*>(g.dst)[swizzleAddr(a, g.swizzleKey)] = 0;
        }
    }
}

__global__ void __launch_bounds__(kTileThreads) foldTileKernel(const __grid_constant__ TileItem it) {
    __shared__ __align__(16) unsigned char smem[kTileSmemBytes];
    for (long long tile = blockIdx.x; tile < it.tiles; tile += gridDim.x) {
        tileBody(it, tile, smem);
        __syncthreads();
    }
}

__global__ void __launch_bounds__(kTileThreads) foldTileBatchKernel(const TileItem* __restrict__ items,
                                                                    const long long* __restrict__ tileStart, int nitems) {
    __shared__ __align__(16) unsigned char smem[kTileSmemBytes];
    __shared__ TileItem it;
    int lo = 0, hi = nitems - 1;
    const long long b = blockIdx.x;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (tileStart[mid] <= b) {
            lo = mid;
        } else {
            hi = mid - 1;
        }
    }
    {
        const int words = sizeof(TileItem) / 4;
        const unsigned int* s = reinterpret_cast<const unsigned int*>(items + lo);
        unsigned int* d = reinterpret_cast<unsigned int*>(&it);
        for (int i = threadIdx.x; i < words; i += kTileThreads) d[i] = s[i];
    }
    __syncthreads();
    tileBody(it, b - tileStart[lo], smem);
}

// ---------------------------------------------------------------------------- host side
// Canonical form: drop unit dims; merge neighbours that are contiguous in the source as well and
// are not singled out by a fill box, a per-axis operation or a per-channel fill table.
static void canonicalize(GenParams& g) {
    auto referenced = [&](int k) {
        for (int i = 0; i < g.nOps; ++i)
            if (g.ops[i].dim == k) return true;
        for (int b = 0; b < g.nBoxes; ++b)
            if (g.box[b].table && g.box[b].tableDim == k) return true;
        return false;
    };
    auto boxFree = [&](int k) {
        for (int b = 0; b < g.nBoxes; ++b)
            if (g.box[b].lo[k] > 0 || g.box[b].hi[k] < g.shape[k]) return false;
        return true;
    };
    auto removeDim = [&](int k) {
        for (int j = k; j + 1 < g.rank; ++j) {
            g.shape[j] = g.shape[j + 1];
            g.stride[j] = g.stride[j + 1];
            for (int b = 0; b < g.nBoxes; ++b) {
                g.box[b].lo[j] = g.box[b].lo[j + 1];
                g.box[b].hi[j] = g.box[b].hi[j + 1];
            }
        }
        for (int i = 0; i < g.nOps; ++i)
            if (g.ops[i].dim > k) --g.ops[i].dim;
        for (int b = 0; b < g.nBoxes; ++b)
            if (g.box[b].table && g.box[b].tableDim > k) --g.box[b].tableDim;
        --g.rank;
    };
    // unit dims (a unit dim referenced by an op keeps coordinate 0: fold its offset into the op)
    for (int k = g.rank - 1; k >= 0 && g.rank > 1; --k) {
        if (g.shape[k] != 1 || !boxFree(k)) continue;
        if (referenced(k)) continue;
        removeDim(k);
    }
    for (int k = g.rank - 2; k >= 0; --k) {
        if (g.stride[k] == g.stride[k + 1] * g.shape[k + 1] && boxFree(k) && boxFree(k + 1) && !referenced(k) &&
            !referenced(k + 1)) {
            g.shape[k + 1] *= g.shape[k];
            for (int b = 0; b < g.nBoxes; ++b) {
                g.box[b].lo[k + 1] = 0;
                g.box[b].hi[k + 1] = g.shape[k + 1];
            }
            removeDim(k);
        }
    }
}

bool makeTileItem(const GenParams& p, TileItem* out) {
    if (!(p.outMode == OUT_RAW || p.outMode == OUT_CAST)) return false;
    if (p.rank < 1 || p.outElems <= 0) return false;
    TileItem it;
    std::memset(&it, 0, sizeof(it));
    it.g = p;
    canonicalize(it.g);
    GenParams& g = it.g;
    for (int k = 0; k < g.rank; ++k)
        if (g.shape[k] <= 0) return false;
    long long s = 1;
    for (int k = g.rank - 1; k >= 0; --k) {
        it.outStride[k] = s;
        s *= g.shape[k];
    }
    const int px = g.rank - 1;
    it.esIn = tagBytes(g.srcTag);
    it.py = -1;
    if (g.stride[px] != 1) {
        for (int k = g.rank - 2; k >= 0; --k) {
            if (g.stride[k] == 1 && g.shape[k] > 1) {
                it.py = k;
                break;
            }
        }
    }
    it.needCoords = 0;
    for (int i = 0; i < g.nOps; ++i)
        if (g.ops[i].dim >= 0) it.needCoords = 1;
    if (it.py >= 0) {
        const long long maxElems = it.esIn == 8 ? 2048 : 4096;
        it.ty = static_cast<int>(std::min<long long>(g.shape[it.py], 64));
        it.tx = static_cast<int>(std::min<long long>(g.shape[px], std::max<long long>(1, maxElems / it.ty)));
        while (static_cast<long long>(it.tx) * (it.ty * it.esIn + 4) > kTileSmemBytes && it.tx > 1) it.tx /= 2;
    } else {
        it.ty = 1;
        it.tx = static_cast<int>(std::min<long long>(g.shape[px], 2048));
    }
    it.tilesX = (g.shape[px] + it.tx - 1) / it.tx;
    it.tilesY = it.py >= 0 ? (g.shape[it.py] + it.ty - 1) / it.ty : 1;
    long long outer = 1;
    for (int k = 0; k < g.rank - 1; ++k)
        if (k != it.py) outer *= g.shape[k];
    it.tiles = it.tilesX * it.tilesY * outer;
    if (it.tiles <= 0 || it.tiles > 0x7FFFFFFFLL) return false;
    *out = it;
    return true;
}

void launchTile(Context* ctx, const TileItem& it) {
    if (ctx->batching) {
        ctx->tileBatch.push_back(it);
        return;
    }
    const int grid = static_cast<int>(std::min<long long>(it.tiles, ctx->smCount * 64LL));
    foldTileKernel<<<grid, kTileThreads, 0, ctx->stream>>>(it);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
}

void flushTileBatch(Context* ctx) {
    std::vector<TileItem> pending;
    pending.swap(ctx->tileBatch);
    size_t first = 0;
    while (first < pending.size()) {
        std::vector<long long> start;
        long long total = 0;
        size_t last = first;
        while (last < pending.size() && total + pending[last].tiles <= 0x7FFFFFFFLL) {
            start.push_back(total);
            total += pending[last].tiles;
            ++last;
        }
        const int n = static_cast<int>(last - first);
        if (n == 1) {
            const bool was = ctx->batching;
            ctx->batching = false;
            launchTile(ctx, pending[first]);
            ctx->batching = was;
        } else {
            TileItem* itemsDev = static_cast<TileItem*>(ctx->arena.alloc(sizeof(TileItem) * n));
            long long* startDev = static_cast<long long*>(ctx->arena.alloc(sizeof(long long) * n));
            copyH2D(ctx, itemsDev, pending.data() + first, sizeof(TileItem) * n);
            copyH2D(ctx, startDev, start.data(), sizeof(long long) * n);
            foldTileBatchKernel<<<static_cast<unsigned int>(total), kTileThreads, 0, ctx->stream>>>(itemsDev, startDev, n);
            B2_CUDA(cudaGetLastError());
            ++ctx->launches;
        }
        first = last;
    }
}

}  // namespace b200c
