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
#include <cstddef>
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


// swizzled position of byte address a (16-byte chunks move inside 512-byte blocks, the low 4 bits stay)
__device__ __forceinline__ long long swz(long long a, int key) {
    return swizzleAddr(a, key);
}

// fast == 1: the tile is a run of nx elements contiguous in source and output; bytes are copied as they are
__device__ __forceinline__ void copyTile(const GenParams& g, long long srcElem, long long outElem, int nx, int es) {
    const unsigned char* src = static_cast<const unsigned char*>(g.src) + srcElem * es;
    unsigned char* dst = static_cast<unsigned char*>(g.dst);
    const long long outByte = outElem * es;
    const long long bytes = static_cast<long long>(nx) * es;
    const bool vec = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | static_cast<uintptr_t>(outByte)) & 15) == 0;
    const long long nvec = vec ? bytes / 16 : 0;
    for (long long v0 = threadIdx.x; v0 < nvec; v0 += 4 * kTileThreads) {  // four loads in flight per thread
        uint4 x[4];
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (v0 + r * kTileThreads < nvec) x[r] = __ldg(reinterpret_cast<const uint4*>(src) + v0 + r * kTileThreads);
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (v0 + r * kTileThreads < nvec)
                *reinterpret_cast<uint4*>(dst + swz(outByte + (v0 + r * kTileThreads) * 16, g.swizzleKey)) = x[r];
    }
    for (long long b = nvec * 16 + threadIdx.x; b < bytes; b += kTileThreads) dst[swz(outByte + b, g.swizzleKey)] = src[b];
}

// byte i of a register array of 32-bit words, i known at compile time
#define B2_SEL(i_) ((i_) & 3)
template <int YI>
__device__ __forceinline__ uint4 gather9(const unsigned int (&w)[36]) {
    // output bytes k = 0..15 are source bytes k * 9 + YI of the thread's 144-byte span
    unsigned int o[4];
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        const int i0 = (4 * m + 0) * 9 + YI, i1 = (4 * m + 1) * 9 + YI, i2 = (4 * m + 2) * 9 + YI, i3 = (4 * m + 3) * 9 + YI;
        const unsigned int lo = __byte_perm(w[i0 >> 2], w[i1 >> 2], B2_SEL(i0) | ((4 + B2_SEL(i1)) << 4));
        const unsigned int hi = __byte_perm(w[i2 >> 2], w[i3 >> 2], B2_SEL(i2) | ((4 + B2_SEL(i3)) << 4));
        o[m] = __byte_perm(lo, hi, 0x5410);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}
#undef B2_SEL

// fast == 2: nz blocks of [nx][ny] elements, contiguous in the source, become nz blocks of [ny][nx].
// The source span is staged linearly (128-bit loads where aligned), the output is written in 32-bit
// or 128-bit pieces along x.
__device__ __forceinline__ void transposeTile(const GenParams& g, long long srcElem, long long outElem, int nz, int ny, int nx,
                                              long long outStrideY, int es, unsigned char* smem) {
    const unsigned char* src = static_cast<const unsigned char*>(g.src) + srcElem * es;
    unsigned char* dst = static_cast<unsigned char*>(g.dst);
    const int block = nx * ny;  // elements of one block; also the output stride between blocks
    const int bytes = nz * block * es;
    const int phase = static_cast<int>(reinterpret_cast<uintptr_t>(src) & 15);
    {
        const int head = min(bytes, (16 - phase) & 15);
        const int nvec = (bytes - head) / 16;
        const int tailAt = head + nvec * 16;
        if (threadIdx.x < head) smem[phase + threadIdx.x] = src[threadIdx.x];
        const uint4* s4 = reinterpret_cast<const uint4*>(src + head);
        uint4* d4 = reinterpret_cast<uint4*>(smem + phase + head);
        for (int v0 = threadIdx.x; v0 < nvec; v0 += 4 * kTileThreads) {  // four loads in flight per thread
            uint4 x[4];
#pragma unroll
            for (int r = 0; r < 4; ++r)
                if (v0 + r * kTileThreads < nvec) x[r] = __ldg(s4 + v0 + r * kTileThreads);
#pragma unroll
            for (int r = 0; r < 4; ++r)
                if (v0 + r * kTileThreads < nvec) d4[v0 + r * kTileThreads] = x[r];
        }
        if (threadIdx.x < bytes - tailAt) smem[phase + tailAt + threadIdx.x] = src[tailAt + threadIdx.x];
    }
    __syncthreads();
    const unsigned char* sm = smem + phase;
    const long long outByte0 = outElem * es;
    const bool dst16 = ((reinterpret_cast<uintptr_t>(dst) | static_cast<uintptr_t>(outByte0)) & 15) == 0;
    if (es == 1 && ny == 9 && phase == 0 && (nx & 15) == 0 && dst16 && (outStrideY & 15) == 0) {
        const int unitsX = nx >> 4;
        const int units = nz * unitsX;
        for (int u = threadIdx.x; u < units; u += kTileThreads) {
            const int zi = u / unitsX, xu = u - zi * unitsX;
            unsigned int w[36];
            const uint4* s4 = reinterpret_cast<const uint4*>(sm + (zi * block + xu * 16 * 9));
#pragma unroll
            for (int i = 0; i < 9; ++i) {
                const uint4 v = s4[i];
                w[4 * i] = v.x;
                w[4 * i + 1] = v.y;
                w[4 * i + 2] = v.z;
                w[4 * i + 3] = v.w;
            }
            const long long o = outByte0 + static_cast<long long>(zi) * block + xu * 16;
            *reinterpret_cast<uint4*>(dst + swz(o + 0 * outStrideY, g.swizzleKey)) = gather9<0>(w);
            *reinterpret_cast<uint4*>(dst + swz(o + 1 * outStrideY, g.swizzleKey)) = gather9<1>(w);
            *reinterpret_cast<uint4*>(dst + swz(o + 2 * outStrideY, g.swizzleKey)) = gather9<2>(w);
            *reinterpret_cast<uint4*>(dst + swz(o + 3 * outStrideY, g.swizzleKey)) = gather9<3>(w);
            *reinterpret_cast<uint4*>(dst + swz(o + 4 * outStrideY, g.swizzleKey)) = gather9<4>(w);
            *reinterpret_cast<uint4*>(dst + swz(o + 5 * outStrideY, g.swizzleKey)) = gather9<5>(w);
            *reinterpret_cast<uint4*>(dst + swz(o + 6 * outStrideY, g.swizzleKey)) = gather9<6>(w);
            *reinterpret_cast<uint4*>(dst + swz(o + 7 * outStrideY, g.swizzleKey)) = gather9<7>(w);
            *reinterpret_cast<uint4*>(dst + swz(o + 8 * outStrideY, g.swizzleKey)) = gather9<8>(w);
        }
        return;
    }
    const int perWord = 4 / es;  // es is 1, 2 or 4 here
    const bool words = ((reinterpret_cast<uintptr_t>(dst) | static_cast<uintptr_t>(outByte0)) & 3) == 0 &&
                       ((outStrideY * es) & 3) == 0 && (nx % perWord) == 0 && ((static_cast<long long>(block) * es) & 3) == 0;
    if (words) {
        const int wordsX = nx / perWord;
        const int perBlock = ny * wordsX;
        const int total = nz * perBlock;
        for (int t = threadIdx.x; t < total; t += kTileThreads) {
            const int zi = t / perBlock, r = t - zi * perBlock;
            const int yi = r / wordsX, xw = r - yi * wordsX;
            const unsigned char* b = sm + (zi * block + xw * perWord * ny + yi) * es;
            unsigned int word;
            if (es == 1) {
                word = b[0] | (static_cast<unsigned int>(b[ny]) << 8) | (static_cast<unsigned int>(b[2 * ny]) << 16) |
                       (static_cast<unsigned int>(b[3 * ny]) << 24);
            } else if (es == 2) {
                word = *reinterpret_cast<const unsigned short*>(b) |
                       (static_cast<unsigned int>(*reinterpret_cast<const unsigned short*>(b + 2 * ny)) << 16);
            } else {
                word = *reinterpret_cast<const unsigned int*>(b);
            }
            const long long o = outByte0 + (static_cast<long long>(zi) * block + yi * outStrideY + xw * perWord) * es;
            *reinterpret_cast<unsigned int*>(dst + swz(o, g.swizzleKey)) = word;
        }
        return;
    }
    const int total = nz * block;
    for (int t = threadIdx.x; t < total; t += kTileThreads) {
        const int zi = t / block, r = t - zi * block;
        const int yi = r / nx, xi = r - yi * nx;
        const unsigned char* b = sm + (zi * block + xi * ny + yi) * es;
        const long long o = outByte0 + (static_cast<long long>(zi) * block + yi * outStrideY + xi) * es;
        for (int k = 0; k < es; ++k) dst[swz(o + k, g.swizzleKey)] = b[k];
    }
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
    int nz = 1;
    for (int k = g.rank - 2; k >= 0; --k) {
        if (k == py) continue;
        const bool blocked = it.fast == 2 && it.tz > 1 && k == g.rank - 3;
        const long long s = blocked ? it.tilesZ : g.shape[k];
        const long long q = rest / s;
        long long c = rest - q * s;
        rest = q;
        if (blocked) {
            c *= it.tz;
            nz = static_cast<int>(min(static_cast<long long>(it.tz), g.shape[k] - c));
        }
        coord[k] = c;
        srcBase += c * g.stride[k];
        outBase += c * it.outStride[k];
    }
    const long long x0 = tX * it.tx, y0 = tY * it.ty;
    const int nx = static_cast<int>(min(static_cast<long long>(it.tx), shapeX - x0));
    const int ny = static_cast<int>(min(static_cast<long long>(it.ty), shapeY - y0));
    const int es = it.esIn;
    if (it.fast) {
        if (it.fast == 1) {
            copyTile(g, srcBase + x0, outBase + x0, nx, es);
        } else {
            transposeTile(g, srcBase + x0 * sx, outBase + x0, nz, ny, nx, it.outStride[py], es, smem);
        }
        if (tile == 0) {
            for (long long a = g.dataBytes + threadIdx.x; a < g.totalBytes; a += kTileThreads) {
                static_cast<unsigned char*>(g.dst)[swizzleAddr(a, g.swizzleKey)] = 0;
            }
        }
        return;
    }
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

__global__ void __launch_bounds__(kTileThreads, 5) foldTileBatchKernel(const TileRef* __restrict__ refs,
                                                                    const long long* __restrict__ tileStart, int nitems) {
    __shared__ __align__(16) unsigned char smem[kTileSmemBytes];
    __shared__ TileItem it;
    const long long b = blockIdx.x;
    const int lo = findBatchItem(tileStart, nitems, b);
    const TileRef ref = refs[lo];
    {
        // the shared template, with this item's own buffers put in place of the template's
        constexpr int words = sizeof(TileItem) / 4;
        constexpr int srcWord = offsetof(TileItem, g.src) / 4, dstWord = offsetof(TileItem, g.dst) / 4;
        const unsigned long long srcBits = reinterpret_cast<unsigned long long>(ref.src);
        const unsigned long long dstBits = reinterpret_cast<unsigned long long>(ref.dst);
        const unsigned int* s = reinterpret_cast<const unsigned int*>(ref.templ);
        unsigned int* d = reinterpret_cast<unsigned int*>(&it);
        for (int i = threadIdx.x; i < words; i += kTileThreads) {
            unsigned int v = __ldg(s + i);
            if (i == srcWord) v = static_cast<unsigned int>(srcBits);
            if (i == srcWord + 1) v = static_cast<unsigned int>(srcBits >> 32);
            if (i == dstWord) v = static_cast<unsigned int>(dstBits);
            if (i == dstWord + 1) v = static_cast<unsigned int>(dstBits >> 32);
            d[i] = v;
        }
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
    // views that only move bytes take the vectorised bodies
    const bool raw = g.nOps == 0 && g.nBoxes == 0 && (g.outMode == OUT_RAW || g.outTag == g.srcTag) &&
                     tagBytes(g.outTag) == it.esIn;
    it.fast = 0;
    it.tz = 1;
    it.tilesZ = 1;
    if (raw && it.py < 0 && g.stride[px] == 1) {
        it.fast = 1;
        it.tx = static_cast<int>(std::min<long long>(g.shape[px], 16384 / it.esIn));
    } else if (raw && it.py >= 0 && it.esIn <= 4 && g.stride[px] == g.shape[it.py] &&
               g.shape[it.py] * it.esIn * 16 <= kTileSmemBytes - 16) {
        it.fast = 2;
        const long long ny = g.shape[it.py];
        it.ty = static_cast<int>(ny);
        const long long room = (kTileSmemBytes - 16) / (ny * it.esIn);  // x extent that fits the staging buffer
        it.tx = static_cast<int>(std::min<long long>(g.shape[px], std::max<long long>(16, room / 16 * 16)));
        if (it.tx == g.shape[px] && it.py == g.rank - 2 && g.rank >= 3 && g.stride[g.rank - 3] == g.shape[px] * ny) {
            it.tz = static_cast<int>(std::max<long long>(1, std::min<long long>(g.shape[g.rank - 3], room / g.shape[px])));
            it.tilesZ = (g.shape[g.rank - 3] + it.tz - 1) / it.tz;
        }
    }
    it.tilesX = (g.shape[px] + it.tx - 1) / it.tx;
    it.tilesY = it.py >= 0 ? (g.shape[it.py] + it.ty - 1) / it.ty : 1;
    long long outer = 1;
    for (int k = 0; k < g.rank - 1; ++k)
        if (k != it.py) outer *= (it.tz > 1 && k == g.rank - 3) ? it.tilesZ : g.shape[k];
    it.tiles = it.tilesX * it.tilesY * outer;
    if (it.tiles <= 0 || it.tiles > 0x7FFFFFFFLL) return false;
    *out = it;
    return true;
}

void launchTile(Context* ctx, const TileItem& it) {
    if (ctx->batching) {
        if (ctx->tileSlabs.empty() || ctx->tileSlabs.back().host.size() >= static_cast<size_t>(TileSlab::kCapacity)) {
            TileSlab slab;
            slab.dev = static_cast<TileItem*>(ctx->arena.alloc(sizeof(TileItem) * TileSlab::kCapacity));
            slab.host.reserve(TileSlab::kCapacity);
            ctx->tileSlabs.push_back(std::move(slab));
        }
        TileSlab& slab = ctx->tileSlabs.back();
        TileRef ref;
        ref.templ = slab.dev + slab.host.size();
        ref.src = it.g.src;
        ref.dst = it.g.dst;
        ref.tiles = it.tiles;
        slab.host.push_back(it);
        ctx->tileBatch.push_back(ref);
        ctx->queuedBytes += it.g.outElems * it.esIn;
        return;
    }
    const int grid = static_cast<int>(std::min<long long>(it.tiles, ctx->smCount * 64LL));
    foldTileKernel<<<grid, kTileThreads, 0, ctx->stream>>>(it);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
}

void uploadTileTemplates(Context* ctx, Context* from) {
    for (TileSlab& slab : from->tileSlabs) {
        if (slab.uploaded < slab.host.size()) {
            uploadSmall(ctx, slab.dev + slab.uploaded, slab.host.data() + slab.uploaded,
                        sizeof(TileItem) * (slab.host.size() - slab.uploaded));
            slab.uploaded = slab.host.size();
        }
    }
}

void flushTileBatch(Context* ctx) {
    uploadTileTemplates(ctx, ctx);
    std::vector<TileRef> pending;
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
        TileRef* refsDev = static_cast<TileRef*>(ctx->arena.alloc(sizeof(TileRef) * n));
        appendCoarseIndex(start, total);
        long long* startDev = static_cast<long long*>(ctx->arena.alloc(sizeof(long long) * start.size()));
        uploadSmall(ctx, refsDev, pending.data() + first, sizeof(TileRef) * n);
        uploadSmall(ctx, startDev, start.data(), sizeof(long long) * start.size());
        foldTileBatchKernel<<<static_cast<unsigned int>(total), kTileThreads, 0, ctx->stream>>>(refsDev, startDev, n);
        B2_CUDA(cudaGetLastError());
        ++ctx->launches;
        first = last;
    }
}

}  // namespace b200c
