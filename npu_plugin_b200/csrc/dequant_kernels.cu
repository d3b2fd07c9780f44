// Dequantize of 8-bit storage laid out as contiguous rows: float((q - zp) * double scale), then the
// lazy conversion to the expressed type at copy-out (f32 or f16), as
// src/vpux_compiler/src/dialect/const/attributes/dequantize.cpp:47-94 followed by Content::copyTo.
//
// A row shares one (scale, zero point), so the 256 possible results of a row are computed once --
// with exactly the reference's double-precision expression -- into a shared-memory table in the
// output type (one table per warp), and every element becomes one table lookup.  Loads and stores
// are 128-bit.
#include "runtime.h"

#include <algorithm>

namespace b200c {

namespace {

struct DequantRowsParams {
    const unsigned char* src;
    void* dst;
    long long rows, cols;
    int srcSigned;   // storage is int8 (else uint8)
    int outHalf;     // output f16 (else f32)
    int perAxis;
    double scale;
    long long zp;
    const double* scales;  // per row (already offset to row 0)
    const long long* zps;
    int swizzleKey;
    long long dataBytes, totalBytes;
};

// One warp per (row, chunk of the row): the warp builds the row's table with exactly the reference's
// double-precision expression, then streams its chunk with independent 128-bit loads.  Warps of a
// CTA never wait for one another.
__global__ void __launch_bounds__(256) dequantRowsKernel(const __grid_constant__ DequantRowsParams p, long long chunksPerRow,
                                                         long long chunkElems) {
    __shared__ float lut32All[8][256];
    __shared__ unsigned short lut16All[8][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* lut32 = lut32All[warp];
    unsigned short* lut16 = lut16All[warp];
    const long long work = p.rows * chunksPerRow;
    long long lastRow = -1;
    for (long long w = static_cast<long long>(blockIdx.x) * 8 + warp; w < work; w += static_cast<long long>(gridDim.x) * 8) {
        const long long row = w / chunksPerRow, chunk = w - row * chunksPerRow;
        if (row != lastRow) {
            __syncwarp();
            const double s = p.perAxis ? p.scales[row] : p.scale;
            const long long zp = p.perAxis ? p.zps[row] : p.zp;
#pragma unroll
            for (int e = lane; e < 256; e += 32) {
                const int q = p.srcSigned ? static_cast<int>(static_cast<signed char>(e)) : e;
                const float r = static_cast<float>(static_cast<double>(static_cast<long long>(q) - zp) * s);
                lut32[e] = r;
                lut16[e] = __half_as_ushort(__float2half_rn(r));
            }
            __syncwarp();
            lastRow = row;
        }
        const long long first = chunk * chunkElems;
        const long long n = min(chunkElems, p.cols - first);
        const unsigned char* src = p.src + row * p.cols + first;
        const long long outElem = row * p.cols + first;
        const bool vec = ((reinterpret_cast<uintptr_t>(src) | (p.outHalf ? outElem * 2 : outElem * 4)) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(p.dst) & 15) == 0;
        const long long nvec = vec ? n / 16 : 0;
        unsigned char* d = static_cast<unsigned char*>(p.dst);
        for (long long u0 = 0; u0 < nvec; u0 += 128) {  // four independent loads per lane and round
            uint4 v[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const long long u = u0 + r * 32 + lane;
                if (u < nvec) v[r] = __ldg(reinterpret_cast<const uint4*>(src) + u);
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const long long u = u0 + r * 32 + lane;
                if (u >= nvec) continue;
                const unsigned int wds[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
                if (p.outHalf) {
                    unsigned int o[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const unsigned int b0 = (wds[i >> 1] >> (16 * (i & 1))) & 0xFFu;
                        const unsigned int b1 = (wds[i >> 1] >> (16 * (i & 1) + 8)) & 0xFFu;
                        o[i] = lut16[b0] | (static_cast<unsigned int>(lut16[b1]) << 16);
                    }
                    const long long a = (outElem + u * 16) * 2;
                    *reinterpret_cast<uint4*>(d + swizzleAddr(a, p.swizzleKey)) = make_uint4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<uint4*>(d + swizzleAddr(a + 16, p.swizzleKey)) = make_uint4(o[4], o[5], o[6], o[7]);
                } else {
                    const long long a = (outElem + u * 16) * 4;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float4 f;
                        f.x = lut32[wds[i] & 0xFFu];
                        f.y = lut32[(wds[i] >> 8) & 0xFFu];
                        f.z = lut32[(wds[i] >> 16) & 0xFFu];
                        f.w = lut32[wds[i] >> 24];
                        *reinterpret_cast<float4*>(d + swizzleAddr(a + 16 * i, p.swizzleKey)) = f;
                    }
                }
            }
        }
        for (long long j = nvec * 16 + lane; j < n; j += 32) {
            const unsigned int b = src[j];
            if (p.outHalf) {
                *reinterpret_cast<unsigned short*>(d + swizzleAddr((outElem + j) * 2, p.swizzleKey)) = lut16[b];
            } else {
                *reinterpret_cast<float*>(d + swizzleAddr((outElem + j) * 4, p.swizzleKey)) = lut32[b];
            }
        }
    }
    if (blockIdx.x == 0) {
        for (long long a = p.dataBytes + threadIdx.x; a < p.totalBytes; a += blockDim.x) {
            static_cast<unsigned char*>(p.dst)[swizzleAddr(a, p.swizzleKey)] = 0;
        }
    }
}

}  // namespace

// Handles views of the form "contiguous rows of 8-bit storage, one Dequantize, output f16/f32".
bool tryLaunchDequantRows(Context* ctx, const GenParams& p) {
    if (p.nOps != 1 || p.ops[0].kind != OP_DEQUANT || p.nBoxes != 0 || p.base != 0) return false;
    if (!(p.srcTag == T_U8 || p.srcTag == T_I8)) return false;
    const bool outF32 = (p.outMode == OUT_RAW) || (p.outMode == OUT_CAST && p.outTag == T_F32);
    const bool outF16 = p.outMode == OUT_CAST && p.outTag == T_F16;
    if (!outF32 && !outF16) return false;
    TileItem it;
    if (!makeTileItem(p, &it)) return false;  // canonical form
    const GenParams& g = it.g;
    const ValueOp& op = g.ops[0];
    long long rows = 1, cols = 0;
    if (g.rank == 1 && g.stride[0] == 1 && op.dim < 0) {
        cols = g.shape[0];
    } else if (g.rank == 2 && g.stride[1] == 1 && g.stride[0] == g.shape[1] && (op.dim == 0 || op.dim < 0)) {
        rows = g.shape[0];
        cols = g.shape[1];
    } else {
        return false;
    }
    DequantRowsParams q;
    q.src = static_cast<const unsigned char*>(g.src);
    q.dst = g.dst;
    q.rows = rows;
    q.cols = cols;
    q.srcSigned = g.srcTag == T_I8;
    q.outHalf = outF16 ? 1 : 0;
    q.perAxis = op.dim >= 0;
    q.scale = op.scale;
    q.zp = op.zp;
    q.scales = op.dim >= 0 ? op.scales + op.off : nullptr;
    q.zps = op.dim >= 0 ? op.zps + op.off : nullptr;
    q.swizzleKey = g.swizzleKey;
    q.dataBytes = g.dataBytes;
    q.totalBytes = g.totalBytes;
    // chunks of a row per CTA: long rows are split so the grid covers the machine
    const long long chunkElems = std::max<long long>(4096, (cols + 63) / 64 / 16 * 16);
    const long long chunksPerRow = (cols + chunkElems - 1) / chunkElems;
    const long long work = rows * chunksPerRow;  // one warp each
    const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>((work + 7) / 8, ctx->smCount * 8LL)));
    dequantRowsKernel<<<grid, 256, 0, ctx->stream>>>(q, chunksPerRow, chunkElems);
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
    return true;
}

}  // namespace b200c
