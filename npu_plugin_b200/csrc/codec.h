// Block codec: stream format and the per-block routines shared by the kernels.
//
// This stands where the reference calls BitCompactor
// (src/vpux_compiler/src/utils/bit_compactor_codec.cpp:15-42); the BitCompactor sources are not
// part of the reference tree, so the bitstream below is this library's own and is NOT
// BitCompactor-compatible.  It keeps the contract of that call site: a size bound, lossless
// 64-byte-block coding with per-block mode selection, "not smaller" reported as failure.
//
// Stream layout (little endian):
//   header, 32 bytes : 'B','2','B','C', u32 version = 1, u64 n, u64 nblocks, u32 nsuper, u32 0
//   index            : nsuper x u32 -- byte offset, from the start of the records, of the first
//                      record of every 64-block group (so groups decode independently)
//   records          : one per 64-byte block of the input (the last block is zero extended)
//   zero bytes up to a multiple of 32
// Record = header byte (mode << 5 | w) + payload:
//   0 RAW    64 bytes
//   1 CONST  1 byte (all 64 bytes equal it)
//   2 PACKU  1 byte base (unsigned block minimum) + 8*w bytes, fields (b - base) of w = 1..7 bits
//   3 PACKS  8*w bytes, fields zigzag(int8 b) of w = 1..7 bits
//   4 SPARSE 8-byte mask (bit k of mask byte j = element 8j+k non-zero) + the non-zero bytes
// Fields are packed per group of 8 elements into a little-endian w-byte word, element k at bits
// [k*w, k*w+w).  The smallest record wins; ties go to the smaller mode number.
#pragma once

#include "view.h"

namespace b200c {

constexpr int kCodecHeaderBytes = 32;
constexpr int kCodecBlock = 64;
constexpr int kCodecSuper = 64;  // blocks per index entry

B2_HD unsigned int zigzag8(unsigned int b) {
    const unsigned int s = (b & 0x80u) ? 0xFFu : 0u;
    return ((b << 1) & 0xFFu) ^ s;
}
B2_HD unsigned int unzigzag8(unsigned int z) {
    return ((z >> 1) ^ ((z & 1u) ? 0xFFu : 0u)) & 0xFFu;
}
B2_HD int bitWidth8(unsigned int v) {
    int w = 0;
    while (v) {
        ++w;
        v >>= 1;
    }
    return w;
}

// header byte and record size of one 64-byte block
B2_HD int codecChoose(const unsigned char* b, unsigned char* header, unsigned char* base) {
    unsigned int mn = 255, mx = 0, zor = 0, nnz = 0;
    for (int i = 0; i < 64; ++i) {
        const unsigned int v = b[i];
        mn = v < mn ? v : mn;
        mx = v > mx ? v : mx;
        zor |= zigzag8(v);
        nnz += v != 0;
    }
    int mode = 0, w = 0, size = 65;
    if (mn == mx) {
        mode = 1;
        size = 2;
    }
    const int wu = bitWidth8(mx - mn);
    if (wu >= 1 && wu <= 7 && 2 + 8 * wu < size) {
        mode = 2;
        w = wu;
        size = 2 + 8 * wu;
    }
    const int ws = bitWidth8(zor);
    if (ws >= 1 && ws <= 7 && 1 + 8 * ws < size) {
        mode = 3;
        w = ws;
        size = 1 + 8 * ws;
    }
    if (9 + static_cast<int>(nnz) < size) {
        mode = 4;
        w = 0;
        size = 9 + static_cast<int>(nnz);
    }
    *header = static_cast<unsigned char>((mode << 5) | w);
    *base = static_cast<unsigned char>(mn);
    return size;
}

B2_HD int codecRecordSize(unsigned char header, const unsigned char* payload) {
    const int mode = header >> 5, w = header & 31;
    switch (mode) {
    case 0:
        return 65;
    case 1:
        return 2;
    case 2:
        return 2 + 8 * w;
    case 3:
        return 1 + 8 * w;
    default: {
        int nnz = 0;
        for (int j = 0; j < 8; ++j) {
            unsigned int m = payload[j];
            while (m) {
                nnz += m & 1u;
                m >>= 1;
            }
        }
        return 9 + nnz;
    }
    }
}

B2_HD void codecWriteRecord(const unsigned char* b, unsigned char header, unsigned char base, unsigned char* out) {
    const int mode = header >> 5, w = header & 31;
    int o = 0;
    out[o++] = header;
    switch (mode) {
    case 0:
        for (int i = 0; i < 64; ++i) out[o++] = b[i];
        break;
    case 1:
        out[o++] = base;
        break;
    case 2:
    case 3:
        if (mode == 2) out[o++] = base;
        for (int g = 0; g < 8; ++g) {
            unsigned long long word = 0;
            for (int k = 0; k < 8; ++k) {
                const unsigned int v = b[g * 8 + k];
                const unsigned long long f = mode == 2 ? ((v - base) & 0xFFu) : zigzag8(v);
                word |= f << (k * w);
            }
            for (int j = 0; j < w; ++j) out[o++] = static_cast<unsigned char>(word >> (8 * j));
        }
        break;
    default:
        for (int g = 0; g < 8; ++g) {
            unsigned int m = 0;
            for (int k = 0; k < 8; ++k) m |= static_cast<unsigned int>(b[g * 8 + k] != 0) << k;
            out[o++] = static_cast<unsigned char>(m);
        }
        for (int i = 0; i < 64; ++i)
            if (b[i] != 0) out[o++] = b[i];
        break;
    }
}

// decodes one record into 64 bytes; returns the record size, or -1 for a bad mode
B2_HD int codecReadRecord(const unsigned char* in, unsigned char* b) {
    const unsigned char header = in[0];
    const int mode = header >> 5, w = header & 31;
    int i = 1;
    switch (mode) {
    case 0:
        for (int k = 0; k < 64; ++k) b[k] = in[i++];
        return i;
    case 1:
        for (int k = 0; k < 64; ++k) b[k] = in[1];
        return 2;
    case 2:
    case 3: {
        if (w < 1 || w > 7) return -1;
        const unsigned int base = mode == 2 ? in[i++] : 0;
        for (int g = 0; g < 8; ++g) {
            unsigned long long word = 0;
            for (int j = 0; j < w; ++j) word |= static_cast<unsigned long long>(in[i++]) << (8 * j);
            for (int k = 0; k < 8; ++k) {
                const unsigned int f = static_cast<unsigned int>((word >> (k * w)) & ((1u << w) - 1u));
                b[g * 8 + k] = static_cast<unsigned char>(mode == 2 ? f + base : unzigzag8(f));
            }
        }
        return i;
    }
    case 4: {
        const unsigned char* mask = in + 1;
        i = 9;
        for (int e = 0; e < 64; ++e) b[e] = ((mask[e >> 3] >> (e & 7)) & 1u) ? in[i++] : 0;
        return i;
    }
    default:
        return -1;
    }
}

}  // namespace b200c
