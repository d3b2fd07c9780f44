// Seeded synthetic weights generated on the device, so benchmark inputs never cross PCIe.
// Counter-based: Philox-4x32-10 keyed by the seed, counter = (element group, stream id); every
// element depends only on (seed, stream, index), so any sharding of a tensor gives the same values.
#include "runtime.h"

#include <algorithm>

namespace b200c {

struct Philox4 {
    unsigned int x, y, z, w;
};

__device__ __forceinline__ Philox4 philox4x32_10(unsigned long long counter, unsigned long long stream,
                                                  unsigned long long seed) {
    unsigned int c0 = static_cast<unsigned int>(counter), c1 = static_cast<unsigned int>(counter >> 32);
    unsigned int c2 = static_cast<unsigned int>(stream), c3 = static_cast<unsigned int>(stream >> 32);
    unsigned int k0 = static_cast<unsigned int>(seed), k1 = static_cast<unsigned int>(seed >> 32);
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const unsigned int hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const unsigned int hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const unsigned int n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
        c0 = n0;
        c1 = lo1;
        c2 = n2;
        c3 = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return Philox4{c0, c1, c2, c3};
}

__device__ __forceinline__ float uniform01(unsigned int u) {  // (0, 1]: (k + 1) * 2^-24 for the top 24 bits k
    return (static_cast<float>(u >> 8) + 1.0f) * (1.0f / 16777216.0f);
}

// The generator is specified down to the rounding of every operation, so that a CPU restatement
// produces the same bytes: only IEEE single-precision add / multiply / divide / square root (each
// rounded to nearest, never fused -- the library is built with --fmad=false) and integer arithmetic.
// No math-library function is involved.

// ln(u) for a normal float u in (0, 1]:  u = m * 2^e with m in (sqrt(1/2), sqrt(2)],
// ln m = 2 atanh(s), s = (m - 1) / (m + 1), |s| <= 0.1716, series up to s^9 (next term < 2e-9 relative).
__device__ __forceinline__ float synthLog(float u) {
    const unsigned int bits = __float_as_uint(u);
    int e = static_cast<int>(bits >> 23) - 127;
    float m = __uint_as_float((bits & 0x007FFFFFu) | 0x3F800000u);
    if (m > 1.41421354f) {
        m = m * 0.5f;
        e += 1;
    }
    const float s = (m - 1.0f) / (m + 1.0f);
    const float t = s * s;
    float p = 0.111111112f;
    p = p * t + 0.142857149f;
    p = p * t + 0.2f;
    p = p * t + 0.333333343f;
    const float lnm = 2.0f * (s + s * (t * p));
    return lnm + static_cast<float>(e) * 0.693147182f;
}

// cos and sin of 2*pi*(k / 2^24) for a 24-bit turn fraction k: the top three bits pick the octant, the
// low 21 bits (mirrored in odd octants) give an angle in [0, pi/4] for the Taylor polynomials.
__device__ __forceinline__ void synthSinCosTurn(unsigned int k, float* sn, float* cs) {
    const unsigned int oct = (k >> 21) & 7u, r = k & 0x1FFFFFu;
    const unsigned int rr = (oct & 1u) ? (0x200000u - r) : r;
    const float x = static_cast<float>(rr) * 3.74507039e-07f;  // (pi / 4) / 2^21
    const float t = x * x;
    float ps = 2.75573192e-06f;            // 1/9!
    ps = ps * t - 1.98412701e-04f;         // 1/7!
    ps = ps * t + 8.33333377e-03f;         // 1/5!
    ps = ps * t - 0.166666672f;            // 1/3!
    const float sx = x + x * (t * ps);
    float pc = -2.75573200e-07f;           // 1/10!
    pc = pc * t + 2.48015876e-05f;         // 1/8!
    pc = pc * t - 1.38888892e-03f;         // 1/6!
    pc = pc * t + 4.16666679e-02f;         // 1/4!
    pc = pc * t - 0.5f;
    const float cx = 1.0f + t * pc;
    // octants 0,3,4,7 keep (cos, sin) of the reduced angle, 1,2,5,6 swap them; signs follow the quadrant
    const bool swap = ((oct + 1u) & 2u) != 0;
    const float c = swap ? sx : cx, sv = swap ? cx : sx;
    *cs = ((oct + 2u) & 4u) ? -c : c;      // cosine is negative in octants 2..5
    *sn = (oct & 4u) ? -sv : sv;           // sine is negative in octants 4..7
}

// four samples per counter value
__device__ __forceinline__ void synthFour(int dist, float p0, float p1, Philox4 r, float* out) {
    if (dist == 0) {  // normal(0, p0): two Box-Muller pairs
        const float r0 = sqrtf(-2.0f * synthLog(uniform01(r.x))), r1 = sqrtf(-2.0f * synthLog(uniform01(r.z)));
        float s0, c0, s1, c1;
        synthSinCosTurn(((r.y >> 8) + 1u) & 0xFFFFFFu, &s0, &c0);
        synthSinCosTurn(((r.w >> 8) + 1u) & 0xFFFFFFu, &s1, &c1);
        out[0] = (p0 * r0) * c0;
        out[1] = (p0 * r0) * s0;
        out[2] = (p0 * r1) * c1;
        out[3] = (p0 * r1) * s1;
    } else if (dist == 1) {  // uniform integer in [-127, 127], zero with probability p0
        const unsigned int v[4] = {r.x, r.y, r.z, r.w};
        const unsigned int cut = static_cast<unsigned int>(fminf(p0, 1.0f) * 65535.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float val = static_cast<float>(static_cast<int>((v[i] >> 16) % 255u) - 127);
            out[i] = ((v[i] & 0xFFFFu) < cut) ? 0.0f : val;
        }
    } else {  // discretised Laplace(0, p0) clipped to [-127, 127], zero with probability p1
        const unsigned int v[4] = {r.x, r.y, r.z, r.w};
        const unsigned int cut = static_cast<unsigned int>(fminf(p1, 1.0f) * 255.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float u = uniform01(v[i] & 0xFFFFFF00u);
            const float mag = -(p0 * synthLog(u));
            float q = rintf((v[i] & 0x80u) ? -mag : mag);
            q = fminf(fmaxf(q, -127.0f), 127.0f);
            out[i] = ((v[i] & 0x7Fu) * 2u < cut) ? 0.0f : q;
        }
    }
}

template <typename T>
__device__ __forceinline__ T synthCast(float v);
template <>
__device__ __forceinline__ float synthCast<float>(float v) {
    return v;
}
template <>
__device__ __forceinline__ __half synthCast<__half>(float v) {
    return __float2half_rn(v);
}
template <>
__device__ __forceinline__ signed char synthCast<signed char>(float v) {
    return static_cast<signed char>(static_cast<int>(v));
}

template <typename T>
__global__ void __launch_bounds__(256) synthFillKernel(T* __restrict__ dst, long long count, int dist, float p0, float p1,
                                                       unsigned long long seed, unsigned long long stream) {
    const long long groups = (count + 3) >> 2;
    const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long g = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; g < groups; g += step) {
        float v[4];
        synthFour(dist, p0, p1, philox4x32_10(static_cast<unsigned long long>(g), stream, seed), v);
        const long long first = g << 2;
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (first + i < count) dst[first + i] = synthCast<T>(v[i]);
    }
}

void launchSynthFill(Context* ctx, void* dst, long long count, int dtype, int dist, double p0, double p1,
                     unsigned long long seed, unsigned long long stream) {
    if (count <= 0) return;
    const long long groups = (count + 3) >> 2;
    const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>((groups + 255) / 256, ctx->smCount * 16LL)));
    const float a = static_cast<float>(p0), b = static_cast<float>(p1);
    if (dtype == B200C_F32) {
        synthFillKernel<float><<<grid, 256, 0, ctx->stream>>>(static_cast<float*>(dst), count, dist, a, b, seed, stream);
    } else if (dtype == B200C_F16) {
        synthFillKernel<__half><<<grid, 256, 0, ctx->stream>>>(static_cast<__half*>(dst), count, dist, a, b, seed, stream);
    } else if (dtype == B200C_SI8) {
        synthFillKernel<signed char><<<grid, 256, 0, ctx->stream>>>(static_cast<signed char*>(dst), count, dist, a, b, seed,
                                                                    stream);
    } else {
        throw BadArg("synthetic fill: dtype must be f32, f16 or si8");
    }
    B2_CUDA(cudaGetLastError());
    ++ctx->launches;
}

}  // namespace b200c
