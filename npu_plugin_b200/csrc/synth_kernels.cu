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

__device__ __forceinline__ float uniform01(unsigned int u) {  // (0, 1]
    return (static_cast<float>(u >> 8) + 1.0f) * (1.0f / 16777216.0f);
}

// four samples per counter value
__device__ __forceinline__ void synthFour(int dist, float p0, float p1, Philox4 r, float* out) {
    if (dist == 0) {  // normal(0, p0): two Box-Muller pairs
        const float r0 = sqrtf(-2.0f * logf(uniform01(r.x))), r1 = sqrtf(-2.0f * logf(uniform01(r.z)));
        float s0, c0, s1, c1;
        sincospif(2.0f * uniform01(r.y), &s0, &c0);
        sincospif(2.0f * uniform01(r.w), &s1, &c1);
        out[0] = p0 * r0 * c0;
        out[1] = p0 * r0 * s0;
        out[2] = p0 * r1 * c1;
        out[3] = p0 * r1 * s1;
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
            const float mag = -p0 * logf(u);
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
    if (B2_EMU(ctx)) throw NotBuilt("synthetic fill needs a device");
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
