// TEST INFRASTRUCTURE -- CPU restatement of the library's two measurement helpers: the seeded
// synthetic-weight generator (b200c_synth_fill) and the buffer digest (b200c_digest64_batch).
//
// Neither has a counterpart in the reference compiler: the benchmark configurations define their
// inputs only as "i.i.d. N(0, sigma) from a seed", "uniform int8 with a Bernoulli mask", "discretised
// Laplace", so this repository fixes a generator, and both sides implement the same specification
// independently.  The specification is exact down to the rounding of every operation:
//
//   counter-based Philox-4x32 with 10 rounds, key = seed (low, high word), counter = (group index low,
//   group index high, stream low, stream high); one counter value yields four consecutive samples.
//   uniform(w)      = (float(w >> 8) + 1) * 2^-24                       in (0, 1]
//   ln(u)           = 2 atanh((m-1)/(m+1)) series to s^9  +  e * float(ln 2),  u = m * 2^e, m in (1/sqrt2, sqrt2]
//   cos/sin(2 pi t) = octant reduction of the 24-bit turn fraction + Taylor polynomials on [0, pi/4]
//   normal   : Box-Muller, (sigma * sqrt(-2 ln u0)) * cos / sin, two pairs per counter
//   uniform8 : (w >> 16) % 255 - 127, zero when (w & 0xFFFF) < uint(min(p0,1) * 65535)
//   laplace  : rint(+-(p0 * -ln u)) clipped to +-127, sign from bit 7, zero when (w & 0x7F) * 2 < uint(min(p1,1) * 255)
// using only IEEE single-precision add, multiply, divide and square root (compile with
// -ffp-contract=off) and integer arithmetic, so the CPU and the GPU produce identical bytes.
//
// digest64(bytes, n) = mix(C0 * (n + 1) + sum_j mix(word_j ^ (C1 * (j + 1))))  over the little-endian
// 64-bit words of the buffer (the last one zero-extended), mix = the splitmix64 finaliser; all
// arithmetic modulo 2^64.  The sum makes it order-independent across threads and position-dependent
// through the per-word key.
#include <cmath>
#include <cstdint>
#include <cstring>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

struct Quad {
    uint32_t v[4];
};

Quad philox(uint64_t group, uint64_t stream, uint64_t seed) {
    uint32_t c[4] = {uint32_t(group), uint32_t(group >> 32), uint32_t(stream), uint32_t(stream >> 32)};
    uint32_t k[2] = {uint32_t(seed), uint32_t(seed >> 32)};
    for (int round = 0; round < 10; ++round) {
        const uint64_t p0 = uint64_t(0xD2511F53u) * c[0];
        const uint64_t p1 = uint64_t(0xCD9E8D57u) * c[2];
        const uint32_t n0 = uint32_t(p1 >> 32) ^ c[1] ^ k[0];
        const uint32_t n2 = uint32_t(p0 >> 32) ^ c[3] ^ k[1];
        c[0] = n0;
        c[1] = uint32_t(p1);
        c[2] = n2;
        c[3] = uint32_t(p0);
        k[0] += 0x9E3779B9u;
        k[1] += 0xBB67AE85u;
    }
    return Quad{{c[0], c[1], c[2], c[3]}};
}

float asFloat(uint32_t b) {
    float f;
    std::memcpy(&f, &b, 4);
    return f;
}
uint32_t asBits(float f) {
    uint32_t b;
    std::memcpy(&b, &f, 4);
    return b;
}

float unit(uint32_t w) {
    return (float(w >> 8) + 1.0f) * (1.0f / 16777216.0f);
}

float lnUnit(float u) {
    const uint32_t b = asBits(u);
    int e = int(b >> 23) - 127;
    float m = asFloat((b & 0x007FFFFFu) | 0x3F800000u);
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
    const float inner = t * p;
    const float lnm = 2.0f * (s + s * inner);
    return lnm + float(e) * 0.693147182f;
}

void sinCosTurn(uint32_t k24, float& sn, float& cs) {
    const uint32_t octant = (k24 >> 21) & 7u, low = k24 & 0x1FFFFFu;
    const uint32_t red = (octant & 1u) ? (0x200000u - low) : low;
    const float x = float(red) * 3.74507039e-07f;
    const float t = x * x;
    float a = 2.75573192e-06f;
    a = a * t - 1.98412701e-04f;
    a = a * t + 8.33333377e-03f;
    a = a * t - 0.166666672f;
    const float sinx = x + x * (t * a);
    float b = -2.75573200e-07f;
    b = b * t + 2.48015876e-05f;
    b = b * t - 1.38888892e-03f;
    b = b * t + 4.16666679e-02f;
    b = b * t - 0.5f;
    const float cosx = 1.0f + t * b;
    float c, s;
    switch (octant) {  // written out per octant: angle = octant * pi/4 + (or -) the reduced angle
    case 0: c = cosx; s = sinx; break;
    case 1: c = sinx; s = cosx; break;
    case 2: c = -sinx; s = cosx; break;
    case 3: c = -cosx; s = sinx; break;
    case 4: c = -cosx; s = -sinx; break;
    case 5: c = -sinx; s = -cosx; break;
    case 6: c = sinx; s = -cosx; break;
    default: c = cosx; s = -sinx; break;
    }
    cs = c;
    sn = s;
}

void four(int dist, float p0, float p1, const Quad& q, float out[4]) {
    if (dist == 0) {
        for (int pair = 0; pair < 2; ++pair) {
            const float radius = std::sqrt(-2.0f * lnUnit(unit(q.v[2 * pair])));
            float sn, cs;
            sinCosTurn(((q.v[2 * pair + 1] >> 8) + 1u) & 0xFFFFFFu, sn, cs);
            const float scaled = p0 * radius;
            out[2 * pair] = scaled * cs;
            out[2 * pair + 1] = scaled * sn;
        }
    } else if (dist == 1) {
        const uint32_t cut = uint32_t(std::fmin(p0, 1.0f) * 65535.0f);
        for (int i = 0; i < 4; ++i) {
            const int val = int((q.v[i] >> 16) % 255u) - 127;
            out[i] = (q.v[i] & 0xFFFFu) < cut ? 0.0f : float(val);
        }
    } else {
        const uint32_t cut = uint32_t(std::fmin(p1, 1.0f) * 255.0f);
        for (int i = 0; i < 4; ++i) {
            const float mag = -(p0 * lnUnit(unit(q.v[i] & 0xFFFFFF00u)));
            float r = std::nearbyintf((q.v[i] & 0x80u) ? -mag : mag);
            r = std::fmin(std::fmax(r, -127.0f), 127.0f);
            out[i] = ((q.v[i] & 0x7Fu) * 2u < cut) ? 0.0f : r;
        }
    }
}

// IEEE binary16 from binary32, round to nearest even
uint16_t toHalf(float f) {
    const uint32_t x = asBits(f), sign = (x >> 16) & 0x8000u, a = x & 0x7FFFFFFFu;
    if (a >= 0x7F800000u) return uint16_t(sign | 0x7C00u | (a > 0x7F800000u ? 0x0200u : 0u));
    if (a >= 0x477FF000u) return uint16_t(sign | 0x7C00u);
    if (a >= 0x38800000u) {
        uint32_t h = (((a >> 23) - 112u) << 10) | ((a & 0x007FFFFFu) >> 13);
        const uint32_t rem = a & 0x1FFFu;
        if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;
        return uint16_t(sign | h);
    }
    if (a >= 0x33000000u) {
        const uint32_t shift = 126u - (a >> 23), mant = (a & 0x007FFFFFu) | 0x00800000u;
        uint32_t h = mant >> shift;
        const uint32_t rem = mant & ((1u << shift) - 1u), half = 1u << (shift - 1u);
        if (rem > half || (rem == half && (h & 1u))) ++h;
        return uint16_t(sign | h);
    }
    return uint16_t(sign);
}

uint64_t mix(uint64_t x) {
    x ^= x >> 30;
    x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27;
    x *= 0x94D049BB133111EBull;
    x ^= x >> 31;
    return x;
}

}  // namespace

extern "C" {

// dtype codes as in include/b200const.h: f32 = 0x120, f16 = 0x110, si8 = 0x408
int orc_synth_fill(void* dst, int64_t count, int32_t dtype, int32_t dist, double p0, double p1, uint64_t seed,
                   uint64_t stream) {
    if (count < 0 || dist < 0 || dist > 2) return -1;
    if (dtype != 0x120 && dtype != 0x110 && dtype != 0x408) return -1;
    const int64_t groups = (count + 3) / 4;
    const float a = float(p0), b = float(p1);
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < groups; ++g) {
        float v[4];
        four(dist, a, b, philox(uint64_t(g), stream, seed), v);
        for (int i = 0; i < 4 && 4 * g + i < count; ++i) {
            const int64_t at = 4 * g + i;
            if (dtype == 0x120) {
                static_cast<float*>(dst)[at] = v[i];
            } else if (dtype == 0x110) {
                static_cast<uint16_t*>(dst)[at] = toHalf(v[i]);
            } else {
                static_cast<int8_t*>(dst)[at] = int8_t(int(v[i]));
            }
        }
    }
    return 0;
}

uint64_t orc_digest64(const void* data, uint64_t n) {
    const unsigned char* p = static_cast<const unsigned char*>(data);
    const uint64_t words = (n + 7) / 8;
    uint64_t sum = 0;
#pragma omp parallel for schedule(static) reduction(+ : sum)
    for (int64_t j = 0; j < int64_t(words); ++j) {
        uint64_t w = 0;
        const uint64_t first = uint64_t(j) * 8;
        const uint64_t len = n - first < 8 ? n - first : 8;
        std::memcpy(&w, p + first, len);  // little-endian host
        sum += mix(w ^ (0xD6E8FEB86659FD93ull * (uint64_t(j) + 1)));
    }
    return mix(0x9E3779B97F4A7C15ull * (n + 1) + sum);
}

}  // extern "C"
