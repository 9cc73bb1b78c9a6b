// 64-bit CityHash of 2011 (version 1): the string hash behind categorical feature values.
// The reference keeps the low 32 bits of this hash of a value's string form (catboost/libs/cat_feature/cat_feature.cpp:4-6);
// model files store those numbers, so this function has to reproduce them bit for bit.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <utility>

namespace city1 {
constexpr uint64_t K0 = 0xc3a5c85c97cb3127ULL, K1 = 0xb492b66fbe98f273ULL, K2 = 0x9ae16a3b2f90404fULL,
                   K3 = 0xc949d7c7509e6557ULL, KMUL = 0x9ddfea08eb382d69ULL;
inline uint64_t ld64(const char* p) { uint64_t v; std::memcpy(&v, p, 8); return v; }
inline uint64_t ld32(const char* p) { uint32_t v; std::memcpy(&v, p, 4); return v; }
inline uint64_t ror(uint64_t v, int s) { return s == 0 ? v : ((v >> s) | (v << (64 - s))); }
inline uint64_t smix(uint64_t v) { return v ^ (v >> 47); }
inline uint64_t h16(uint64_t u, uint64_t v) {
    uint64_t a = (u ^ v) * KMUL; a ^= a >> 47;
    uint64_t b = (v ^ a) * KMUL; b ^= b >> 47;
    return b * KMUL;
}
struct P { uint64_t a, b; };
inline P weak32(uint64_t w, uint64_t x, uint64_t y, uint64_t z, uint64_t a, uint64_t b) {
    a += w; b = ror(b + a + z, 21);
    const uint64_t c = a;
    a += x; a += y; b += ror(a, 44);
    return P{a + z, b + c};
}
inline P weak32(const char* s, uint64_t a, uint64_t b) { return weak32(ld64(s), ld64(s + 8), ld64(s + 16), ld64(s + 24), a, b); }

inline uint64_t hash(const char* s, size_t n) {
    if (n <= 16) {
        if (n > 8) { const uint64_t a = ld64(s), b = ld64(s + n - 8); return h16(a, ror(b + n, int(n))) ^ b; }
        if (n >= 4) { const uint64_t a = ld32(s); return h16(n + (a << 3), ld32(s + n - 4)); }
        if (n > 0) {
            const uint8_t a = uint8_t(s[0]), b = uint8_t(s[n >> 1]), c = uint8_t(s[n - 1]);
            const uint32_t y = uint32_t(a) + (uint32_t(b) << 8), z = uint32_t(n) + (uint32_t(c) << 2);
            return smix(y * K2 ^ z * K3) * K2;
        }
        return K2;
    }
    if (n <= 32) {
        const uint64_t a = ld64(s) * K1, b = ld64(s + 8), c = ld64(s + n - 8) * K2, d = ld64(s + n - 16) * K0;
        return h16(ror(a - b, 43) + ror(c, 30) + d, a + ror(b ^ K3, 20) - c + n);
    }
    if (n <= 64) {
        uint64_t z = ld64(s + 24);
        uint64_t a = ld64(s) + (n + ld64(s + n - 16)) * K0;
        uint64_t b = ror(a + z, 52), c = ror(a, 37);
        a += ld64(s + 8); c += ror(a, 7); a += ld64(s + 16);
        const uint64_t vf = a + z, vs = b + ror(a, 31) + c;
        a = ld64(s + 16) + ld64(s + n - 32);
        z = ld64(s + n - 8);
        b = ror(a + z, 52); c = ror(a, 37);
        a += ld64(s + n - 24); c += ror(a, 7); a += ld64(s + n - 16);
        const uint64_t wf = a + z, ws = b + ror(a, 31) + c;
        const uint64_t r = smix((vf + ws) * K2 + (wf + vs) * K0);
        return smix(r * K0 + vs) * K2;
    }
    uint64_t x = ld64(s), y = ld64(s + n - 16) ^ K1, z = ld64(s + n - 56) ^ K0;
    P v = weak32(s + n - 64, n, y), w = weak32(s + n - 32, n * K1, K0);
    z += smix(v.b) * K1; x = ror(z + x, 39) * K1; y = ror(y, 33) * K1;
    size_t left = (n - 1) & ~size_t(63);
    do {
        x = ror(x + y + v.a + ld64(s + 16), 37) * K1;
        y = ror(y + v.b + ld64(s + 48), 42) * K1;
        x ^= w.b; y ^= v.a; z = ror(z ^ w.a, 33);
        v = weak32(s, v.b * K1, x + w.a);
        w = weak32(s + 32, z + w.b, y);
        std::swap(z, x);
        s += 64; left -= 64;
    } while (left != 0);
    return h16(h16(v.a, w.a) + smix(y) * K1 + z, h16(v.b, w.b) + x);
}
}  // namespace city1
