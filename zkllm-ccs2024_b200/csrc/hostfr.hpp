// Host-side BLS12-381 scalar-field arithmetic on standard-form values.
//
// The reference evaluates every host scalar operation (operator+,-,*,/ and inv
// on Fr_t, polynomial.cu:9-151) by launching a one-thread kernel with its own
// cudaMalloc/cudaMemcpy/cudaFree.  Here the same values are computed on the
// CPU: 4 x u64 limbs, Montgomery multiplication through unsigned __int128.
// Inputs and outputs are canonical standard-form integers in [0, r), so the
// results are the same field elements bit for bit.
#pragma once
#include <cstdint>
#include <cstring>

#include "../../include/zkllm_b200.h"

namespace zkb {
namespace hfr {

typedef unsigned __int128 u128;

struct H {   // a value in [0, r), little-endian u64 limbs
    uint64_t l[4];
};

static const H kMod = {{0xffffffff00000001ull, 0x53bda402fffe5bfeull, 0x3339d80809a1d805ull, 0x73eda753299d7d48ull}};
static const H kR2  = {{0xc999e990f3f29c6dull, 0x2b6cedcb87925c23ull, 0x05d314967254398full, 0x0748d9d99f59ff11ull}};
static const uint64_t kM0 = 0xfffffffeffffffffull;   // -r^-1 mod 2^64

inline H zero() { H r = {{0, 0, 0, 0}}; return r; }
inline H from_u64(uint64_t x) { H r = {{x, 0, 0, 0}}; return r; }
inline H load(const zkb_fr_t& a) { H r; std::memcpy(r.l, a.val, 32); return r; }
inline zkb_fr_t store(const H& a) { zkb_fr_t r; std::memcpy(r.val, a.l, 32); return r; }

inline bool geq(const H& a, const H& b) {
    for (int i = 3; i >= 0; --i) {
        if (a.l[i] != b.l[i]) return a.l[i] > b.l[i];
    }
    return true;
}
inline bool eq(const H& a, const H& b) {
    return a.l[0] == b.l[0] && a.l[1] == b.l[1] && a.l[2] == b.l[2] && a.l[3] == b.l[3];
}
inline bool is_zero(const H& a) { return (a.l[0] | a.l[1] | a.l[2] | a.l[3]) == 0; }

inline H raw_sub(const H& a, const H& b, uint64_t* borrow_out) {
    H r; uint64_t borrow = 0;
    for (int i = 0; i < 4; ++i) {
        u128 d = (u128)a.l[i] - b.l[i] - borrow;
        r.l[i] = (uint64_t)d;
        borrow = (uint64_t)(d >> 64) & 1;
    }
    *borrow_out = borrow;
    return r;
}
inline H raw_add(const H& a, const H& b) {   // no carry out for operands below r
    H r; uint64_t carry = 0;
    for (int i = 0; i < 4; ++i) {
        u128 s = (u128)a.l[i] + b.l[i] + carry;
        r.l[i] = (uint64_t)s;
        carry = (uint64_t)(s >> 64);
    }
    return r;
}
inline H add(const H& a, const H& b) {
    H s = raw_add(a, b);
    if (geq(s, kMod)) { uint64_t bo; s = raw_sub(s, kMod, &bo); }
    return s;
}
inline H sub(const H& a, const H& b) {
    uint64_t bo;
    H d = raw_sub(a, b, &bo);
    if (bo) d = raw_add(d, kMod);
    return d;
}
inline H neg(const H& a) { return sub(zero(), a); }

// a*b*2^-256 mod r
inline H mont_mul(const H& a, const H& b) {
    uint64_t t[6] = {0, 0, 0, 0, 0, 0};
    for (int i = 0; i < 4; ++i) {
        uint64_t carry = 0;
        for (int j = 0; j < 4; ++j) {
            u128 cur = (u128)a.l[j] * b.l[i] + t[j] + carry;
            t[j] = (uint64_t)cur;
            carry = (uint64_t)(cur >> 64);
        }
        u128 top = (u128)t[4] + carry;
        t[4] = (uint64_t)top;
        t[5] = (uint64_t)(top >> 64);
        const uint64_t m = t[0] * kM0;
        u128 cur = (u128)m * kMod.l[0] + t[0];
        carry = (uint64_t)(cur >> 64);
        for (int j = 1; j < 4; ++j) {
            cur = (u128)m * kMod.l[j] + t[j] + carry;
            t[j - 1] = (uint64_t)cur;
            carry = (uint64_t)(cur >> 64);
        }
        top = (u128)t[4] + carry;
        t[3] = (uint64_t)top;
        t[4] = t[5] + (uint64_t)(top >> 64);
    }
    H r = {{t[0], t[1], t[2], t[3]}};
    if (t[4] || geq(r, kMod)) { uint64_t bo; r = raw_sub(r, kMod, &bo); }
    return r;
}
inline H to_mont(const H& a) { return mont_mul(a, kR2); }
inline H from_mont(const H& a) { return mont_mul(a, from_u64(1)); }
// standard-form product
inline H mul(const H& a, const H& b) { return mont_mul(to_mont(a), b); }

inline H pow(const H& a, const H& e) {
    H base = to_mont(a);
    H acc = to_mont(from_u64(1));
    for (int i = 0; i < 256; ++i) {
        if ((e.l[i >> 6] >> (i & 63)) & 1) acc = mont_mul(acc, base);
        base = mont_mul(base, base);
    }
    return from_mont(acc);
}
// Fermat inverse, 0 -> 0 (as the reference's device inverse, bls12-381.cu:597-609)
inline H inv(const H& a) {
    uint64_t bo;
    H e = raw_sub(kMod, from_u64(2), &bo);
    return pow(a, e);
}

// (1-u) + (2u-1) t evaluated at v: 2uv - u - v + 1   (polynomial.cu:355-360)
inline H eq_eval(const H& u, const H& v) {
    H uv = mul(u, v);
    return add(sub(add(uv, uv), add(u, v)), from_u64(1));
}

// sum c[i] x^i  (polynomial.cu:296-304)
inline H poly_eval(const H* c, int n, const H& x) {
    H acc = zero();
    for (int i = n - 1; i >= 0; --i) acc = add(mul(acc, x), c[i]);
    return acc;
}

}  // namespace hfr
}  // namespace zkb
