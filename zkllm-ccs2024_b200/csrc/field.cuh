// Montgomery arithmetic for the two BLS12-381 prime fields on sm_100a.
//
//   Fr : 255-bit scalar field, 8 x u32 little-endian limbs, radix 2^256
//   Fq : 381-bit base field,  12 x u32 little-endian limbs, radix 2^384
//
// Semantics follow the reference's blstrs__scalar__Scalar_* / blstrs__fp__Fp_*
// device functions (bls12-381.cu:289-622 and :641-1044): add/sub are canonical
// modular operations on values in [0, p); mont_mul(a, b) returns a*b*R^-1 mod p
// in [0, p).  The implementation is independent of that code: one interleaved
// (CIOS) multiply-and-reduce pass in which the running sum is held as two
// register arrays, one for the even-aligned 64-bit partial products and one for
// the odd-aligned ones, so that every mad.lo/mad.hi pair extends a single carry
// chain and no partial product needs a separate carry fix-up.
#pragma once
#include <cstdint>

namespace zkb {

// ---------------------------------------------------------------------------
// Carry-chain PTX primitives.  Every wrapper is `asm volatile` so that the
// compiler keeps them in program order: the condition-code register is an
// implicit operand that ordinary data-flow analysis does not see.
// ---------------------------------------------------------------------------
#define ZKB_DEV __device__ __forceinline__

ZKB_DEV uint32_t ptx_mul_lo(uint32_t a, uint32_t b) {
    uint32_t r; asm volatile("mul.lo.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b)); return r;
}
ZKB_DEV uint32_t ptx_mul_hi(uint32_t a, uint32_t b) {
    uint32_t r; asm volatile("mul.hi.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b)); return r;
}
// acc = a*b(lo) + acc, sets CC
ZKB_DEV void ptx_mad_lo_cc(uint32_t& acc, uint32_t a, uint32_t b) {
    asm volatile("mad.lo.cc.u32 %0, %1, %2, %0;" : "+r"(acc) : "r"(a), "r"(b));
}
// acc = a*b(lo) + acc + CC, sets CC
ZKB_DEV void ptx_madc_lo_cc(uint32_t& acc, uint32_t a, uint32_t b) {
    asm volatile("madc.lo.cc.u32 %0, %1, %2, %0;" : "+r"(acc) : "r"(a), "r"(b));
}
// acc = a*b(hi) + acc, sets CC
ZKB_DEV void ptx_mad_hi_cc(uint32_t& acc, uint32_t a, uint32_t b) {
    asm volatile("mad.hi.cc.u32 %0, %1, %2, %0;" : "+r"(acc) : "r"(a), "r"(b));
}
// acc = a*b(hi) + acc + CC, sets CC
ZKB_DEV void ptx_madc_hi_cc(uint32_t& acc, uint32_t a, uint32_t b) {
    asm volatile("madc.hi.cc.u32 %0, %1, %2, %0;" : "+r"(acc) : "r"(a), "r"(b));
}
// dst = a*b(lo) + c + CC, sets CC
ZKB_DEV uint32_t ptx_madc_lo_cc3(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r; asm volatile("madc.lo.cc.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c)); return r;
}
// dst = a*b(hi) + c + CC, sets CC
ZKB_DEV uint32_t ptx_madc_hi_cc3(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r; asm volatile("madc.hi.cc.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c)); return r;
}
ZKB_DEV void ptx_add_cc(uint32_t& acc, uint32_t a) {
    asm volatile("add.cc.u32 %0, %0, %1;" : "+r"(acc) : "r"(a));
}
ZKB_DEV void ptx_addc_cc(uint32_t& acc, uint32_t a) {
    asm volatile("addc.cc.u32 %0, %0, %1;" : "+r"(acc) : "r"(a));
}
ZKB_DEV void ptx_addc(uint32_t& acc, uint32_t a) {
    asm volatile("addc.u32 %0, %0, %1;" : "+r"(acc) : "r"(a));
}
ZKB_DEV uint32_t ptx_add_cc3(uint32_t a, uint32_t b) {
    uint32_t r; asm volatile("add.cc.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b)); return r;
}
ZKB_DEV uint32_t ptx_addc_cc3(uint32_t a, uint32_t b) {
    uint32_t r; asm volatile("addc.cc.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b)); return r;
}
ZKB_DEV uint32_t ptx_addc3(uint32_t a, uint32_t b) {
    uint32_t r; asm volatile("addc.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b)); return r;
}
ZKB_DEV uint32_t ptx_sub_cc3(uint32_t a, uint32_t b) {
    uint32_t r; asm volatile("sub.cc.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b)); return r;
}
ZKB_DEV uint32_t ptx_subc_cc3(uint32_t a, uint32_t b) {
    uint32_t r; asm volatile("subc.cc.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b)); return r;
}
ZKB_DEV uint32_t ptx_subc3(uint32_t a, uint32_t b) {
    uint32_t r; asm volatile("subc.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b)); return r;
}

// ---------------------------------------------------------------------------
// Field parameter packs.  Limb tables are function-local constexpr arrays so
// that fully unrolled device code folds them to immediates.
// ---------------------------------------------------------------------------
struct FrParams {
    static constexpr int N = 8;
    static constexpr uint32_t M0 = 0xffffffffu;   // -r^-1 mod 2^32
    __host__ __device__ static constexpr uint32_t mod(int i) {
        constexpr uint32_t t[8] = {0x00000001u, 0xffffffffu, 0xfffe5bfeu, 0x53bda402u,
                                   0x09a1d805u, 0x3339d808u, 0x299d7d48u, 0x73eda753u};
        return t[i];
    }
    __host__ __device__ static constexpr uint32_t one(int i) {        // 2^256 mod r
        constexpr uint32_t t[8] = {0xfffffffeu, 0x00000001u, 0x00034802u, 0x5884b7fau,
                                   0xecbc4ff5u, 0x998c4fefu, 0xacc5056fu, 0x1824b159u};
        return t[i];
    }
    __host__ __device__ static constexpr uint32_t r2(int i) {         // 2^512 mod r
        constexpr uint32_t t[8] = {0xf3f29c6du, 0xc999e990u, 0x87925c23u, 0x2b6cedcbu,
                                   0x7254398fu, 0x05d31496u, 0x9f59ff11u, 0x0748d9d9u};
        return t[i];
    }
};

struct FqParams {
    static constexpr int N = 12;
    static constexpr uint32_t M0 = 0xfffcfffdu;   // -p^-1 mod 2^32
    __host__ __device__ static constexpr uint32_t mod(int i) {
        constexpr uint32_t t[12] = {0xffffaaabu, 0xb9feffffu, 0xb153ffffu, 0x1eabfffeu,
                                    0xf6b0f624u, 0x6730d2a0u, 0xf38512bfu, 0x64774b84u,
                                    0x434bacd7u, 0x4b1ba7b6u, 0x397fe69au, 0x1a0111eau};
        return t[i];
    }
    __host__ __device__ static constexpr uint32_t one(int i) {        // 2^384 mod p
        constexpr uint32_t t[12] = {0x0002fffdu, 0x76090000u, 0xc40c0002u, 0xebf4000bu,
                                    0x53c758bau, 0x5f489857u, 0x70525745u, 0x77ce5853u,
                                    0xa256ec6du, 0x5c071a97u, 0xfa80e493u, 0x15f65ec3u};
        return t[i];
    }
    __host__ __device__ static constexpr uint32_t r2(int i) {         // 2^768 mod p
        constexpr uint32_t t[12] = {0x1c341746u, 0xf4df1f34u, 0x09d104f1u, 0x0a76e6a6u,
                                    0x4c95b6d5u, 0x8de5476cu, 0x939d83c0u, 0x67eb88a9u,
                                    0xb519952du, 0x9a793e85u, 0x92cae3aau, 0x11988fe5u};
        return t[i];
    }
};

// A field element: N little-endian u32 limbs.  16-byte alignment lets the
// kernels move elements with 128-bit loads and stores.
template <class P>
struct __align__(16) Fe {
    uint32_t v[P::N];
};
using Fr = Fe<FrParams>;   // layout-compatible with the reference's Fr_t (8 x u32)
using Fq = Fe<FqParams>;   // layout-compatible with the reference's Fp_t (12 x u32)

template <class P> ZKB_DEV Fe<P> fe_zero() {
    Fe<P> r;
#pragma unroll
    for (int i = 0; i < P::N; ++i) r.v[i] = 0;
    return r;
}
template <class P> ZKB_DEV Fe<P> fe_mont_one() {
    Fe<P> r;
#pragma unroll
    for (int i = 0; i < P::N; ++i) r.v[i] = P::one(i);
    return r;
}
template <class P> ZKB_DEV Fe<P> fe_r2() {
    Fe<P> r;
#pragma unroll
    for (int i = 0; i < P::N; ++i) r.v[i] = P::r2(i);
    return r;
}
template <class P> ZKB_DEV bool fe_is_zero(const Fe<P>& a) {
    uint32_t acc = 0;
#pragma unroll
    for (int i = 0; i < P::N; ++i) acc |= a.v[i];
    return acc == 0;
}
template <class P> ZKB_DEV bool fe_eq(const Fe<P>& a, const Fe<P>& b) {
    uint32_t acc = 0;
#pragma unroll
    for (int i = 0; i < P::N; ++i) acc |= a.v[i] ^ b.v[i];
    return acc == 0;
}

// r = a - p if a >= p else a   (a < 2p, no carry above limb N-1)
template <class P> ZKB_DEV void fe_final_sub(Fe<P>& a) {
    constexpr int N = P::N;
    uint32_t t[N];
    t[0] = ptx_sub_cc3(a.v[0], P::mod(0));
#pragma unroll
    for (int i = 1; i < N; ++i) t[i] = ptx_subc_cc3(a.v[i], P::mod(i));
    uint32_t borrow = ptx_subc3(0u, 0u);   // 0 if a >= p, 0xffffffff if a < p
#pragma unroll
    for (int i = 0; i < N; ++i) a.v[i] = borrow ? a.v[i] : t[i];
}

// (a + b) mod p, inputs and output in [0, p)
template <class P> ZKB_DEV Fe<P> fe_add(const Fe<P>& a, const Fe<P>& b) {
    constexpr int N = P::N;
    Fe<P> r;
    r.v[0] = ptx_add_cc3(a.v[0], b.v[0]);
#pragma unroll
    for (int i = 1; i < N - 1; ++i) r.v[i] = ptx_addc_cc3(a.v[i], b.v[i]);
    r.v[N - 1] = ptx_addc3(a.v[N - 1], b.v[N - 1]);   // 2p < 2^(32N): no carry out
    fe_final_sub(r);
    return r;
}

// (a - b) mod p
template <class P> ZKB_DEV Fe<P> fe_sub(const Fe<P>& a, const Fe<P>& b) {
    constexpr int N = P::N;
    Fe<P> r;
    r.v[0] = ptx_sub_cc3(a.v[0], b.v[0]);
#pragma unroll
    for (int i = 1; i < N; ++i) r.v[i] = ptx_subc_cc3(a.v[i], b.v[i]);
    uint32_t borrow = ptx_subc3(0u, 0u);              // all-ones when a < b
    // add back p masked by the borrow
    r.v[0] = ptx_add_cc3(r.v[0], P::mod(0) & borrow);
#pragma unroll
    for (int i = 1; i < N - 1; ++i) r.v[i] = ptx_addc_cc3(r.v[i], P::mod(i) & borrow);
    r.v[N - 1] = ptx_addc3(r.v[N - 1], P::mod(N - 1) & borrow);
    return r;
}

template <class P> ZKB_DEV Fe<P> fe_neg(const Fe<P>& a) {
    return fe_sub(fe_zero<P>(), a);
}
template <class P> ZKB_DEV Fe<P> fe_dbl(const Fe<P>& a) { return fe_add(a, a); }

// ---------------------------------------------------------------------------
// Montgomery product.
//
// The running sum T is kept as two limb arrays: `ev` holds the 64-bit products
// that start on an even limb, `od` those that start on an odd limb, i.e.
//     T = sum ev[k] 2^(32k) + 2^32 * sum od[k] 2^(32k).
// Adding x*y (x an N-limb number, y one limb) is then two independent carry
// chains of N multiply-adds each.  After the Montgomery step makes limb 0 zero,
// dividing by 2^32 swaps the roles of the two arrays; the orphaned limb ev[1]
// is folded into the head of the next pair of chains.
//
// Bound: with a, b < p the sum before each division is below 2^33 * p, which
// fits the N+1 limbs that (ev, od) cover for both fields (p < 2^(32N-1)).
// ---------------------------------------------------------------------------
template <class P>
ZKB_DEV void mont_reduce_step(uint32_t* ev, uint32_t* od) {
    constexpr int N = P::N;
    const uint32_t m = ev[0] * P::M0;
    ptx_mad_lo_cc(od[0], P::mod(1), m);
    ptx_madc_hi_cc(od[1], P::mod(1), m);
#pragma unroll
    for (int i = 2; i < N; i += 2) {
        ptx_madc_lo_cc(od[i], P::mod(i + 1), m);
        ptx_madc_hi_cc(od[i + 1], P::mod(i + 1), m);
    }
    ptx_mad_lo_cc(ev[0], P::mod(0), m);
    ptx_madc_hi_cc(ev[1], P::mod(0), m);
#pragma unroll
    for (int i = 2; i < N; i += 2) {
        ptx_madc_lo_cc(ev[i], P::mod(i), m);
        ptx_madc_hi_cc(ev[i + 1], P::mod(i), m);
    }
    ptx_addc(od[N - 1], 0u);
}

// One operand-limb step.  On entry `x` is the even array of the previous step
// (x[0] == 0) and `y` its odd array; on exit `y` is the even array (y[0] == 0)
// and `x` the odd array of T' = (T/2^32 + a*bj + m*p).
template <class P>
ZKB_DEV void mont_mad_step(uint32_t* x, uint32_t* y, const uint32_t* a, uint32_t bj) {
    constexpr int N = P::N;
    ptx_add_cc(y[0], x[1]);
#pragma unroll
    for (int i = 0; i < N - 2; i += 2) {
        x[i]     = ptx_madc_lo_cc3(a[i + 1], bj, x[i + 2]);
        x[i + 1] = ptx_madc_hi_cc3(a[i + 1], bj, x[i + 3]);
    }
    x[N - 2] = ptx_madc_lo_cc3(a[N - 1], bj, 0u);
    x[N - 1] = ptx_madc_hi_cc3(a[N - 1], bj, 0u);   // cannot carry out
    ptx_mad_lo_cc(y[0], a[0], bj);
    ptx_madc_hi_cc(y[1], a[0], bj);
#pragma unroll
    for (int i = 2; i < N; i += 2) {
        ptx_madc_lo_cc(y[i], a[i], bj);
        ptx_madc_hi_cc(y[i + 1], a[i], bj);
    }
    ptx_addc(x[N - 1], 0u);
    mont_reduce_step<P>(y, x);
}

template <class P>
ZKB_DEV Fe<P> mont_mul(const Fe<P>& a, const Fe<P>& b) {
    constexpr int N = P::N;
    static_assert(N % 2 == 0, "limb count must be even");
    uint32_t s[N], t[N];
    // first operand limb: plain products, nothing to accumulate onto
#pragma unroll
    for (int i = 0; i < N; i += 2) {
        s[i]     = ptx_mul_lo(a.v[i], b.v[0]);
        s[i + 1] = ptx_mul_hi(a.v[i], b.v[0]);
        t[i]     = ptx_mul_lo(a.v[i + 1], b.v[0]);
        t[i + 1] = ptx_mul_hi(a.v[i + 1], b.v[0]);
    }
    mont_reduce_step<P>(s, t);
#pragma unroll
    for (int j = 1; j < N; j += 2) {
        mont_mad_step<P>(s, t, a.v, b.v[j]);              // even: t, odd: s
        if (j + 1 < N) mont_mad_step<P>(t, s, a.v, b.v[j + 1]);   // even: s, odd: t
    }
    // N is even, so the loop ends after a (s, t) step: even array t, odd array s.
    Fe<P> r;
    r.v[0] = ptx_add_cc3(s[0], t[1]);
#pragma unroll
    for (int i = 1; i < N - 1; ++i) r.v[i] = ptx_addc_cc3(s[i], t[i + 1]);
    r.v[N - 1] = ptx_addc3(s[N - 1], 0u);
    fe_final_sub(r);
    return r;
}

template <class P> ZKB_DEV Fe<P> mont_sqr(const Fe<P>& a) { return mont_mul(a, a); }

// standard -> Montgomery and back
template <class P> ZKB_DEV Fe<P> to_mont(const Fe<P>& a) { return mont_mul(a, fe_r2<P>()); }
template <class P> ZKB_DEV Fe<P> from_mont(const Fe<P>& a) {
    Fe<P> one = fe_zero<P>();
    one.v[0] = 1;
    return mont_mul(a, one);
}

// a^(p-2) in Montgomery form (maps 0 to 0, like the reference's Fermat inverse,
// bls12-381.cu:597-609).  Plain square-and-multiply over the bits of p-2.
template <class P> __host__ __device__ constexpr uint32_t fe_pm2_limb(int i) {
    // limb i of p - 2, with the borrow rippled through at compile time
    uint32_t borrow = 2u, out = 0u;
    for (int k = 0; k <= i; ++k) {
        const uint32_t m = P::mod(k);
        out = m - borrow;
        borrow = (m < borrow) ? 1u : 0u;
    }
    return out;
}

template <class P> ZKB_DEV Fe<P> mont_inv_fermat(const Fe<P>& a) {
    constexpr int N = P::N;
    Fe<P> res = fe_mont_one<P>();
    Fe<P> base = a;
    uint32_t ex[N];
#pragma unroll
    for (int i = 0; i < N; ++i) ex[i] = fe_pm2_limb<P>(i);
#pragma unroll 1
    for (int i = 0; i < N; ++i) {
        const uint32_t e = ex[i];
        const int nbits = 32;
#pragma unroll 1
        for (int k = 0; k < nbits; ++k) {
            if ((e >> k) & 1u) res = mont_mul(res, base);
            base = mont_sqr(base);
        }
    }
    return res;
}

// x / 2^s mod p for x in [0, p) and 1 <= s <= 31: add the multiple m p that clears the low s bits
// (m = -x / p mod 2^s), then shift; the sum is below 2^s p, which fits N + 1 limbs.
template <class P> ZKB_DEV void fe_div_pow2(Fe<P>& x, uint32_t s) {
    constexpr int N = P::N;
    const uint32_t m = (x.v[0] * P::M0) & ((1u << s) - 1u);
    uint32_t t[N + 1];
#pragma unroll
    for (int i = 0; i < N; ++i) t[i] = x.v[i];
    ptx_mad_lo_cc(t[0], P::mod(0), m);
#pragma unroll
    for (int i = 1; i < N; ++i) ptx_madc_lo_cc(t[i], P::mod(i), m);
    t[N] = ptx_addc3(0u, 0u);
    ptx_mad_hi_cc(t[1], P::mod(0), m);
#pragma unroll
    for (int i = 1; i < N; ++i) ptx_madc_hi_cc(t[i + 1], P::mod(i), m);
#pragma unroll
    for (int i = 0; i < N; ++i) x.v[i] = __funnelshift_r(t[i], t[i + 1], s);
}

// 1/a in Montgomery form for a in Montgomery form; 0 maps to 0 like the
// reference's Fermat inverse (bls12-381.cu:597-609), with the same value for
// every other input.  Binary extended Euclid on plain integers with u, v both
// odd: each pass replaces the larger of the two by their difference and strips all
// its trailing zero bits at once (up to 31 per pass), while x1, x2 follow so
// that u = x1 a, v = x2 a (mod p); the division of x1 by 2^s is one short
// multiply-add pass (fe_div_pow2).  The order of u and v is handled with selects,
// not branches, so the lanes of a warp stay together; about 0.7 * bits(p) passes,
// capped above the worst case bits(u) + bits(v).
template <class P> ZKB_DEV Fe<P> mont_inv(const Fe<P>& a) {
    constexpr int N = P::N;
    if (fe_is_zero(a)) return a;
    Fe<P> u = a, v, x1 = fe_zero<P>(), x2 = fe_zero<P>();
#pragma unroll
    for (int i = 0; i < N; ++i) v.v[i] = P::mod(i);
    x1.v[0] = 1u;
#pragma unroll 1
    for (int it = 0; it < 64 * N + 64; ++it) {
        if (u.v[0] & 1u) {
            // d = u - v; on a borrow the roles swap: v <- u, u <- v - u
            Fe<P> d;
            d.v[0] = ptx_sub_cc3(u.v[0], v.v[0]);
#pragma unroll
            for (int i = 1; i < N; ++i) d.v[i] = ptx_subc_cc3(u.v[i], v.v[i]);
            const uint32_t borrow = ptx_subc3(0u, 0u);      // all-ones when u < v
            if (fe_is_zero(d)) break;                        // u == v == gcd == 1
            Fe<P> nd;
            nd.v[0] = ptx_sub_cc3(0u, d.v[0]);
#pragma unroll
            for (int i = 1; i < N - 1; ++i) nd.v[i] = ptx_subc_cc3(0u, d.v[i]);
            nd.v[N - 1] = ptx_subc3(0u, d.v[N - 1]);
            Fe<P> xa, xc;
#pragma unroll
            for (int i = 0; i < N; ++i) {
                v.v[i] = borrow ? u.v[i] : v.v[i];
                u.v[i] = borrow ? nd.v[i] : d.v[i];
                xa.v[i] = borrow ? x2.v[i] : x1.v[i];
                xc.v[i] = borrow ? x1.v[i] : x2.v[i];
            }
            x1 = fe_sub(xa, xc);
            x2 = xc;
        }
        // u is even and not zero: strip up to 31 trailing zero bits
        uint32_t s = u.v[0] ? (uint32_t)(__ffs((int)u.v[0]) - 1) : 31u;
        if (s > 31u) s = 31u;
#pragma unroll
        for (int i = 0; i < N - 1; ++i) u.v[i] = __funnelshift_r(u.v[i], u.v[i + 1], s);
        u.v[N - 1] >>= s;
        fe_div_pow2(x1, s);
    }
    // u = v = 1 = x1 (a R): x1 is (a R)^-1 as a plain residue; the Montgomery form of 1/a is that times R^2
    return mont_mul(mont_mul(x1, fe_r2<P>()), fe_r2<P>());
}

// ---------------------------------------------------------------------------
// Small-integer conversions used by the fixed-point file formats
// (fr-tensor.cu:686-711 and :924-945).
// ---------------------------------------------------------------------------
ZKB_DEV Fr fr_from_u64(unsigned long long x) {
    Fr r = fe_zero<FrParams>();
    r.v[0] = (uint32_t)x;
    r.v[1] = (uint32_t)(x >> 32);
    return r;
}
ZKB_DEV Fr fr_from_i64(long long x) {
    if (x >= 0) return fr_from_u64((unsigned long long)x);
    return fe_neg(fr_from_u64(0ull - (unsigned long long)x));
}
ZKB_DEV bool fr_fits_u64(const Fr& a) {
    return (a.v[2] | a.v[3] | a.v[4] | a.v[5] | a.v[6] | a.v[7]) == 0;
}
// Same mapping as scalar_to_long: a value that is not a small non-negative
// integer is read as -(r - a); magnitudes beyond 64 bits collapse to 0.
ZKB_DEV long long fr_to_i64(const Fr& a) {
    if (fr_fits_u64(a) && !(a.v[1] >> 31))
        return (long long)(((unsigned long long)a.v[1] << 32) | a.v[0]);
    Fr n = fe_neg(a);
    unsigned long long mag = fr_fits_u64(n) ? (((unsigned long long)n.v[1] << 32) | n.v[0]) : 0ull;
    return -(long long)mag;
}
ZKB_DEV int fr_to_i32(const Fr& a) {
    const uint32_t hi = a.v[1] | a.v[2] | a.v[3] | a.v[4] | a.v[5] | a.v[6] | a.v[7];
    if (!hi && !(a.v[0] >> 31)) return (int)a.v[0];
    Fr n = fe_neg(a);
    const uint32_t nhi = n.v[1] | n.v[2] | n.v[3] | n.v[4] | n.v[5] | n.v[6] | n.v[7];
    const uint32_t mag = nhi ? 0u : n.v[0];
    return -(int)mag;
}

// 128-bit vector moves for field elements
template <class P> ZKB_DEV Fe<P> fe_load(const Fe<P>* p) {
    Fe<P> r;
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < P::N / 4; ++i) {
        uint4 w = q[i];
        r.v[4 * i] = w.x; r.v[4 * i + 1] = w.y; r.v[4 * i + 2] = w.z; r.v[4 * i + 3] = w.w;
    }
    return r;
}
template <class P> ZKB_DEV void fe_store(Fe<P>* p, const Fe<P>& a) {
    uint4* q = reinterpret_cast<uint4*>(p);
#pragma unroll
    for (int i = 0; i < P::N / 4; ++i)
        q[i] = make_uint4(a.v[4 * i], a.v[4 * i + 1], a.v[4 * i + 2], a.v[4 * i + 3]);
}

}  // namespace zkb
