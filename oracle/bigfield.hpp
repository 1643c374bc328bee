// TEST INFRASTRUCTURE ONLY - CPU restatement used as the checker and as the
// timed CPU baseline.  Nothing in the product library includes this file.
//
// Prime-field arithmetic for BLS12-381 Fr (4 x u64) and Fq (6 x u64) on the
// host, Montgomery multiplication through unsigned __int128, plus the Jacobian
// G1 group law.  The reference keeps these operations in vendored third-party
// device code (bls12-381.cu:289-1044 field ops, :1361-1464 group law); this is
// an independent implementation of the same mathematics, checked against the
// Python big-integer oracle (oracle/pyref.py) in tests/test_oracle_cpp.py.
#pragma once
#include <cstdint>
#include <cstring>

namespace zko {

typedef unsigned __int128 u128;

template <int N>
struct Big {
    uint64_t l[N];
};

template <int N>
struct FieldParams;

template <>
struct FieldParams<4> {   // Fr
    static constexpr uint64_t mod[4] = {0xffffffff00000001ull, 0x53bda402fffe5bfeull, 0x3339d80809a1d805ull, 0x73eda753299d7d48ull};
    static constexpr uint64_t r2[4] = {0xc999e990f3f29c6dull, 0x2b6cedcb87925c23ull, 0x05d314967254398full, 0x0748d9d99f59ff11ull};
    static constexpr uint64_t m0 = 0xfffffffeffffffffull;
};
template <>
struct FieldParams<6> {   // Fq
    static constexpr uint64_t mod[6] = {0xb9feffffffffaaabull, 0x1eabfffeb153ffffull, 0x6730d2a0f6b0f624ull,
                                        0x64774b84f38512bfull, 0x4b1ba7b6434bacd7ull, 0x1a0111ea397fe69aull};
    static constexpr uint64_t r2[6] = {0xf4df1f341c341746ull, 0x0a76e6a609d104f1ull, 0x8de5476c4c95b6d5ull,
                                       0x67eb88a9939d83c0ull, 0x9a793e85b519952dull, 0x11988fe592cae3aaull};
    static constexpr uint64_t m0 = 0x89f3fffcfffcfffdull;
};

template <int N>
struct Field {
    typedef Big<N> E;
    typedef FieldParams<N> P;

    static E zero() { E r; std::memset(&r, 0, sizeof(r)); return r; }
    static E from_u64(uint64_t x) { E r = zero(); r.l[0] = x; return r; }
    static E modulus() { E r; for (int i = 0; i < N; ++i) r.l[i] = P::mod[i]; return r; }
    static bool is_zero(const E& a) { uint64_t t = 0; for (int i = 0; i < N; ++i) t |= a.l[i]; return t == 0; }
    static bool eq(const E& a, const E& b) { return std::memcmp(&a, &b, sizeof(E)) == 0; }
    static bool geq(const E& a, const E& b) {
        for (int i = N - 1; i >= 0; --i) if (a.l[i] != b.l[i]) return a.l[i] > b.l[i];
        return true;
    }
    static E raw_add(const E& a, const E& b, uint64_t* carry) {
        E r; uint64_t c = 0;
        for (int i = 0; i < N; ++i) { u128 s = (u128)a.l[i] + b.l[i] + c; r.l[i] = (uint64_t)s; c = (uint64_t)(s >> 64); }
        *carry = c; return r;
    }
    static E raw_sub(const E& a, const E& b, uint64_t* borrow) {
        E r; uint64_t bo = 0;
        for (int i = 0; i < N; ++i) { u128 d = (u128)a.l[i] - b.l[i] - bo; r.l[i] = (uint64_t)d; bo = (uint64_t)(d >> 64) & 1; }
        *borrow = bo; return r;
    }
    static E add(const E& a, const E& b) {
        uint64_t c, bo; E s = raw_add(a, b, &c);
        if (c || geq(s, modulus())) s = raw_sub(s, modulus(), &bo);
        return s;
    }
    static E sub(const E& a, const E& b) {
        uint64_t bo, c; E d = raw_sub(a, b, &bo);
        if (bo) d = raw_add(d, modulus(), &c);
        return d;
    }
    static E neg(const E& a) { return sub(zero(), a); }
    static E dbl(const E& a) { return add(a, a); }
    // a*b*2^(-64N) mod p
    static E mmul(const E& a, const E& b) {
        uint64_t t[N + 2];
        for (int i = 0; i < N + 2; ++i) t[i] = 0;
        for (int i = 0; i < N; ++i) {
            uint64_t carry = 0;
            for (int j = 0; j < N; ++j) {
                u128 cur = (u128)a.l[j] * b.l[i] + t[j] + carry;
                t[j] = (uint64_t)cur; carry = (uint64_t)(cur >> 64);
            }
            u128 top = (u128)t[N] + carry;
            t[N] = (uint64_t)top; t[N + 1] = (uint64_t)(top >> 64);
            const uint64_t m = t[0] * P::m0;
            u128 cur = (u128)m * P::mod[0] + t[0];
            carry = (uint64_t)(cur >> 64);
            for (int j = 1; j < N; ++j) {
                cur = (u128)m * P::mod[j] + t[j] + carry;
                t[j - 1] = (uint64_t)cur; carry = (uint64_t)(cur >> 64);
            }
            top = (u128)t[N] + carry;
            t[N - 1] = (uint64_t)top;
            t[N] = t[N + 1] + (uint64_t)(top >> 64);
        }
        E r; for (int i = 0; i < N; ++i) r.l[i] = t[i];
        uint64_t bo;
        if (t[N] || geq(r, modulus())) r = raw_sub(r, modulus(), &bo);
        return r;
    }
    static E r2() { E r; for (int i = 0; i < N; ++i) r.l[i] = P::r2[i]; return r; }
    static E to_mont(const E& a) { return mmul(a, r2()); }
    static E from_mont(const E& a) { return mmul(a, from_u64(1)); }
    static E mul_std(const E& a, const E& b) { return mmul(to_mont(a), b); }   // standard-form product
    static E pow_mont(const E& a_mont, const E& e) {
        E acc = to_mont(from_u64(1)), base = a_mont;
        for (int i = 0; i < 64 * N; ++i) {
            if ((e.l[i >> 6] >> (i & 63)) & 1) acc = mmul(acc, base);
            base = mmul(base, base);
        }
        return acc;
    }
    static E inv_mont(const E& a_mont) {   // Fermat, 0 -> 0
        uint64_t bo; E e = raw_sub(modulus(), from_u64(2), &bo);
        return pow_mont(a_mont, e);
    }
    static E inv_std(const E& a) { return from_mont(inv_mont(to_mont(a))); }
};

typedef Field<4> Fr;
typedef Field<6> Fq;
typedef Big<4> FrE;
typedef Big<6> FqE;

// ---- G1, Jacobian over Montgomery-form Fq; Z == 0 is the identity -----------------
struct G1 { FqE x, y, z; };
struct G1A { FqE x, y; bool inf; };

inline G1 g1_zero() { G1 r; r.x = r.y = r.z = Fq::zero(); return r; }
inline bool g1_is_zero(const G1& p) { return Fq::is_zero(p.z); }
inline G1 g1_neg(const G1& p) { G1 r = p; r.y = Fq::neg(p.y); return r; }

inline G1 g1_double(const G1& p) {   // dbl-2009-l
    if (g1_is_zero(p)) return p;
    FqE A = Fq::mmul(p.x, p.x), B = Fq::mmul(p.y, p.y), C = Fq::mmul(B, B);
    FqE t = Fq::add(p.x, B);
    FqE D = Fq::dbl(Fq::sub(Fq::sub(Fq::mmul(t, t), A), C));
    FqE E = Fq::add(Fq::dbl(A), A), F = Fq::mmul(E, E);
    G1 r;
    r.x = Fq::sub(F, Fq::dbl(D));
    r.y = Fq::sub(Fq::mmul(E, Fq::sub(D, r.x)), Fq::dbl(Fq::dbl(Fq::dbl(C))));
    r.z = Fq::dbl(Fq::mmul(p.y, p.z));
    return r;
}
inline G1 g1_add(const G1& p, const G1& q) {   // add-2007-bl
    if (g1_is_zero(p)) return q;
    if (g1_is_zero(q)) return p;
    FqE Z1Z1 = Fq::mmul(p.z, p.z), Z2Z2 = Fq::mmul(q.z, q.z);
    FqE U1 = Fq::mmul(p.x, Z2Z2), U2 = Fq::mmul(q.x, Z1Z1);
    FqE S1 = Fq::mmul(Fq::mmul(p.y, q.z), Z2Z2), S2 = Fq::mmul(Fq::mmul(q.y, p.z), Z1Z1);
    FqE H = Fq::sub(U2, U1), rr = Fq::sub(S2, S1);
    if (Fq::is_zero(H)) return Fq::is_zero(rr) ? g1_double(p) : g1_zero();
    rr = Fq::dbl(rr);
    FqE H2 = Fq::dbl(H), I = Fq::mmul(H2, H2), J = Fq::mmul(H, I), V = Fq::mmul(U1, I);
    G1 r;
    r.x = Fq::sub(Fq::sub(Fq::mmul(rr, rr), J), Fq::dbl(V));
    r.y = Fq::sub(Fq::mmul(rr, Fq::sub(V, r.x)), Fq::dbl(Fq::mmul(S1, J)));
    FqE zz = Fq::add(p.z, q.z);
    r.z = Fq::mmul(Fq::sub(Fq::sub(Fq::mmul(zz, zz), Z1Z1), Z2Z2), H);
    return r;
}
inline G1 g1_add_affine(const G1& p, const G1A& q) {   // madd-2007-bl
    if (q.inf) return p;
    if (g1_is_zero(p)) { G1 r; r.x = q.x; r.y = q.y; r.z = Fq::to_mont(Fq::from_u64(1)); return r; }
    FqE Z1Z1 = Fq::mmul(p.z, p.z), U2 = Fq::mmul(q.x, Z1Z1), S2 = Fq::mmul(Fq::mmul(q.y, p.z), Z1Z1);
    FqE H = Fq::sub(U2, p.x), rr = Fq::sub(S2, p.y);
    if (Fq::is_zero(H)) return Fq::is_zero(rr) ? g1_double(p) : g1_zero();
    rr = Fq::dbl(rr);
    FqE HH = Fq::mmul(H, H), I = Fq::dbl(Fq::dbl(HH)), J = Fq::mmul(H, I), V = Fq::mmul(p.x, I);
    G1 r;
    r.x = Fq::sub(Fq::sub(Fq::mmul(rr, rr), J), Fq::dbl(V));
    r.y = Fq::sub(Fq::mmul(rr, Fq::sub(V, r.x)), Fq::dbl(Fq::mmul(p.y, J)));
    FqE zh = Fq::add(p.z, H);
    r.z = Fq::sub(Fq::sub(Fq::mmul(zh, zh), Z1Z1), HH);
    return r;
}
inline G1A g1_to_affine(const G1& p) {
    G1A r;
    if (g1_is_zero(p)) { r.x = r.y = Fq::zero(); r.inf = true; return r; }
    FqE zi = Fq::inv_mont(p.z), zi2 = Fq::mmul(zi, zi);
    r.x = Fq::mmul(p.x, zi2);
    r.y = Fq::mmul(p.y, Fq::mmul(zi2, zi));
    r.inf = false;
    return r;
}
inline G1A g1a_neg(const G1A& p) { G1A r = p; r.y = Fq::neg(p.y); return r; }

}  // namespace zko
