// BLS12-381 G1 group law on Jacobian coordinates over Montgomery-form Fq.
//
// Memory layout matches the reference's G1Jacobian_t / G1Affine_t
// (bls12-381.cuh:424-433): three (two) consecutive 12-limb Fq values.  The
// identity is any triple with Z == 0, as in the reference.  The formulas are the
// textbook ones the reference also uses (bls12-381.cu:1361-1464): doubling
// "dbl-2009-l", mixed addition "madd-2007-bl", full addition "add-2007-bl" for
// the curve y^2 = x^3 + 4 (a = 0).  Representatives (X:Y:Z) are not unique, so
// equality with the reference is defined on the affine point (X/Z^2, Y/Z^3).
#pragma once
#include "field.cuh"

namespace zkb {

struct __align__(16) G1Jac { Fq x, y, z; };   // 144 bytes
struct __align__(16) G1Aff { Fq x, y; };      //  96 bytes; (0,0) encodes the identity

#ifdef ZKB_FQ_NOINLINE
__device__ __noinline__ static Fq fq_mul(const Fq& a, const Fq& b) { return mont_mul<FqParams>(a, b); }
#else
ZKB_DEV Fq fq_mul(const Fq& a, const Fq& b) { return mont_mul<FqParams>(a, b); }
#endif
ZKB_DEV Fq fq_sqr(const Fq& a) { return fq_mul(a, a); }
ZKB_DEV Fq fq_add(const Fq& a, const Fq& b) { return fe_add<FqParams>(a, b); }
ZKB_DEV Fq fq_sub(const Fq& a, const Fq& b) { return fe_sub<FqParams>(a, b); }
ZKB_DEV Fq fq_dbl(const Fq& a) { return fe_add<FqParams>(a, a); }

ZKB_DEV G1Jac g1_identity() {
    G1Jac r;
    r.x = fe_zero<FqParams>(); r.y = fe_zero<FqParams>(); r.z = fe_zero<FqParams>();
    return r;
}
ZKB_DEV bool g1_is_identity(const G1Jac& p) { return fe_is_zero(p.z); }
ZKB_DEV bool g1_aff_is_identity(const G1Aff& p) { return fe_is_zero(p.x) && fe_is_zero(p.y); }

ZKB_DEV G1Jac g1_neg(const G1Jac& p) {
    G1Jac r = p;
    r.y = fe_neg<FqParams>(p.y);
    return r;
}
ZKB_DEV G1Aff g1_aff_neg(const G1Aff& p) {
    G1Aff r = p;
    r.y = fe_neg<FqParams>(p.y);   // -(0) = 0 keeps the identity encoding
    return r;
}

// 2M + 5S
ZKB_DEV G1Jac g1_double(const G1Jac& p) {
    if (g1_is_identity(p)) return p;
    Fq a = fq_sqr(p.x);
    Fq b = fq_sqr(p.y);
    Fq c = fq_sqr(b);
    Fq d = fq_sub(fq_sub(fq_sqr(fq_add(p.x, b)), a), c);
    d = fq_dbl(d);
    Fq e = fq_add(fq_dbl(a), a);
    Fq f = fq_sqr(e);
    G1Jac r;
    r.z = fq_mul(p.y, p.z);
    r.z = fq_dbl(r.z);
    r.x = fq_sub(f, fq_dbl(d));
    Fq c8 = fq_dbl(fq_dbl(fq_dbl(c)));
    r.y = fq_sub(fq_mul(e, fq_sub(d, r.x)), c8);
    return r;
}

// Jacobian + affine, 7M + 4S.  Handles identity operands, P + P and P + (-P).
ZKB_DEV G1Jac g1_add_mixed(const G1Jac& p, const G1Aff& q) {
    if (g1_aff_is_identity(q)) return p;
    if (g1_is_identity(p)) {
        G1Jac r;
        r.x = q.x; r.y = q.y; r.z = fe_mont_one<FqParams>();
        return r;
    }
    Fq z1z1 = fq_sqr(p.z);
    Fq u2 = fq_mul(q.x, z1z1);
    Fq s2 = fq_mul(fq_mul(q.y, p.z), z1z1);
    Fq h = fq_sub(u2, p.x);
    Fq rr = fq_sub(s2, p.y);
    if (fe_is_zero(h)) {
        if (fe_is_zero(rr)) return g1_double(p);
        return g1_identity();
    }
    rr = fq_dbl(rr);
    Fq hh = fq_sqr(h);
    Fq i = fq_dbl(fq_dbl(hh));
    Fq j = fq_mul(h, i);
    Fq v = fq_mul(p.x, i);
    G1Jac r;
    r.x = fq_sub(fq_sub(fq_sqr(rr), j), fq_dbl(v));
    Fq t = fq_mul(p.y, j);
    r.y = fq_sub(fq_mul(rr, fq_sub(v, r.x)), fq_dbl(t));
    r.z = fq_sub(fq_sub(fq_sqr(fq_add(p.z, h)), z1z1), hh);
    return r;
}

// Jacobian + Jacobian, 11M + 5S.
ZKB_DEV G1Jac g1_add(const G1Jac& p, const G1Jac& q) {
    if (g1_is_identity(p)) return q;
    if (g1_is_identity(q)) return p;
    Fq z1z1 = fq_sqr(p.z);
    Fq z2z2 = fq_sqr(q.z);
    Fq u1 = fq_mul(p.x, z2z2);
    Fq u2 = fq_mul(q.x, z1z1);
    Fq s1 = fq_mul(fq_mul(p.y, q.z), z2z2);
    Fq s2 = fq_mul(fq_mul(q.y, p.z), z1z1);
    Fq h = fq_sub(u2, u1);
    Fq rr = fq_sub(s2, s1);
    if (fe_is_zero(h)) {
        if (fe_is_zero(rr)) return g1_double(p);
        return g1_identity();
    }
    rr = fq_dbl(rr);
    Fq i = fq_sqr(fq_dbl(h));
    Fq j = fq_mul(h, i);
    Fq v = fq_mul(u1, i);
    G1Jac r;
    r.x = fq_sub(fq_sub(fq_sqr(rr), j), fq_dbl(v));
    Fq t = fq_mul(s1, j);
    r.y = fq_sub(fq_mul(rr, fq_sub(v, r.x)), fq_dbl(t));
    r.z = fq_mul(fq_sub(fq_sub(fq_sqr(fq_add(p.z, q.z)), z1z1), z2z2), h);
    return r;
}

// ---------------------------------------------------------------------------
// Extended Jacobian ("XYZZ") accumulator: x = X / ZZ, y = Y / ZZZ with
// ZZ^3 == ZZZ^2; ZZZ == 0 is the identity.  Adding an affine point costs
// 8M + 2S ("madd-2008-s") against 7M + 4S for Jacobian coordinates, and a
// squaring costs a full product here, so a long chain of mixed additions is
// one product per step cheaper.  Used only for running sums inside kernels;
// results leave as Jacobian points.
// ---------------------------------------------------------------------------
struct __align__(16) G1Xyzz { Fq x, y, zz, zzz; };

ZKB_DEV G1Xyzz xyzz_identity() {
    G1Xyzz r;
    r.x = fe_zero<FqParams>(); r.y = fe_zero<FqParams>(); r.zz = fe_zero<FqParams>(); r.zzz = fe_zero<FqParams>();
    return r;
}
ZKB_DEV bool xyzz_is_identity(const G1Xyzz& p) { return fe_is_zero(p.zzz); }

// 2 * q for an affine q that is not the identity ("mdbl-2008-s-1", a = 0)
ZKB_DEV G1Xyzz xyzz_double_affine(const G1Aff& q) {
    const Fq u = fq_dbl(q.y);
    const Fq v = fq_sqr(u);
    const Fq w = fq_mul(u, v);
    const Fq s = fq_mul(q.x, v);
    const Fq xx = fq_sqr(q.x);
    const Fq m = fq_add(fq_dbl(xx), xx);
    G1Xyzz r;
    r.x = fq_sub(fq_sqr(m), fq_dbl(s));
    r.y = fq_sub(fq_mul(m, fq_sub(s, r.x)), fq_mul(w, q.y));
    r.zz = v;
    r.zzz = w;
    return r;
}

// 2 * p ("dbl-2008-s-1", a = 0): 6M + 3S
ZKB_DEV G1Xyzz xyzz_double(const G1Xyzz& p) {
    if (xyzz_is_identity(p)) return p;
    const Fq u = fq_dbl(p.y);
    const Fq v = fq_sqr(u);
    const Fq w = fq_mul(u, v);
    const Fq s = fq_mul(p.x, v);
    const Fq xx = fq_sqr(p.x);
    const Fq m = fq_add(fq_dbl(xx), xx);
    G1Xyzz r;
    r.x = fq_sub(fq_sqr(m), fq_dbl(s));
    r.y = fq_sub(fq_mul(m, fq_sub(s, r.x)), fq_mul(w, p.y));
    r.zz = fq_mul(v, p.zz);
    r.zzz = fq_mul(w, p.zzz);
    return r;
}

// XYZZ + affine.  Handles identity operands, P + P and P + (-P).
ZKB_DEV G1Xyzz xyzz_add_mixed(const G1Xyzz& p, const G1Aff& q) {
    if (g1_aff_is_identity(q)) return p;
    if (xyzz_is_identity(p)) {
        G1Xyzz r;
        r.x = q.x; r.y = q.y; r.zz = fe_mont_one<FqParams>(); r.zzz = fe_mont_one<FqParams>();
        return r;
    }
    const Fq u2 = fq_mul(q.x, p.zz);
    const Fq s2 = fq_mul(q.y, p.zzz);
    const Fq h = fq_sub(u2, p.x);
    const Fq rr = fq_sub(s2, p.y);
    if (fe_is_zero(h)) {
        if (fe_is_zero(rr)) return xyzz_double_affine(q);
        return xyzz_identity();
    }
    const Fq hh = fq_sqr(h);
    const Fq hhh = fq_mul(h, hh);
    const Fq v = fq_mul(p.x, hh);
    G1Xyzz r;
    r.x = fq_sub(fq_sub(fq_sqr(rr), hhh), fq_dbl(v));
    r.y = fq_sub(fq_mul(rr, fq_sub(v, r.x)), fq_mul(p.y, hhh));
    r.zz = fq_mul(p.zz, hh);
    r.zzz = fq_mul(p.zzz, hhh);
    return r;
}

// The same point in Jacobian coordinates with Z = ZZZ: Z^2 = ZZ^3, Z^3 = ZZZ^3.
ZKB_DEV G1Jac xyzz_to_jac(const G1Xyzz& p) {
    G1Jac r;
    r.x = fq_mul(p.x, fq_sqr(p.zz));
    r.y = fq_mul(p.y, fq_sqr(p.zzz));
    r.z = p.zzz;
    return r;
}

// k * p for a 256-bit scalar given as 8 raw little-endian limbs (the reference
// reads the standard-form scalar bits directly, g1-tensor.cu:445-453).
// Left-to-right double-and-add; the result is the same group element.
__device__ __noinline__ static G1Jac g1_mul_bits(const G1Jac& p, const Fr& k) {
    G1Jac acc = g1_identity();
    bool started = false;
#pragma unroll 1
    for (int i = 255; i >= 0; --i) {
        if (started) acc = g1_double(acc);
        if ((k.v[i >> 5] >> (i & 31)) & 1u) {
            acc = g1_add(acc, p);
            started = true;
        }
    }
    return acc;
}

// 128-bit vector moves
ZKB_DEV G1Jac g1_load(const G1Jac* p) {
    G1Jac r;
    r.x = fe_load(&p->x); r.y = fe_load(&p->y); r.z = fe_load(&p->z);
    return r;
}
ZKB_DEV void g1_store(G1Jac* p, const G1Jac& a) {
    fe_store(&p->x, a.x); fe_store(&p->y, a.y); fe_store(&p->z, a.z);
}
ZKB_DEV G1Aff g1_aff_load(const G1Aff* p) {
    G1Aff r;
    r.x = fe_load(&p->x); r.y = fe_load(&p->y);
    return r;
}
ZKB_DEV void g1_aff_store(G1Aff* p, const G1Aff& a) {
    fe_store(&p->x, a.x); fe_store(&p->y, a.y);
}

}  // namespace zkb
