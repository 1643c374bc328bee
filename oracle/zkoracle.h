/* TEST INFRASTRUCTURE ONLY - C interface of the CPU restatement (libzkoracle.so).
 * Layouts: Fr = 8 x u32 standard form, G1 = 36 x u32 Jacobian in Montgomery form. */
#ifndef ZKORACLE_H
#define ZKORACLE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
int zko_threads(void);
void zko_fr_mul(const uint32_t* a, const uint32_t* b, uint32_t* out, size_t n);
void zko_fr_inv(const uint32_t* a, uint32_t* out, size_t n);
void zko_g1_add(const uint32_t* a, const uint32_t* b, uint32_t* out, size_t n);
void zko_g1_to_affine_jac(const uint32_t* a, uint32_t* out, size_t n);
void zko_g1_mul(const uint32_t* g, const uint32_t* k, uint32_t* out, size_t n);
void zko_commit_int_ref(const uint32_t* gens, size_t n, const int32_t* scalars, size_t m, uint32_t* out, int threads);
void zko_commit_int_pippenger(const uint32_t* gens, size_t n, const int32_t* scalars, size_t m, uint32_t* out, int threads);
void zko_mle_eval(const uint32_t* a, size_t n, const uint32_t* u, unsigned k, uint32_t* out);
int zko_zkip(const uint32_t* claim, const uint32_t* a, const uint32_t* b, size_t n, const uint32_t* u, unsigned k,
             uint32_t* polys, uint32_t* final_claim);
int zko_zkfc_prove(const uint32_t* X, const uint32_t* W, const uint32_t* Y, size_t B, size_t I, size_t O,
                   const uint32_t* ub, const uint32_t* ui, const uint32_t* uo, uint32_t* polys, uint32_t* claims);
int zko_tlookup_prove(const uint32_t* S, const uint32_t* T, const uint32_t* m, size_t D, size_t N,
                      const uint32_t* alpha, const uint32_t* beta, const uint32_t* u, const uint32_t* v,
                      uint32_t* polys, uint32_t* final_claim, int threads);
/* Commitment::me_open (commitment.cu:79-125): t[n] in the form the caller holds (raw limbs are read as scalar bits),
 * gens[n] Jacobian, u[k] standard form.  proof gets 3k+1 Jacobian points, out the final scalar. */
void zko_me_open(const uint32_t* t, const uint32_t* gens, size_t n, const uint32_t* u, unsigned k, uint32_t* proof, uint32_t* out);
#ifdef __cplusplus
}
#endif
#endif
