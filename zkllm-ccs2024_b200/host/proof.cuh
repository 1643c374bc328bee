// Proof primitives (reference: proof.cuh:13-50): claims, weight-claim
// verification, the product-of-tensors sumcheck and the three legacy
// adjacent-pair sumchecks.
#ifndef PROOF_CUH
#define PROOF_CUH

#include <random>
#include <vector>

#include "bls12-381.cuh"
#include "fr-tensor.cuh"
#include "g1-tensor.cuh"
#include "polynomial.cuh"

struct Claim {
    Fr_t claim;
    std::vector<std::vector<Fr_t>> u;
    std::vector<uint> dims;
};

struct Weight;
void verifyWeightClaim(const Weight& w, const Claim& c);

bool operator==(const Fr_t& a, const Fr_t& b);
bool operator!=(const Fr_t& a, const Fr_t& b);

// sumcheck of prod_k X_k weighted by eq(u, .): appends one degree-K polynomial per round
Fr_t multi_hadamard_sumchecks(const Fr_t& claim, const vector<FrTensor>& Xs, const vector<Fr_t>& u, const vector<Fr_t>& v,
                              vector<Polynomial>& proof);

// Legacy sumchecks over adjacent pairs.  Their product terms carry the factor
// 2^-256 that the reference's kernels leave on them (proof.cu:23-26, 116-119).
vector<Fr_t> inner_product_sumcheck(const FrTensor& a, const FrTensor& b, vector<Fr_t> u);
vector<Fr_t> hadamard_product_sumcheck(const FrTensor& a, const FrTensor& b, vector<Fr_t> u, vector<Fr_t> v);
vector<Fr_t> binary_sumcheck(const FrTensor& a, vector<Fr_t> u, vector<Fr_t> v);

#endif
