// LogUp-style lookup arguments (reference: tlookup.cuh:11-52): a generic table,
// a range table [low, low + len) and a range table with mapped values.
#ifndef TLOOKUP_CUH
#define TLOOKUP_CUH

#include "bls12-381.cuh"
#include "fr-tensor.cuh"
#include "polynomial.cuh"
#include "proof.cuh"

class tLookup {
public:
    FrTensor table;
    tLookup(const FrTensor& table);

    // multiplicities of D table indices (a device array of uint)
    FrTensor prep(const uint* indices, const uint D);

    // S: looked-up values (D, a power of two, a multiple of the table size), m: multiplicities
    Fr_t prove(const FrTensor& S, const FrTensor& m, const Fr_t& alpha, const Fr_t& beta, const vector<Fr_t>& u,
               const vector<Fr_t>& v, vector<Polynomial>& proof);
};

class tLookupRange : public tLookup {
public:
    const int low;
    tLookupRange(int low, uint len);

    FrTensor prep(const int* vals, const uint D);   // device ints
    FrTensor prep(const FrTensor& vals);
    using tLookup::prove;
};

class tLookupRangeMapping : public tLookupRange {
public:
    FrTensor mapped_vals;
    tLookupRangeMapping(int low, uint len, const FrTensor& mapped_vals);

    using tLookupRange::prep;
    // (mapped values, multiplicities)
    pair<FrTensor, FrTensor> operator()(const int* vals, const uint D);
    pair<FrTensor, FrTensor> operator()(const FrTensor& mvals);

    Fr_t prove(const FrTensor& S_in, const FrTensor& S_out, const FrTensor& m, const Fr_t& r, const Fr_t& alpha, const Fr_t& beta,
               const vector<Fr_t>& u, const vector<Fr_t>& v, vector<Polynomial>& proof);
};

#endif
