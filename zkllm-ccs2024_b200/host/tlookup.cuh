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
    tLookup(const FrTensor& table_values);

    // multiplicities of n table indices (a device array of uint)
    FrTensor prep(const uint* device_indices, const uint n);

    // S: looked-up values (D, a power of two, a multiple of the table size), m: multiplicities
    Fr_t prove(const FrTensor& S, const FrTensor& m, const Fr_t& alpha, const Fr_t& beta,
               const vector<Fr_t>& u, const vector<Fr_t>& v, vector<Polynomial>& transcript);

protected:
    // set by tLookupRange: entry j of the table is range_first + j, so the index of a looked-up
    // value is known without a search (the prover then reads 1/(S + beta) from the table's inverses)
    bool is_range = false;
    int range_first = 0;
};

class tLookupRange : public tLookup {
public:
    const int low;
    tLookupRange(int first, uint count);            // table = first, first + 1, ..., padded to a power of two

    using tLookup::prove;
    FrTensor prep(const FrTensor& values);
    FrTensor prep(const int* device_values, const uint n);
};

class tLookupRangeMapping : public tLookupRange {
public:
    FrTensor mapped_vals;
    tLookupRangeMapping(int first, uint count, const FrTensor& images);

    using tLookupRange::prep;
    // (mapped values, multiplicities)
    pair<FrTensor, FrTensor> operator()(const FrTensor& values);
    pair<FrTensor, FrTensor> operator()(const int* device_values, const uint n);

    // lookup of the pairs (S_in, S_out) combined as S_in + r * S_out
    Fr_t prove(const FrTensor& S_in, const FrTensor& S_out, const FrTensor& m, const Fr_t& r, const Fr_t& alpha,
               const Fr_t& beta, const vector<Fr_t>& u, const vector<Fr_t>& v, vector<Polynomial>& transcript);
};

#endif
