// Division of fixed-point values by a power-of-two scale with a range proof of
// the remainder (reference: rescaling.cuh:11-22).
#ifndef RESCALING_CUH
#define RESCALING_CUH

#include <cstddef>

#include "bls12-381.cuh"
#include "fr-tensor.cuh"
#include "proof.cuh"
#include "tlookup.cuh"

class Rescaling {
public:
    uint scaling_factor;
    tLookupRange tl_rem;        // remainders lie in [-sf/2, sf/2)
    Rescaling decomp(const FrTensor& X, FrTensor& rem);
    FrTensor* rem_tensor_ptr;   // remainders of the last operator() call

    Rescaling(uint scaling_factor);
    FrTensor operator()(const FrTensor& X);
    vector<Claim> prove(const FrTensor& X, const FrTensor& X_);
    ~Rescaling();
};

#endif
