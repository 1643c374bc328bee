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
    Rescaling(uint divisor);
    ~Rescaling();

    uint scaling_factor;        // the divisor
    tLookupRange tl_rem;        // remainders lie in [-divisor/2, divisor/2)
    FrTensor* rem_tensor_ptr;   // remainders of the last operator() call (owned)

    // quotient rounded to nearest; keeps the remainders for prove()
    FrTensor operator()(const FrTensor& values);
    // values = quotients * divisor + remainders at a random point, and the remainders' range proof
    vector<Claim> prove(const FrTensor& values, const FrTensor& quotients);
    Rescaling decomp(const FrTensor& values, FrTensor& remainders);   // declared by the reference, defined nowhere
};

#endif
