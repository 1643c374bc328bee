// ReLU on fixed-point values with the rescaling folded in: decomposition into
// sign, magnitude and centred remainder (reference: zkrelu.cuh:11-22).  The
// reference's prove() is empty; so is this one.
#ifndef ZKRELU_CUH
#define ZKRELU_CUH

#include <cstddef>

#include "bls12-381.cuh"
#include "fr-tensor.cuh"
#include "proof.cuh"
#include "tlookup.cuh"

class zkReLU {
public:
    zkReLU(uint divisor);
    ~zkReLU();

    uint scaling_factor;   // the divisor of the rescaling
    tLookupRange tl_rem;   // remainders lie in [-divisor/2, divisor/2)
    // parts of the last operator() call (owned): sign bit, magnitude, remainder, remainder multiplicities
    FrTensor *sign_tensor_ptr, *abs_tensor_ptr, *rem_tensor_ptr, *m_tensor_ptr;

    // max(round(values / divisor), 0); keeps the parts
    FrTensor operator()(const FrTensor& values);
    FrTensor decomp(const FrTensor& values, FrTensor& sign_out, FrTensor& abs_out, FrTensor& rem_out);
    void prove(const FrTensor& pre_activation, const FrTensor& activation);
};

#endif
