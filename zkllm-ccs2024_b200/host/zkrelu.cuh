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
    uint scaling_factor;
    tLookupRange tl_rem;   // table for the remainder
    FrTensor decomp(const FrTensor& X, FrTensor& sign, FrTensor& abs, FrTensor& rem);
    FrTensor *sign_tensor_ptr, *abs_tensor_ptr, *rem_tensor_ptr, *m_tensor_ptr;

    zkReLU(uint scaling_factor);
    FrTensor operator()(const FrTensor& X);
    void prove(const FrTensor& Z, const FrTensor& A);
    ~zkReLU();
};

#endif
