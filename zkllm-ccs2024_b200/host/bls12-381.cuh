// Type names of the reference's field and curve header, for code that includes
// "bls12-381.cuh" directly.  Only the data layouts are provided (the reference's
// bls12-381.cuh:116-120, 221-225, 424-433); the arithmetic lives in the CUDA
// library behind the C ABI.
#pragma once
#include "../../include/zkllm_b200.h"

typedef zkb_fr_t blstrs__scalar__Scalar;
typedef zkb_fq_t blstrs__fp__Fp;
typedef zkb_g1_affine_t blstrs__g1__G1Affine_affine;
typedef zkb_g1_t blstrs__g1__G1Affine_jacobian;
