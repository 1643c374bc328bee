// Pedersen/Hyrax row commitment (reference: commitment.cuh:8-36).  A Commitment
// is the tensor of generators; commit* return one G1 point per row of the
// committed tensor, open/me_open return the multilinear opening.
#ifndef COMMITMENT_CUH
#define COMMITMENT_CUH

#include "fr-tensor.cuh"
#include "g1-tensor.cuh"
#include "proof.cuh"

class Commitment : public G1TensorJacobian {
public:
    using G1TensorJacobian::G1TensorJacobian;
    using G1TensorJacobian::operator+;
    using G1TensorJacobian::operator-;
    using G1TensorJacobian::operator*;
    using G1TensorJacobian::operator*=;

    // t holds t.size / size rows of `size` scalars
    static Commitment random(uint n_generators);

    G1TensorJacobian commit_int(const FrTensor& values) const;                    // scalars that encode int32 values
    G1TensorJacobian commit_int_multi(const vector<FrTensor>& tensors) const;     // rows of several tensors, concatenated
    G1TensorJacobian commit(const FrTensor& values) const;                        // full-width scalars

    // opening of the committed tensor at `point`: rows folded by the high challenges, then me_open
    Fr_t open(const FrTensor& values, const G1TensorJacobian& row_commitments, const vector<Fr_t>& point) const;
    static Fr_t me_open(const FrTensor& row, const Commitment& gens, vector<Fr_t>::const_iterator first,
                        vector<Fr_t>::const_iterator last, vector<G1Jacobian_t>& transcript);
};

// a committed parameter: generators, padded integer weights, row commitments
struct Weight {
    Commitment generator;
    FrTensor weight;
    G1TensorJacobian com;
    uint in_dim, out_dim;
};

// reads the three files one parameter has (-pp.bin, -int.bin, -commitment.bin)
Weight create_weight(string pp_file, string int_file, string commitment_file, uint in_dim, uint out_dim);

#endif
