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
    G1TensorJacobian commit(const FrTensor& t) const;                      // full-width scalars
    G1TensorJacobian commit_int(const FrTensor& t) const;                  // scalars that encode int32 values
    G1TensorJacobian commit_int_multi(const vector<FrTensor>& t) const;    // rows of several tensors, concatenated

    Fr_t open(const FrTensor& t, const G1TensorJacobian& c, const vector<Fr_t>& u) const;

    static Commitment random(uint size);
    static Fr_t me_open(const FrTensor& t, const Commitment& generators, vector<Fr_t>::const_iterator begin,
                        vector<Fr_t>::const_iterator end, vector<G1Jacobian_t>& proof);
};

struct Weight {
    Commitment generator;
    FrTensor weight;
    G1TensorJacobian com;
    uint in_dim;
    uint out_dim;
};

Weight create_weight(string generator_filename, string weight_filename, string com_filename, uint in_dim, uint out_dim);

#endif
