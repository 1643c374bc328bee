// G1 point tensors on the device (reference: g1-tensor.cuh:10-187).  Coordinates
// are Montgomery-form Fq; a Jacobian point with Z == 0 is the identity.  All group
// arithmetic runs in the CUDA library behind the C ABI.
#ifndef G1_TENSOR_CUH
#define G1_TENSOR_CUH

#include <iomanip>
#include <iostream>

#include "bls12-381.cuh"
#include "fr-tensor.cuh"
using namespace std;

typedef blstrs__fp__Fp Fp_t;

ostream& operator<<(ostream& os, const Fp_t& x);
ostream& operator<<(ostream& os, const G1Affine_t& g);
ostream& operator<<(ostream& os, const G1Jacobian_t& g);

// The BLS12-381 G1 generator and the field's Montgomery one, (coordinate * 2^384) mod p.
extern const Fp_t G1_generator_x_mont;
extern const Fp_t G1_generator_y_mont;
extern const Fp_t G1_ONE;
extern const G1Affine_t G1Affine_generator;
extern const G1Jacobian_t G1Jacobian_generator;
extern const G1Jacobian_t G1Jacobian_ZERO;

class G1Tensor {
public:
    const uint size;
    G1Tensor(uint size);
};

class G1TensorAffine;
class G1TensorJacobian;

class G1TensorAffine : public G1Tensor {
public:
    G1Affine_t* gpu_data;

    G1TensorAffine(const G1TensorAffine&);
    G1TensorAffine(uint size);
    G1TensorAffine(uint size, const G1Affine_t&);
    G1TensorAffine(uint size, const G1Affine_t* cpu_data);
    G1TensorAffine(const string& filename);
    ~G1TensorAffine();

    void save(const string& filename) const;
    G1Affine_t operator()(uint idx) const;
    G1TensorAffine operator-() const;
};

class G1TensorJacobian : public G1Tensor {
public:
    G1Jacobian_t* gpu_data;

    G1TensorJacobian(const G1TensorJacobian&);
    G1TensorJacobian(uint size);
    G1TensorJacobian(uint size, const G1Jacobian_t&);
    G1TensorJacobian(uint size, const G1Jacobian_t* cpu_data);
    G1TensorJacobian(const G1TensorAffine& affine_tensor);
    G1TensorJacobian(const string& filename);
    ~G1TensorJacobian();

    void save(const string& filename) const;
    G1Jacobian_t operator()(uint) const;

    G1TensorJacobian operator-() const;
    G1TensorJacobian operator+(const G1TensorJacobian&) const;
    G1TensorJacobian operator+(const G1TensorAffine&) const;
    G1TensorJacobian operator+(const G1Jacobian_t&) const;
    G1TensorJacobian operator+(const G1Affine_t&) const;
    G1TensorJacobian& operator+=(const G1TensorJacobian&);
    G1TensorJacobian& operator+=(const G1TensorAffine&);
    G1TensorJacobian& operator+=(const G1Jacobian_t&);
    G1TensorJacobian& operator+=(const G1Affine_t&);
    G1TensorJacobian operator-(const G1TensorJacobian&) const;
    G1TensorJacobian operator-(const G1TensorAffine&) const;
    G1TensorJacobian operator-(const G1Jacobian_t&) const;
    G1TensorJacobian operator-(const G1Affine_t&) const;
    G1TensorJacobian& operator-=(const G1TensorJacobian&);
    G1TensorJacobian& operator-=(const G1TensorAffine&);
    G1TensorJacobian& operator-=(const G1Jacobian_t&);
    G1TensorJacobian& operator-=(const G1Affine_t&);

    G1Jacobian_t sum() const;
    // out[i] = scalars[i] * (*this)[i mod size]; the scalar tensor may hold several rows
    G1TensorJacobian operator*(const FrTensor&) const;
    G1TensorJacobian& operator*=(const FrTensor&);
    // multilinear extension "in the exponent"
    G1Jacobian_t operator()(const vector<Fr_t>& u) const;
    G1TensorJacobian rowwise_sum(uint nrow, uint ncol) const;
};

#endif
