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

// affine points (x, y), Montgomery coordinates
class G1TensorAffine : public G1Tensor {
public:
    G1Affine_t* gpu_data;

    G1TensorAffine(uint n);                               // uninitialised
    G1TensorAffine(uint n, const G1Affine_t& fill);
    G1TensorAffine(uint n, const G1Affine_t* host_points);
    G1TensorAffine(const string& path);                   // raw file, 96 bytes per point
    G1TensorAffine(const G1TensorAffine& src);
    ~G1TensorAffine();

    G1Affine_t operator()(uint index) const;
    G1TensorAffine operator-() const;
    void save(const string& path) const;
};

// Jacobian points (X, Y, Z), Z = 0 for the identity
class G1TensorJacobian : public G1Tensor {
public:
    G1Jacobian_t* gpu_data;

    G1TensorJacobian(uint n);                             // uninitialised
    G1TensorJacobian(uint n, const G1Jacobian_t& fill);
    G1TensorJacobian(uint n, const G1Jacobian_t* host_points);
    G1TensorJacobian(const string& path);                 // raw file, 144 bytes per point
    G1TensorJacobian(const G1TensorAffine& src);
    G1TensorJacobian(const G1TensorJacobian& src);
    ~G1TensorJacobian();

    G1Jacobian_t operator()(uint index) const;
    void save(const string& path) const;

    // elementwise group operations; a single point on the right is applied to every element
    G1TensorJacobian operator-() const;
    G1TensorJacobian operator+(const G1TensorJacobian& rhs) const;
    G1TensorJacobian operator-(const G1TensorJacobian& rhs) const;
    G1TensorJacobian operator+(const G1TensorAffine& rhs) const;
    G1TensorJacobian operator-(const G1TensorAffine& rhs) const;
    G1TensorJacobian operator+(const G1Jacobian_t& point) const;
    G1TensorJacobian operator-(const G1Jacobian_t& point) const;
    G1TensorJacobian operator+(const G1Affine_t& point) const;
    G1TensorJacobian operator-(const G1Affine_t& point) const;
    G1TensorJacobian& operator+=(const G1TensorJacobian& rhs);
    G1TensorJacobian& operator-=(const G1TensorJacobian& rhs);
    G1TensorJacobian& operator+=(const G1TensorAffine& rhs);
    G1TensorJacobian& operator-=(const G1TensorAffine& rhs);
    G1TensorJacobian& operator+=(const G1Jacobian_t& point);
    G1TensorJacobian& operator-=(const G1Jacobian_t& point);
    G1TensorJacobian& operator+=(const G1Affine_t& point);
    G1TensorJacobian& operator-=(const G1Affine_t& point);

    // out[i] = scalars[i] * (*this)[i mod size]; the scalar tensor may hold several rows
    G1TensorJacobian operator*(const FrTensor& scalars) const;
    G1TensorJacobian& operator*=(const FrTensor& scalars);

    G1Jacobian_t sum() const;
    G1TensorJacobian rowwise_sum(uint rows, uint cols) const;
    // multilinear extension "in the exponent"
    G1Jacobian_t operator()(const vector<Fr_t>& point) const;
};

#endif
