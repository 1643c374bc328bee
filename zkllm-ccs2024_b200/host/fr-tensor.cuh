// FrTensor: a device array of BLS12-381 scalars in standard (non-Montgomery)
// form.  Same public interface as the reference's class (fr-tensor.cuh:69-177),
// so that code written against it compiles unchanged; every method forwards the
// device work to the CUDA library through its C ABI and returns when the result
// is complete, as the reference's methods do.
#ifndef FR_TENSOR_CUH
#define FR_TENSOR_CUH

#include <iomanip>
#include <iostream>
#include <random>
#include <string>
#include <utility>
#include <vector>

#include "bls12-381.cuh"

using namespace std;

typedef blstrs__scalar__Scalar Fr_t;
typedef blstrs__g1__G1Affine_affine G1Affine_t;
typedef blstrs__g1__G1Affine_jacobian G1Jacobian_t;

ostream& operator<<(ostream& os, const Fr_t& x);

// challenge vector of `len` field elements below r (see zkllm_ext.hpp for seeding)
vector<Fr_t> random_vec(uint len);
uint ceilLog2(uint num);

template <typename T>
std::vector<T> concatenate(const std::vector<std::vector<T>>& vecs);

class FrTensor {
public:
    Fr_t* gpu_data;
    const uint size;

    // construction, copies, files
    FrTensor(uint size);
    FrTensor(uint size, const Fr_t* cpu_data);
    FrTensor(uint size, const int* cpu_data);
    FrTensor(uint size, const long* cpu_data);
    FrTensor(uint size, const float* cpu_data, unsigned long scaling_factor);
    FrTensor(uint size, const double* cpu_data, unsigned long scaling_factor);
    FrTensor(const FrTensor& t);
    FrTensor(const string& filename);
    ~FrTensor();
    FrTensor& operator=(const FrTensor& x);
    static FrTensor from_int_bin(const string& filename);
    static FrTensor from_long_bin(const string& filename);
    void save(const string& filename) const;
    void save_int(const string& filename) const;
    void save_long(const string& filename) const;
    static FrTensor random_int(uint size, uint num_bits);
    static FrTensor random(uint size);

    // element read
    Fr_t operator()(uint idx) const;

    // field arithmetic, elementwise or against one broadcast value
    FrTensor operator+(const FrTensor& t) const;
    FrTensor operator+(const Fr_t& x) const;
    FrTensor operator-(const FrTensor& t) const;
    FrTensor operator-(const Fr_t& x) const;
    FrTensor operator*(const FrTensor& t) const;
    FrTensor operator*(const Fr_t& x) const;
    FrTensor operator-() const;
    FrTensor& operator+=(const FrTensor& t);
    FrTensor& operator+=(const Fr_t& x);
    FrTensor& operator-=(const FrTensor& t);
    FrTensor& operator-=(const Fr_t& x);
    FrTensor& operator*=(const FrTensor& t);
    FrTensor& operator*=(const Fr_t& x);
    FrTensor& mont();
    FrTensor& unmont();

    // reductions and multilinear extensions
    Fr_t sum() const;
    Fr_t operator()(const vector<Fr_t>& u) const;
    FrTensor partial_me(const vector<Fr_t>& u, uint window_size) const;
    FrTensor partial_me(const vector<Fr_t>& u, uint cur_dim, uint window_size) const;
    Fr_t multi_dim_me(const vector<vector<Fr_t>>& us, const vector<uint>& shape) const;

    // layout
    std::pair<FrTensor, FrTensor> split(uint window_size) const;
    FrTensor pad(const vector<uint>& shape, const Fr_t& pad_val = {0, 0, 0, 0, 0, 0, 0, 0}) const;
    FrTensor transpose(uint M, uint N) const;
    FrTensor trunc(uint begin_idx, uint end_idx) const;
    static FrTensor matmul(const FrTensor& x, const FrTensor& y, uint M, uint N, uint P);
};

ostream& operator<<(ostream& os, const FrTensor& A);
FrTensor catTensors(const vector<FrTensor>& vec);

#endif
