// zkReLU over the C ABI (reference: zkrelu.cu).
#include "zkrelu.cuh"

#include "zkllm_ext.hpp"

using zkllm::check;

zkReLU::zkReLU(uint scaling_factor)
    : scaling_factor(scaling_factor), tl_rem(-static_cast<int>(scaling_factor >> 1), scaling_factor), sign_tensor_ptr(nullptr),
      abs_tensor_ptr(nullptr), rem_tensor_ptr(nullptr), m_tensor_ptr(nullptr) {}

zkReLU::~zkReLU() {
    delete sign_tensor_ptr;
    delete abs_tensor_ptr;
    delete rem_tensor_ptr;
    delete m_tensor_ptr;
}

FrTensor zkReLU::decomp(const FrTensor& X, FrTensor& sign, FrTensor& abs, FrTensor& rem) {
    FrTensor res(X.size);
    check(zkb_relu_decomp(X.gpu_data, scaling_factor, sign.gpu_data, abs.gpu_data, rem.gpu_data, res.gpu_data, X.size, nullptr));
    check(zkb_sync(nullptr));
    return res;
}

FrTensor zkReLU::operator()(const FrTensor& X) {
    delete sign_tensor_ptr;
    delete abs_tensor_ptr;
    delete rem_tensor_ptr;
    delete m_tensor_ptr;
    m_tensor_ptr = nullptr;
    sign_tensor_ptr = new FrTensor(X.size);
    abs_tensor_ptr = new FrTensor(X.size);
    rem_tensor_ptr = new FrTensor(X.size);
    FrTensor res = decomp(X, *sign_tensor_ptr, *abs_tensor_ptr, *rem_tensor_ptr);
    m_tensor_ptr = new FrTensor(tl_rem.prep(*rem_tensor_ptr));   // multiplicities of the remainders in their table
    return res;
}

// the reference leaves this proof unwritten (zkrelu.cu:57-59)
void zkReLU::prove(const FrTensor& Z, const FrTensor& A) {
    (void)Z;
    (void)A;
}
