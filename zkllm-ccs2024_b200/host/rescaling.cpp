// Rescaling over the C ABI (reference: rescaling.cu).
#include "rescaling.cuh"

#include <stdexcept>

#include "zkllm_ext.hpp"

using zkllm::check;

Rescaling::Rescaling(uint scaling_factor)
    : scaling_factor(scaling_factor), tl_rem(-static_cast<int>(scaling_factor >> 1), scaling_factor), rem_tensor_ptr(nullptr) {}

Rescaling::~Rescaling() {
    if (rem_tensor_ptr) delete rem_tensor_ptr;
}

FrTensor Rescaling::operator()(const FrTensor& X) {
    if (rem_tensor_ptr) delete rem_tensor_ptr;
    rem_tensor_ptr = new FrTensor(X.size);
    FrTensor out(X.size);
    check(zkb_rescale(X.gpu_data, scaling_factor, out.gpu_data, rem_tensor_ptr->gpu_data, X.size, nullptr));
    check(zkb_sync(nullptr));
    return out;
}

vector<Claim> Rescaling::prove(const FrTensor& X, const FrTensor& X_) {
    if (X.size != X_.size) throw std::runtime_error("Error: the size of X and X_ should be the same.");
    auto u = random_vec(ceilLog2(X.size));
    auto v = random_vec(ceilLog2(X.size));
    auto rand_temp = random_vec(2);
    vector<Polynomial> proof;
    if (!rem_tensor_ptr) throw std::runtime_error("Rescaling::prove called before operator()");
    auto rem = rem_tensor_ptr->pad({rem_tensor_ptr->size});
    auto m = tl_rem.prep(rem);
    if (X(u) != X_(u) * Fr_t({scaling_factor, 0, 0, 0, 0, 0, 0, 0}) + rem(u)) throw std::runtime_error("Error: the rem is not correct.");
    tl_rem.prove(rem, m, rand_temp[0], rand_temp[1], u, v, proof);
    cout << "Rescaling proof complete." << endl;
    return {};
}
