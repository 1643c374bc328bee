// zkFC / zkip over the C ABI (reference: zkfc.cu).
#include "zkfc.cuh"

#include <stdexcept>

#include "zkllm_ext.hpp"

using zkllm::check;

static const Fr_t kZero = {{0, 0, 0, 0, 0, 0, 0, 0}};
static const Fr_t kOne = {{1, 0, 0, 0, 0, 0, 0, 0}};
static const Fr_t* ptr_or_dummy(const vector<Fr_t>& u) { return u.empty() ? &kZero : u.data(); }

zkFC::zkFC(uint input_size, uint output_size, const FrTensor& weight)
    : inputSize(input_size), outputSize(output_size), has_bias(false), weights(weight), bias(output_size) {
    if (weight.size != input_size * output_size) throw std::runtime_error("weight size does not match");
}

zkFC::zkFC(uint input_size, uint output_size, const FrTensor& weight, const FrTensor& bias)
    : inputSize(input_size), outputSize(output_size), has_bias(true), weights(weight), bias(bias) {
    if (weight.size != input_size * output_size) throw std::runtime_error("weight size does not match");
    if (bias.size != output_size) throw std::runtime_error("bias size does not match");
}

static FrTensor from_device_floats(const float* d_ptr, uint n, unsigned long scale) {
    FrTensor out(n);
    check(zkb_fr_from_f32(d_ptr, scale, out.gpu_data, n, nullptr));
    check(zkb_sync(nullptr));
    return out;
}

zkFC zkFC::from_float_gpu_ptr(uint input_size, uint output_size, unsigned long scaling_factor, float* weight_ptr, float* bias_ptr) {
    // the bias lives at the scale of a product of two scaled values
    return zkFC(input_size, output_size, from_device_floats(weight_ptr, input_size * output_size, scaling_factor),
                from_device_floats(bias_ptr, output_size, scaling_factor * scaling_factor));
}
zkFC zkFC::from_float_gpu_ptr(uint input_size, uint output_size, unsigned long scaling_factor, float* weight_ptr) {
    return zkFC(input_size, output_size, from_device_floats(weight_ptr, input_size * output_size, scaling_factor));
}
FrTensor zkFC::load_float_gpu_input(uint batch_size, uint input_size, unsigned long scaling_factor, float* input_ptr) {
    return from_device_floats(input_ptr, batch_size * input_size, scaling_factor);
}

FrTensor zkFC::operator()(const FrTensor& X) const {
    if (X.size % inputSize) throw std::runtime_error("input size does not match");
    const uint batch = X.size / inputSize;
    FrTensor out(batch * outputSize);
    check(zkb_fr_matmul(X.gpu_data, weights.gpu_data, out.gpu_data, batch, inputSize, outputSize, nullptr));
    if (has_bias) check(zkb_fr_add_bias(out.gpu_data, bias.gpu_data, batch, outputSize, nullptr));
    check(zkb_sync(nullptr));
    return out;
}

static void record(const char* label, const vector<Fr_t>& scalars) {
    if (auto* sink = zkllm::transcript_sink()) {
        zkllm::Transcript::Entry e;
        e.label = label;
        e.scalars = scalars;
        sink->entries.push_back(e);
    }
}

vector<Claim> zkFC::prove(const FrTensor& X, const FrTensor& Y) const {
    if (has_bias) throw std::runtime_error("Cleaned-up version not implemented for zkFC with bias. Use zkFCStacked instead.");
    const uint batch = X.size / inputSize;
    auto u_batch = random_vec(ceilLog2(batch));
    auto u_input = random_vec(ceilLog2(inputSize));
    auto u_output = random_vec(ceilLog2(outputSize));
    if (Y.size != batch * outputSize) throw std::runtime_error("Incompatible dimensions");
    vector<Fr_t> polys(3 * u_input.size() + 1), claims(4);
    check(zkb_zkfc_prove(X.gpu_data, weights.gpu_data, Y.gpu_data, batch, inputSize, outputSize, ptr_or_dummy(u_batch),
                         ptr_or_dummy(u_input), ptr_or_dummy(u_output), polys.data(), claims.data(), nullptr));
    polys.resize(3 * u_input.size());
    polys.insert(polys.end(), claims.begin(), claims.end());
    record("zkFC::prove", polys);
    vector<Claim> out;
    out.push_back({claims[3], vector<vector<Fr_t>>({u_input, u_output}), vector<uint>({inputSize, outputSize})});
    return out;
}

Fr_t zkip(const Fr_t& claim, const FrTensor& a, const FrTensor& b, const vector<Fr_t>& u, vector<Polynomial>& proof) {
    if (u.empty()) return claim;
    if (a.size != b.size) throw std::runtime_error("a.size != b.size");
    vector<Fr_t> polys(3 * u.size());
    Fr_t final_claim;
    const int rc = zkb_zkip(&claim, a.gpu_data, b.gpu_data, a.size, u.data(), (unsigned)u.size(), polys.data(), &final_claim, nullptr);
    if (rc == ZKB_OK || rc == ZKB_ERR_VERIFY)
        for (size_t r = 0; r < u.size(); ++r) proof.push_back(Polynomial(vector<Fr_t>(polys.begin() + 3 * r, polys.begin() + 3 * r + 3)));
    check(rc);
    polys.push_back(final_claim);
    record("zkip", polys);
    return final_claim;
}

// ---- stacked variants (reference: zkfc.cu:153-307) -----------------------------------------
// All rounds over the leading `num` axis and the inner-product rounds over D in one call: each stack
// round is one fused kernel (coefficient sums weighted by eq over the lower half of the stack, and the fold).
Fr_t zkip_stacked(const Fr_t& claim, const FrTensor& A, const FrTensor& B, const vector<Fr_t>& uN, const vector<Fr_t>& uD,
                  const vector<Fr_t> vN, uint N, uint D, vector<Polynomial>& proof) {
    if (uN.empty()) return zkip(claim, A, B, uD, proof);
    if (A.size != N * D) throw std::runtime_error("a.size != N * D");
    if (B.size != N * D) throw std::runtime_error("b.size != N * D");
    if (vN.size() < uN.size()) throw std::runtime_error("zkip_stacked: fewer fold challenges than stack variables");
    const size_t rounds = uN.size() + uD.size();
    vector<Fr_t> polys(3 * rounds + 1);
    Fr_t final_claim;
    // the reference pairs uN[i] with vN[i] from the back of both vectors
    const vector<Fr_t> v_used(vN.end() - uN.size(), vN.end());
    const int rc = zkb_zkip_stacked(&claim, A.gpu_data, B.gpu_data, N, D, uN.data(), v_used.data(), (unsigned)uN.size(),
                                    ptr_or_dummy(uD), (unsigned)uD.size(), polys.data(), &final_claim, nullptr);
    if (rc == ZKB_OK || rc == ZKB_ERR_VERIFY)
        for (size_t r = 0; r < rounds; ++r) proof.push_back(Polynomial(vector<Fr_t>(polys.begin() + 3 * r, polys.begin() + 3 * r + 3)));
    check(rc);
    polys.resize(3 * rounds);
    polys.push_back(final_claim);
    record("zkip_stacked", polys);
    return final_claim;
}

static FrTensor cat_weights(const vector<zkFC>& layers) {
    vector<FrTensor> w;
    for (auto& l : layers) w.push_back(l.weights);
    return catTensors(w);
}
static FrTensor cat_biases(const vector<zkFC>& layers) {
    vector<FrTensor> b;
    for (auto& l : layers) b.push_back(l.bias);
    return catTensors(b);
}

zkFCStacked::zkFCStacked(bool has_bias, uint num, uint batch_size, uint input_size, uint output_size, const vector<zkFC>& layers,
                         const vector<FrTensor>& Xs, const vector<FrTensor>& Ys)
    : has_bias(has_bias), num(num), batchSize(batch_size), inputSize(input_size), outputSize(output_size),
      X(catTensors(Xs)), W(cat_weights(layers)), b(cat_biases(layers)), Y(catTensors(Ys)) {
    if (X.size != num * batchSize * inputSize) throw std::runtime_error("X size does not match");
    if (Y.size != num * batchSize * outputSize) throw std::runtime_error("Y size does not match");
    if (W.size != num * inputSize * outputSize) throw std::runtime_error("W size does not match");
    if (has_bias && b.size != num * outputSize) throw std::runtime_error("b size does not match");
}

void zkFCStacked::prove(vector<Polynomial>& proof) const {
    auto u_num = random_vec(ceilLog2(num));
    auto v_num = random_vec(ceilLog2(num));
    auto u_batch = random_vec(ceilLog2(batchSize));
    auto u_input = random_vec(ceilLog2(inputSize));
    auto u_output = random_vec(ceilLog2(outputSize));
    prove(u_num, v_num, u_batch, u_input, u_output, proof);
}

void zkFCStacked::prove(const vector<Fr_t>& u_num, const vector<Fr_t>& v_num, const vector<Fr_t>& u_batch,
                        const vector<Fr_t>& u_input, const vector<Fr_t>& u_output, vector<Polynomial>& proof) const {
    auto claim = Y.multi_dim_me({u_num, u_batch, u_output}, {num, batchSize, outputSize});
    if (has_bias) {
        FrTensor ones(batchSize);
        check(zkb_memset0(ones.gpu_data, sizeof(Fr_t) * (size_t)batchSize, nullptr));
        ones += kOne;
        claim = claim - ones(u_batch) * b.multi_dim_me({u_num, u_output}, {num, outputSize});
    }
    auto X_reduced = X.partial_me(u_batch, batchSize, inputSize);
    auto W_reduced = W.partial_me(u_output, outputSize, 1);
    auto final_claim = zkip_stacked(claim, X_reduced, W_reduced, u_num, u_input, v_num, num, inputSize, proof);
    auto opening = X.multi_dim_me({v_num, u_batch, u_input}, {num, batchSize, inputSize}) *
                   W.multi_dim_me({v_num, u_input, u_output}, {num, inputSize, outputSize});
    if (final_claim != opening) throw std::runtime_error("final claim != opening");
}
