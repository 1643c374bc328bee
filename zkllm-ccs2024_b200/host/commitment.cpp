// Commitment over the C ABI (reference: commitment.cu).
#include "commitment.cuh"

#include <stdexcept>

#include "zkllm_ext.hpp"

using zkllm::check;

Commitment Commitment::random(uint size) {
    Commitment out(size, G1Jacobian_generator);
    out *= FrTensor::random(size);
    return out;
}

G1TensorJacobian Commitment::commit(const FrTensor& t) const {
    if (t.size % size != 0) throw std::runtime_error("Commitment::commit - Incompatible dimensions");
    G1TensorJacobian out(t.size / size);
    check(zkb_commit(gpu_data, size, t.gpu_data, t.size, out.gpu_data, nullptr));
    check(zkb_sync(nullptr));
    return out;
}

G1TensorJacobian Commitment::commit_int(const FrTensor& t) const {
    if (t.size % size != 0) throw std::runtime_error("Commitment::commit_int - Incompatible dimensions");
    G1TensorJacobian out(t.size / size);
    check(zkb_commit_int(gpu_data, size, t.gpu_data, t.size, out.gpu_data, nullptr));
    check(zkb_sync(nullptr));
    return out;
}

G1TensorJacobian Commitment::commit_int_multi(const vector<FrTensor>& ts) const {
    uint rows = 0;
    for (auto& t : ts) {
        if (t.size % size != 0) throw std::runtime_error("Commitment::commit_int_multi - Incompatible dimensions");
        rows += t.size / size;
    }
    G1TensorJacobian out(rows);
    uint done = 0;
    for (auto& t : ts) {
        check(zkb_commit_int(gpu_data, size, t.gpu_data, t.size, out.gpu_data + done, nullptr));
        done += t.size / size;
    }
    check(zkb_sync(nullptr));
    return out;
}

Fr_t Commitment::me_open(const FrTensor& t, const Commitment& generators, vector<Fr_t>::const_iterator begin,
                         vector<Fr_t>::const_iterator end, vector<G1Jacobian_t>& proof) {
    if (t.size != generators.size)
        throw std::runtime_error("Commitment::me_open - Incompatible dimensions " + std::to_string(t.size) + " " +
                                 std::to_string(generators.size));
    const vector<Fr_t> u(begin, end >= begin ? end : begin);
    static const Fr_t dummy = {{0, 0, 0, 0, 0, 0, 0, 0}};
    vector<G1Jacobian_t> elems(3 * u.size() + 1);
    Fr_t opening;
    check(zkb_me_open(t.gpu_data, generators.gpu_data, t.size, u.empty() ? &dummy : u.data(), (unsigned)u.size(), elems.data(),
                      &opening, nullptr));
    proof.insert(proof.end(), elems.begin(), elems.end());
    if (auto* sink = zkllm::transcript_sink()) {
        zkllm::Transcript::Entry e;
        e.label = "me_open";
        e.points = elems;
        e.scalars.push_back(opening);
        sink->entries.push_back(e);
    }
    return opening;
}

Fr_t Commitment::open(const FrTensor& t, const G1TensorJacobian& com, const vector<Fr_t>& u) const {
    const uint k_out = ceilLog2(com.size);
    if (u.size() < k_out) throw std::runtime_error("Commitment::open - not enough challenges");
    const vector<Fr_t> u_out(u.end() - k_out, u.end());
    const vector<Fr_t> u_in(u.begin(), u.end() - k_out);
    // The reference also evaluates the commitment tensor at u_out here and drops the
    // result (commitment.cu:137); it has no effect on the value returned.
    vector<G1Jacobian_t> proof;
    if (u_out.empty()) return me_open(t, *this, u_in.begin(), u_in.end(), proof);
    return me_open(t.partial_me(u_out, t.size / com.size), *this, u_in.begin(), u_in.end(), proof);
}

Weight create_weight(string generator_filename, string weight_filename, string com_filename, uint in_dim, uint out_dim) {
    Commitment generator(generator_filename);
    FrTensor weight = FrTensor::from_int_bin(weight_filename);
    G1TensorJacobian com(com_filename);
    return {generator, weight, com, in_dim, out_dim};
}
