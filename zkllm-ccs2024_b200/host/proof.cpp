// Proof primitives over the C ABI (reference: proof.cu).
#include "proof.cuh"

#include <stdexcept>

#include "commitment.cuh"
#include "zkllm_ext.hpp"

using zkllm::check;

void verifyWeightClaim(const Weight& w, const Claim& c) {
    vector<Fr_t> u_cat = concatenate(vector<vector<Fr_t>>({c.u[1], c.u[0]}));
    auto w_padded = w.weight.pad({w.in_dim, w.out_dim});
    auto opening = w.generator.open(w_padded, w.com, u_cat);
    if (opening != c.claim) throw std::runtime_error("verifyWeightClaim: opening != c.claim");
    cout << "Opening complete" << endl;
}

// ---- openings in flight (zkllm_ext.hpp) ----------------------------------------------------
struct zkllm::WeightOpenings::Pending {
    void* handle = nullptr;
    FrTensor* row = nullptr;          // the weights folded by the high challenges: input of the opening in flight
    Fr_t expected;
    size_t rounds = 0;
};
zkllm::WeightOpenings::WeightOpenings() {}
zkllm::WeightOpenings::~WeightOpenings() {
    for (Pending* p : pending_) {
        if (p->handle) zkb_me_open_end(p->handle, nullptr, nullptr);
        delete p->row;
        delete p;
    }
}
void zkllm::WeightOpenings::add(const Weight& w, const Claim& c) {
    // verifyWeightClaim and Commitment::open up to the call of me_open
    const vector<Fr_t> u_cat = concatenate(vector<vector<Fr_t>>({c.u[1], c.u[0]}));
    auto w_padded = w.weight.pad({w.in_dim, w.out_dim});
    const uint k_out = ceilLog2(w.com.size);
    if (u_cat.size() < k_out) throw std::runtime_error("Commitment::open - not enough challenges");
    const vector<Fr_t> u_out(u_cat.end() - k_out, u_cat.end());
    const vector<Fr_t> u_in(u_cat.begin(), u_cat.end() - k_out);
    Pending* p = new Pending;
    pending_.push_back(p);
    p->expected = c.claim;
    p->rounds = u_in.size();
    p->row = u_out.empty() ? new FrTensor(w_padded) : new FrTensor(w_padded.partial_me(u_out, w_padded.size / w.com.size));
    if (p->row->size != w.generator.size)
        throw std::runtime_error("Commitment::me_open - Incompatible dimensions " + std::to_string(p->row->size) + " " +
                                 std::to_string(w.generator.size));
    static const Fr_t dummy = {{0, 0, 0, 0, 0, 0, 0, 0}};
    zkllm::check(zkb_me_open_begin(p->row->gpu_data, w.generator.gpu_data, p->row->size, u_in.empty() ? &dummy : u_in.data(),
                                   (unsigned)u_in.size(), nullptr, &p->handle));
}
void zkllm::WeightOpenings::finish() {
    std::vector<Pending*> todo;
    todo.swap(pending_);
    std::string failure;
    for (Pending* p : todo) {
        vector<G1Jacobian_t> elems(3 * p->rounds + 1);
        Fr_t opening;
        const int rc = p->handle ? zkb_me_open_end(p->handle, elems.data(), &opening) : ZKB_ERR_ARG;
        p->handle = nullptr;
        if (rc != ZKB_OK && failure.empty()) failure = zkb_last_error();
        if (rc == ZKB_OK) {
            if (auto* sink = zkllm::transcript_sink()) {
                zkllm::Transcript::Entry e;
                e.label = "me_open";
                e.points = elems;
                e.scalars.push_back(opening);
                sink->entries.push_back(e);
            }
            if (opening != p->expected) { if (failure.empty()) failure = "verifyWeightClaim: opening != c.claim"; }
            else cout << "Opening complete" << endl;
        }
        delete p->row;
        delete p;
    }
    if (!failure.empty()) throw std::runtime_error(failure);
}

bool operator==(const Fr_t& a, const Fr_t& b) {
    for (int i = 0; i < 8; ++i)
        if (a.val[i] != b.val[i]) return false;
    return true;
}
bool operator!=(const Fr_t& a, const Fr_t& b) { return !(a == b); }

static const Fr_t* ptr_or_dummy(const vector<Fr_t>& u) {
    static const Fr_t dummy = {{0, 0, 0, 0, 0, 0, 0, 0}};
    return u.empty() ? &dummy : u.data();
}

Fr_t multi_hadamard_sumchecks(const Fr_t& claim, const vector<FrTensor>& Xs, const vector<Fr_t>& u, const vector<Fr_t>& v,
                              vector<Polynomial>& proof) {
    const uint N = Xs[0].size;
    if (N == 1) return claim;
    if ((N & (N - 1)) != 0) throw std::runtime_error("N is not a power of 2");
    for (auto& X : Xs)
        if (X.size != N) throw std::runtime_error("Xs[i] size is not N");
    const unsigned K = (unsigned)Xs.size(), k = ceilLog2(N);
    if (u.size() < k || v.size() < k) throw std::runtime_error("multi_hadamard_sumchecks: not enough challenges");
    vector<const zkb_fr_t*> ptrs(K);
    for (unsigned i = 0; i < K; ++i) ptrs[i] = Xs[i].gpu_data;
    vector<Fr_t> coefs((size_t)k * (K + 1));
    Fr_t final_claim;
    // the reference consumes u and v from the back, one per halving: the last k of each
    const int rc = zkb_multi_hadamard(&claim, ptrs.data(), K, N, u.data() + (u.size() - k), v.data() + (v.size() - k), coefs.data(),
                                      &final_claim, nullptr);
    if (rc == ZKB_OK || rc == ZKB_ERR_VERIFY) {
        // polynomials computed before a failed check were already pushed by the reference
        for (unsigned r = 0; r < k; ++r)
            proof.push_back(Polynomial(vector<Fr_t>(coefs.begin() + (size_t)r * (K + 1), coefs.begin() + (size_t)(r + 1) * (K + 1))));
    }
    check(rc);
    if (auto* sink = zkllm::transcript_sink()) {
        zkllm::Transcript::Entry e;
        e.label = "multi_hadamard";
        e.scalars = coefs;
        e.scalars.push_back(final_claim);
        sink->entries.push_back(e);
    }
    return final_claim;
}

vector<Fr_t> inner_product_sumcheck(const FrTensor& a, const FrTensor& b, vector<Fr_t> u) {
    if (a.size != b.size) throw std::runtime_error("Incompatible dimensions");
    vector<Fr_t> proof(3 * u.size() + 2);
    check(zkb_inner_product_sumcheck(a.gpu_data, b.gpu_data, a.size, ptr_or_dummy(u), (unsigned)u.size(), proof.data(), nullptr));
    return proof;
}

vector<Fr_t> hadamard_product_sumcheck(const FrTensor& a, const FrTensor& b, vector<Fr_t> u, vector<Fr_t> v) {
    if (u.size() != v.size()) throw std::runtime_error("Incompatible dimensions 1");
    if (a.size != b.size) throw std::runtime_error("Incompatible dimensions 2");
    if (u.size() >= 1 && a.size <= (1u << (u.size() - 1))) throw std::runtime_error("Incompatible dimensions 3");
    if (a.size > (1u << u.size())) throw std::runtime_error("Incompatible dimensions 4");
    vector<Fr_t> proof(3 * u.size() + 2);
    check(zkb_hadamard_product_sumcheck(a.gpu_data, b.gpu_data, a.size, ptr_or_dummy(u), ptr_or_dummy(v), (unsigned)u.size(),
                                        proof.data(), nullptr));
    return proof;
}

vector<Fr_t> binary_sumcheck(const FrTensor& a, vector<Fr_t> u, vector<Fr_t> v) {
    if (u.size() != v.size()) throw std::runtime_error("Incompatible dimensions");
    vector<Fr_t> proof(3 * u.size() + 1);
    check(zkb_binary_sumcheck(a.gpu_data, a.size, ptr_or_dummy(u), ptr_or_dummy(v), (unsigned)u.size(), proof.data(), nullptr));
    return proof;
}
