// Lookup arguments over the C ABI (reference: tlookup.cu).
#include "tlookup.cuh"

#include <stdexcept>

#include "zkllm_ext.hpp"

using zkllm::check;

namespace {
struct DevU32 {   // scoped device array of uint
    uint* p = nullptr;
    explicit DevU32(size_t n) {
        void* q = nullptr;
        check(zkb_malloc(&q, sizeof(uint) * n));
        p = static_cast<uint*>(q);
    }
    ~DevU32() { zkb_free_default_stream(p); }
};
const Fr_t kZero = {{0, 0, 0, 0, 0, 0, 0, 0}};
}  // namespace

tLookup::tLookup(const FrTensor& table) : table(table) {}

FrTensor tLookup::prep(const uint* indices, const uint D) {
    FrTensor m(table.size);
    check(zkb_tlookup_prep(indices, D, table.size, m.gpu_data, nullptr));
    check(zkb_sync(nullptr));
    return m;
}

// Runs the whole argument; the reference never appends to `proof` on this path
// (tlookup.cu:324-370), so neither does this, but the round polynomials go to
// the transcript sink when one is installed.
// `indexed_by` (optional): a tensor of D range values whose offsets from `first` are the table indices of S.
static Fr_t lookup_prove(const FrTensor& S, const FrTensor& T, const FrTensor& m, const Fr_t& alpha, const Fr_t& beta,
                         const vector<Fr_t>& u, const vector<Fr_t>& v, const FrTensor* indexed_by = nullptr, int first = 0) {
    const uint D = S.size, N = m.size;
    if (u.size() != ceilLog2(D)) throw std::runtime_error("u.size() != ceilLog2(D)");
    if (v.size() != ceilLog2(D)) throw std::runtime_error("v.size() != ceilLog2(D)");
    vector<Fr_t> polys(4 * u.size() + 1);
    Fr_t final_claim;
    if (indexed_by && D > N) {
        DevU32 idx(D);
        check(zkb_tlookup_range_indices(indexed_by->gpu_data, first, idx.p, D, nullptr));
        check(zkb_tlookup_prove_indexed(S.gpu_data, idx.p, T.gpu_data, m.gpu_data, D, N, &alpha, &beta, u.empty() ? &kZero : u.data(),
                                        v.empty() ? &kZero : v.data(), polys.data(), &final_claim, nullptr));
    } else {
        check(zkb_tlookup_prove(S.gpu_data, T.gpu_data, m.gpu_data, D, N, &alpha, &beta, u.empty() ? &kZero : u.data(),
                                v.empty() ? &kZero : v.data(), polys.data(), &final_claim, nullptr));
    }
    if (auto* sink = zkllm::transcript_sink()) {
        zkllm::Transcript::Entry e;
        e.label = "tLookup";
        e.scalars.assign(polys.begin(), polys.begin() + 4 * u.size());
        e.scalars.push_back(final_claim);
        sink->entries.push_back(e);
    }
    return final_claim;
}

Fr_t tLookup::prove(const FrTensor& S, const FrTensor& m, const Fr_t& alpha, const Fr_t& beta, const vector<Fr_t>& u,
                    const vector<Fr_t>& v, vector<Polynomial>& proof) {
    (void)proof;
    const uint D = S.size;
    if (m.size != table.size) throw std::runtime_error("m.size != table.size");
    const uint N = m.size;
    if (D != 1u << ceilLog2(D) || N != 1u << ceilLog2(N) || D % N != 0)
        throw std::runtime_error("D or N is not power of 2, or D is not divisible by N");
    return lookup_prove(S, table, m, alpha, beta, u, v, is_range ? &S : nullptr, range_first);
}

static FrTensor range_table(int low, uint len) {
    FrTensor t(1u << ceilLog2(len));
    check(zkb_tlookup_range_table(low, len, t.size, t.gpu_data, nullptr));
    check(zkb_sync(nullptr));
    return t;
}

tLookupRange::tLookupRange(int low, uint len) : tLookup(range_table(low, len)), low(low) {
    is_range = true;
    range_first = low;
}

// vals[i] - low as a table index, for device ints
static void int_indices(const int* d_vals, int low, uint* d_idx, uint D) {
    // through the field path: ints -> Fr -> low limb of (v - low); equal to the
    // reference's unsigned (v - low) for every value inside the table's range
    FrTensor fr(D);
    check(zkb_fr_from_i32(d_vals, fr.gpu_data, D, nullptr));
    check(zkb_tlookup_range_indices(fr.gpu_data, low, d_idx, D, nullptr));
    check(zkb_sync(nullptr));
}

FrTensor tLookupRange::prep(const int* vals, const uint D) {
    DevU32 idx(D);
    int_indices(vals, low, idx.p, D);
    return tLookup::prep(idx.p, D);
}

FrTensor tLookupRange::prep(const FrTensor& vals) {
    DevU32 idx(vals.size);
    check(zkb_tlookup_range_indices(vals.gpu_data, low, idx.p, vals.size, nullptr));
    return tLookup::prep(idx.p, vals.size);
}

tLookupRangeMapping::tLookupRangeMapping(int low, uint len, const FrTensor& mvals)
    : tLookupRange(low, len), mapped_vals(1u << ceilLog2(len)) {
    if (mvals.size != len) throw std::runtime_error("mvals.size != len");
    // padding repeats the last mapped value
    check(zkb_memset0(mapped_vals.gpu_data, sizeof(Fr_t) * (size_t)mapped_vals.size, nullptr));
    mapped_vals += mvals(mvals.size - 1);
    check(zkb_memcpy_d2d(mapped_vals.gpu_data, mvals.gpu_data, sizeof(Fr_t) * (size_t)mvals.size, nullptr));
    check(zkb_sync(nullptr));
}

pair<FrTensor, FrTensor> tLookupRangeMapping::operator()(const int* vals, const uint D) {
    DevU32 idx(D);
    int_indices(vals, low, idx.p, D);
    auto m = tLookup::prep(idx.p, D);
    FrTensor y(D);
    check(zkb_fr_gather(idx.p, mapped_vals.gpu_data, y.gpu_data, D, nullptr));
    check(zkb_sync(nullptr));
    return {y, m};
}

pair<FrTensor, FrTensor> tLookupRangeMapping::operator()(const FrTensor& vals) {
    DevU32 idx(vals.size);
    check(zkb_tlookup_range_indices(vals.gpu_data, low, idx.p, vals.size, nullptr));
    auto m = tLookup::prep(idx.p, vals.size);
    FrTensor y(vals.size);
    check(zkb_fr_gather(idx.p, mapped_vals.gpu_data, y.gpu_data, vals.size, nullptr));
    check(zkb_sync(nullptr));
    return {y, m};
}

Fr_t tLookupRangeMapping::prove(const FrTensor& S_in, const FrTensor& S_out, const FrTensor& m, const Fr_t& r, const Fr_t& alpha,
                                const Fr_t& beta, const vector<Fr_t>& u, const vector<Fr_t>& v, vector<Polynomial>& proof) {
    const uint D = S_in.size;
    if (m.size != table.size) throw std::runtime_error("m.size != table.size");
    const uint N = m.size;
    if (D != 1u << ceilLog2(D)) {
        // pad to a power of two with the first table entry and count the padding in m[0]
        auto S_in_ = S_in.pad({D}, table(0u));
        auto S_out_ = S_out.pad({D}, mapped_vals(0u));
        FrTensor m_(m);
        Fr_t m0 = m_(0u);
        m0 = m0 + Fr_t{{(1u << ceilLog2(D)) - D, 0, 0, 0, 0, 0, 0, 0}};
        check(zkb_memcpy_h2d(m_.gpu_data, &m0, sizeof(Fr_t), nullptr));
        return prove(S_in_, S_out_, m_, r, alpha, beta, u, v, proof);
    }
    if (N != 1u << ceilLog2(N) || D % N != 0) throw std::runtime_error("N is not power of 2, or D is not divisible by N");
    auto S_com = S_in + S_out * r;
    auto T_com = table + mapped_vals * r;
    return lookup_prove(S_com, T_com, m, alpha, beta, u, v, &S_in, low);
}
