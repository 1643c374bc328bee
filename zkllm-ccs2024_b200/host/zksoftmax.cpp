// zkSoftmax / zkAttn over the C ABI (reference: zksoftmax.cu).
#include "zksoftmax.cuh"

#include <stdexcept>

#include "zkllm_ext.hpp"

using zkllm::check;

static const Fr_t kZero = {{0, 0, 0, 0, 0, 0, 0, 0}};
static const Fr_t kOne = {{1, 0, 0, 0, 0, 0, 0, 0}};

zkSoftmax::zkSoftmax(const vector<uint>& bs, uint L, uint M, unsigned long scaling_factor_in, const vector<double>& thetas, uint m,
                     uint n, uint d, uint E)
    : bs(bs), K(bs.size()), L(L), M(M), scaling_factor_in(scaling_factor_in), thetas(thetas), m(m), n(n), d(d), E(E),
      least_significant_segments(), other_segments() {
    if (K - L - M != thetas.size()) throw std::invalid_argument("bs and thetas must have the same size");
    if (K <= L + M) throw std::invalid_argument("K must be greater than L + M");

    // weight of digit i in the mixed-radix expansion
    vector<unsigned long> weight(K);
    weight[0] = 1L;
    for (uint i = 1; i < K; ++i) weight[i] = weight[i - 1] * static_cast<unsigned long>(bs[i - 1]);

    for (uint i = 0; i < L; ++i) least_significant_segments.push_back({0, bs[i]});
    for (uint i = L; i < K - M; ++i) {
        // table[x] = round(theta * exp(-weight * x / (sf * sqrt(d))))
        FrTensor mapped(bs[i]);
        check(zkb_softmax_table(thetas[i - L], (double)scaling_factor_in, (double)d, (double)weight[i], bs[i], mapped.gpu_data, nullptr));
        check(zkb_sync(nullptr));
        other_segments.push_back({0, bs[i], mapped});
    }
    for (uint i = K - M; i < K; ++i) {
        // the most significant digits must be zero: indicator table {1, 0, 0, ...}
        vector<int> ind(bs[i], 0);
        ind[0] = 1;
        FrTensor mapped(bs[i], ind.data());
        other_segments.push_back({0, bs[i], mapped});
    }
}

FrTensor zkSoftmax::compute(const FrTensor& X, FrTensor& shift, FrTensor& X_shifted, vector<FrTensor>& X_segments,
                            vector<FrTensor>& Y_segments, vector<FrTensor>& m_segments) {
    if (X.size != m * n) throw std::invalid_argument("X must be m * n");
    if (shift.size != m) throw std::invalid_argument("shift must be m");
    if (X_shifted.size != X.size) throw std::invalid_argument("X_shifted must be the same size as X");

    check(zkb_softmax_shift(X.gpu_data, shift.gpu_data, X_shifted.gpu_data, m, n, (double)scaling_factor_in, (double)d, nullptr));

    // digit i of element g lands at digits[i * N + g]
    const uint N = m * n;
    void* raw = nullptr;
    check(zkb_malloc(&raw, sizeof(Fr_t) * (size_t)N * K));
    Fr_t* digits = static_cast<Fr_t*>(raw);
    int rc = zkb_softmax_decompose(X_shifted.gpu_data, bs.data(), K, digits, N, nullptr);
    if (rc == ZKB_OK) rc = zkb_sync(nullptr);
    if (rc != ZKB_OK) { zkb_free_default_stream(raw); check(rc); }

    FrTensor out(N);
    try {
        check(zkb_memset0(out.gpu_data, sizeof(Fr_t) * (size_t)N, nullptr));
        out += kOne;
        for (uint i = 0; i < K; ++i) {
            X_segments.push_back({N});
            check(zkb_memcpy_d2d(X_segments[i].gpu_data, digits + (size_t)i * N, sizeof(Fr_t) * (size_t)N, nullptr));
            check(zkb_sync(nullptr));
            if (i < L) {
                m_segments.push_back(least_significant_segments[i].prep(X_segments[i]));
            } else {
                auto p = other_segments[i - L](X_segments[i]);
                Y_segments.push_back(p.first);
                m_segments.push_back(p.second);
                out *= p.first;
            }
        }
    } catch (...) {
        zkb_free_default_stream(raw);
        throw;
    }
    zkb_free_default_stream(raw);
    return out;
}

Fr_t zkSoftmax::prove(const FrTensor& Y, const FrTensor& X, const FrTensor& shift, const FrTensor& X_shifted,
                      const vector<FrTensor>& X_segments, const vector<FrTensor>& Y_segments, const vector<FrTensor>& m_segments,
                      const vector<Fr_t>& u_Y, const vector<Fr_t>& v_Y, const Fr_t& r_seg, const Fr_t& alpha_seg, const Fr_t& beta_seg,
                      vector<Polynomial>& proof) {
    (void)X_shifted;
    const uint N = Y.size;
    if (X.size != N) throw std::invalid_argument("X and Y must have the same size " + to_string(X.size) + " " + to_string(Y.size));

    // Y is the elementwise product of the segment outputs
    auto claim_Y = Y(u_Y);
    multi_hadamard_sumchecks(claim_Y, Y_segments, u_Y, v_Y, proof);

    // every digit is in its table (and maps to its output)
    for (uint i = 0; i < L; ++i) least_significant_segments[i].prove(X_segments[i], m_segments[i], alpha_seg, beta_seg, u_Y, v_Y, proof);
    for (uint i = L; i < K; ++i)
        other_segments[i - L].prove(X_segments[i], Y_segments[i - L], m_segments[i], r_seg, alpha_seg, beta_seg, u_Y, v_Y, proof);

    // the digits recompose to shift - X at v_Y
    Fr_t recomposed = kZero;
    for (int i = (int)bs.size() - 1; i >= 0; --i) recomposed = recomposed * Fr_t({bs[i], 0, 0, 0, 0, 0, 0, 0}) + X_segments[i](v_Y);
    vector<Fr_t> v_rows(v_Y.begin() + ceilLog2(n), v_Y.end());
    auto shift_opening = shift(v_rows);
    auto X_opening = X(v_Y);
    if (shift_opening - recomposed != X_opening) throw std::runtime_error("X claim is not correct");
    return X_opening;
}

// ---- attention wrappers -----------------------------------------------------------------------
zkAttn::zkAttn(unsigned long sf_Q, unsigned long sf_K, const vector<uint>& bs, uint L, uint M, const vector<double>& thetas, uint m,
               uint n, uint d, uint E)
    : zkSoftmax(bs, L, M, sf_Q * sf_K, thetas, m, n, d, E) {}

FrTensor zkAttn::compute(const FrTensor& Q, const FrTensor& K, const FrTensor& V, FrTensor& sm_in, FrTensor& sm_out,
                         FrTensor& sm_shift, FrTensor& sm_in_shifted, vector<FrTensor>& sm_in_segments,
                         vector<FrTensor>& sm_out_segments, vector<FrTensor>& sm_m_segments) {
    if (Q.size != m * d) throw std::invalid_argument("Q must be m * d");
    if (K.size != n * d) throw std::invalid_argument("K must be n * d");
    if (V.size != n * d) throw std::invalid_argument("V must be n * d");
    sm_in = FrTensor::matmul(Q, K.transpose(n, d), m, d, n);
    sm_out = zkSoftmax::compute(sm_in, sm_shift, sm_in_shifted, sm_in_segments, sm_out_segments, sm_m_segments);
    return FrTensor::matmul(sm_out, V, m, n, d);
}

vector<Claim> zkAttn::prove(const FrTensor& Q, const FrTensor& K, const FrTensor& V, const FrTensor& out, const FrTensor& sm_out,
                            const FrTensor& sm_in, const FrTensor& sm_shift, const FrTensor& sm_in_shifted,
                            const vector<FrTensor>& sm_in_segments, const vector<FrTensor>& sm_out_segments,
                            const vector<FrTensor>& sm_m_segments) {
    auto u_matmul_out = random_vec(ceilLog2(m));
    auto v_matmul_out = random_vec(ceilLog2(n));
    auto w_matmul_out = random_vec(ceilLog2(d));
    auto v_sm = random_vec(ceilLog2(m) + ceilLog2(n));
    auto temp_rand = random_vec(3);
    auto v_matmul_in = random_vec(ceilLog2(d));
    vector<Polynomial> proof;
    this->prove(Q, K, V, out, sm_out, sm_in, sm_shift, sm_in_shifted, sm_in_segments, sm_out_segments, sm_m_segments, u_matmul_out,
                v_matmul_out, w_matmul_out, v_sm, temp_rand[0], temp_rand[1], temp_rand[2], v_matmul_in, proof);
    cout << "zkAttn proof complete." << endl;
    return {};
}

Fr_t zkAttn::prove(const FrTensor& Q, const FrTensor& K, const FrTensor& V, const FrTensor& out, const FrTensor& sm_out,
                   const FrTensor& sm_in, const FrTensor& sm_shift, const FrTensor& sm_in_shifted,
                   const vector<FrTensor>& sm_in_segments, const vector<FrTensor>& sm_out_segments,
                   const vector<FrTensor>& sm_m_segments, const vector<Fr_t>& u_matmul_out, const vector<Fr_t>& v_matmul_out,
                   const vector<Fr_t>& w_matmul_out, const vector<Fr_t>& v_sm, const Fr_t& r_seg, const Fr_t& alpha_seg,
                   const Fr_t& beta_seg, const vector<Fr_t>& v_matmul_in, vector<Polynomial>& proof) {
    // out = sm_out * V
    auto out_claim = out.multi_dim_me({u_matmul_out, w_matmul_out}, {m, d});
    auto out_matmul_claim = zkip(out_claim, sm_out.partial_me(u_matmul_out, m, n), V.partial_me(w_matmul_out, d, 1), v_matmul_out, proof);
    auto V_claim = V.multi_dim_me({v_matmul_out, w_matmul_out}, {n, d});
    auto sm_out_claim = sm_out.multi_dim_me({u_matmul_out, v_matmul_out}, {m, n});
    if (out_matmul_claim != V_claim * sm_out_claim) throw std::runtime_error("out_matmul_claim is not correct");

    // softmax
    auto sm_in_claim = zkSoftmax::prove(sm_out, sm_in, sm_shift, sm_in_shifted, sm_in_segments, sm_out_segments, sm_m_segments,
                                        concatenate<Fr_t>({v_matmul_out, u_matmul_out}), v_sm, r_seg, alpha_seg, beta_seg, proof);

    // sm_in = Q * K^T, opened at v_sm
    vector<Fr_t> u_matmul_in(v_sm.end() - ceilLog2(m), v_sm.end());
    vector<Fr_t> w_matmul_in(v_sm.begin(), v_sm.end() - ceilLog2(m));
    return zkip(sm_in_claim, Q.partial_me(u_matmul_in, m, d), K.partial_me(w_matmul_in, n, d), v_matmul_in, proof);
}

zkAttnStacked::zkAttnStacked(uint num, unsigned long sf_Q, unsigned long sf_K, const vector<uint>& bs, uint L, uint M,
                             const vector<double>& thetas, uint m, uint n, uint d, uint E)
    : zkAttn(sf_Q, sf_K, bs, L, M, thetas, m, n, d, E), num(num) {}

Fr_t zkAttnStacked::prove(const FrTensor& Q, const FrTensor& K, const FrTensor& V, const FrTensor& out, const FrTensor& sm_out,
                          const FrTensor& sm_in, const FrTensor& sm_shift, const FrTensor& sm_in_shifted,
                          const vector<FrTensor>& sm_in_segments, const vector<FrTensor>& sm_out_segments,
                          const vector<FrTensor>& sm_m_segments, const vector<Fr_t>& u_matmul_out_num,
                          const vector<Fr_t>& v_matmul_out_num, const vector<Fr_t>& u_matmul_out, const vector<Fr_t>& v_matmul_out,
                          const vector<Fr_t>& w_matmul_out, const vector<Fr_t>& v_sm, const Fr_t& r_seg, const Fr_t& alpha_seg,
                          const Fr_t& beta_seg, const vector<Fr_t>& v_matmul_in_num, const vector<Fr_t>& v_matmul_in,
                          vector<Polynomial>& proof) {
    auto out_claim = out.multi_dim_me({u_matmul_out_num, u_matmul_out, w_matmul_out}, {num, m, d});
    auto out_matmul_claim = zkip_stacked(out_claim, sm_out.partial_me(u_matmul_out, m, n), V.partial_me(w_matmul_out, d, 1),
                                         u_matmul_out_num, v_matmul_out, v_matmul_out_num, num, n, proof);
    auto V_claim = V.multi_dim_me({v_matmul_out_num, v_matmul_out, w_matmul_out}, {num, n, d});
    auto sm_out_claim = sm_out.multi_dim_me({v_matmul_out_num, u_matmul_out, v_matmul_out}, {num, m, n});
    if (out_matmul_claim != V_claim * sm_out_claim) throw std::runtime_error("out_matmul_claim is not correct");

    auto sm_in_claim = zkSoftmax::prove(sm_out, sm_in, sm_shift, sm_in_shifted, sm_in_segments, sm_out_segments, sm_m_segments,
                                        concatenate<Fr_t>({v_matmul_out, u_matmul_out, v_matmul_out_num}), v_sm, r_seg, alpha_seg,
                                        beta_seg, proof);

    const uint kn = ceilLog2(num), km = ceilLog2(m);
    vector<Fr_t> u_matmul_in_num(v_sm.end() - kn, v_sm.end());
    vector<Fr_t> u_matmul_in(v_sm.end() - kn - km, v_sm.end() - kn);
    vector<Fr_t> w_matmul_in(v_sm.begin(), v_sm.end() - kn - km);
    return zkip_stacked(sm_in_claim, Q.partial_me(u_matmul_in, m, d), K.partial_me(w_matmul_in, n, d), u_matmul_in_num, v_matmul_in,
                        v_matmul_in_num, num, d, proof);
}

// Declared by the reference (zksoftmax.cuh:66-68) and never defined there; given
// the same shape as zkAttn's: draw the challenges, run the explicit-challenge proof.
vector<Claim> zkAttnStacked::prove(const FrTensor& Q, const FrTensor& K, const FrTensor& V, const FrTensor& out,
                                   const FrTensor& sm_out, const FrTensor& sm_in, const FrTensor& sm_shift,
                                   const FrTensor& sm_in_shifted, const vector<FrTensor>& sm_in_segments,
                                   const vector<FrTensor>& sm_out_segments, const vector<FrTensor>& sm_m_segments) {
    const uint kn = ceilLog2(num), km = ceilLog2(m), kk = ceilLog2(n), kd = ceilLog2(d);
    auto temp_rand = random_vec(3);
    vector<Polynomial> proof;
    this->prove(Q, K, V, out, sm_out, sm_in, sm_shift, sm_in_shifted, sm_in_segments, sm_out_segments, sm_m_segments,
                random_vec(kn), random_vec(kn), random_vec(km), random_vec(kk), random_vec(kd), random_vec(kn + km + kk),
                temp_rand[0], temp_rand[1], temp_rand[2], random_vec(kn), random_vec(kd), proof);
    cout << "zkAttnStacked proof complete." << endl;
    return {};
}
