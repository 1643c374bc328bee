// TEST INFRASTRUCTURE ONLY.  One source, two builds: it uses nothing but the public
// class API that the reference's headers and zkllm-ccs2024_b200/host/ both
// declare (zkfc.cuh, zksoftmax.cuh, fr-tensor.cuh, polynomial.cuh), so the same
// program runs the reference's own CUDA code (oracle/Makefile: `make ref-api`,
// _ref/api_check_ref) and this repository's library (`make api`, _build/api_check).
// Inputs and challenges come from a fixed integer generator, so the two builds
// print the same lines when the implementations agree.  Covered here are the
// parts of the API that no stage driver reaches: zkip_stacked / zkFCStacked
// (zkfc.cu:153-307), zkAttn / zkAttnStacked (zksoftmax.cu:222-320), zkReLU
// (zkrelu.cu:3-66), and FrTensor::split, Commitment::commit_int_multi, FrTensor::random*.  Every
// prove() below throws if one of its verifier equations fails.
//
// usage: api_check <fcstacked|attn|attnstacked|relu|misc>
// output: "poly<i> <coefficients>" per round polynomial, "final <Fr>", "ok 1".
#include <iostream>
#include <string>
#include <vector>

#include "commitment.cuh"
#include "fr-tensor.cuh"
#include "polynomial.cuh"
#include "zkfc.cuh"
#include "zkrelu.cuh"
#include "zksoftmax.cuh"

using namespace std;

// xorshift64*: the same stream in both builds
struct Gen {
    unsigned long s;
    explicit Gen(unsigned long seed) : s(seed) {}
    unsigned long next() {
        s ^= s >> 12; s ^= s << 25; s ^= s >> 27;
        return s * 2685821657736338717UL;
    }
    int small(int bound) { return (int)(next() % (2UL * bound)) - bound; }
    Fr_t fr() {   // below 2^254: a canonical field element
        Fr_t x;
        for (int i = 0; i < 8; ++i) x.val[i] = (uint)next();
        x.val[7] &= 0x3fffffffu;
        return x;
    }
    vector<Fr_t> vec(uint n) {
        vector<Fr_t> v(n);
        for (auto& x : v) x = fr();
        return v;
    }
    FrTensor ints(uint n, int bound) {
        vector<int> h(n);
        for (auto& x : h) x = small(bound);
        return FrTensor(n, h.data());
    }
};

static void print_tensor(const char* key, const FrTensor& t) {
    cout << key;
    for (uint i = 0; i < t.size; ++i) cout << " " << t(i);
    cout << endl;
}

static void print_polys(vector<Polynomial>& ps) {
    for (size_t i = 0; i < ps.size(); ++i) cout << "poly" << i << " " << ps[i] << endl;
}

static int fc_stacked() {
    const uint num = 4, batch = 8, in = 16, out = 8;
    Gen g(0x5EED0001);
    vector<zkFC> layers;
    vector<FrTensor> Xs, Ys;
    for (uint l = 0; l < num; ++l) {
        layers.push_back(zkFC(in, out, g.ints(in * out, 3000)));
        Xs.push_back(g.ints(batch * in, 3000));
        Ys.push_back(layers.back()(Xs.back()));
    }
    zkFCStacked stacked(false, num, batch, in, out, layers, Xs, Ys);
    vector<Polynomial> proof;
    stacked.prove(g.vec(2), g.vec(2), g.vec(3), g.vec(4), g.vec(3), proof);
    print_polys(proof);
    cout << "ok 1" << endl;
    return 0;
}

// the driver's softmax parameters (self-attn.cu:87); the tables need m * n >= 2^20
static const vector<uint> kBs = {1 << 8, 1 << 20, 1 << 20};
static const vector<double> kThetas = {1 << 18, 1 << 22};

static int attn() {
    const uint m = 1024, n = 1024, d = 16;
    Gen g(0x5EED0002);
    FrTensor Q = g.ints(m * d, 1 << 16), K = g.ints(n * d, 1 << 16), V = g.ints(n * d, 1 << 16);
    zkAttn at(1 << 16, 1 << 16, kBs, 1, 0, kThetas, m, n, d, 1);
    FrTensor sm_in(m * n), sm_out(m * n), shift(m), shifted(m * n);
    vector<FrTensor> in_seg, out_seg, m_seg;
    FrTensor out = at.compute(Q, K, V, sm_in, sm_out, shift, shifted, in_seg, out_seg, m_seg);
    cout << "out0 " << out(0u) << endl << "out_last " << out(out.size - 1) << endl;
    vector<Polynomial> proof;
    auto u_out = g.vec(10), v_out = g.vec(10), w_out = g.vec(4), v_sm = g.vec(20), t = g.vec(3), v_in = g.vec(4);
    Fr_t fin = at.prove(Q, K, V, out, sm_out, sm_in, shift, shifted, in_seg, out_seg, m_seg, u_out, v_out, w_out, v_sm, t[0], t[1],
                        t[2], v_in, proof);
    print_polys(proof);
    cout << "final " << fin << endl << "ok 1" << endl;
    return 0;
}

static int attn_stacked() {
    const uint num = 2, m = 1024, n = 1024, d = 16;
    Gen g(0x5EED0003);
    // per-head tensors, stacked along a leading axis; the softmax intermediates come from
    // one zkSoftmax over all num * m rows (the stacked class has no compute of its own)
    vector<FrTensor> Qs, Ks, Vs, ins;
    for (uint h = 0; h < num; ++h) {
        Qs.push_back(g.ints(m * d, 1 << 16));
        Ks.push_back(g.ints(n * d, 1 << 16));
        Vs.push_back(g.ints(n * d, 1 << 16));
        ins.push_back(FrTensor::matmul(Qs[h], Ks[h].transpose(n, d), m, d, n));
    }
    FrTensor Q = catTensors(Qs), K = catTensors(Ks), V = catTensors(Vs), sm_in = catTensors(ins);
    zkSoftmax sm(kBs, 1, 0, 1UL << 32, kThetas, num * m, n, d, 1);
    FrTensor shift(num * m), shifted(num * m * n);
    vector<FrTensor> in_seg, out_seg, m_seg;
    FrTensor sm_out = sm.compute(sm_in, shift, shifted, in_seg, out_seg, m_seg);
    vector<FrTensor> outs;
    for (uint h = 0; h < num; ++h) {
        FrTensor y_h = sm_out.trunc(h * m * n, (h + 1) * m * n);
        outs.push_back(FrTensor::matmul(y_h, Vs[h], m, n, d));
    }
    FrTensor out = catTensors(outs);
    zkAttnStacked at(num, 1 << 16, 1 << 16, kBs, 1, 0, kThetas, m, n, d, 1);
    vector<Polynomial> proof;
    auto un = g.vec(1), vn = g.vec(1), u_out = g.vec(10), v_out = g.vec(10), w_out = g.vec(4), v_sm = g.vec(21), t = g.vec(3);
    auto vin_n = g.vec(1), v_in = g.vec(4);
    Fr_t fin = at.prove(Q, K, V, out, sm_out, sm_in, shift, shifted, in_seg, out_seg, m_seg, un, vn, u_out, v_out, w_out, v_sm, t[0],
                        t[1], t[2], vin_n, v_in, proof);
    print_polys(proof);
    cout << "final " << fin << endl << "ok 1" << endl;
    return 0;
}

static int relu() {
    Gen g(0x5EED0004);
    const uint n = 1 << 12;
    vector<long> h(n);
    for (auto& x : h) x = (long)(g.next() % (1UL << 41)) - (1L << 40);
    h[0] = 0; h[1] = 32768; h[2] = -32768; h[3] = -32769; h[4] = 65536;
    FrTensor X(n, h.data());
    zkReLU act(1 << 16);
    FrTensor res = act(X);
    print_tensor("out_res", res);
    print_tensor("out_sign", *act.sign_tensor_ptr);
    print_tensor("out_abs", *act.abs_tensor_ptr);
    print_tensor("out_rem", *act.rem_tensor_ptr);
    cout << "out_m_sum " << act.m_tensor_ptr->sum() << endl;
    act.prove(X, res);
    cout << "ok 1" << endl;
    return 0;
}

// FrTensor::split with ragged windows (fr-tensor.cu:562-585), Commitment::commit_int_multi against
// commit_int of each tensor (commitment.cu:60-77), FrTensor::random / random_int value ranges
// (fr-tensor.cu:444-510).  The random draws differ from run to run, so only their ranges are printed.
static int misc() {
    Gen g(0x5EED0005);
    FrTensor t = g.ints(37, 1 << 20);
    for (uint window : {5u, 1u, 36u, 16u}) {
        auto halves = t.split(window);
        print_tensor(("out_split" + to_string(window) + "_0").c_str(), halves.first);
        print_tensor(("out_split" + to_string(window) + "_1").c_str(), halves.second);
    }
    Commitment gens(8, G1Jacobian_generator);
    gens *= g.ints(8, 1 << 30);
    vector<FrTensor> ts;
    ts.push_back(g.ints(16, 8000));
    ts.push_back(g.ints(8, 8000));
    ts.push_back(g.ints(24, 1 << 30));
    G1TensorJacobian all = gens.commit_int_multi(ts);
    cout << "out_multi_rows " << all.size << endl;
    bool same = true;
    uint row = 0;
    for (auto& x : ts) {
        G1TensorJacobian c = gens.commit_int(x);
        for (uint i = 0; i < c.size; ++i, ++row) {
            G1TensorJacobian diff = G1TensorJacobian(1, all(row)) - G1TensorJacobian(1, c(i));
            const G1Jacobian_t d = diff(0u);
            for (int k = 0; k < 12; ++k) same = same && d.z.val[k] == 0;   // the identity has Z = 0
        }
    }
    cout << "ok_multi " << (same && row == all.size) << endl;
    const uint bits = 12, n = 4096;
    FrTensor ri = FrTensor::random_int(n, bits);
    FrTensor shifted = ri + Fr_t{{1u << (bits - 1), 0, 0, 0, 0, 0, 0, 0}};
    bool in_range = true, varied = false;
    for (uint i = 0; i < n; ++i) {
        const Fr_t x = shifted(i);
        for (int k = 1; k < 8; ++k) in_range = in_range && x.val[k] == 0;
        in_range = in_range && x.val[0] < (1u << bits);
        varied = varied || x.val[0] != shifted(0u).val[0];
    }
    cout << "ok_random_int " << (in_range && varied) << endl;
    FrTensor rf = FrTensor::random(n);
    bool canonical = true, wide = false;
    for (uint i = 0; i < n; ++i) {
        const Fr_t x = rf(i);
        canonical = canonical && x.val[7] < 1944954707u;
        wide = wide || x.val[7] != 0;
    }
    cout << "ok_random " << (canonical && wide) << endl;
    cout << "ok 1" << endl;
    return 0;
}

int main(int argc, char** argv) {
    const string cmd = argc > 1 ? argv[1] : "";
    try {
        if (cmd == "fcstacked") return fc_stacked();
        if (cmd == "attn") return attn();
        if (cmd == "attnstacked") return attn_stacked();
        if (cmd == "relu") return relu();
        if (cmd == "misc") return misc();
        cerr << "usage: api_check <fcstacked|attn|attnstacked|relu|misc>" << endl;
        return 2;
    } catch (const std::exception& e) {
        cout << "exception " << e.what() << endl;
        return 1;
    }
}
