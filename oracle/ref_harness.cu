// TEST INFRASTRUCTURE ONLY.  Drives the reference's own, unmodified CUDA code
// (compiled from its sources in place, see oracle/Makefile) on input files and
// prints what it computes, so that
//   - tests/golden/make_golden.py can record golden vectors that pin the oracle, and
//   - bench.py --impl reference can time the reference on the benchmark inputs.
// This file contains no reference code: it includes the reference's headers and
// calls its public classes and (for the lookup rounds, whose polynomials the
// reference computes and drops) two of its non-static functions.
//
// usage: ref_harness <command> <args...>; every tensor argument is a raw .bin file
// (Fr: 32 B standard form; int: int32; G1: 144 B Jacobian, Montgomery form).
// Output: one "key value..." line per result on stdout, Fr as 0x<64 hex>,
// G1 as (0x<96 hex>, 0x.., 0x..) in Montgomery form.
#include <chrono>
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#include "commitment.cuh"
#include "fr-tensor.cuh"
#include "g1-tensor.cuh"
#include "ioutils.cuh"
#include "polynomial.cuh"
#include "proof.cuh"
#include "rescaling.cuh"
#include "tlookup.cuh"
#include "zkfc.cuh"
#include "zksoftmax.cuh"

using namespace std;

// non-static functions of the reference's tlookup.cu (tlookup.cu:184, :245)
Polynomial tLookup_phase1_step_poly(const FrTensor& A, const FrTensor& S, const Fr_t& alpha, const Fr_t& beta, const Fr_t& C,
                                    const vector<Fr_t>& u);
Polynomial tLookup_phase2_step_poly(const FrTensor& A, const FrTensor& S, const FrTensor& B, const FrTensor& T, const FrTensor& m,
                                    const Fr_t& alpha_, const Fr_t& beta, const Fr_t& inv_size_ratio, const Fr_t& alpha_sq,
                                    const vector<Fr_t>& u);

static vector<Fr_t> load_vec(const string& fn) {
    if (fn == "-") return {};
    FrTensor t(fn);
    vector<Fr_t> out(t.size);
    cudaMemcpy(out.data(), t.gpu_data, sizeof(Fr_t) * t.size, cudaMemcpyDeviceToHost);
    return out;
}
static void print_tensor(const string& key, const FrTensor& t) {
    vector<Fr_t> h(t.size);
    cudaMemcpy(h.data(), t.gpu_data, sizeof(Fr_t) * t.size, cudaMemcpyDeviceToHost);
    cout << key;
    for (auto& x : h) cout << " " << x;
    cout << endl;
}
static void print_g1s(const string& key, const vector<G1Jacobian_t>& v) {
    cout << key;
    for (auto& g : v) cout << " " << g.x << " " << g.y << " " << g.z;
    cout << endl;
}
static void print_g1_tensor(const string& key, const G1TensorJacobian& t) {
    vector<G1Jacobian_t> h(t.size);
    cudaMemcpy(h.data(), t.gpu_data, sizeof(G1Jacobian_t) * t.size, cudaMemcpyDeviceToHost);
    print_g1s(key, h);
}
static void print_polys(const string& key, vector<Polynomial>& ps) {
    for (size_t i = 0; i < ps.size(); ++i) cout << key << i << " " << ps[i] << endl;
}
static double now_s() {
    return chrono::duration<double>(chrono::steady_clock::now().time_since_epoch()).count();
}

int main(int argc, char** argv) {
    if (argc < 2) { cerr << "usage: ref_harness <command> ..." << endl; return 2; }
    const string cmd = argv[1];
    auto arg = [&](int i) { return string(argv[i]); };
    try {
        if (cmd == "frops") {                       // a b
            FrTensor a(arg(2)), b(arg(3));
            print_tensor("add", a + b);
            print_tensor("sub", a - b);
            print_tensor("mul", a * b);
            print_tensor("neg", -a);
            FrTensor m(a); m.mont(); print_tensor("mont", m);
            FrTensor um(a); um.unmont(); print_tensor("unmont", um);
            cout << "sum " << a.sum() << endl;
            Fr_t x = b(0);
            print_tensor("adds", a + x);
            print_tensor("subs", a - x);
            print_tensor("muls", a * x);
            cout << "host_add " << (a(0) + x) << endl;
            cout << "host_sub " << (a(0) - x) << endl;
            cout << "host_mul " << (a(0) * x) << endl;
            cout << "host_div " << (a(0) / x) << endl;
            cout << "host_inv " << inv(x) << endl;
        } else if (cmd == "ints") {                 // int.bin
            FrTensor a = FrTensor::from_int_bin(arg(2));
            print_tensor("from_int", a);
            a.save_int(arg(3));
            a.save_long(arg(4));
        } else if (cmd == "me") {                   // t u
            FrTensor t(arg(2));
            cout << "me " << t(load_vec(arg(3))) << endl;
        } else if (cmd == "partial_me") {           // t u cur_dim window
            FrTensor t(arg(2));
            print_tensor("partial_me", t.partial_me(load_vec(arg(3)), (uint)stoul(arg(4)), (uint)stoul(arg(5))));
        } else if (cmd == "partial_me_window") {    // t u window
            FrTensor t(arg(2));
            print_tensor("partial_me_window", t.partial_me(load_vec(arg(3)), (uint)stoul(arg(4))));
        } else if (cmd == "multi_dim_me") {         // t u0 u1 d0 d1
            FrTensor t(arg(2));
            cout << "multi_dim_me " << t.multi_dim_me({load_vec(arg(3)), load_vec(arg(4))}, {(uint)stoul(arg(5)), (uint)stoul(arg(6))}) << endl;
        } else if (cmd == "layout") {               // t d0 d1
            FrTensor t(arg(2));
            uint d0 = stoul(arg(3)), d1 = stoul(arg(4));
            print_tensor("pad", t.pad({d0, d1}));
            print_tensor("transpose", t.transpose(d0, d1));
        } else if (cmd == "matmul") {               // x y M N P
            FrTensor x(arg(2)), y(arg(3));
            print_tensor("matmul", FrTensor::matmul(x, y, stoul(arg(4)), stoul(arg(5)), stoul(arg(6))));
        } else if (cmd == "zkip") {                 // claim a b u
            FrTensor a(arg(3)), b(arg(4));
            vector<Polynomial> proof;
            Fr_t fc = zkip(load_vec(arg(2))[0], a, b, load_vec(arg(5)), proof);
            print_polys("poly", proof);
            cout << "final " << fc << endl;
        } else if (cmd == "zkfc") {                 // X W Y B I O ub ui uo : the body of zkFC::prove with given challenges
            FrTensor X(arg(2)), W(arg(3)), Y(arg(4));
            uint B = stoul(arg(5)), I = stoul(arg(6)), O = stoul(arg(7));
            auto ub = load_vec(arg(8)), ui = load_vec(arg(9)), uo = load_vec(arg(10));
            zkFC fc(I, O, W);
            print_tensor("forward", fc(X));
            auto claim = Y.multi_dim_me({ub, uo}, {B, O});
            auto X_red = X.partial_me(ub, B, I);
            auto W_red = W.partial_me(uo, O, 1);
            vector<Polynomial> proof;
            auto final_claim = zkip(claim, X_red, W_red, ui, proof);
            auto claim_X = X.multi_dim_me({ub, ui}, {B, I});
            auto claim_W = W.multi_dim_me({ui, uo}, {I, O});
            print_polys("poly", proof);
            cout << "claim " << claim << endl << "final " << final_claim << endl;
            cout << "claim_x " << claim_X << endl << "claim_w " << claim_W << endl;
            print_tensor("x_red", X_red);
            print_tensor("w_red", W_red);
            cout << "ok " << (claim_X * claim_W == final_claim) << endl;
        } else if (cmd == "tlookup") {              // S(int.bin) low len alpha beta u v : range lookup, all round polynomials
            FrTensor S = FrTensor::from_int_bin(arg(2));
            tLookupRange tl(stoi(arg(3)), stoul(arg(4)));
            auto m = tl.prep(S);
            print_tensor("table", tl.table);
            print_tensor("m", m);
            Fr_t alpha = load_vec(arg(5))[0], beta = load_vec(arg(6))[0];
            auto u = load_vec(arg(7)), v = load_vec(arg(8));
            vector<Polynomial> proof;
            cout << "final " << tl.prove(S, m, alpha, beta, u, v, proof) << endl;
            // replay the rounds with the reference's own step functions to expose the polynomials
            const uint D = S.size, N = m.size;
            FrTensor A = S, B = tl.table;           // sized buffers
            {
                FrTensor Sb = S + beta, Tb = tl.table + beta;
                vector<Fr_t> hs(D), ht(N);
                cudaMemcpy(hs.data(), Sb.gpu_data, sizeof(Fr_t) * D, cudaMemcpyDeviceToHost);
                cudaMemcpy(ht.data(), Tb.gpu_data, sizeof(Fr_t) * N, cudaMemcpyDeviceToHost);
                for (auto& x : hs) x = inv(x);
                for (auto& x : ht) x = inv(x);
                cudaMemcpy(A.gpu_data, hs.data(), sizeof(Fr_t) * D, cudaMemcpyHostToDevice);
                cudaMemcpy(B.gpu_data, ht.data(), sizeof(Fr_t) * N, cudaMemcpyHostToDevice);
            }
            print_tensor("A", A);
            const uint k1 = ceilLog2(D / N);
            vector<Fr_t> v1(v.begin(), v.begin() + k1), v2(v.begin() + k1, v.end());
            Fr_t alpha_sq = alpha * alpha;
            Fr_t C = alpha_sq - (B * m).sum();
            Fr_t a_cur = alpha;
            const Fr_t TWO_INV_ = inv(Fr_t{2, 0, 0, 0, 0, 0, 0, 0});
            Fr_t ratio = Fr_t{N, 0, 0, 0, 0, 0, 0, 0} / Fr_t{D, 0, 0, 0, 0, 0, 0, 0};
            FrTensor cA = A, cS = S;
            int round = 0;
            while (v1.size()) {
                auto p = tLookup_phase1_step_poly(cA, cS, a_cur, beta, C, u);
                cout << "poly" << round++ << " " << p << endl;
                // fold MSB-first with v1.back(): lo + v (hi - lo)
                uint half = cA.size / 2;
                FrTensor loA = cA.trunc(0, half), hiA = cA.trunc(half, cA.size), loS = cS.trunc(0, half), hiS = cS.trunc(half, cS.size);
                FrTensor nA = loA + (hiA - loA) * v1.back(), nS = loS + (hiS - loS) * v1.back();
                a_cur = a_cur * Polynomial::eq(u.back(), v1.back());
                C = C * TWO_INV_;
                u.pop_back(); v1.pop_back();
                FrTensor tA(nA), tS(nS);
                cA.~FrTensor(); new (&cA) FrTensor(tA);
                cS.~FrTensor(); new (&cS) FrTensor(tS);
            }
            FrTensor cB = B, cT = tl.table, cm = m;
            while (v2.size()) {
                auto p = tLookup_phase2_step_poly(cA, cS, cB, cT, cm, a_cur, beta, ratio, alpha_sq, u);
                cout << "poly" << round++ << " " << p << endl;
                uint half = cm.size / 2;
                auto fold = [&](FrTensor& t) {
                    FrTensor lo = t.trunc(0, half), hi = t.trunc(half, t.size);
                    FrTensor n = lo + (hi - lo) * v2.back();
                    t.~FrTensor(); new (&t) FrTensor(n);
                };
                if (half >= 1) { fold(cA); fold(cS); fold(cB); fold(cT); fold(cm); }
                Fr_t e = Polynomial::eq(u.back(), v2.back());
                a_cur = a_cur * e;
                alpha_sq = alpha_sq * e;
                u.pop_back(); v2.pop_back();
            }
        } else if (cmd == "mapping") {              // S_in(int.bin) low len mapped(Fr) r alpha beta u v
            FrTensor S = FrTensor::from_int_bin(arg(2));
            FrTensor mapped(arg(5));
            tLookupRangeMapping tl(stoi(arg(3)), stoul(arg(4)), mapped);
            auto p = tl(S);
            print_tensor("y", p.first);
            print_tensor("m", p.second);
            vector<Polynomial> proof;
            cout << "final " << tl.prove(S, p.first, p.second, load_vec(arg(6))[0], load_vec(arg(7))[0], load_vec(arg(8))[0],
                                         load_vec(arg(9)), load_vec(arg(10)), proof) << endl;
        } else if (cmd == "hadamard") {             // claim u v X0 X1 ...
            vector<FrTensor> Xs;
            for (int i = 5; i < argc; ++i) Xs.push_back(FrTensor(arg(i)));
            vector<Polynomial> proof;
            cout << "final " << multi_hadamard_sumchecks(load_vec(arg(2))[0], Xs, load_vec(arg(3)), load_vec(arg(4)), proof) << endl;
            print_polys("poly", proof);
        } else if (cmd == "legacy") {               // a b u v
            FrTensor a(arg(2)), b(arg(3));
            auto u = load_vec(arg(4)), v = load_vec(arg(5));
            auto hp = hadamard_product_sumcheck(a, b, u, v);
            cout << "hp"; for (auto& x : hp) cout << " " << x; cout << endl;
            auto ip = inner_product_sumcheck(a, b, u);
            cout << "ip"; for (auto& x : ip) cout << " " << x; cout << endl;
            auto bn = binary_sumcheck(a, u, v);
            cout << "bin"; for (auto& x : bn) cout << " " << x; cout << endl;
        } else if (cmd == "rescale") {              // X(long.bin as Fr file) sf
            FrTensor X(arg(2));
            Rescaling rs(stoul(arg(3)));
            print_tensor("out", rs(X));
            print_tensor("rem", *rs.rem_tensor_ptr);
        } else if (cmd == "softmax") {              // X(Fr) m n d : the driver's parameters (self-attn.cu:87)
            FrTensor X(arg(2));
            uint m = stoul(arg(3)), n = stoul(arg(4)), d = stoul(arg(5));
            zkSoftmax sm({1 << 8, 1 << 20, 1 << 20}, 1, 0, 1UL << 32, {1 << 18, 1 << 22}, m, n, d, 1);
            FrTensor shift(m), X_shifted(m * n);
            vector<FrTensor> Xs, Ys, ms;
            FrTensor Y = sm.compute(X, shift, X_shifted, Xs, Ys, ms);
            print_tensor("shift", shift);
            print_tensor("y", Y);
            for (size_t i = 0; i < Xs.size(); ++i) print_tensor("xseg" + to_string(i), Xs[i]);
            for (size_t i = 0; i < Ys.size(); ++i) print_tensor("yseg" + to_string(i), Ys[i]);
            if (argc > 6) {                         // u v r alpha beta: the proof
                vector<Polynomial> proof;
                cout << "final " << sm.prove(Y, X, shift, X_shifted, Xs, Ys, ms, load_vec(arg(6)), load_vec(arg(7)),
                                             load_vec(arg(8))[0], load_vec(arg(9))[0], load_vec(arg(10))[0], proof) << endl;
                print_polys("poly", proof);
            }
        } else if (cmd == "g1ops") {                // gens(G1) scalars(Fr) u
            G1TensorJacobian g(arg(2));
            FrTensor s(arg(3));
            print_g1_tensor("mul", g * s);
            print_g1_tensor("add", g + g);
            print_g1s("sum", {g.sum()});
            auto u = load_vec(arg(4));
            print_g1s("me", {g(u)});
        } else if (cmd == "commit") {               // gens(G1) ints(int.bin) full(Fr) u
            Commitment gen(arg(2));
            FrTensor t = FrTensor::from_int_bin(arg(3));
            auto com = gen.commit_int(t);
            print_g1_tensor("commit_int", com);
            FrTensor f(arg(4));
            print_g1_tensor("commit", gen.commit(f));
            auto u = load_vec(arg(5));
            cout << "open " << gen.open(t, com, u) << endl;
            // the same call sequence as Commitment::open with the proof kept
            const vector<Fr_t> u_out(u.end() - ceilLog2(com.size), u.end());
            const vector<Fr_t> u_in(u.begin(), u.end() - ceilLog2(com.size));
            vector<G1Jacobian_t> proof;
            auto folded = t.partial_me(u_out, t.size / com.size);
            cout << "me_open " << Commitment::me_open(folded, gen, u_in.begin(), u_in.end(), proof) << endl;
            print_g1s("proof", proof);
        } else if (cmd == "bench-commit") {         // gens(G1) ints(int.bin) steps warmup
            Commitment gen(arg(2));
            FrTensor t = FrTensor::from_int_bin(arg(3));
            int steps = stoi(arg(4)), warm = stoi(arg(5));
            cudaDeviceSynchronize();
            for (int i = 0; i < warm; ++i) { auto c = gen.commit_int(t); }
            cudaDeviceSynchronize();
            for (int i = 0; i < steps; ++i) {
                double t0 = now_s();
                auto c = gen.commit_int(t);
                cudaDeviceSynchronize();
                cout << "step_s " << (now_s() - t0) << endl;
                if (i == steps - 1) c.save(arg(6));
            }
        } else if (cmd == "bench-zkfc") {           // X W Y B I O ub ui uo steps warmup : body of zkFC::prove
            FrTensor X(arg(2)), W(arg(3)), Y(arg(4));
            uint B = stoul(arg(5)), I = stoul(arg(6)), O = stoul(arg(7));
            auto ub = load_vec(arg(8)), ui = load_vec(arg(9)), uo = load_vec(arg(10));
            int steps = stoi(arg(11)), warm = stoi(arg(12));
            for (int i = 0; i < warm + steps; ++i) {
                cudaDeviceSynchronize();
                double t0 = now_s();
                auto claim = Y.multi_dim_me({ub, uo}, {B, O});
                auto X_red = X.partial_me(ub, B, I);
                auto W_red = W.partial_me(uo, O, 1);
                vector<Polynomial> proof;
                auto final_claim = zkip(claim, X_red, W_red, ui, proof);
                auto claim_X = X.multi_dim_me({ub, ui}, {B, I});
                auto claim_W = W.multi_dim_me({ui, uo}, {I, O});
                bool ok = (claim_X * claim_W == final_claim);
                cudaDeviceSynchronize();
                if (i >= warm) cout << "step_s " << (now_s() - t0) << endl;
                if (i == warm + steps - 1) cout << "final " << final_claim << endl << "ok " << ok << endl;
            }
        } else if (cmd == "bench-tlookup") {        // S(int.bin) low len alpha beta u v steps warmup : prep + prove
            FrTensor S = FrTensor::from_int_bin(arg(2));
            tLookupRange tl(stoi(arg(3)), stoul(arg(4)));
            Fr_t alpha = load_vec(arg(5))[0], beta = load_vec(arg(6))[0];
            auto u = load_vec(arg(7)), v = load_vec(arg(8));
            int steps = stoi(arg(9)), warm = stoi(arg(10));
            for (int i = 0; i < warm + steps; ++i) {
                cudaDeviceSynchronize();
                double t0 = now_s();
                auto m = tl.prep(S);
                vector<Polynomial> proof;
                Fr_t fc = tl.prove(S, m, alpha, beta, u, v, proof);
                cudaDeviceSynchronize();
                if (i >= warm) cout << "step_s " << (now_s() - t0) << endl;
                if (i == warm + steps - 1) cout << "final " << fc << endl;
            }
        } else {
            cerr << "unknown command " << cmd << endl;
            return 2;
        }
        cudaError_t e = cudaDeviceSynchronize();
        if (e != cudaSuccess) { cerr << "cuda error: " << cudaGetErrorString(e) << endl; return 3; }
    } catch (const std::exception& ex) {
        cout << "exception " << ex.what() << endl;
        return 1;
    }
    return 0;
}
