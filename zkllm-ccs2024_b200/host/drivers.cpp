// Per-layer stage drivers with the reference's command lines and .bin hand-off
// files (reference: ppgen.cu, commit-param.cu, rmsnorm.cu, self-attn.cu, ffn.cu,
// skip-connection.cu).  One executable; the stage is the first argument, or the
// name the program was invoked under (a symlink called `ffn` runs the ffn stage):
//
//   zkllm-driver ppgen <size> <out-pp.bin>
//   zkllm-driver commit-param <pp.bin> <int.bin> <out-commitment.bin> <in_dim> <out_dim>
//   zkllm-driver rmsnorm <input|post_attention> <in.bin> <seq> <embed> <workdir> <layer-prefix> <out.bin>
//   zkllm-driver self-attn <linear|attn> <in.bin> <seq> <embed> <workdir> <layer-prefix> <out.bin>
//   zkllm-driver ffn <in.bin> <seq> <embed> <hidden> <workdir> <layer-prefix> <out.bin>
//   zkllm-driver skip-connection <x.bin> <y.bin> <out.bin>
//   zkllm-driver batch <script|->      (no counterpart in the reference)
//
// `batch` reads one stage command per line ("ffn in.bin 2048 4096 ..."; blank
// lines and lines starting with # are skipped) and runs them in this one
// process, so a whole layer pays for one CUDA context and one module load
// instead of one per stage.  After each line it prints "[batch] <stage> <s> s"
// to stderr; with ZKLLM_PROFILE=1 it also prints the library's per-kernel times.
// The first failing stage ends the batch with its exception.
//
// Several driver processes, one per GPU, can share the proofs of one layer: with
// ZKLLM_PROOF_WORLD=P and ZKLLM_PROOF_RANK=r every process computes all the outputs
// (they are cheap next to the proofs, and each process needs them as inputs of its
// proofs), while every proof of the layer (a rescaling lookup, a zkFC sumcheck with
// the opening of its weight, the softmax proof, ...) is run by exactly one process.
// The proofs are independent of one another (each draws its own challenges), so
// the processes exchange nothing; the layer is proven when all of them exit 0.
// The deal is the same in every process: each proof goes to the process with the
// least estimated work so far; a batch line "begin-layer" starts the deal afresh, so
// that every layer of a batch is dealt out the same way.  Give every process its own
// working directory for the hand-off files and the same <workdir> for the parameters.
// Each stage computes its fixed-point outputs in the field, proves them and
// throws if a verifier equation fails, printing the reference's progress lines.
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <functional>
#include <map>
#include <sstream>
#include <string>

#include "../../include/zkllm_b200.h"

#include "commitment.cuh"
#include "fr-tensor.cuh"
#include "proof.cuh"
#include "rescaling.cuh"
#include "zkfc.cuh"
#include "zksoftmax.cuh"
#include "zkllm_ext.hpp"

namespace {

typedef std::vector<std::string> Args;

// With ZKLLM_PROFILE=1: wall seconds since the previous mark, to stderr.
struct StepClock {
    std::chrono::steady_clock::time_point last = std::chrono::steady_clock::now();
    bool on = std::getenv("ZKLLM_PROFILE") && std::getenv("ZKLLM_PROFILE")[0] == '1';
    void mark(const char* what) {
        if (!on) return;
        const auto now = std::chrono::steady_clock::now();
        cerr << "[step] " << what << " " << std::chrono::duration<double>(now - last).count() << " s" << endl;
        last = now;
    }
};

// Which of the P cooperating driver processes proves the next proof (see the head of this file).
class ProofShare {
public:
    void configure(int rank, int world) {
        if (world < 1 || rank < 0 || rank >= world) throw std::runtime_error("ZKLLM_PROOF_RANK / ZKLLM_PROOF_WORLD: bad values");
        rank_ = rank;
        load_.assign(world, 0.0);
    }
    void begin_layer() { load_.assign(load_.size(), 0.0); }
    // cost: estimated milliseconds of the proof; only the ratios matter
    bool take(double cost) {
        size_t to = 0;
        for (size_t i = 1; i < load_.size(); ++i)
            if (load_[i] < load_[to]) to = i;
        load_[to] += cost;
        ++dealt_;
        if ((int)to != rank_) return false;
        ++mine_;
        return true;
    }
    void report() const {
        if (load_.size() < 2) return;
        double most = 0;
        for (double l : load_) most = std::max(most, l);
        cerr << "[share] process " << rank_ << " of " << load_.size() << ": " << mine_ << " of " << dealt_
             << " proofs; last layer: estimated " << load_[rank_] << " ms here, " << most << " ms on the busiest" << endl;
    }

private:
    int rank_ = 0;
    std::vector<double> load_ = std::vector<double>(1, 0.0);
    unsigned long dealt_ = 0, mine_ = 0;
};

ProofShare g_share;

template <class Body>
void proof(double cost, Body&& body) {
    if (g_share.take(cost)) body();
}

// Estimates in milliseconds on one B200, from the stage clocks of the 7B-shape layer.
double cost_lookup(size_t values) { return 1.0 + 1.0e-6 * values; }             // Rescaling::prove
double cost_weight_claim(size_t weights) { return 4.0 + 2.0e-6 * weights; }     // zkFC::prove + the opening
double cost_sumcheck(size_t values) { return 1.0 + 0.3e-6 * values; }

// generator, int weights and commitment of one parameter of one layer
Weight load_param(const std::string& workdir, const std::string& prefix, const std::string& name, uint in_dim, uint out_dim) {
    return create_weight(workdir + "/" + name + "-pp.bin", workdir + "/" + prefix + "-" + name + "-int.bin",
                         workdir + "/" + prefix + "-" + name + "-commitment.bin", in_dim, out_dim);
}

// forward + rescale + both proofs of one linear layer; returns the rescaled output
struct Linear {
    Weight w;
    zkFC fc;
    Rescaling rs;
    Linear(const Weight& weight, uint in_dim, uint out_dim, uint scale) : w(weight), fc(in_dim, out_dim, w.weight), rs(scale) {}
};

int run_ppgen(const Args& a) {
    const uint size = std::stoi(a.at(0));
    Commitment::random(1u << ceilLog2(size)).save(a.at(1));
    return 0;
}

int run_commit_param(const Args& a) {
    Commitment generator(a.at(0));
    if (generator.size != (1u << ceilLog2(generator.size))) throw std::runtime_error("Generator size has to be a power of 2");
    const uint in_dim = std::stoi(a.at(3)), out_dim = std::stoi(a.at(4));
    FrTensor param = FrTensor::from_int_bin(a.at(1));
    cout << "Param size: " << param.size << endl << "In dim: " << in_dim << endl << "Out dim: " << out_dim << endl;
    auto padded = param.pad({in_dim, out_dim});
    auto com = generator.commit_int(padded);
    cout << "Generator size: " << generator.size << endl << "Unpadded param size: " << param.size << endl;
    cout << "Padded param size: " << padded.size << endl << "Commitment size: " << com.size << endl;
    com.save(a.at(2));
    return 0;
}

int run_rmsnorm(const Args& a) {
    const std::string which = a.at(0);
    const uint seq = std::stoi(a.at(2)), embed = std::stoi(a.at(3));
    auto weight = load_param(a.at(4), a.at(5), which + "_layernorm.weight", 1, embed);
    FrTensor X = FrTensor::from_int_bin(a.at(1));
    FrTensor rms_inv = FrTensor::from_int_bin("rms_inv_temp.bin");   // written by the Python side, one value per row
    Rescaling rs_gain(1 << 16), rs_out(1 << 16);
    zkFC gain(1, embed, weight.weight);
    auto g_rms = gain(rms_inv);                 // outer product [seq, embed]
    auto g_rms_ = rs_gain(g_rms);
    auto Y = g_rms_ * X;
    auto Y_ = rs_out(Y);
    Y_.save_int(a.at(6));
    proof(cost_lookup(Y.size), [&] { rs_out.prove(Y, Y_); });
    proof(cost_sumcheck(Y.size),
          [&] { hadamard_product_sumcheck(g_rms_, X, random_vec(ceilLog2(Y.size)), random_vec(ceilLog2(Y.size))); });
    proof(cost_lookup(g_rms.size), [&] { rs_gain.prove(g_rms, g_rms_); });
    zkllm::WeightOpenings openings;
    proof(cost_weight_claim(embed), [&] { openings.add(weight, gain.prove(rms_inv, g_rms)[0]); });
    openings.finish();
    (void)seq;
    return 0;
}

int run_self_attn(const Args& a) {
    const std::string mode = a.at(0);
    const uint seq = std::stoi(a.at(2)), embed = std::stoi(a.at(3));
    if (mode == "linear") {
        FrTensor input = FrTensor::from_int_bin(a.at(1));
        const char* names[3] = {"q", "k", "v"};
        std::vector<Linear*> layers;
        std::vector<FrTensor> raw, scaled;
        for (const char* nm : names) {
            layers.push_back(new Linear(load_param(a.at(4), a.at(5), std::string("self_attn.") + nm + "_proj.weight", embed, embed),
                                        embed, embed, 1 << 16));
            raw.push_back(layers.back()->fc(input));
            scaled.push_back(layers.back()->rs(raw.back()));
        }
        scaled[0].save_int("temp_Q.bin");
        scaled[1].save_int("temp_K.bin");
        scaled[2].save_int("temp_V.bin");
        // the openings are started first (the reference opens k, then q, then v) and run beside the lookups
        zkllm::WeightOpenings openings;
        for (int i : {1, 0, 2})
            proof(cost_weight_claim((size_t)embed * embed), [&] { openings.add(layers[i]->w, layers[i]->fc.prove(input, raw[i])[0]); });
        for (int i = 0; i < 3; ++i) proof(cost_lookup(raw[i].size), [&] { layers[i]->rs.prove(raw[i], scaled[i]); });
        openings.finish();
        for (auto* l : layers) delete l;
        cout << "QKV linear proof successfully verified!" << endl;
        return 0;
    }
    if (mode == "attn") {
        auto Q = FrTensor::from_int_bin("temp_Q.bin");
        auto K = FrTensor::from_int_bin("temp_K.bin");
        auto V = FrTensor::from_int_bin("temp_V.bin");
        const uint d = Q.size / seq;   // all heads together, as the reference does
        auto X = FrTensor::matmul(Q, K.transpose(seq, d), seq, d, seq);
        zkSoftmax softmax({1 << 8, 1 << 20, 1 << 20}, 1, 0, 1UL << 32, {1 << 18, 1 << 22}, seq, seq, d, 1);
        Rescaling rs1(1 << 20), rs2(1 << 20);
        FrTensor shift(seq), X_shifted(seq * seq);
        vector<FrTensor> X_segments, Y_segments, m_segments;
        FrTensor Y = softmax.compute(X, shift, X_shifted, X_segments, Y_segments, m_segments);
        Y.save_long("temp_head_Y.bin");
        auto out = FrTensor::matmul(Y, V, seq, seq, d);
        auto out_ = rs2(out);
        auto out__ = rs1(out_);
        out__.save_int("temp_head_out.bin");
        proof(cost_lookup(out_.size), [&] { rs1.prove(out_, out__); });
        proof(cost_lookup(out.size), [&] { rs2.prove(out, out_); });
        auto temp_rand = random_vec(3);
        vector<Polynomial> polys;
        proof(cost_sumcheck(Y.size + V.size), [&] {
            auto u1 = random_vec(ceilLog2(seq));
            auto u2 = random_vec(ceilLog2(d));
            auto ud = random_vec(ceilLog2(seq));
            auto claim = out.multi_dim_me({u1, u2}, {seq, d});
            zkip(claim, Y.partial_me(u1, seq, seq), V.partial_me(u2, d, 1), ud, polys);
        });
        proof(8.0 * cost_lookup(Y.size), [&] {   // three segment lookups, the products between them and the row sums
            auto u_sm = random_vec(ceilLog2(Y.size));
            auto v_sm = random_vec(ceilLog2(Y.size));
            softmax.prove(Y, X, shift, X_shifted, X_segments, Y_segments, m_segments, u_sm, v_sm, temp_rand[0], temp_rand[1],
                          temp_rand[2], polys);
        });
        proof(cost_sumcheck(X.size + Q.size + K.size), [&] {
            auto u1_ = random_vec(ceilLog2(seq));
            auto u2_ = random_vec(ceilLog2(seq));
            auto ud_ = random_vec(ceilLog2(d));
            auto claim_ = X.multi_dim_me({u1_, u2_}, {seq, seq});
            zkip(claim_, Q.partial_me(u1_, seq, d), K.partial_me(u2_, seq, d), ud_, polys);
        });
        cout << "Self attention proof successfully verified!" << endl;
        return 0;
    }
    return 0;
}

int run_ffn(const Args& a) {
    StepClock clk;
    const uint seq = std::stoi(a.at(1)), embed = std::stoi(a.at(2)), hidden = std::stoi(a.at(3));
    const std::string workdir = a.at(4), prefix = a.at(5);
    Linear up(load_param(workdir, prefix, "mlp.up_proj.weight", embed, hidden), embed, hidden, 1 << 16);
    Linear gate(load_param(workdir, prefix, "mlp.gate_proj.weight", embed, hidden), embed, hidden, 1 << 20);
    Linear down(load_param(workdir, prefix, "mlp.down_proj.weight", hidden, embed), hidden, embed, 1 << 16);
    Rescaling hidden_rescale(1 << 16);
    FrTensor swiglu_values = FrTensor::from_int_bin("swiglu-table.bin");   // written by the Python side
    tLookupRangeMapping swiglu(-(1 << 21), 1 << 22, swiglu_values);
    clk.mark("load parameters");

    FrTensor input = FrTensor::from_int_bin(a.at(0));
    auto up_out = up.fc(input);
    auto up_out_ = up.rs(up_out);
    auto gate_out = gate.fc(input);
    auto gate_out_ = gate.rs(gate_out);
    auto act = swiglu(gate_out_);   // (activations, multiplicities)
    auto temp_rand = random_vec(3);
    auto swiglu_u = random_vec(ceilLog2(seq * hidden));
    auto swiglu_v = random_vec(ceilLog2(seq * hidden));
    vector<Polynomial> swiglu_proof;
    auto down_in = act.first * up_out_;
    auto down_in_ = hidden_rescale(down_in);
    auto down_out = down.fc(down_in_);
    auto down_out_ = down.rs(down_out);
    clk.mark("forward");
    down_out.save_int(a.at(6));   // the reference saves the value before the last rescaling
    clk.mark("save");

    const size_t n_weights = (size_t)embed * hidden;
    // the three matmul proofs first: their openings then run beside the lookups below
    zkllm::WeightOpenings openings;
    proof(cost_weight_claim(n_weights), [&] { openings.add(up.w, up.fc.prove(input, up_out)[0]); });
    proof(cost_weight_claim(n_weights), [&] { openings.add(gate.w, gate.fc.prove(input, gate_out)[0]); });
    proof(cost_weight_claim(n_weights), [&] { openings.add(down.w, down.fc.prove(down_in_, down_out)[0]); });
    clk.mark("fc proofs, openings started");
    proof(cost_lookup(down_out.size), [&] { down.rs.prove(down_out, down_out_); });
    clk.mark("down rescale prove");
    proof(cost_lookup(down_in.size), [&] { hidden_rescale.prove(down_in, down_in_); });
    clk.mark("hidden rescale prove");
    proof(cost_lookup(gate_out_.size), [&] {
        swiglu.prove(gate_out_, act.first, act.second, temp_rand[0], temp_rand[1], temp_rand[2], swiglu_u, swiglu_v, swiglu_proof);
    });
    cout << "SwiGLU proof complete." << endl;
    clk.mark("swiglu prove");
    proof(cost_lookup(gate_out.size), [&] { gate.rs.prove(gate_out, gate_out_); });
    clk.mark("gate rescale prove");
    proof(cost_lookup(up_out.size), [&] { up.rs.prove(up_out, up_out_); });
    clk.mark("up rescale prove");
    openings.finish();
    clk.mark("openings finished");
    return 0;
}

int run_skip(const Args& a) {
    FrTensor x = FrTensor::from_int_bin(a.at(0));
    FrTensor y = FrTensor::from_int_bin(a.at(1));
    (x + y).save_int(a.at(2));
    return 0;
}

typedef std::map<std::string, std::pair<std::function<int(const Args&)>, size_t>> StageTable;

const StageTable& stage_table() {
    static const StageTable stages = {
        {"ppgen", {run_ppgen, 2}},         {"commit-param", {run_commit_param, 5}}, {"rmsnorm", {run_rmsnorm, 7}},
        {"self-attn", {run_self_attn, 7}}, {"ffn", {run_ffn, 7}},                   {"skip-connection", {run_skip, 3}}};
    return stages;
}

int run_batch(const Args& a) {
    std::ifstream file;
    if (a.at(0) != "-") {
        file.open(a.at(0));
        if (!file) throw std::runtime_error("batch: cannot open " + a.at(0));
    }
    std::istream& in = a.at(0) == "-" ? std::cin : file;
    const char* prof_env = std::getenv("ZKLLM_PROFILE");
    const bool profile = prof_env && prof_env[0] == '1';
    if (profile) zkb_profile_enable(1);
    // generators, weights, commitments and the activations handed from stage to stage stay on the device
    // (every file is still written); ZKLLM_RESIDENT=0 reads every file from disk again, as separate processes do
    const char* res_env = std::getenv("ZKLLM_RESIDENT");
    zkllm::set_resident_files(!(res_env && res_env[0] == '0'));
    // ZKLLM_PRIORITY_STREAM=1: this process's own work runs on a high-priority stream, so that while openings are in
    // flight on the library's streams its short kernels are scheduled ahead of the openings' long-running blocks.  Off by
    // default: the sumchecks then start sooner and the openings end later, and a layer takes the same time.
    const char* prio_env = std::getenv("ZKLLM_PRIORITY_STREAM");
    void* work_stream = nullptr;
    if (prio_env && prio_env[0] == '1' && zkb_stream_create(1, &work_stream) == ZKB_OK) zkb_set_default_stream(work_stream);
    // output files go to the disk from a writer thread while the stage proves; each is complete before its line is answered
    const char* def_env = std::getenv("ZKLLM_DEFERRED_SAVES");
    zkllm::set_deferred_saves(!(def_env && def_env[0] == '0'));
    zkllm::ResidentStats before = zkllm::resident_stats();
    std::string line;
    while (std::getline(in, line)) {
        std::istringstream words(line);
        Args cmd;
        for (std::string w; words >> w;) cmd.push_back(w);
        if (cmd.empty() || cmd[0][0] == '#') continue;
        const std::string stage = cmd[0];
        if (stage == "begin-layer") {
            g_share.begin_layer();
            cerr << "[batch] begin-layer 0 s" << endl;
            continue;
        }
        if (!stage_table().count(stage)) throw std::runtime_error("batch: unknown stage " + stage);
        cmd.erase(cmd.begin());
        if (cmd.size() < stage_table().at(stage).second) throw std::runtime_error("batch: too few arguments for " + stage);
        if (profile) zkb_profile_reset();
        const auto t0 = std::chrono::steady_clock::now();
        const int rc = stage_table().at(stage).first(cmd);
        zkllm::flush_saves();
        const double secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        const zkllm::ResidentStats now = zkllm::resident_stats();
        cerr << "[files] " << stage << " loads from disk " << now.loads_from_disk - before.loads_from_disk << " ("
             << (now.bytes_from_disk - before.bytes_from_disk) / 1048576 << " MiB), from the device "
             << now.loads_from_device - before.loads_from_device << " (" << (now.bytes_from_device - before.bytes_from_device) / 1048576
             << " MiB)" << endl;
        before = now;
        cerr << "[batch] " << stage << (stage == "self-attn" || stage == "rmsnorm" ? " " + cmd[0] : "") << " " << secs << " s" << endl;
        if (profile) {
            std::vector<char> buf(1 << 16);
            if (zkb_profile_read(buf.data(), buf.size()) == 0) cerr << buf.data();
        }
        if (rc) return rc;
    }
    g_share.report();
    return 0;
}

}  // namespace

int main(int argc, char* argv[]) {
    StageTable stages = stage_table();
    stages["batch"] = {run_batch, 1};
    std::string self = argv[0];
    const size_t slash = self.find_last_of('/');
    if (slash != std::string::npos) self = self.substr(slash + 1);
    int first = 1;
    std::string stage = self;
    if (!stages.count(stage)) {
        if (argc < 2 || !stages.count(argv[1])) {
            cerr << "usage: " << self << " <ppgen|commit-param|rmsnorm|self-attn|ffn|skip-connection|batch> <stage arguments>" << endl;
            return 2;
        }
        stage = argv[1];
        first = 2;
    }
    Args args(argv + first, argv + argc);
    if (const char* world = std::getenv("ZKLLM_PROOF_WORLD")) {
        const char* rank = std::getenv("ZKLLM_PROOF_RANK");
        try {
            g_share.configure(rank ? std::stoi(rank) : 0, std::stoi(world));
        } catch (const std::exception& ex) {
            cerr << "ZKLLM_PROOF_RANK / ZKLLM_PROOF_WORLD: " << ex.what() << endl;
            return 2;
        }
    }
    if (args.size() < stages.at(stage).second) {
        cerr << stage << ": expected " << stages.at(stage).second << " arguments" << endl;
        return 2;
    }
    return stages.at(stage).first(args);
}
