// FrTensor over the C ABI (reference: fr-tensor.cu).  Error texts are the
// reference's, so callers that match on what() keep working.
#include "fr-tensor.cuh"

#include <climits>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <mutex>
#include <stdexcept>

#include "ioutils.cuh"
#include "zkllm_ext.hpp"

namespace zkllm {

void check(int rc) {
    if (rc == ZKB_OK) return;
    throw std::runtime_error(zkb_last_error());
}

namespace {
std::mutex g_seed_mu;
bool g_seeded = false;
bool g_seeded_by_env = false;
std::mt19937_64 g_seed_rng;
bool g_env_checked = false;
Transcript* g_sink = nullptr;
}  // namespace

void seed_challenges(uint64_t seed) {
    std::lock_guard<std::mutex> lk(g_seed_mu);
    g_seeded = true;
    g_seeded_by_env = false;
    g_env_checked = true;
    g_seed_rng.seed(seed);
}
void unseed_challenges() {
    std::lock_guard<std::mutex> lk(g_seed_mu);
    g_seeded = false;
    g_env_checked = true;
}
void set_transcript_sink(Transcript* sink) { g_sink = sink; }
Transcript* transcript_sink() { return g_sink; }

// fills `out` with `words` 32-bit words from the seeded stream; false when unseeded.
// for_generators: the draw makes tensor values (FrTensor::random*, hence Commitment::random and
// ppgen).  Those honour only a seed set by seed_challenges(): a seed left in the environment
// must not make commitment generators with predictable discrete logarithms.
static bool seeded_words(uint32_t* out, size_t words, bool for_generators = false) {
    std::lock_guard<std::mutex> lk(g_seed_mu);
    if (!g_env_checked) {
        g_env_checked = true;
        if (const char* e = std::getenv("ZKLLM_CHALLENGE_SEED")) {
            g_seeded = true;
            g_seeded_by_env = true;
            g_seed_rng.seed(std::strtoull(e, nullptr, 0));
            std::cerr << "zkllm: ZKLLM_CHALLENGE_SEED is set - verifier challenges are deterministic (testing only, not sound)"
                      << std::endl;
        }
    }
    if (!g_seeded || (for_generators && g_seeded_by_env)) return false;
    for (size_t i = 0; i < words; ++i) out[i] = (uint32_t)g_seed_rng();
    return true;
}

}  // namespace zkllm

using zkllm::check;

static const uint32_t kTopLimbBound = 1944954707u;   // r >> 224: keeps a random value below r

ostream& operator<<(ostream& os, const Fr_t& x) {
    os << "0x" << std::hex;
    for (int i = 7; i >= 0; --i) os << std::setfill('0') << std::setw(8) << x.val[i];
    return os << std::dec << std::setw(0) << std::setfill(' ');
}

vector<Fr_t> random_vec(uint len) {
    vector<Fr_t> out(len);
    if (len == 0) return out;
    vector<uint32_t> words(8 * (size_t)len);
    if (!zkllm::seeded_words(words.data(), words.size())) {
        std::random_device rd;
        std::mt19937 mt(rd());
        std::uniform_int_distribution<unsigned int> dist(0, UINT_MAX);
        for (auto& w : words) w = dist(mt);
    }
    for (uint i = 0; i < len; ++i) {
        for (int k = 0; k < 8; ++k) out[i].val[k] = words[8 * (size_t)i + k];
        out[i].val[7] %= kTopLimbBound;
    }
    return out;
}

uint ceilLog2(uint num) {
    if (num == 0) return 0;
    uint bits = 0;
    for (uint v = num - 1; v > 0; v >>= 1) ++bits;
    return bits;
}

template <typename T>
std::vector<T> concatenate(const std::vector<std::vector<T>>& vecs) {
    std::vector<T> all;
    for (const auto& v : vecs) all.insert(all.end(), v.begin(), v.end());
    return all;
}
template std::vector<Fr_t> concatenate(const std::vector<std::vector<Fr_t>>& vecs);

// ---- storage ------------------------------------------------------------------------
static Fr_t* dev_alloc_fr(uint n) {
    void* p = nullptr;
    check(zkb_malloc(&p, sizeof(Fr_t) * (size_t)n));
    return static_cast<Fr_t*>(p);
}

FrTensor::FrTensor(uint size) : gpu_data(dev_alloc_fr(size)), size(size) {}

FrTensor::FrTensor(uint size, const Fr_t* cpu_data) : gpu_data(dev_alloc_fr(size)), size(size) {
    check(zkb_memcpy_h2d(gpu_data, cpu_data, sizeof(Fr_t) * (size_t)size, nullptr));
}

template <class T, class F>
static void upload_and_convert(Fr_t* dst, const T* cpu, uint n, F convert) {
    void* tmp = nullptr;
    check(zkb_malloc(&tmp, sizeof(T) * (size_t)n));
    int rc = zkb_memcpy_h2d(tmp, cpu, sizeof(T) * (size_t)n, nullptr);
    if (rc == ZKB_OK) rc = convert(static_cast<const T*>(tmp), dst);
    if (rc == ZKB_OK) rc = zkb_sync(nullptr);
    zkb_free_default_stream(tmp);
    check(rc);
}

FrTensor::FrTensor(uint size, const int* cpu_data) : gpu_data(dev_alloc_fr(size)), size(size) {
    upload_and_convert(gpu_data, cpu_data, size, [&](const int* d, Fr_t* o) { return zkb_fr_from_i32(d, o, size, nullptr); });
}
FrTensor::FrTensor(uint size, const long* cpu_data) : gpu_data(dev_alloc_fr(size)), size(size) {
    upload_and_convert(gpu_data, cpu_data, size,
                       [&](const long* d, Fr_t* o) { return zkb_fr_from_i64(reinterpret_cast<const int64_t*>(d), o, size, nullptr); });
}
FrTensor::FrTensor(uint size, const float* cpu_data, unsigned long scaling_factor) : gpu_data(dev_alloc_fr(size)), size(size) {
    upload_and_convert(gpu_data, cpu_data, size,
                       [&](const float* d, Fr_t* o) { return zkb_fr_from_f32(d, scaling_factor, o, size, nullptr); });
}
FrTensor::FrTensor(uint size, const double* cpu_data, unsigned long scaling_factor) : gpu_data(dev_alloc_fr(size)), size(size) {
    upload_and_convert(gpu_data, cpu_data, size,
                       [&](const double* d, Fr_t* o) { return zkb_fr_from_f64(d, scaling_factor, o, size, nullptr); });
}

FrTensor::FrTensor(const FrTensor& t) : gpu_data(dev_alloc_fr(t.size)), size(t.size) {
    check(zkb_memcpy_d2d(gpu_data, t.gpu_data, sizeof(Fr_t) * (size_t)size, nullptr));
    check(zkb_sync(nullptr));
}

FrTensor::FrTensor(const string& filename) : gpu_data(nullptr), size(findsize(filename) / sizeof(Fr_t)) {
    gpu_data = dev_alloc_fr(size);
    loadbin(filename, gpu_data, sizeof(Fr_t) * size);
}

FrTensor::~FrTensor() {
    zkb_free_default_stream(gpu_data);
    gpu_data = nullptr;
}

FrTensor& FrTensor::operator=(const FrTensor& t) {
    if (size != t.size) throw std::runtime_error("Incompatible dimensions");
    check(zkb_memcpy_d2d(gpu_data, t.gpu_data, sizeof(Fr_t) * (size_t)size, nullptr));
    check(zkb_sync(nullptr));
    return *this;
}

FrTensor FrTensor::from_int_bin(const string& filename) {
    const uint n = findsize(filename) / sizeof(int);
    FrTensor out(n);
    void* tmp = nullptr;
    check(zkb_malloc(&tmp, sizeof(int) * (size_t)n));
    loadbin(filename, tmp, sizeof(int) * n);
    int rc = zkb_fr_from_i32(static_cast<const int32_t*>(tmp), out.gpu_data, n, nullptr);
    if (rc == ZKB_OK) rc = zkb_sync(nullptr);
    zkb_free_default_stream(tmp);
    check(rc);
    return out;
}

FrTensor FrTensor::from_long_bin(const string& filename) {
    const uint n = findsize(filename) / sizeof(long);
    FrTensor out(n);
    void* tmp = nullptr;
    check(zkb_malloc(&tmp, sizeof(long) * (size_t)n));
    loadbin(filename, tmp, sizeof(long) * n);
    int rc = zkb_fr_from_i64(static_cast<const int64_t*>(tmp), out.gpu_data, n, nullptr);
    if (rc == ZKB_OK) rc = zkb_sync(nullptr);
    zkb_free_default_stream(tmp);
    check(rc);
    return out;
}

void FrTensor::save(const string& filename) const { savebin(filename, gpu_data, sizeof(Fr_t) * size); }

void FrTensor::save_int(const string& filename) const {
    void* tmp = nullptr;
    check(zkb_malloc(&tmp, sizeof(int) * (size_t)size));
    int rc = zkb_fr_to_i32(gpu_data, static_cast<int32_t*>(tmp), size, nullptr);
    if (rc == ZKB_OK) rc = zkb_sync(nullptr);
    if (rc == ZKB_OK) savebin(filename, tmp, sizeof(int) * size);
    zkb_free_default_stream(tmp);
    check(rc);
}

void FrTensor::save_long(const string& filename) const {
    void* tmp = nullptr;
    check(zkb_malloc(&tmp, sizeof(long) * (size_t)size));
    int rc = zkb_fr_to_i64(gpu_data, static_cast<int64_t*>(tmp), size, nullptr);
    if (rc == ZKB_OK) rc = zkb_sync(nullptr);
    if (rc == ZKB_OK) savebin(filename, tmp, sizeof(long) * size);
    zkb_free_default_stream(tmp);
    check(rc);
}

// Host-side generators stand in for the reference's cuRAND kernels
// (fr-tensor.cu:444-510); the streams were never reproducible there either.
static void fill_random_words(vector<uint32_t>& words) {
    if (zkllm::seeded_words(words.data(), words.size(), true)) return;
    std::random_device rd;
    std::mt19937_64 rng(rd());
    for (auto& w : words) w = (uint32_t)rng();
}

FrTensor FrTensor::random_int(uint size, uint num_bits) {
    vector<uint32_t> words(size);
    fill_random_words(words);
    vector<int> vals(size);
    const uint32_t mask = num_bits >= 32 ? 0xffffffffu : ((1u << num_bits) - 1u);
    const long half = 1L << (num_bits - 1);
    vector<long> lv(size);
    for (uint i = 0; i < size; ++i) lv[i] = (long)(words[i] & mask) - half;
    return FrTensor(size, lv.data());
}

FrTensor FrTensor::random(uint size) {
    vector<uint32_t> words(8 * (size_t)size);
    fill_random_words(words);
    vector<Fr_t> h(size);
    for (uint i = 0; i < size; ++i) {
        for (int k = 0; k < 8; ++k) h[i].val[k] = words[8 * (size_t)i + k];
        h[i].val[7] %= kTopLimbBound;
    }
    return FrTensor(size, h.data());
}

Fr_t FrTensor::operator()(uint idx) const {
    Fr_t out;
    check(zkb_memcpy_d2h(&out, gpu_data + idx, sizeof(Fr_t), nullptr));
    return out;
}

// ---- arithmetic -------------------------------------------------------------------------
typedef int (*BinFn)(const zkb_fr_t*, const zkb_fr_t*, zkb_fr_t*, size_t, void*);
typedef int (*ScalarFn)(const zkb_fr_t*, const zkb_fr_t*, zkb_fr_t*, size_t, void*);

static FrTensor binary(const FrTensor& a, const FrTensor& b, BinFn fn) {
    if (a.size != b.size) throw std::runtime_error("Incompatible dimensions");
    FrTensor out(a.size);
    check(fn(a.gpu_data, b.gpu_data, out.gpu_data, a.size, nullptr));
    check(zkb_sync(nullptr));
    return out;
}
static FrTensor& binary_inplace(FrTensor& a, const FrTensor& b, BinFn fn) {
    if (a.size != b.size) throw std::runtime_error("Incompatible dimensions");
    check(fn(a.gpu_data, b.gpu_data, a.gpu_data, a.size, nullptr));
    check(zkb_sync(nullptr));
    return a;
}
static FrTensor scalar(const FrTensor& a, const Fr_t& x, ScalarFn fn) {
    FrTensor out(a.size);
    check(fn(a.gpu_data, &x, out.gpu_data, a.size, nullptr));
    check(zkb_sync(nullptr));
    return out;
}
static FrTensor& scalar_inplace(FrTensor& a, const Fr_t& x, ScalarFn fn) {
    check(fn(a.gpu_data, &x, a.gpu_data, a.size, nullptr));
    check(zkb_sync(nullptr));
    return a;
}

FrTensor FrTensor::operator+(const FrTensor& t) const { return binary(*this, t, zkb_fr_add); }
FrTensor FrTensor::operator-(const FrTensor& t) const { return binary(*this, t, zkb_fr_sub); }
FrTensor FrTensor::operator*(const FrTensor& t) const { return binary(*this, t, zkb_fr_mul); }
FrTensor FrTensor::operator+(const Fr_t& x) const { return scalar(*this, x, zkb_fr_add_scalar); }
FrTensor FrTensor::operator-(const Fr_t& x) const { return scalar(*this, x, zkb_fr_sub_scalar); }
FrTensor FrTensor::operator*(const Fr_t& x) const { return scalar(*this, x, zkb_fr_mul_scalar); }
FrTensor& FrTensor::operator+=(const FrTensor& t) { return binary_inplace(*this, t, zkb_fr_add); }
FrTensor& FrTensor::operator-=(const FrTensor& t) { return binary_inplace(*this, t, zkb_fr_sub); }
FrTensor& FrTensor::operator*=(const FrTensor& t) { return binary_inplace(*this, t, zkb_fr_mul); }
FrTensor& FrTensor::operator+=(const Fr_t& x) { return scalar_inplace(*this, x, zkb_fr_add_scalar); }
FrTensor& FrTensor::operator-=(const Fr_t& x) { return scalar_inplace(*this, x, zkb_fr_sub_scalar); }
FrTensor& FrTensor::operator*=(const Fr_t& x) { return scalar_inplace(*this, x, zkb_fr_mul_scalar); }

FrTensor FrTensor::operator-() const {
    FrTensor out(size);
    check(zkb_fr_neg(gpu_data, out.gpu_data, size, nullptr));
    check(zkb_sync(nullptr));
    return out;
}
FrTensor& FrTensor::mont() {
    check(zkb_fr_mont(gpu_data, gpu_data, size, nullptr));
    check(zkb_sync(nullptr));
    return *this;
}
FrTensor& FrTensor::unmont() {
    check(zkb_fr_unmont(gpu_data, gpu_data, size, nullptr));
    check(zkb_sync(nullptr));
    return *this;
}

// ---- reductions ---------------------------------------------------------------------------
Fr_t FrTensor::sum() const {
    Fr_t out;
    check(zkb_fr_sum(gpu_data, size, &out, nullptr));
    return out;
}

static const Fr_t* data_or_dummy(const vector<Fr_t>& u) {
    static const Fr_t dummy = {{0, 0, 0, 0, 0, 0, 0, 0}};
    return u.empty() ? &dummy : u.data();
}

Fr_t FrTensor::operator()(const vector<Fr_t>& u) const {
    Fr_t out;
    check(zkb_fr_mle_eval(gpu_data, size, data_or_dummy(u), (unsigned)u.size(), &out, nullptr));
    return out;
}

FrTensor FrTensor::partial_me(const vector<Fr_t>& u, uint window_size) const {
    if (u.size() >= 1 && size <= window_size * (1u << (u.size() - 1))) throw std::runtime_error("partial_me: Incompatible dimensions");
    if (u.empty()) return *this;
    const size_t nwin = ((size_t)size + window_size - 1) / window_size;
    const size_t groups = (nwin + ((size_t)1 << u.size()) - 1) >> u.size();
    FrTensor out((uint)(groups * window_size));
    size_t out_n = 0;
    check(zkb_fr_partial_me_window(gpu_data, size, u.data(), (unsigned)u.size(), window_size, out.gpu_data, &out_n, nullptr));
    check(zkb_sync(nullptr));
    return out;
}

FrTensor FrTensor::partial_me(const vector<Fr_t>& u, uint cur_dim, uint window_size) const {
    if (cur_dim <= ((1u << u.size()) >> 1)) throw std::runtime_error("cur_dim <= ((1<<u.size()) >> 1)");
    if (cur_dim > (1u << u.size())) throw std::runtime_error("cur_dim > (1<<u.size())");
    if (u.empty()) return *this;
    if (size % (cur_dim * window_size) != 0) throw std::runtime_error("t.size % (cur_dim * window_size) != 0");
    FrTensor out(size / cur_dim);
    check(zkb_fr_partial_me(gpu_data, size, u.data(), (unsigned)u.size(), cur_dim, window_size, out.gpu_data, nullptr));
    check(zkb_sync(nullptr));
    return out;
}

Fr_t FrTensor::multi_dim_me(const vector<vector<Fr_t>>& us, const vector<uint>& shape) const {
    if (shape.size() != us.size()) throw std::runtime_error("Incompatible dimensions");
    if (shape.empty()) return (*this)(0u);
    if (shape.size() == 1) return (*this)(us[0]);
    if (shape.size() == 2) {
        // one fused call: rows against eq(us[1]), then against eq(us[0])
        if (shape[1] <= ((1u << us[1].size()) >> 1)) throw std::runtime_error("cur_dim <= ((1<<u.size()) >> 1)");
        if (shape[1] > (1u << us[1].size())) throw std::runtime_error("cur_dim > (1<<u.size())");
        if (size % shape[1] != 0) throw std::runtime_error("t.size % (cur_dim * window_size) != 0");
        Fr_t out;
        check(zkb_fr_mle_eval_2d(gpu_data, size / shape[1], shape[1], data_or_dummy(us[0]), (unsigned)us[0].size(),
                                 data_or_dummy(us[1]), (unsigned)us[1].size(), &out, nullptr));
        return out;
    }
    FrTensor folded = partial_me(us.back(), shape.back(), 1);
    return folded.multi_dim_me({us.begin(), us.end() - 1}, {shape.begin(), shape.end() - 1});
}

// ---- layout --------------------------------------------------------------------------------
std::pair<FrTensor, FrTensor> FrTensor::split(uint window_size) const {
    if (window_size < 1 || window_size >= size) throw std::runtime_error("Invalid window size.");
    const uint windows_in = (size + window_size - 1) / window_size;
    const uint out_size = ((windows_in + 1) / 2) * window_size;
    std::pair<FrTensor, FrTensor> out{out_size, out_size};
    check(zkb_fr_split_window(gpu_data, size, window_size, out.first.gpu_data, out.second.gpu_data, out_size, nullptr));
    check(zkb_sync(nullptr));
    return out;
}

FrTensor FrTensor::pad(const vector<uint>& shape, const Fr_t& pad_val) const {
    uint total = 1;
    for (uint s : shape) total *= s;
    if (total != size) throw std::runtime_error("pad: cum_shape != size");
    const uint last = shape.back();
    const uint last_p = 1u << ceilLog2(last);
    const uint rows = total / last;
    FrTensor out(rows * last_p);
    check(zkb_fr_pad_last(gpu_data, rows, last, last_p, &pad_val, out.gpu_data, nullptr));
    check(zkb_sync(nullptr));
    if (shape.size() == 1) return out;
    vector<uint> rest(shape.begin(), shape.end() - 1);
    rest.back() *= last_p;
    return out.pad(rest, pad_val);
}

FrTensor FrTensor::transpose(uint M, uint N) const {
    if (size != M * N) throw std::runtime_error("transpose: incompatible dimensions");
    FrTensor out(N * M);
    check(zkb_fr_transpose(gpu_data, M, N, out.gpu_data, nullptr));
    check(zkb_sync(nullptr));
    return out;
}

FrTensor FrTensor::trunc(uint begin_idx, uint end_idx) const {
    if (begin_idx >= end_idx || end_idx > size) throw std::runtime_error("trunc: invalid indices");
    FrTensor out(end_idx - begin_idx);
    check(zkb_memcpy_d2d(out.gpu_data, gpu_data + begin_idx, sizeof(Fr_t) * (size_t)out.size, nullptr));
    check(zkb_sync(nullptr));
    return out;
}

FrTensor FrTensor::matmul(const FrTensor& x, const FrTensor& y, uint M, uint N, uint P) {
    if (x.size != M * N || y.size != N * P) throw std::runtime_error("matmul: incompatible dimensions");
    FrTensor out(M * P);
    check(zkb_fr_matmul(x.gpu_data, y.gpu_data, out.gpu_data, M, N, P, nullptr));
    check(zkb_sync(nullptr));
    return out;
}

ostream& operator<<(ostream& os, const FrTensor& A) {
    vector<Fr_t> h(A.size);
    if (A.size) check(zkb_memcpy_d2h(h.data(), A.gpu_data, sizeof(Fr_t) * (size_t)A.size, nullptr));
    os << '[';
    for (uint i = 0; i < A.size; ++i) os << h[i] << (i + 1 < A.size ? "\n" : "");
    return os << ']';
}

FrTensor catTensors(const vector<FrTensor>& vec) {
    const uint each = vec[0].size;
    for (uint i = 1; i < vec.size(); ++i) {
        if (vec[i].size != each) {
            cout << "tensor size does not match: vec[0].size = " << each << ", vec[" << i << "].size = " << vec[i].size << "!" << endl;
            throw std::runtime_error("tensor size does not match!");
        }
    }
    FrTensor out((uint)vec.size() * each);
    for (uint i = 0; i < vec.size(); ++i)
        check(zkb_memcpy_d2d(out.gpu_data + (size_t)i * each, vec[i].gpu_data, sizeof(Fr_t) * (size_t)each, nullptr));
    check(zkb_sync(nullptr));
    return out;
}
