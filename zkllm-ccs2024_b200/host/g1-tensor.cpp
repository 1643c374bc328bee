// G1 tensors over the C ABI (reference: g1-tensor.cu).
#include "g1-tensor.cuh"

#include <cstring>
#include <stdexcept>

#include "ioutils.cuh"
#include "zkllm_ext.hpp"

using zkllm::check;

// (coordinate * 2^384) mod p of the standard generator, and 2^384 mod p
const Fp_t G1_generator_x_mont = {{0xfd530c16u, 0x5cb38790u, 0x9976fff5u, 0x7817fc67u, 0x143ba1c1u, 0x154f95c7u,
                                   0xf3d0e747u, 0xf0ae6acdu, 0x21dbf440u, 0xedce6eccu, 0x9e0bfb75u, 0x12017741u}};
const Fp_t G1_generator_y_mont = {{0x0ce72271u, 0xbaac93d5u, 0x7918fd8eu, 0x8c22631au, 0x570725ceu, 0xdd595f13u,
                                   0x50405194u, 0x51ac5829u, 0xad0059c0u, 0x0e1c8c3fu, 0x5008a26au, 0x0bbc3efcu}};
const Fp_t G1_ONE = {{0x0002fffdu, 0x76090000u, 0xc40c0002u, 0xebf4000bu, 0x53c758bau, 0x5f489857u,
                      0x70525745u, 0x77ce5853u, 0xa256ec6du, 0x5c071a97u, 0xfa80e493u, 0x15f65ec3u}};
const G1Affine_t G1Affine_generator = {G1_generator_x_mont, G1_generator_y_mont};
const G1Jacobian_t G1Jacobian_generator = {G1_generator_x_mont, G1_generator_y_mont, G1_ONE};
const G1Jacobian_t G1Jacobian_ZERO = {};

static void print_limbs(ostream& os, const uint32_t* v, int n) {
    os << "0x" << std::hex;
    for (int i = n - 1; i >= 0; --i) os << std::setfill('0') << std::setw(8) << v[i];
    os << std::dec << std::setw(0) << std::setfill(' ');
}
ostream& operator<<(ostream& os, const Fp_t& x) { print_limbs(os, x.val, 12); return os; }
ostream& operator<<(ostream& os, const G1Affine_t& g) { return os << "(" << g.x << ", " << g.y << ")"; }
ostream& operator<<(ostream& os, const G1Jacobian_t& g) { return os << "(" << g.x << ", " << g.y << ", " << g.z << ")"; }

G1Tensor::G1Tensor(uint size) : size(size) {}

template <class T>
static T* dev_alloc(uint n) {
    void* p = nullptr;
    check(zkb_malloc(&p, sizeof(T) * (size_t)n));
    return static_cast<T*>(p);
}

// ---- affine ---------------------------------------------------------------------------------
G1TensorAffine::G1TensorAffine(const G1TensorAffine& t) : G1Tensor(t.size), gpu_data(dev_alloc<G1Affine_t>(t.size)) {
    check(zkb_memcpy_d2d(gpu_data, t.gpu_data, sizeof(G1Affine_t) * (size_t)size, nullptr));
    check(zkb_sync(nullptr));
}
G1TensorAffine::G1TensorAffine(uint size) : G1Tensor(size), gpu_data(dev_alloc<G1Affine_t>(size)) {}
G1TensorAffine::G1TensorAffine(uint size, const G1Affine_t& g) : G1Tensor(size), gpu_data(dev_alloc<G1Affine_t>(size)) {
    std::vector<G1Affine_t> h(size, g);
    if (size) check(zkb_memcpy_h2d(gpu_data, h.data(), sizeof(G1Affine_t) * (size_t)size, nullptr));
}
G1TensorAffine::G1TensorAffine(uint size, const G1Affine_t* cpu_data) : G1Tensor(size), gpu_data(dev_alloc<G1Affine_t>(size)) {
    if (size) check(zkb_memcpy_h2d(gpu_data, cpu_data, sizeof(G1Affine_t) * (size_t)size, nullptr));
}
G1TensorAffine::G1TensorAffine(const string& filename) : G1Tensor(findsize(filename) / sizeof(G1Affine_t)), gpu_data(nullptr) {
    gpu_data = dev_alloc<G1Affine_t>(size);
    loadbin(filename, gpu_data, sizeof(G1Affine_t) * size);
}
G1TensorAffine::~G1TensorAffine() {
    zkb_free_default_stream(gpu_data);
    gpu_data = nullptr;
}
void G1TensorAffine::save(const string& filename) const { savebin(filename, gpu_data, sizeof(G1Affine_t) * size); }
G1Affine_t G1TensorAffine::operator()(uint idx) const {
    G1Affine_t out;
    check(zkb_memcpy_d2h(&out, gpu_data + idx, sizeof(G1Affine_t), nullptr));
    return out;
}
G1TensorAffine G1TensorAffine::operator-() const {
    // negate through the Jacobian kernels: lift, negate, normalise
    G1TensorJacobian j(*this);
    G1TensorJacobian n = -j;
    G1TensorAffine out(size);
    check(zkb_g1_to_affine(n.gpu_data, out.gpu_data, size, nullptr));
    check(zkb_sync(nullptr));
    return out;
}

// ---- Jacobian --------------------------------------------------------------------------------
G1TensorJacobian::G1TensorJacobian(const G1TensorJacobian& t) : G1Tensor(t.size), gpu_data(dev_alloc<G1Jacobian_t>(t.size)) {
    check(zkb_memcpy_d2d(gpu_data, t.gpu_data, sizeof(G1Jacobian_t) * (size_t)size, nullptr));
    check(zkb_sync(nullptr));
}
G1TensorJacobian::G1TensorJacobian(uint size) : G1Tensor(size), gpu_data(dev_alloc<G1Jacobian_t>(size)) {}
G1TensorJacobian::G1TensorJacobian(uint size, const G1Jacobian_t& g) : G1Tensor(size), gpu_data(dev_alloc<G1Jacobian_t>(size)) {
    check(zkb_g1_fill(gpu_data, &g, size, nullptr));
    check(zkb_sync(nullptr));
}
G1TensorJacobian::G1TensorJacobian(uint size, const G1Jacobian_t* cpu_data) : G1Tensor(size), gpu_data(dev_alloc<G1Jacobian_t>(size)) {
    if (size) check(zkb_memcpy_h2d(gpu_data, cpu_data, sizeof(G1Jacobian_t) * (size_t)size, nullptr));
}
G1TensorJacobian::G1TensorJacobian(const G1TensorAffine& a) : G1Tensor(a.size), gpu_data(dev_alloc<G1Jacobian_t>(a.size)) {
    check(zkb_g1_from_affine(a.gpu_data, gpu_data, size, nullptr));
    check(zkb_sync(nullptr));
}
G1TensorJacobian::G1TensorJacobian(const string& filename) : G1Tensor(findsize(filename) / sizeof(G1Jacobian_t)), gpu_data(nullptr) {
    gpu_data = dev_alloc<G1Jacobian_t>(size);
    loadbin(filename, gpu_data, sizeof(G1Jacobian_t) * size);
}
G1TensorJacobian::~G1TensorJacobian() {
    zkb_free_default_stream(gpu_data);
    gpu_data = nullptr;
}
void G1TensorJacobian::save(const string& filename) const { savebin(filename, gpu_data, sizeof(G1Jacobian_t) * size); }
G1Jacobian_t G1TensorJacobian::operator()(uint idx) const {
    G1Jacobian_t out;
    check(zkb_memcpy_d2h(&out, gpu_data + idx, sizeof(G1Jacobian_t), nullptr));
    return out;
}

static G1Jacobian_t lift(const G1Affine_t& a) {
    G1Jacobian_t j;
    j.x = a.x; j.y = a.y; j.z = G1_ONE;
    return j;
}

G1TensorJacobian G1TensorJacobian::operator-() const {
    G1TensorJacobian out(size);
    check(zkb_g1_neg(gpu_data, out.gpu_data, size, nullptr));
    check(zkb_sync(nullptr));
    return out;
}

typedef int (*G1BinFn)(const zkb_g1_t*, const zkb_g1_t*, zkb_g1_t*, size_t, void*);

static void g1_binary(const G1TensorJacobian& a, const G1Jacobian_t* b, uint b_size, G1Jacobian_t* out, G1BinFn fn) {
    if (a.size != b_size) throw std::runtime_error("Incompatible dimensions");
    check(fn(a.gpu_data, b, out, a.size, nullptr));
    check(zkb_sync(nullptr));
}
// (*this) +/- one broadcast point
static void g1_broadcast(const G1TensorJacobian& a, G1Jacobian_t x, bool negate, G1Jacobian_t* out) {
    if (negate) {
        // negate the single point on the device: fill, negate, read back
        G1TensorJacobian one(1, x);
        G1TensorJacobian neg = -one;
        x = neg(0);
    }
    check(zkb_g1_add_scalar(a.gpu_data, &x, out, a.size, nullptr));
    check(zkb_sync(nullptr));
}

G1TensorJacobian G1TensorJacobian::operator+(const G1TensorJacobian& t) const {
    G1TensorJacobian out(size);
    g1_binary(*this, t.gpu_data, t.size, out.gpu_data, zkb_g1_add);
    return out;
}
G1TensorJacobian G1TensorJacobian::operator+(const G1TensorAffine& t) const { return *this + G1TensorJacobian(t); }
G1TensorJacobian G1TensorJacobian::operator+(const G1Jacobian_t& x) const {
    G1TensorJacobian out(size);
    g1_broadcast(*this, x, false, out.gpu_data);
    return out;
}
G1TensorJacobian G1TensorJacobian::operator+(const G1Affine_t& x) const { return *this + lift(x); }
G1TensorJacobian& G1TensorJacobian::operator+=(const G1TensorJacobian& t) {
    g1_binary(*this, t.gpu_data, t.size, gpu_data, zkb_g1_add);
    return *this;
}
G1TensorJacobian& G1TensorJacobian::operator+=(const G1TensorAffine& t) { return *this += G1TensorJacobian(t); }
G1TensorJacobian& G1TensorJacobian::operator+=(const G1Jacobian_t& x) {
    g1_broadcast(*this, x, false, gpu_data);
    return *this;
}
G1TensorJacobian& G1TensorJacobian::operator+=(const G1Affine_t& x) { return *this += lift(x); }

G1TensorJacobian G1TensorJacobian::operator-(const G1TensorJacobian& t) const {
    G1TensorJacobian out(size);
    g1_binary(*this, t.gpu_data, t.size, out.gpu_data, zkb_g1_sub);
    return out;
}
G1TensorJacobian G1TensorJacobian::operator-(const G1TensorAffine& t) const { return *this - G1TensorJacobian(t); }
G1TensorJacobian G1TensorJacobian::operator-(const G1Jacobian_t& x) const {
    G1TensorJacobian out(size);
    g1_broadcast(*this, x, true, out.gpu_data);
    return out;
}
G1TensorJacobian G1TensorJacobian::operator-(const G1Affine_t& x) const { return *this - lift(x); }
G1TensorJacobian& G1TensorJacobian::operator-=(const G1TensorJacobian& t) {
    g1_binary(*this, t.gpu_data, t.size, gpu_data, zkb_g1_sub);
    return *this;
}
G1TensorJacobian& G1TensorJacobian::operator-=(const G1TensorAffine& t) { return *this -= G1TensorJacobian(t); }
G1TensorJacobian& G1TensorJacobian::operator-=(const G1Jacobian_t& x) {
    g1_broadcast(*this, x, true, gpu_data);
    return *this;
}
G1TensorJacobian& G1TensorJacobian::operator-=(const G1Affine_t& x) { return *this -= lift(x); }

G1Jacobian_t G1TensorJacobian::sum() const {
    G1Jacobian_t out;
    check(zkb_g1_sum(gpu_data, size, &out, nullptr));
    return out;
}

G1TensorJacobian G1TensorJacobian::operator*(const FrTensor& scalars) const {
    if (scalars.size % size != 0) throw std::runtime_error("Incompatible dimensions");
    G1TensorJacobian out(scalars.size);
    check(zkb_g1_mul(gpu_data, size, scalars.gpu_data, scalars.size, out.gpu_data, nullptr));
    check(zkb_sync(nullptr));
    return out;
}
G1TensorJacobian& G1TensorJacobian::operator*=(const FrTensor& scalars) {
    if (size != scalars.size) throw std::runtime_error("Incompatible dimensions 01");
    check(zkb_g1_mul(gpu_data, size, scalars.gpu_data, size, gpu_data, nullptr));
    check(zkb_sync(nullptr));
    return *this;
}

G1Jacobian_t G1TensorJacobian::operator()(const vector<Fr_t>& u) const {
    static const Fr_t dummy = {{0, 0, 0, 0, 0, 0, 0, 0}};
    G1Jacobian_t out;
    check(zkb_g1_mle_eval(gpu_data, size, u.empty() ? &dummy : u.data(), (unsigned)u.size(), &out, nullptr));
    return out;
}

G1TensorJacobian G1TensorJacobian::rowwise_sum(uint nrow, uint ncol) const {
    if (size != nrow * ncol) throw std::runtime_error("Incompatible dimensions");
    G1TensorJacobian out(nrow);
    check(zkb_g1_rowwise_sum(gpu_data, nrow, ncol, out.gpu_data, nullptr));
    check(zkb_sync(nullptr));
    return out;
}
