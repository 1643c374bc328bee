// Host Fr operators and Polynomial (reference: polynomial.cu:9-373).
#include "polynomial.cuh"

#include "../csrc/hostfr.hpp"

using namespace zkb;

static inline hfr::H L(const Fr_t& a) { return hfr::load(a); }
static inline Fr_t S(const hfr::H& h) { return hfr::store(h); }

Fr_t operator+(const Fr_t& a, const Fr_t& b) { return S(hfr::add(L(a), L(b))); }
Fr_t operator-(const Fr_t& a, const Fr_t& b) { return S(hfr::sub(L(a), L(b))); }
Fr_t operator-(const Fr_t& a) { return S(hfr::neg(L(a))); }
Fr_t operator*(const Fr_t& a, const Fr_t& b) { return S(hfr::mul(L(a), L(b))); }
Fr_t inv(const Fr_t& a) { return S(hfr::inv(L(a))); }
Fr_t operator/(const Fr_t& a, const Fr_t& b) { return S(hfr::mul(L(a), hfr::inv(L(b)))); }

static const Fr_t kZero = {{0, 0, 0, 0, 0, 0, 0, 0}};
static const Fr_t kOne = {{1, 0, 0, 0, 0, 0, 0, 0}};

Polynomial::Polynomial() : coefs_(), degree_(0) {}
Polynomial::Polynomial(int degree) : coefs_((size_t)degree + 1, kZero), degree_(degree) {}
Polynomial::Polynomial(int degree, Fr_t* coefficients) : coefs_(coefficients, coefficients + degree + 1), degree_(degree) {}
Polynomial::Polynomial(const Polynomial& other) : coefs_(other.coefs_), degree_(other.degree_) {}
Polynomial::Polynomial(const Fr_t& constant) : coefs_(1, constant), degree_(0) {}
Polynomial::Polynomial(const vector<Fr_t>& coefficients) : coefs_(coefficients), degree_((int)coefficients.size() - 1) {}
Polynomial::~Polynomial() {}

Polynomial& Polynomial::operator=(const Polynomial& other) {
    coefs_ = other.coefs_;
    degree_ = other.degree_;
    return *this;
}

Polynomial Polynomial::operator+(const Polynomial& other) {
    const size_t n = coefs_.size(), m = other.coefs_.size();
    Polynomial out((int)(n > m ? n : m) - 1);
    for (size_t i = 0; i < out.coefs_.size(); ++i) {
        if (i < n && i < m) out.coefs_[i] = coefs_[i] + other.coefs_[i];
        else out.coefs_[i] = i < n ? coefs_[i] : other.coefs_[i];
    }
    return out;
}

// Where only the right operand has a coefficient the reference's kernel copies it
// without negating (polynomial.cu:208-219); kept, since every caller subtracts a
// polynomial of lower or equal degree.
Polynomial Polynomial::operator-(const Polynomial& other) {
    const size_t n = coefs_.size(), m = other.coefs_.size();
    Polynomial out((int)(n > m ? n : m) - 1);
    for (size_t i = 0; i < out.coefs_.size(); ++i) {
        if (i < n && i < m) out.coefs_[i] = coefs_[i] - other.coefs_[i];
        else out.coefs_[i] = i < n ? coefs_[i] : other.coefs_[i];
    }
    return out;
}

Polynomial Polynomial::operator*(const Polynomial& other) {
    const int n = (int)coefs_.size(), m = (int)other.coefs_.size();
    Polynomial out(degree_ + other.degree_);
    for (int i = 0; i < n + m - 1; ++i) {
        Fr_t acc = kZero;
        for (int j = (i - m + 1 > 0 ? i - m + 1 : 0); j <= (i < n - 1 ? i : n - 1); ++j) acc = acc + coefs_[j] * other.coefs_[i - j];
        out.coefs_[i] = acc;
    }
    return out;
}

Polynomial Polynomial::operator-() {
    Polynomial out(degree_);
    for (size_t i = 0; i < coefs_.size(); ++i) out.coefs_[i] = -coefs_[i];
    return out;
}

Polynomial& Polynomial::operator+=(const Polynomial& other) { return *this = *this + other; }
Polynomial& Polynomial::operator-=(const Polynomial& other) { return *this = *this - other; }
Polynomial& Polynomial::operator*=(const Polynomial& other) { return *this = *this * other; }

Fr_t Polynomial::operator()(const Fr_t& x) {
    Fr_t acc = kZero, pw = kOne;
    for (size_t i = 0; i < coefs_.size(); ++i) {
        acc = acc + coefs_[i] * pw;
        pw = pw * x;
    }
    return acc;
}

int Polynomial::getDegree() const { return degree_; }

void Polynomial::setCoefficients(int degree, Fr_t* coefficients) {
    degree_ = degree;
    coefs_.assign(coefficients, coefficients + degree + 1);
}

std::ostream& operator<<(std::ostream& os, const Polynomial& poly) {
    for (const auto& c : poly.coefs_) os << c << " ";
    return os;
}

Polynomial Polynomial::eq(const Fr_t& u) {
    Polynomial p(1);
    p.coefs_[0] = kOne - u;
    p.coefs_[1] = (u + u) - kOne;
    return p;
}

Fr_t Polynomial::eq(const Fr_t& u, const Fr_t& v) {
    const Fr_t uv = u * v;
    return ((uv + uv) - (u + v)) + kOne;
}
