// Host scalar algebra on Fr_t and small dense polynomials (reference:
// polynomial.cuh:8-47).  The reference runs each of these as a one-thread kernel
// with its own allocation; here they are plain CPU arithmetic on canonical
// standard-form values, which yields the same field elements.
#ifndef POLYNOMIAL_CUH
#define POLYNOMIAL_CUH

#include "fr-tensor.cuh"

// field arithmetic on single elements (canonical standard form in, canonical out)
Fr_t operator+(const Fr_t& lhs, const Fr_t& rhs);
Fr_t operator-(const Fr_t& lhs, const Fr_t& rhs);
Fr_t operator*(const Fr_t& lhs, const Fr_t& rhs);
Fr_t operator/(const Fr_t& num, const Fr_t& den);   // den = 0 gives 0, as the Fermat inverse does
Fr_t operator-(const Fr_t& x);
Fr_t inv(const Fr_t& x);

// coefficients are stored low degree first; degree = number of coefficients - 1
class Polynomial {
public:
    Polynomial();                                   // the zero polynomial
    Polynomial(const Fr_t& c0);                     // a constant
    Polynomial(const vector<Fr_t>& low_first);
    Polynomial(int deg);                            // deg + 1 zero coefficients
    Polynomial(int deg, Fr_t* low_first);           // copies deg + 1 values
    Polynomial(const Polynomial& src);
    ~Polynomial();

    Polynomial& operator=(const Polynomial& src);
    Polynomial operator-();
    Polynomial operator+(const Polynomial& rhs);
    Polynomial& operator+=(const Polynomial& rhs);
    Polynomial operator-(const Polynomial& rhs);
    Polynomial& operator-=(const Polynomial& rhs);
    Polynomial operator*(const Polynomial& rhs);     // schoolbook product
    Polynomial& operator*=(const Polynomial& rhs);

    Fr_t operator()(const Fr_t& at);                // Horner evaluation

    void setCoefficients(int deg, Fr_t* low_first);
    int getDegree() const;

    // (1 - u) + (2u - 1) t, and its value at t = v
    static Polynomial eq(const Fr_t& u);
    static Fr_t eq(const Fr_t& u, const Fr_t& v);

    // not in the reference: read access to the coefficients (host memory)
    const vector<Fr_t>& coefficients() const { return coefs_; }

    friend std::ostream& operator<<(std::ostream& out, const Polynomial& p);

private:
    vector<Fr_t> coefs_;
    int degree_;
};

#endif
