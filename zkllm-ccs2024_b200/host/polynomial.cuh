// Host scalar algebra on Fr_t and small dense polynomials (reference:
// polynomial.cuh:8-47).  The reference runs each of these as a one-thread kernel
// with its own allocation; here they are plain CPU arithmetic on canonical
// standard-form values, which yields the same field elements.
#ifndef POLYNOMIAL_CUH
#define POLYNOMIAL_CUH

#include "fr-tensor.cuh"

Fr_t operator+(const Fr_t& a, const Fr_t& b);
Fr_t operator-(const Fr_t& a, const Fr_t& b);
Fr_t operator-(const Fr_t& a);
Fr_t operator*(const Fr_t& a, const Fr_t& b);
Fr_t operator/(const Fr_t& a, const Fr_t& b);
Fr_t inv(const Fr_t& a);

// coefficients are stored low degree first; degree = number of coefficients - 1
class Polynomial {
public:
    Polynomial();
    Polynomial(int degree);
    Polynomial(int degree, Fr_t* coefficients);
    Polynomial(const Polynomial& other);
    Polynomial(const Fr_t& constant);
    Polynomial(const vector<Fr_t>& coefficients);
    ~Polynomial();

    Polynomial& operator=(const Polynomial& other);
    Polynomial operator+(const Polynomial& other);
    Polynomial operator-(const Polynomial& other);
    Polynomial operator*(const Polynomial& other);
    Polynomial operator-();
    Polynomial& operator+=(const Polynomial& other);
    Polynomial& operator-=(const Polynomial& other);
    Polynomial& operator*=(const Polynomial& other);

    Fr_t operator()(const Fr_t& x);

    int getDegree() const;
    void setCoefficients(int degree, Fr_t* coefficients);

    // (1 - u) + (2u - 1) t, and its value at t = v
    static Polynomial eq(const Fr_t& u);
    static Fr_t eq(const Fr_t& u, const Fr_t& v);

    // not in the reference: read access to the coefficients (host memory)
    const vector<Fr_t>& coefficients() const { return coefs_; }

    friend std::ostream& operator<<(std::ostream& os, const Polynomial& poly);

private:
    vector<Fr_t> coefs_;
    int degree_;
};

#endif
