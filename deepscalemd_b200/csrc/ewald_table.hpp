// Host-side builder of the real-space Ewald tables the pair kernel evaluates.
//
// Same table geometry as the reference's list kernel (include/ewald_real_table.h:26-35): r^2 is split by its float
// exponent and its top 5 mantissa bits into intervals of constant relative width, starting at r^2 = 2^-1; an interval
// holds a cubic in t in [0, 1), the position inside the interval, for
//     energy(r2) = erfc(alpha r) / r
//     force(r2)  = (erfc(alpha r) / r + 2 alpha / sqrt(pi) exp(-alpha^2 r^2)) / r^2        (= F / r per unit q_i q_j k)
// The cubics interpolate the functions at the four Chebyshev nodes of the interval; here they are found by Newton's
// divided differences and expanded to monomial coefficients (fp64), then rounded to float.
#pragma once

#include <algorithm>
#include <cmath>
#include <vector>

namespace dsmd {

constexpr int kEwaldBits = 5;                   // 32 intervals per octave of r^2
constexpr int kEwaldFirstExponent = -1;         // table starts at r^2 = 0.5
constexpr int kEwaldMaxOctaves = 16;
constexpr unsigned kEwaldBaseBits = static_cast<unsigned>(127 + kEwaldFirstExponent) << 23;
constexpr int kEwaldIndexShift = 23 - kEwaldBits;

inline int ewald_intervals(double cutoff_sq) {
    const int top = static_cast<int>(std::ceil(std::log2(std::max(cutoff_sq, 1.0))));
    const int octaves = std::min(std::max(top - kEwaldFirstExponent, 1), kEwaldMaxOctaves);
    return octaves << kEwaldBits;
}

// coef[2 * i] = force cubic of interval i, coef[2 * i + 1] = energy cubic, each {c0, c1, c2, c3}.
inline std::vector<float> ewald_build_table(double alpha, int intervals) {
    std::vector<float> coef(static_cast<size_t>(intervals) * 8, 0.0f);
    const double pi = 3.14159265358979323846;
    const double gauss = 2.0 * alpha / std::sqrt(pi);
    double node[4];
    for (int k = 0; k < 4; ++k) node[k] = 0.5 * (1.0 - std::cos((2 * k + 1) * pi / 8.0));
    const int per_octave = 1 << kEwaldBits;
    for (int iv = 0; iv < intervals; ++iv) {
        const double base = std::ldexp(1.0, kEwaldFirstExponent + iv / per_octave);
        const double start = base * (1.0 + static_cast<double>(iv % per_octave) / per_octave);
        const double width = base / per_octave;
        double f[2][4];
        for (int k = 0; k < 4; ++k) {
            const double r2 = start + node[k] * width, r = std::sqrt(r2);
            const double e = std::erfc(alpha * r) / r;
            f[0][k] = (e + gauss * std::exp(-alpha * alpha * r2)) / r2;
            f[1][k] = e;
        }
        for (int which = 0; which < 2; ++which) {
            // Newton form: p(t) = d0 + d1 (t - n0) + d2 (t - n0)(t - n1) + d3 (t - n0)(t - n1)(t - n2)
            long double d[4] = {f[which][0], f[which][1], f[which][2], f[which][3]};
            for (int level = 1; level < 4; ++level)
                for (int k = 3; k >= level; --k) d[k] = (d[k] - d[k - 1]) / (node[k] - node[k - level]);
            // expand to monomials by Horner-style nesting from the innermost term outwards
            long double c[4] = {d[3], 0.0L, 0.0L, 0.0L};   // polynomial so far, degree grows by one per step
            int degree = 0;
            for (int k = 2; k >= 0; --k) {
                long double next[4] = {0.0L, 0.0L, 0.0L, 0.0L};
                for (int m = 0; m <= degree; ++m) {          // multiply by (t - node[k])
                    next[m + 1] += c[m];
                    next[m] -= c[m] * node[k];
                }
                next[0] += d[k];
                ++degree;
                for (int m = 0; m < 4; ++m) c[m] = next[m];
            }
            float* out = &coef[(static_cast<size_t>(iv) * 2 + which) * 4];
            for (int m = 0; m < 4; ++m) out[m] = static_cast<float>(static_cast<double>(c[m]));
        }
    }
    return coef;
}

// Bisection of erfc(alpha rc) = tolerance on [1e-4, 10 / rc], 100 halvings (src/force_calculator_cuda.cu:6821-6828).
inline double ewald_alpha_for(double cutoff, double tolerance = 1e-5) {
    double a = 1e-4, b = 10.0 / cutoff;
    for (int it = 0; it < 100; ++it) {
        const double m = 0.5 * (a + b);
        if (std::erfc(m * cutoff) > tolerance) a = m; else b = m;
    }
    return 0.5 * (a + b);
}

}  // namespace dsmd
