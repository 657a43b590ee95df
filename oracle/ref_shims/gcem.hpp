// Stand-in for the gcem compile-time math library: the reference only calls gcem::pow(2*pi, -D/2) in a constexpr
// initialiser (D = 2 or 3).  This pow is constexpr for exponents that are multiples of 1/2 (integer power times a
// Newton square root evaluated in long double), which covers every call site.
#pragma once

namespace gcem {
namespace shim_detail {
constexpr long double newton_sqrt(long double x, long double guess, int iterations) {
    return iterations == 0 ? guess : newton_sqrt(x, 0.5L * (guess + x / guess), iterations - 1);
}
constexpr long double sqrt_ld(long double x) { return x <= 0 ? 0.0L : newton_sqrt(x, x > 1 ? x : 1.0L, 64); }
constexpr long double ipow(long double x, long long n) {
    return n == 0 ? 1.0L : (n < 0 ? 1.0L / ipow(x, -n) : ((n & 1) ? x * ipow(x * x, n / 2) : ipow(x * x, n / 2)));
}
}  // namespace shim_detail

template <typename T1, typename T2>
#if defined(__CUDACC__)
__host__ __device__
#endif
    constexpr T1
    pow(T1 base, T2 exponent) {
    // exponent = h / 2 with integer h
    const long long doubled = static_cast<long long>(exponent * T2(2));
    const long double b = static_cast<long double>(base);
    const long double whole = shim_detail::ipow(b, doubled / 2);
    const long long rem = doubled % 2;  // -1, 0 or 1
    const long double root = shim_detail::sqrt_ld(b);
    return static_cast<T1>(rem == 0 ? whole : (rem > 0 ? whole * root : whole / root));
}
}  // namespace gcem
