// Stand-in for the small part of the GLM vector library that the reference's gmc extension sources use
// (vec<2|3>, mat<2x2|3x3>, a handful of free functions).  Written for the reference-build recipe in this folder: the
// reference's own glm checkout is an empty clone target, and no glm is installed.  This is test infrastructure; it is
// not part of the product library.  Conventions follow GLM's documented interface: matrices are column-major,
// `m[i]` is column i, `mat(a, b, c)` takes columns, `outerProduct(c, r)` is c * r^T.
#pragma once

#include <cmath>
#include <cstddef>

#if defined(__CUDACC__)
#define GLM_FUNC_QUALIFIER __host__ __device__ inline
#else
#define GLM_FUNC_QUALIFIER inline
#endif
#define GLM_SHIM_FN GLM_FUNC_QUALIFIER

namespace glm {

using length_t = int;

template <int N, typename T> struct vec;

template <typename T> struct vec<2, T> {
    T x, y;
    using value_type = T;
    GLM_SHIM_FN vec() : x(T(0)), y(T(0)) {}
    GLM_SHIM_FN explicit vec(T s) : x(s), y(s) {}
    GLM_SHIM_FN vec(T a, T b) : x(a), y(b) {}
    template <typename A, typename B> GLM_SHIM_FN vec(A a, B b) : x(T(a)), y(T(b)) {}
    template <typename U> GLM_SHIM_FN vec(const vec<2, U>& o) : x(T(o.x)), y(T(o.y)) {}
    template <typename U> GLM_SHIM_FN explicit vec(const vec<3, U>& o) : x(T(o.x)), y(T(o.y)) {}
    GLM_SHIM_FN T& operator[](int i) { return (&x)[i]; }
    GLM_SHIM_FN const T& operator[](int i) const { return (&x)[i]; }
    static GLM_SHIM_FN constexpr int length() { return 2; }
};

template <typename T> struct vec<3, T> {
    T x, y, z;
    using value_type = T;
    GLM_SHIM_FN vec() : x(T(0)), y(T(0)), z(T(0)) {}
    GLM_SHIM_FN explicit vec(T s) : x(s), y(s), z(s) {}
    GLM_SHIM_FN vec(T a, T b, T c) : x(a), y(b), z(c) {}
    template <typename A, typename B, typename C> GLM_SHIM_FN vec(A a, B b, C c) : x(T(a)), y(T(b)), z(T(c)) {}
    template <typename U, typename C> GLM_SHIM_FN vec(const vec<2, U>& o, C c) : x(T(o.x)), y(T(o.y)), z(T(c)) {}
    template <typename U> GLM_SHIM_FN vec(const vec<3, U>& o) : x(T(o.x)), y(T(o.y)), z(T(o.z)) {}
    GLM_SHIM_FN T& operator[](int i) { return (&x)[i]; }
    GLM_SHIM_FN const T& operator[](int i) const { return (&x)[i]; }
    static GLM_SHIM_FN constexpr int length() { return 3; }
};

// ---- vector arithmetic (component-wise) ----
#define GLM_SHIM_VEC_BINOP(OP)                                                                                         \
    template <int N, typename T> GLM_SHIM_FN vec<N, T> operator OP(const vec<N, T>& a, const vec<N, T>& b) {           \
        vec<N, T> r;                                                                                                   \
        for (int i = 0; i < N; ++i) r[i] = a[i] OP b[i];                                                               \
        return r;                                                                                                      \
    }                                                                                                                  \
    template <int N, typename T> GLM_SHIM_FN vec<N, T> operator OP(const vec<N, T>& a, T s) {                          \
        vec<N, T> r;                                                                                                   \
        for (int i = 0; i < N; ++i) r[i] = a[i] OP s;                                                                  \
        return r;                                                                                                      \
    }                                                                                                                  \
    template <int N, typename T> GLM_SHIM_FN vec<N, T> operator OP(T s, const vec<N, T>& a) {                          \
        vec<N, T> r;                                                                                                   \
        for (int i = 0; i < N; ++i) r[i] = s OP a[i];                                                                  \
        return r;                                                                                                      \
    }                                                                                                                  \
    template <int N, typename T> GLM_SHIM_FN vec<N, T>& operator OP##=(vec<N, T>& a, const vec<N, T>& b) {             \
        for (int i = 0; i < N; ++i) a[i] OP## = b[i];                                                                  \
        return a;                                                                                                      \
    }                                                                                                                  \
    template <int N, typename T> GLM_SHIM_FN vec<N, T>& operator OP##=(vec<N, T>& a, T s) {                            \
        for (int i = 0; i < N; ++i) a[i] OP## = s;                                                                     \
        return a;                                                                                                      \
    }
GLM_SHIM_VEC_BINOP(+)
GLM_SHIM_VEC_BINOP(-)
GLM_SHIM_VEC_BINOP(*)
GLM_SHIM_VEC_BINOP(/)
#undef GLM_SHIM_VEC_BINOP

template <int N, typename T> GLM_SHIM_FN vec<N, T> operator-(const vec<N, T>& a) {
    vec<N, T> r;
    for (int i = 0; i < N; ++i) r[i] = -a[i];
    return r;
}
template <int N, typename T> GLM_SHIM_FN vec<N, T> operator+(const vec<N, T>& a) { return a; }
template <int N, typename T> GLM_SHIM_FN bool operator==(const vec<N, T>& a, const vec<N, T>& b) {
    bool e = true;
    for (int i = 0; i < N; ++i) e = e && (a[i] == b[i]);
    return e;
}
template <int N, typename T> GLM_SHIM_FN bool operator!=(const vec<N, T>& a, const vec<N, T>& b) { return !(a == b); }

// ---- matrices: C columns of R rows ----
template <int C, int R, typename T> struct mat {
    using col_type = vec<R, T>;
    using value_type = T;
    col_type value[C];

    GLM_SHIM_FN mat() {}
    GLM_SHIM_FN explicit mat(T diagonal) {
        for (int c = 0; c < C; ++c)
            if (c < R) value[c][c] = diagonal;
    }
    GLM_SHIM_FN mat(const col_type& c0, const col_type& c1) {
        static_assert(C == 2, "two columns");
        value[0] = c0;
        value[1] = c1;
    }
    GLM_SHIM_FN mat(const col_type& c0, const col_type& c1, const col_type& c2) {
        static_assert(C == 3, "three columns");
        value[0] = c0;
        value[1] = c1;
        value[2] = c2;
    }
    // scalars in column-major order
    GLM_SHIM_FN mat(T a, T b, T c, T d) {
        static_assert(C == 2 && R == 2, "2x2");
        value[0] = col_type(a, b);
        value[1] = col_type(c, d);
    }
    GLM_SHIM_FN mat(T a, T b, T c, T d, T e, T f, T g, T h, T i) {
        static_assert(C == 3 && R == 3, "3x3");
        value[0] = col_type(a, b, c);
        value[1] = col_type(d, e, f);
        value[2] = col_type(g, h, i);
    }
    template <typename U> GLM_SHIM_FN mat(const mat<C, R, U>& o) {
        for (int c = 0; c < C; ++c) value[c] = col_type(o[c]);
    }
    GLM_SHIM_FN col_type& operator[](int i) { return value[i]; }
    GLM_SHIM_FN const col_type& operator[](int i) const { return value[i]; }
    static GLM_SHIM_FN constexpr int length() { return C; }
};

#define GLM_SHIM_MAT_CWISE(OP)                                                                                         \
    template <int C, int R, typename T> GLM_SHIM_FN mat<C, R, T> operator OP(const mat<C, R, T>& a,                    \
                                                                            const mat<C, R, T>& b) {                   \
        mat<C, R, T> r;                                                                                                \
        for (int c = 0; c < C; ++c) r[c] = a[c] OP b[c];                                                               \
        return r;                                                                                                      \
    }                                                                                                                  \
    template <int C, int R, typename T> GLM_SHIM_FN mat<C, R, T>& operator OP##=(mat<C, R, T>& a,                      \
                                                                                const mat<C, R, T>& b) {               \
        for (int c = 0; c < C; ++c) a[c] OP## = b[c];                                                                  \
        return a;                                                                                                      \
    }
GLM_SHIM_MAT_CWISE(+)
GLM_SHIM_MAT_CWISE(-)
#undef GLM_SHIM_MAT_CWISE

#define GLM_SHIM_MAT_SCALAR(OP)                                                                                        \
    template <int C, int R, typename T> GLM_SHIM_FN mat<C, R, T> operator OP(const mat<C, R, T>& a, T s) {             \
        mat<C, R, T> r;                                                                                                \
        for (int c = 0; c < C; ++c) r[c] = a[c] OP s;                                                                  \
        return r;                                                                                                      \
    }                                                                                                                  \
    template <int C, int R, typename T> GLM_SHIM_FN mat<C, R, T> operator OP(T s, const mat<C, R, T>& a) {             \
        mat<C, R, T> r;                                                                                                \
        for (int c = 0; c < C; ++c) r[c] = s OP a[c];                                                                  \
        return r;                                                                                                      \
    }                                                                                                                  \
    template <int C, int R, typename T> GLM_SHIM_FN mat<C, R, T>& operator OP##=(mat<C, R, T>& a, T s) {               \
        for (int c = 0; c < C; ++c) a[c] OP## = s;                                                                     \
        return a;                                                                                                      \
    }
GLM_SHIM_MAT_SCALAR(*)
GLM_SHIM_MAT_SCALAR(/)
GLM_SHIM_MAT_SCALAR(+)
GLM_SHIM_MAT_SCALAR(-)
#undef GLM_SHIM_MAT_SCALAR

template <int C, int R, typename T> GLM_SHIM_FN mat<C, R, T> operator-(const mat<C, R, T>& a) {
    mat<C, R, T> r;
    for (int c = 0; c < C; ++c) r[c] = -a[c];
    return r;
}

// matrix * column vector: linear combination of the columns
template <int C, int R, typename T> GLM_SHIM_FN vec<R, T> operator*(const mat<C, R, T>& m, const vec<C, T>& v) {
    vec<R, T> r = m[0] * v[0];
    for (int c = 1; c < C; ++c) r = r + m[c] * v[c];
    return r;
}
// row vector * matrix
template <int C, int R, typename T> GLM_SHIM_FN vec<C, T> operator*(const vec<R, T>& v, const mat<C, R, T>& m) {
    vec<C, T> r;
    for (int c = 0; c < C; ++c) {
        T s = v[0] * m[c][0];
        for (int k = 1; k < R; ++k) s = s + v[k] * m[c][k];
        r[c] = s;
    }
    return r;
}
template <int N, typename T> GLM_SHIM_FN mat<N, N, T> operator*(const mat<N, N, T>& a, const mat<N, N, T>& b) {
    mat<N, N, T> r;
    for (int c = 0; c < N; ++c) r[c] = a * b[c];
    return r;
}
template <int N, typename T> GLM_SHIM_FN mat<N, N, T>& operator*=(mat<N, N, T>& a, const mat<N, N, T>& b) {
    a = a * b;
    return a;
}
template <int C, int R, typename T> GLM_SHIM_FN bool operator==(const mat<C, R, T>& a, const mat<C, R, T>& b) {
    bool e = true;
    for (int c = 0; c < C; ++c) e = e && (a[c] == b[c]);
    return e;
}

// ---- free functions ----
template <int N, typename T> GLM_SHIM_FN T dot(const vec<N, T>& a, const vec<N, T>& b) {
    T s = a[0] * b[0];
    for (int i = 1; i < N; ++i) s = s + a[i] * b[i];
    return s;
}
template <int N, typename T> GLM_SHIM_FN T length(const vec<N, T>& a) {
    using std::sqrt;
    return sqrt(dot(a, a));
}
template <int N, typename T> GLM_SHIM_FN vec<N, T> normalize(const vec<N, T>& a) {
    using std::sqrt;
    return a * (T(1) / sqrt(dot(a, a)));
}
template <typename T> GLM_SHIM_FN vec<3, T> cross(const vec<3, T>& a, const vec<3, T>& b) {
    return vec<3, T>(a.y * b.z - b.y * a.z, a.z * b.x - b.z * a.x, a.x * b.y - b.x * a.y);
}
template <int N, typename T> GLM_SHIM_FN vec<N, T> sqrt(const vec<N, T>& a) {
    vec<N, T> r;
    for (int i = 0; i < N; ++i) r[i] = std::sqrt(a[i]);
    return r;
}
template <int N, typename T> GLM_SHIM_FN vec<N, T> abs(const vec<N, T>& a) {
    vec<N, T> r;
    for (int i = 0; i < N; ++i) r[i] = a[i] < T(0) ? -a[i] : a[i];
    return r;
}
template <int N, typename T> GLM_SHIM_FN vec<N, T> min(const vec<N, T>& a, const vec<N, T>& b) {
    vec<N, T> r;
    for (int i = 0; i < N; ++i) r[i] = b[i] < a[i] ? b[i] : a[i];
    return r;
}
template <int N, typename T> GLM_SHIM_FN vec<N, T> max(const vec<N, T>& a, const vec<N, T>& b) {
    vec<N, T> r;
    for (int i = 0; i < N; ++i) r[i] = a[i] < b[i] ? b[i] : a[i];
    return r;
}
// c * r^T: column j of the result is c scaled by r[j]
template <int N, typename T> GLM_SHIM_FN mat<N, N, T> outerProduct(const vec<N, T>& c, const vec<N, T>& r) {
    mat<N, N, T> m;
    for (int j = 0; j < N; ++j) m[j] = c * r[j];
    return m;
}
template <int C, int R, typename T> GLM_SHIM_FN mat<R, C, T> transpose(const mat<C, R, T>& m) {
    mat<R, C, T> t;
    for (int c = 0; c < C; ++c)
        for (int r = 0; r < R; ++r) t[r][c] = m[c][r];
    return t;
}
template <typename T> GLM_SHIM_FN T determinant(const mat<2, 2, T>& m) { return m[0][0] * m[1][1] - m[1][0] * m[0][1]; }
template <typename T> GLM_SHIM_FN T determinant(const mat<3, 3, T>& m) {
    return m[0][0] * (m[1][1] * m[2][2] - m[2][1] * m[1][2]) - m[1][0] * (m[0][1] * m[2][2] - m[2][1] * m[0][2]) +
           m[2][0] * (m[0][1] * m[1][2] - m[1][1] * m[0][2]);
}
template <typename T> GLM_SHIM_FN mat<2, 2, T> inverse(const mat<2, 2, T>& m) {
    const T inv_det = T(1) / (m[0][0] * m[1][1] - m[1][0] * m[0][1]);
    return mat<2, 2, T>(m[1][1] * inv_det, -m[0][1] * inv_det, -m[1][0] * inv_det, m[0][0] * inv_det);
}
template <typename T> GLM_SHIM_FN mat<3, 3, T> inverse(const mat<3, 3, T>& m) {
    const T inv_det = T(1) / determinant(m);
    mat<3, 3, T> r;
    r[0][0] = +(m[1][1] * m[2][2] - m[2][1] * m[1][2]) * inv_det;
    r[1][0] = -(m[1][0] * m[2][2] - m[2][0] * m[1][2]) * inv_det;
    r[2][0] = +(m[1][0] * m[2][1] - m[2][0] * m[1][1]) * inv_det;
    r[0][1] = -(m[0][1] * m[2][2] - m[2][1] * m[0][2]) * inv_det;
    r[1][1] = +(m[0][0] * m[2][2] - m[2][0] * m[0][2]) * inv_det;
    r[2][1] = -(m[0][0] * m[2][1] - m[2][0] * m[0][1]) * inv_det;
    r[0][2] = +(m[0][1] * m[1][2] - m[1][1] * m[0][2]) * inv_det;
    r[1][2] = -(m[0][0] * m[1][2] - m[1][0] * m[0][2]) * inv_det;
    r[2][2] = +(m[0][0] * m[1][1] - m[1][0] * m[0][1]) * inv_det;
    return r;
}

}  // namespace glm
