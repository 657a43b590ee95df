/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE. CPU restatement of the reference's mixture evaluation, used
 * only as the checker in tests / smoke and as the timed CPU baseline of the benchmark.
 *
 * Follows, line by line in meaning:
 *   forward  : src/gmc/cpp/extensions/evaluate_inversed/parallel_implementation.cu:23-55
 *              (one work item per query point, serial loop over components), with the per-pair
 *              math of gpe::evaluate_inversed, src/gmc/cpp/extensions/util/gaussian.h:82-95
 *   backward : parallel_implementation.cu:133-173 with gpe::grad::evaluate_inversed,
 *              src/gmc/cpp/extensions/util/grad/gaussian.h:19-66 and the cofactor matrix of
 *              util/grad/glm.h:16-51
 * The reference runs these bodies under OpenMP with one thread per CUDA thread of a 128-wide block
 * (parallel_start.h:92-111) and accumulates gradients with CAS-loop atomics; here the OpenMP loop runs
 * over query points and each thread keeps a private gradient buffer that is summed at the end, which
 * gives the same sums without atomics.
 *
 * Two instantiations: float (the arithmetic the reference uses; timed as the CPU baseline) and double
 * (the parity oracle for the 1e-4 relative check).
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define GMC_PI 3.14159265358979323846

#define DEFINE_EVAL(T, SUFFIX, EXP, SQRT)                                                                          \
    static inline T det_##SUFFIX(const T* S, int D) {                                                              \
        if (D == 2) return S[0] * S[3] - S[1] * S[2];                                                              \
        return S[0] * (S[4] * S[8] - S[5] * S[7]) - S[1] * (S[3] * S[8] - S[5] * S[6]) +                           \
               S[2] * (S[3] * S[7] - S[4] * S[6]);                                                                 \
    }                                                                                                              \
    /* cofactor matrix = d det / d S (util/grad/glm.h:16-51) */                                                    \
    static inline void cofactor_##SUFFIX(const T* S, int D, T* C) {                                                \
        if (D == 2) {                                                                                              \
            C[0] = S[3]; C[1] = -S[2]; C[2] = -S[1]; C[3] = S[0];                                                  \
            return;                                                                                                \
        }                                                                                                          \
        for (int i = 0; i < 3; ++i)                                                                                \
            for (int j = 0; j < 3; ++j) {                                                                          \
                const int i1 = i < 1, i2 = 2 - (i >> 1), j1 = j < 1, j2 = 2 - (j >> 1);                            \
                const T m = S[i1 * 3 + j1] * S[i2 * 3 + j2] - S[i1 * 3 + j2] * S[i2 * 3 + j1];                     \
                C[i * 3 + j] = (((i ^ j) & 1) == 0) ? m : -m;                                                      \
            }                                                                                                      \
    }                                                                                                              \
    void oracle_eval_forward_##SUFFIX(const T* mixture, const T* xes, T* out, int B, int L, int G, int D, int Bx,  \
                                      int Lx, int N) {                                                             \
        const int RF = 1 + D + D * D;                                                                              \
        const T factor = (T)pow(2.0 * GMC_PI, -0.5 * D);                                                           \
        const long long rows = (long long)B * L * N;                                                               \
        _Pragma("omp parallel for schedule(static)") for (long long r = 0; r < rows; ++r) {                        \
            const int n = (int)(r % N);                                                                            \
            const int bl = (int)(r / N);                                                                           \
            const int b = bl / L, l = bl % L;                                                                      \
            const int bx = b < Bx - 1 ? b : Bx - 1, lx = l < Lx - 1 ? l : Lx - 1;                                   \
            const T* x = xes + (((size_t)bx * Lx + lx) * N + n) * D;                                               \
            T sum = 0;                                                                                             \
            for (int g = 0; g < G; ++g) {                                                                          \
                const T* ga = mixture + ((size_t)bl * G + g) * RF;                                                 \
                const T* S = ga + 1 + D;                                                                           \
                T t[3], St[3], v = 0;                                                                              \
                for (int i = 0; i < D; ++i) t[i] = x[i] - ga[1 + i];                                               \
                for (int i = 0; i < D; ++i) {                                                                      \
                    St[i] = 0;                                                                                     \
                    for (int j = 0; j < D; ++j) St[i] += S[i * D + j] * t[j];                                      \
                    v += t[i] * St[i];                                                                             \
                }                                                                                                  \
                v *= (T)-0.5;                                                                                      \
                const T norm = SQRT(det_##SUFFIX(S, D)) * factor;                                                  \
                sum += ga[0] * norm * EXP(v);                                                                      \
            }                                                                                                      \
            out[r] = sum;                                                                                          \
        }                                                                                                          \
    }                                                                                                              \
    void oracle_eval_backward_##SUFFIX(const T* grad_out, const T* mixture, const T* xes, T* grad_mixture,         \
                                       T* grad_xes, int B, int L, int G, int D, int Bx, int Lx, int N) {           \
        const int RF = 1 + D + D * D;                                                                              \
        const T factor = (T)pow(2.0 * GMC_PI, -0.5 * D);                                                           \
        const size_t gm_count = (size_t)B * L * G * RF;                                                            \
        const size_t gx_count = (size_t)Bx * Lx * N * D;                                                           \
        if (grad_mixture) memset(grad_mixture, 0, gm_count * sizeof(T));                                           \
        if (grad_xes) memset(grad_xes, 0, gx_count * sizeof(T));                                                   \
        for (int bl = 0; bl < B * L; ++bl) {                                                                       \
            const int b = bl / L, l = bl % L;                                                                      \
            const int bx = b < Bx - 1 ? b : Bx - 1, lx = l < Lx - 1 ? l : Lx - 1;                                   \
            _Pragma("omp parallel") {                                                                              \
                T* priv = (T*)calloc((size_t)G * RF, sizeof(T));                                                   \
                _Pragma("omp for schedule(static)") for (int n = 0; n < N; ++n) {                                  \
                    const T* x = xes + (((size_t)bx * Lx + lx) * N + n) * D;                                       \
                    const T incoming = grad_out[(size_t)bl * N + n];                                               \
                    T gx[3] = {0, 0, 0};                                                                           \
                    for (int g = 0; g < G; ++g) {                                                                  \
                        const T* ga = mixture + ((size_t)bl * G + g) * RF;                                         \
                        const T* S = ga + 1 + D;                                                                   \
                        T t[3], St[3], v = 0;                                                                      \
                        for (int i = 0; i < D; ++i) t[i] = x[i] - ga[1 + i];                                       \
                        for (int i = 0; i < D; ++i) {                                                              \
                            St[i] = 0;                                                                             \
                            for (int j = 0; j < D; ++j) St[i] += S[i * D + j] * t[j];                              \
                            v += t[i] * St[i];                                                                     \
                        }                                                                                          \
                        v *= (T)-0.5;                                                                              \
                        const T det = det_##SUFFIX(S, D);                                                          \
                        const T root = SQRT(det);                                                                  \
                        const T norm = root * factor;                                                              \
                        const T e = EXP(v);                                                                        \
                        T* gg = priv + (size_t)g * RF;                                                             \
                        gg[0] += norm * e * incoming;                                                              \
                        const T grad_norm = ga[0] * e * incoming;                                                  \
                        const T grad_v = ga[0] * norm * incoming * e;                                              \
                        const T grad_det = grad_norm * factor / (2 * root);                                        \
                        /* grad_t = -grad_v * S t (symmetric S); d/dx = grad_t, d/dmu = -grad_t */                 \
                        T SSt[3];                                                                                  \
                        for (int i = 0; i < D; ++i) {                                                              \
                            SSt[i] = 0;                                                                            \
                            for (int j = 0; j < D; ++j) SSt[i] += S[j * D + i] * t[j];                             \
                        }                                                                                          \
                        T cof[9];                                                                                  \
                        cofactor_##SUFFIX(S, D, cof);                                                              \
                        for (int i = 0; i < D; ++i) {                                                              \
                            const T grad_t = (T)-0.5 * grad_v * (St[i] + SSt[i]);                                  \
                            gx[i] += grad_t;                                                                       \
                            gg[1 + i] -= grad_t;                                                                   \
                            for (int j = 0; j < D; ++j)                                                            \
                                gg[1 + D + i * D + j] += (T)-0.5 * grad_v * t[i] * t[j] + grad_det * cof[i * D + j]; \
                        }                                                                                          \
                    }                                                                                              \
                    if (grad_xes) {                                                                                \
                        T* dst = grad_xes + (((size_t)bx * Lx + lx) * N + n) * D;                                  \
                        for (int i = 0; i < D; ++i) {                                                              \
                            if (Bx == B && Lx == L) dst[i] += gx[i];                                               \
                            else {                                                                                 \
                                _Pragma("omp atomic") dst[i] += gx[i];                                             \
                            }                                                                                      \
                        }                                                                                          \
                    }                                                                                              \
                }                                                                                                  \
                if (grad_mixture) {                                                                                \
                    _Pragma("omp critical") {                                                                      \
                        T* dst = grad_mixture + (size_t)bl * G * RF;                                               \
                        for (size_t i = 0; i < (size_t)G * RF; ++i) dst[i] += priv[i];                             \
                    }                                                                                              \
                }                                                                                                  \
                free(priv);                                                                                        \
            }                                                                                                      \
        }                                                                                                          \
    }

DEFINE_EVAL(float, f32, expf, sqrtf)
DEFINE_EVAL(double, f64, exp, sqrt)

/* torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the timed CPU baseline asks for all cores instead. */
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
