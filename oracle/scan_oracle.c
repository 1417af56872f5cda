/*
 * CPU oracle for the first-order gated linear scan.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the sequential algorithm of the reference's CPU
 * path.  It exists to check the CUDA kernels and to serve as a timed CPU baseline;
 * nothing on the product path may link, import or call it.
 *
 * Reference being restated (paths inside the unixpickle/scanscam project):
 *   forward : src/scanscam_cpu.hpp:9-28   (simple_linear_scan_cpu_kernel)
 *   backward: src/scanscam_cpu.hpp:54-78  (simple_linear_scan_backward_cpu_kernel)
 *   second opinion: scanscam/baseline.py:8-40 (naive per-timestep torch loops)
 *
 * Arithmetic contract: every step is one multiply and one add, each rounded
 * separately in the working precision (the reference source has no fused
 * multiply-add; build this file with -ffp-contract=off so the compiler does not
 * introduce one).  With that, the results are bit-identical to the reference's
 * CPU extension; tests/test_oracle.py pins this against vectors produced by the
 * reference itself.
 *
 * Layouts:
 *   "rows" functions work on a dense [rows, T] matrix, scan axis innermost.
 *   "cl" (channels-last) functions work on a dense [N, T, C] array and scan over
 *   the middle axis; they restate what the reference obtains by running the same
 *   loops on a transposed view (scanscam/op.py:28-29, scanscam/cuda_test.py:138-141).
 *
 * Optional carry arguments model a shard of a longer sequence:
 *   h_in[r]    value of h just before the first step of the shard (NULL = 0)
 *   gb_in[r]   value of a_{t+1}*gb_{t+1} entering the last step (NULL = 0)
 *   h_prev[r]  value of h just before the first step, used for ga at step 0 (NULL = 0)
 * With all of them NULL the functions are exactly the reference's.
 */
#include <stddef.h>
#include <stdint.h>

#define DEFINE_ORACLE(SUFFIX, real)                                                          \
    void oracle_scan_fwd_##SUFFIX(const real *gate, const real *value, real *out,            \
                                  int64_t rows, int64_t T, const real *h_in)                 \
    {                                                                                        \
        for (int64_t r = 0; r < rows; r++) {                                                 \
            const real *g = gate + r * T;                                                    \
            const real *v = value + r * T;                                                   \
            real *o = out + r * T;                                                           \
            real acc = h_in ? h_in[r] : (real)0;                                             \
            for (int64_t t = 0; t < T; t++) {                                                \
                acc *= g[t];                                                                 \
                acc += v[t];                                                                 \
                o[t] = acc;                                                                  \
            }                                                                                \
        }                                                                                    \
    }                                                                                        \
                                                                                             \
    void oracle_scan_bwd_##SUFFIX(const real *gate, const real *h, const real *gout,         \
                                  real *ggate, real *gvalue, int64_t rows, int64_t T,        \
                                  const real *gb_in, const real *h_prev)                     \
    {                                                                                        \
        for (int64_t r = 0; r < rows; r++) {                                                 \
            const int64_t base = r * T;                                                      \
            real d = gb_in ? gb_in[r] : (real)0;                                             \
            for (int64_t t = T - 1; t >= 0; t--) {                                           \
                real prev = t > 0 ? h[base + t - 1] : (h_prev ? h_prev[r] : (real)0);        \
                d += gout[base + t];                                                         \
                gvalue[base + t] = d;                                                        \
                ggate[base + t] = d * prev;                                                  \
                d *= gate[base + t];                                                         \
            }                                                                                \
        }                                                                                    \
    }                                                                                        \
                                                                                             \
    void oracle_scan_cl_fwd_##SUFFIX(const real *gate, const real *value, real *out,         \
                                     int64_t N, int64_t T, int64_t C)                        \
    {                                                                                        \
        for (int64_t n = 0; n < N; n++) {                                                    \
            for (int64_t c = 0; c < C; c++) {                                                \
                real acc = (real)0;                                                          \
                for (int64_t t = 0; t < T; t++) {                                            \
                    const int64_t i = (n * T + t) * C + c;                                   \
                    acc *= gate[i];                                                          \
                    acc += value[i];                                                         \
                    out[i] = acc;                                                            \
                }                                                                            \
            }                                                                                \
        }                                                                                    \
    }                                                                                        \
                                                                                             \
    void oracle_scan_cl_bwd_##SUFFIX(const real *gate, const real *h, const real *gout,      \
                                     real *ggate, real *gvalue, int64_t N, int64_t T,        \
                                     int64_t C)                                              \
    {                                                                                        \
        for (int64_t n = 0; n < N; n++) {                                                    \
            for (int64_t c = 0; c < C; c++) {                                                \
                real d = (real)0;                                                            \
                for (int64_t t = T - 1; t >= 0; t--) {                                       \
                    const int64_t i = (n * T + t) * C + c;                                   \
                    real prev = t > 0 ? h[i - C] : (real)0;                                  \
                    d += gout[i];                                                            \
                    gvalue[i] = d;                                                           \
                    ggate[i] = d * prev;                                                     \
                    d *= gate[i];                                                            \
                }                                                                            \
            }                                                                                \
        }                                                                                    \
    }

DEFINE_ORACLE(f32, float)
DEFINE_ORACLE(f64, double)
