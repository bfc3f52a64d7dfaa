/* CPU restatement of the reference project's "dequantise, then matmul" path for packed
 * groupwise INT2 / INT4 weights.  TEST INFRASTRUCTURE ONLY: it is the checker for the
 * larger parity cases and the thing timed as the CPU baseline; the product library never
 * links or calls it.
 *
 * What it follows (paths inside the reference project, ai_accel_lab v5.0.0):
 *   unpack_groupwise_int2   ai_accel_lab/kernels/groupwise_int2.py:122-130
 *   unpack_groupwise_int4   ai_accel_lab/kernels/groupwise_int4.py:63-69
 *   reference_linear        ai_accel_lab/kernels/groupwise_int2.py:133-135, groupwise_int4.py:72-73
 *   outlier term            ai_accel_lab/kernels/decode_int2.py:147-151
 *   residual term           ai_accel_lab/optimize/hybrid_int2.py:104-106
 *   CPU forward             ai_accel_lab/optimize/hybrid_int2.py:96-107, hybrid_int4.py:36-37
 *
 * Like the reference's CPU branch it works in two passes: the whole [N,K] matrix is
 * dequantised into memory first, then multiplied.  Dequantisation is float32
 * (level_f32 * float32(scale_f16)), the dot products accumulate in double, so the result is
 * the "fp32-accumulate reference" the GPU kernels are compared against.
 * Parallelised over output rows with OpenMP; bit-identical for any thread count.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static const float kInt2Levels[4] = {-1.0f, -1.0f / 3.0f, 1.0f / 3.0f, 1.0f}; /* groupwise_int2.py:18 */

static float half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static float bf16_to_float(uint16_t h) {
    uint32_t bits = (uint32_t)h << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

int qref_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1; a timing run asks for the cores it may use. */
void qref_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* codes[N, Kpad] <- packed; bits = 2: byte b holds columns 4b..4b+3 in bit pairs 0,2,4,6
 * (groupwise_int2.py:124); bits = 4: low nibble = even column (groupwise_int4.py:65). */
void qref_unpack_codes(const uint8_t* packed, int64_t n, int64_t kpad, int bits, uint8_t* codes) {
    const int64_t rowb = kpad * bits / 8;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
        const uint8_t* p = packed + r * rowb;
        uint8_t* c = codes + r * kpad;
        if (bits == 2) {
            for (int64_t b = 0; b < rowb; ++b) {
                c[4 * b + 0] = p[b] & 3; c[4 * b + 1] = (p[b] >> 2) & 3;
                c[4 * b + 2] = (p[b] >> 4) & 3; c[4 * b + 3] = (p[b] >> 6) & 3;
            }
        } else {
            for (int64_t b = 0; b < rowb; ++b) { c[2 * b] = p[b] & 15; c[2 * b + 1] = p[b] >> 4; }
        }
    }
}

/* w[N, K] (float32, row stride K) <- level * float32(scale); the padded tail columns are dropped. */
void qref_dequant_f32(const uint8_t* packed, const uint16_t* scales, int64_t n, int64_t kpad, int64_t k,
                      int group, int bits, float* w) {
    const int64_t rowb = kpad * bits / 8, ng = kpad / group;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
        const uint8_t* p = packed + r * rowb;
        float* o = w + r * k;
        for (int64_t c = 0; c < k; ++c) {
            const float s = half_to_float(scales[r * ng + c / group]);
            float v;
            if (bits == 2) v = kInt2Levels[(p[c >> 2] >> (2 * (c & 3))) & 3];
            else v = (float)((int)((p[c >> 1] >> (4 * (c & 1))) & 15) - 8);
            o[c] = v * s;
        }
    }
}

/* Whole forward: y[M,N] (float32) = x[:, :K] . W^T + x[:, idx] . OW^T + (x . V^T) . U^T + bias, then act.
 * x is fp16 (x_is_bf16 = 0) or bf16 bit patterns [M, ldx].  wbuf is caller scratch of N*K floats
 * (the materialised matrix, as in the reference).  act: 0 none, 1 relu, 2 silu. */
void qref_forward(const uint16_t* x, int64_t ldx, int x_is_bf16, int m,
                  const uint8_t* packed, const uint16_t* scales, int64_t n, int64_t kpad, int64_t k,
                  int group, int bits, const uint16_t* bias,
                  const int32_t* out_idx, const uint16_t* out_w, int oc,
                  const uint16_t* res_u, const uint16_t* res_v, int rank, int act,
                  float* wbuf, float* y) {
    qref_dequant_f32(packed, scales, n, kpad, k, group, bits, wbuf);          /* pass 1 */
    float* xf = (float*)malloc(sizeof(float) * (size_t)m * (size_t)kpad);
    for (int i = 0; i < m; ++i)
        for (int64_t c = 0; c < kpad; ++c)
            xf[i * kpad + c] = x_is_bf16 ? bf16_to_float(x[i * ldx + c]) : half_to_float(x[i * ldx + c]);
    double* t = NULL;
    if (rank > 0) { /* t[m][r] = x . V[r] */
        t = (double*)malloc(sizeof(double) * (size_t)m * (size_t)rank);
        for (int i = 0; i < m; ++i)
            for (int r = 0; r < rank; ++r) {
                double a = 0;
                for (int64_t c = 0; c < k; ++c) a += (double)xf[i * kpad + c] * (double)half_to_float(res_v[r * k + c]);
                t[i * rank + r] = a;
            }
    }
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n; ++r) {                                           /* pass 2 */
        const float* wr = wbuf + r * k;
        for (int i = 0; i < m; ++i) {
            const float* xr = xf + i * kpad;
            double a0 = 0, a1 = 0, a2 = 0, a3 = 0;
            int64_t c = 0;
            for (; c + 4 <= k; c += 4) {
                a0 += (double)wr[c] * xr[c]; a1 += (double)wr[c + 1] * xr[c + 1];
                a2 += (double)wr[c + 2] * xr[c + 2]; a3 += (double)wr[c + 3] * xr[c + 3];
            }
            for (; c < k; ++c) a0 += (double)wr[c] * xr[c];
            double a = (a0 + a1) + (a2 + a3);
            for (int j = 0; j < oc; ++j)
                a += (double)half_to_float(out_w[r * oc + j]) * (double)xr[out_idx[j]];
            for (int q = 0; q < rank; ++q) a += (double)half_to_float(res_u[r * rank + q]) * t[i * rank + q];
            if (bias) a += (double)half_to_float(bias[r]);
            if (act == 1) a = a > 0 ? a : 0;
            else if (act == 2) a = a / (1.0 + exp(-a));
            y[(int64_t)i * n + r] = (float)a;
        }
    }
    free(xf);
    free(t);
}
