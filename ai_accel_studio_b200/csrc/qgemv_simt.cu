// CUDA-core (no tensor core) fused GEMV for packed groupwise INT2 / INT4 weights, M <= 4.
//
// This is the general kernel: any N, any group size the format allows, any alignment.  It is
// also the literal "in-register unpack + group-scale dequant fused into an fp32 dot product"
// design: one warp owns two output rows, its lanes stride over K in units of 16 / 4 / 1 packed
// bytes, the activation tile lives in shared memory as fp32 and every product is an fp32 FMA.
//
// Arithmetic per weight (the reason this kernel is instruction-issue bound rather than HBM
// bound on B200 -- about 2 + M issue slots per weight against a budget of ~1.4 (INT2) or ~2.8
// (INT4) slots per weight at full HBM rate):
//   1 LOP3   (h & field_mask) | 0x4B000000     -> float 2^23 + code * radix^j  (code left in place)
//   1 FADD   - (2^23 + offset * radix^j)       -> (code - offset) * radix^j, exact
//   M FFMA   with x[k] pre-multiplied by radix^-j when it was staged (exact, power of two)
// INT2 levels are (2c-3)/3: the packed half-word is shifted left once so that the field holds
// 2c, the offset is 3, and the factor 1/3 is folded into the group scale.  INT4 levels are c-8.
// The group scale multiplies the fp32 partial sum of a unit once.
//
// Replaces the Triton kernels _decode_gemv (ai_accel_lab/kernels/decode_int2.py:43-96) and
// _decode_int4_gemv (ai_accel_lab/kernels/groupwise_int4.py:85-107) of the reference project.
#include "qgemv_common.cuh"

namespace qgemv {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kRowsPerWarp = 2;
constexpr int kRowsPerBlock = kWarps * kRowsPerWarp;
constexpr int kTileFloats = 2048;  // fp32 activations per row of x held in shared memory

// (code - offset) * radix^j for the 16-bit half-word h; INT2: 8 codes, INT4: 4 codes.
template <int BITS, int J>
__device__ __forceinline__ float field_value(uint32_t h) {
    if constexpr (BITS == 2) {
        // h already shifted left by one: bits 2J+1..2J+2 hold 2c.
        const uint32_t f = (h & (6u << (2 * J))) | 0x4B000000u;
        return __uint_as_float(f) - (8388608.0f + 3.0f * float(1u << (2 * J)));
    } else {
        const uint32_t f = (h & (15u << (4 * J))) | 0x4B000000u;
        return __uint_as_float(f) - (8388608.0f + 8.0f * float(1u << (4 * J)));
    }
}

// Accumulate one 16-bit half-word (8 INT2 codes or 4 INT4 codes) against M rows of staged x.
// xs points at the float4-interleaved activations of this unit: element w of the unit lives
// at xs[(w / 4) * stride4 * 4 + (w % 4)] for each m at distance mstride.
template <int BITS, int M>
__device__ __forceinline__ void half_word(uint32_t h, const float* xs, int stride4, int mstride,
                                          int first_w, float (&p)[M]) {
    constexpr int CODES = 16 / BITS;
    if constexpr (BITS == 2) h <<= 1;
#pragma unroll
    for (int q = 0; q < CODES / 4; ++q) {
        float w[4];
        if constexpr (BITS == 2) {
            if (q == 0) { w[0] = field_value<2, 0>(h); w[1] = field_value<2, 1>(h); w[2] = field_value<2, 2>(h); w[3] = field_value<2, 3>(h); }
            else        { w[0] = field_value<2, 4>(h); w[1] = field_value<2, 5>(h); w[2] = field_value<2, 6>(h); w[3] = field_value<2, 7>(h); }
        } else {
            w[0] = field_value<4, 0>(h); w[1] = field_value<4, 1>(h); w[2] = field_value<4, 2>(h); w[3] = field_value<4, 3>(h);
        }
        const int i4 = (first_w >> 2) + q;
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const float4 xv = *reinterpret_cast<const float4*>(xs + m * mstride + (size_t)i4 * stride4 * 4);
            p[m] = fmaf(w[0], xv.x, p[m]);
            p[m] = fmaf(w[1], xv.y, p[m]);
            p[m] = fmaf(w[2], xv.z, p[m]);
            p[m] = fmaf(w[3], xv.w, p[m]);
        }
    }
}

template <int BITS, int M, int U, bool BF16>
__global__ void __launch_bounds__(kThreads) qgemv_simt_kernel(const Args a) {
    using XT = typename Act16<BF16>::T;
    constexpr int CPB = 8 / BITS;           // codes per packed byte
    constexpr int UC = U * CPB;             // codes per unit (one lane, one load)
    constexpr int UC4 = UC < 4 ? 4 : UC;    // floats of shared memory a unit occupies
    constexpr int KT = kTileFloats / UC4 * UC;  // codes per K tile
    constexpr int NU = KT / UC;             // units per tile
    constexpr int RADIX_LOG2 = BITS;        // INT2 -> 4^-j = 2^-2j ; INT4 -> 16^-j = 2^-4j
    constexpr int JMASK = 16 / BITS - 1;    // j = k mod (codes per half-word)

    __shared__ __align__(16) float xs[M * kTileFloats];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row0 = blockIdx.x * kRowsPerBlock + warp * kRowsPerWarp;
    const XT* x = static_cast<const XT*>(a.x);

    float acc[kRowsPerWarp][M];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) acc[r][m] = 0.0f;

    int rows[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) rows[r] = min(row0 + r, a.n - 1);

    for (int k0 = 0; k0 < a.kpad; k0 += KT) {
        const int kt = min(KT, a.kpad - k0);
        __syncthreads();
        // Stage x[:, k0:k0+kt] as fp32, pre-scaled by radix^-(k mod codes-per-half-word), in
        // unit-interleaved order: code w of unit u -> float ((w/4) * NU + u) * 4 + (w % 4).
        for (int i = tid; i < M * KT; i += kThreads) {
            const int m = i / KT, kk = i - m * KT;
            float v = 0.0f;
            if (kk < kt) v = Act16<BF16>::to_float(x[(size_t)m * a.ldx + k0 + kk]);
            v = ldexpf(v, -RADIX_LOG2 * (kk & JMASK));
            const int u = kk / UC, w = kk - u * UC;
            xs[m * kTileFloats + ((w >> 2) * NU + u) * 4 + (w & 3)] = v;
        }
        __syncthreads();

        const int nu = kt / UC;
        for (int u = lane; u < nu; u += 32) {
            const int kcode = k0 + u * UC;
            const int g = kcode / a.group;
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r) {
                const uint8_t* prow = a.packed + (size_t)rows[r] * a.ldp + (size_t)(kcode / CPB);
                float s = __half2float(a.scales[(size_t)rows[r] * a.lds + g]);
                if constexpr (BITS == 2) s *= (1.0f / 3.0f);
                float p[M];
#pragma unroll
                for (int m = 0; m < M; ++m) p[m] = 0.0f;
                const float* xu = xs + u * 4;
                if constexpr (U == 16) {
                    const uint4 v = *reinterpret_cast<const uint4*>(prow);
                    const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        half_word<BITS, M>(wv[q] & 0xffffu, xu, NU, kTileFloats, (2 * q) * (16 / BITS), p);
                        half_word<BITS, M>(wv[q] >> 16, xu, NU, kTileFloats, (2 * q + 1) * (16 / BITS), p);
                    }
                } else if constexpr (U == 4) {
                    const uint32_t wv = *reinterpret_cast<const uint32_t*>(prow);
                    half_word<BITS, M>(wv & 0xffffu, xu, NU, kTileFloats, 0, p);
                    half_word<BITS, M>(wv >> 16, xu, NU, kTileFloats, 16 / BITS, p);
                } else {
                    // One byte: its codes sit at j = (codes per byte) * (byte parity) + i of a half-word.
                    const uint32_t b = *prow;
                    const int odd = (kcode / CPB) & 1;
                    const uint32_t h = b << (8 * odd);
                    float w[4] = {0.f, 0.f, 0.f, 0.f};
                    if constexpr (BITS == 2) {
                        const uint32_t h2 = h << 1;
                        if (odd) { w[0] = field_value<2, 4>(h2); w[1] = field_value<2, 5>(h2); w[2] = field_value<2, 6>(h2); w[3] = field_value<2, 7>(h2); }
                        else     { w[0] = field_value<2, 0>(h2); w[1] = field_value<2, 1>(h2); w[2] = field_value<2, 2>(h2); w[3] = field_value<2, 3>(h2); }
                    } else {
                        if (odd) { w[0] = field_value<4, 2>(h); w[1] = field_value<4, 3>(h); }
                        else     { w[0] = field_value<4, 0>(h); w[1] = field_value<4, 1>(h); }
                    }
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        const float4 xv = *reinterpret_cast<const float4*>(xu + m * kTileFloats);
                        p[m] = fmaf(w[0], xv.x, p[m]);
                        p[m] = fmaf(w[1], xv.y, p[m]);
                        if constexpr (BITS == 2) {
                            p[m] = fmaf(w[2], xv.z, p[m]);
                            p[m] = fmaf(w[3], xv.w, p[m]);
                        }
                    }
                }
#pragma unroll
                for (int m = 0; m < M; ++m) acc[r][m] = fmaf(s, p[m], acc[r][m]);
            }
        }
    }

    // Exact-fp16 outlier columns and the rank-r residual, spread over the lanes.
    if (a.oc > 0) {
        for (int j = lane; j < a.oc; j += 32) {
            const int col = a.oidx[j];
            float xv[M];
#pragma unroll
            for (int m = 0; m < M; ++m)
                xv[m] = (col >= 0 && col < a.kpad) ? Act16<BF16>::to_float(x[(size_t)m * a.ldx + col]) : 0.0f;
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r) {
                const float w = __half2float(a.ow[(size_t)rows[r] * a.ldow + j]);
#pragma unroll
                for (int m = 0; m < M; ++m) acc[r][m] = fmaf(w, xv[m], acc[r][m]);
            }
        }
    }
    if (a.rank > 0) {
        for (int q = lane; q < a.rank; q += 32) {
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r) {
                const float w = __half2float(a.ru[(size_t)rows[r] * a.ldu + q]);
#pragma unroll
                for (int m = 0; m < M; ++m) acc[r][m] = fmaf(w, a.t[m * kMaxRank + q], acc[r][m]);
            }
        }
    }

#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float v = acc[r][m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            acc[r][m] = v;
        }

    if (lane == 0) {
        XT* y = static_cast<XT*>(a.y);
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            const int row = row0 + r;
            if (row >= a.n) continue;
            const float b = a.bias ? __half2float(a.bias[row]) : 0.0f;
#pragma unroll
            for (int m = 0; m < M; ++m)
                y[(size_t)m * a.ldy + row] = Act16<BF16>::from_float(apply_act(acc[r][m] + b, a.act));
        }
    }
}

// t[m][r] = sum_{k < Korig} res_v[r, k] * x[m, k]   (fp32).  One block per residual row r.
// Launched in full stream order (so x is final once any block of it runs); the fused kernel
// that follows carries the programmatic-serialisation attribute, may start as soon as every
// block here has executed griddepcontrol.launch_dependents, reads x at once and reads t only
// after its own griddepcontrol.wait.
template <bool BF16>
__global__ void __launch_bounds__(256) residual_t_kernel(const Args a) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    using XT = typename Act16<BF16>::T;
    const int r = blockIdx.x;
    const XT* x = static_cast<const XT*>(a.x);
    const __half* v = a.rv + (size_t)r * a.ldv;
    float s[QGEMV_MAX_M] = {0.f, 0.f, 0.f, 0.f};
    const bool vec = (reinterpret_cast<uintptr_t>(v) % 16 == 0) && (a.ldv % 8 == 0) &&
                     (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (a.ldx % 8 == 0);
    const int k8 = vec ? a.korig / 8 : 0;
    for (int i = threadIdx.x; i < k8; i += blockDim.x) {
        const uint4 vv = reinterpret_cast<const uint4*>(v)[i];
        const __half* vh = reinterpret_cast<const __half*>(&vv);
        for (int m = 0; m < a.m; ++m) {
            const uint4 xv = *reinterpret_cast<const uint4*>(x + (size_t)m * a.ldx + (size_t)i * 8);
            const XT* xh = reinterpret_cast<const XT*>(&xv);
#pragma unroll
            for (int q = 0; q < 8; ++q) s[m] = fmaf(__half2float(vh[q]), Act16<BF16>::to_float(xh[q]), s[m]);
        }
    }
    for (int k = k8 * 8 + threadIdx.x; k < a.korig; k += blockDim.x)
        for (int m = 0; m < a.m; ++m)
            s[m] = fmaf(__half2float(v[k]), Act16<BF16>::to_float(x[(size_t)m * a.ldx + k]), s[m]);
    __shared__ float red[8][QGEMV_MAX_M];
#pragma unroll
    for (int m = 0; m < QGEMV_MAX_M; ++m) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s[m] += __shfl_xor_sync(0xffffffffu, s[m], o);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5][m] = s[m];
    }
    __syncthreads();
    if (threadIdx.x < a.m) {
        float tot = 0.0f;
        for (int i = 0; i < 8; ++i) tot += red[i][threadIdx.x];
        a.t[threadIdx.x * kMaxRank + r] = tot;
    }
}

template <int BITS, int M, int U>
int launch_simt_bmu(const Args& a, bool bf16, cudaStream_t s) {
    dim3 grid((a.n + kRowsPerBlock - 1) / kRowsPerBlock), block(kThreads);
    if (bf16) qgemv_simt_kernel<BITS, M, U, true><<<grid, block, 0, s>>>(a);
    else      qgemv_simt_kernel<BITS, M, U, false><<<grid, block, 0, s>>>(a);
    return check_launch("qgemv_simt_kernel");
}

template <int BITS, int M>
int launch_simt_bm(const Args& a, bool bf16, int unit, cudaStream_t s) {
    if (unit == 16) return launch_simt_bmu<BITS, M, 16>(a, bf16, s);
    if (unit == 4) return launch_simt_bmu<BITS, M, 4>(a, bf16, s);
    return launch_simt_bmu<BITS, M, 1>(a, bf16, s);
}

template <int BITS>
int launch_simt_b(const Args& a, bool bf16, int unit, cudaStream_t s) {
    switch (a.m) {
        case 1: return launch_simt_bm<BITS, 1>(a, bf16, unit, s);
        case 2: return launch_simt_bm<BITS, 2>(a, bf16, unit, s);
        case 3: return launch_simt_bm<BITS, 3>(a, bf16, unit, s);
        default: return launch_simt_bm<BITS, 4>(a, bf16, unit, s);
    }
}

}  // namespace

int launch_residual_t(const Args& a, bool bf16, cudaStream_t s) {
    dim3 grid(a.rank), block(256);
    if (bf16) residual_t_kernel<true><<<grid, block, 0, s>>>(a);
    else      residual_t_kernel<false><<<grid, block, 0, s>>>(a);
    return check_launch("residual_t_kernel");
}

int launch_simt(const Args& a, int bits, bool bf16, int unit_bytes, cudaStream_t s) {
    return bits == 2 ? launch_simt_b<2>(a, bf16, unit_bytes, s) : launch_simt_b<4>(a, bf16, unit_bytes, s);
}

const char* simt_name(int bits, int m, int unit_bytes) {
    static const char* names[2][3] = {{"simt_int2_u16", "simt_int2_u4", "simt_int2_u1"},
                                      {"simt_int4_u16", "simt_int4_u4", "simt_int4_u1"}};
    (void)m;
    return names[bits == 2 ? 0 : 1][unit_bytes == 16 ? 0 : unit_bytes == 4 ? 1 : 2];
}

}  // namespace qgemv
