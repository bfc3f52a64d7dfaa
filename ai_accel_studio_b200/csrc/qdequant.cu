// Dense dequantisation and code expansion for packed groupwise INT2 / INT4 weights.
//
// Bit-exact restatement of the reference project's torch expressions
//   unpack_groupwise_int2  ai_accel_lab/kernels/groupwise_int2.py:122-130
//   unpack_groupwise_int4  ai_accel_lab/kernels/groupwise_int4.py:63-69
// for dtype float32, float16 and bfloat16: the level table is first rounded to the output
// type, the fp16 scale is converted to the output type, and their product is rounded once.
// Used for the M > 4 (prefill) path, where the dense matrix feeds a library GEMM, and by the
// tests that pin "unpacked codes bit-exact".
#include <type_traits>

#include "qgemv_common.cuh"

namespace qgemv {
namespace {

// (-1, -1/3, 1/3, 1) rounded to each output type (round-to-nearest-even from the exact value).
__device__ __forceinline__ float level2_f32(int c) {
    return c == 0 ? -1.0f : c == 1 ? -0.3333333432674408f : c == 2 ? 0.3333333432674408f : 1.0f;
}
__device__ __forceinline__ __half level2_f16(int c) {
    const unsigned short bits = c == 0 ? 0xBC00u : c == 1 ? 0xB555u : c == 2 ? 0x3555u : 0x3C00u;
    return __ushort_as_half(bits);
}
__device__ __forceinline__ float level2_bf16(int c) {  // bf16 value held in a float
    const unsigned int bits = c == 0 ? 0xBF800000u : c == 1 ? 0xBEAB0000u : c == 2 ? 0x3EAB0000u : 0x3F800000u;
    return __uint_as_float(bits);
}

template <int BITS, int DT>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ packed, long long ldp,
                                                      const __half* __restrict__ scales, long long lds,
                                                      int n, int korig, int group, void* __restrict__ out,
                                                      long long ldo) {
    constexpr int CPB = 8 / BITS;
    const int bytes_per_row = (korig + CPB - 1) / CPB;
    const long long total = (long long)n * bytes_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int row = (int)(i / bytes_per_row), b = (int)(i - (long long)row * bytes_per_row);
        const uint32_t byte = packed[(size_t)row * ldp + b];
        const int kbase = b * CPB;
        const __half s16 = scales[(size_t)row * lds + kbase / group];   // a byte never straddles a group
#pragma unroll
        for (int j = 0; j < CPB; ++j) {
            const int k = kbase + j;
            if (k >= korig) break;
            const int c = (byte >> (BITS * j)) & ((1 << BITS) - 1);
            const size_t o = (size_t)row * ldo + k;
            if constexpr (DT == QGEMV_F32) {
                const float lv = BITS == 2 ? level2_f32(c) : float(c - 8);
                static_cast<float*>(out)[o] = __fmul_rn(lv, __half2float(s16));
            } else if constexpr (DT == QGEMV_F16) {
                const __half lv = BITS == 2 ? level2_f16(c) : __int2half_rn(c - 8);
                static_cast<__half*>(out)[o] = __float2half_rn(__fmul_rn(__half2float(lv), __half2float(s16)));
            } else {
                const float lv = BITS == 2 ? level2_bf16(c) : float(c - 8);
                const float sb = __bfloat162float(__float2bfloat16_rn(__half2float(s16)));
                static_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(__fmul_rn(lv, sb));
            }
        }
    }
}

// One element, rounded exactly as the scalar kernel above does.
template <int BITS, int DT>
__device__ __forceinline__ auto dequant_one(int c, __half s16) {
    if constexpr (DT == QGEMV_F32) {
        const float lv = BITS == 2 ? level2_f32(c) : float(c - 8);
        return __fmul_rn(lv, __half2float(s16));
    } else if constexpr (DT == QGEMV_F16) {
        const __half lv = BITS == 2 ? level2_f16(c) : __int2half_rn(c - 8);
        return __float2half_rn(__fmul_rn(__half2float(lv), __half2float(s16)));
    } else {
        const float lv = BITS == 2 ? level2_bf16(c) : float(c - 8);
        const float sb = __bfloat162float(__float2bfloat16_rn(__half2float(s16)));
        return __float2bfloat16_rn(__fmul_rn(lv, sb));
    }
}

// Vector path: a thread turns one aligned 32-bit word of codes (8 INT4 or 16 INT2 weights) into 16-byte
// stores; consecutive threads take consecutive words, so loads and stores are fully coalesced.
// Needs 4-byte aligned packed rows, 16-byte aligned output rows, and K and the group size multiples of
// the weights per word (a word then never straddles a group or the end of a row).
template <int BITS, int DT>
__global__ void __launch_bounds__(256) dequant_vec_kernel(const uint8_t* __restrict__ packed, long long ldp,
                                                          const __half* __restrict__ scales, long long lds,
                                                          int n, int korig, int group, void* __restrict__ out,
                                                          long long ldo) {
    constexpr int WPW = 32 / BITS;                                    // weights per word
    using OT = std::conditional_t<DT == QGEMV_F32, float, std::conditional_t<DT == QGEMV_F16, __half, __nv_bfloat16>>;
    constexpr int VEC = 16 / (int)sizeof(OT);                         // elements per 16-byte store
    const int words_per_row = korig / WPW;
    const long long total = (long long)n * words_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int row = (int)(i / words_per_row), wi = (int)(i - (long long)row * words_per_row);
        const uint32_t word = *reinterpret_cast<const uint32_t*>(packed + (size_t)row * ldp + (size_t)wi * 4);
        const int kbase = wi * WPW;
        const __half s16 = scales[(size_t)row * lds + kbase / group];
        OT* o = static_cast<OT*>(out) + (size_t)row * ldo + kbase;
#pragma unroll
        for (int v = 0; v < WPW / VEC; ++v) {
            __align__(16) OT vals[VEC];
#pragma unroll
            for (int j = 0; j < VEC; ++j)
                vals[j] = dequant_one<BITS, DT>((int)((word >> (BITS * (v * VEC + j))) & ((1u << BITS) - 1u)), s16);
            *reinterpret_cast<uint4*>(o + v * VEC) = *reinterpret_cast<const uint4*>(vals);
        }
    }
}

template <int BITS>
__global__ void __launch_bounds__(256) unpack_codes_kernel(const uint8_t* __restrict__ packed, long long ldp,
                                                           int n, int kpad, uint8_t* __restrict__ codes,
                                                           long long ldc) {
    constexpr int CPB = 8 / BITS;
    const int bytes_per_row = kpad / CPB;
    const long long total = (long long)n * bytes_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int row = (int)(i / bytes_per_row), b = (int)(i - (long long)row * bytes_per_row);
        const uint32_t byte = packed[(size_t)row * ldp + b];
        uint8_t* o = codes + (size_t)row * ldc + (size_t)b * CPB;
#pragma unroll
        for (int j = 0; j < CPB; ++j) o[j] = (uint8_t)((byte >> (BITS * j)) & ((1 << BITS) - 1));
    }
}

inline int grid_for(long long total) {
    long long blocks = (total + 255) / 256;
    const long long cap = 148LL * 16;
    return (int)(blocks < 1 ? 1 : blocks > cap ? cap : blocks);
}

}  // namespace
}  // namespace qgemv

using namespace qgemv;

extern "C" int qdequant(int bits, const uint8_t* packed, int64_t ldp, const void* scales, int64_t lds,
                        int n, int k_padded, int k_original, int group,
                        void* out, int64_t ld_out, int out_dtype, void* stream) {
    if (!packed || !scales || !out || n <= 0 || k_padded <= 0 || k_original <= 0 || k_original > k_padded) {
        set_error("qdequant: null pointer or non-positive size");
        return QGEMV_ERR_BAD_ARG;
    }
    if ((bits != 2 && bits != 4) || out_dtype < QGEMV_F16 || out_dtype > QGEMV_F32) {
        set_error("qdequant: bits must be 2 or 4 and out_dtype f16/bf16/f32");
        return QGEMV_ERR_BAD_ARG;
    }
    if (group <= 0 || group % (8 / bits) || k_padded % group || ldp < (int64_t)k_padded * bits / 8 ||
        lds < k_padded / group || ld_out < k_original) {
        set_error("qdequant: inconsistent group / padded K / leading dimensions");
        return QGEMV_ERR_SHAPE;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int cpb = 8 / bits, wpw = 32 / bits;
    const size_t esize = out_dtype == QGEMV_F32 ? 4 : 2;
    const bool vec = reinterpret_cast<uintptr_t>(packed) % 4 == 0 && ldp % 4 == 0 && k_original % wpw == 0 && group % wpw == 0 &&
                     reinterpret_cast<uintptr_t>(out) % 16 == 0 && (ld_out * esize) % 16 == 0;
    const long long total = vec ? (long long)n * (k_original / wpw) : (long long)n * ((k_original + cpb - 1) / cpb);
    const int grid = grid_for(total);
    const __half* sc = static_cast<const __half*>(scales);
#define QD_LAUNCH(B, D)                                                                                              \
    do {                                                                                                             \
        if (vec) dequant_vec_kernel<B, D><<<grid, 256, 0, s>>>(packed, ldp, sc, lds, n, k_original, group, out, ld_out); \
        else dequant_kernel<B, D><<<grid, 256, 0, s>>>(packed, ldp, sc, lds, n, k_original, group, out, ld_out);     \
    } while (0)
    if (bits == 2) {
        if (out_dtype == QGEMV_F32) QD_LAUNCH(2, QGEMV_F32);
        else if (out_dtype == QGEMV_F16) QD_LAUNCH(2, QGEMV_F16);
        else QD_LAUNCH(2, QGEMV_BF16);
    } else {
        if (out_dtype == QGEMV_F32) QD_LAUNCH(4, QGEMV_F32);
        else if (out_dtype == QGEMV_F16) QD_LAUNCH(4, QGEMV_F16);
        else QD_LAUNCH(4, QGEMV_BF16);
    }
#undef QD_LAUNCH
    return check_launch("dequant_kernel");
}

extern "C" int qunpack_codes(int bits, const uint8_t* packed, int64_t ldp, int n, int k_padded,
                             uint8_t* codes, int64_t ld_codes, void* stream) {
    if (!packed || !codes || n <= 0 || k_padded <= 0 || (bits != 2 && bits != 4)) {
        set_error("qunpack_codes: null pointer, non-positive size or bits not 2/4");
        return QGEMV_ERR_BAD_ARG;
    }
    if (k_padded % (8 / bits) || ldp < (int64_t)k_padded * bits / 8 || ld_codes < k_padded) {
        set_error("qunpack_codes: inconsistent padded K / leading dimensions");
        return QGEMV_ERR_SHAPE;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int grid = grid_for((long long)n * (k_padded / (8 / bits)));
    if (bits == 2) unpack_codes_kernel<2><<<grid, 256, 0, s>>>(packed, ldp, n, k_padded, codes, ld_codes);
    else           unpack_codes_kernel<4><<<grid, 256, 0, s>>>(packed, ldp, n, k_padded, codes, ld_codes);
    return check_launch("unpack_codes_kernel");
}
