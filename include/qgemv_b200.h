/* qgemv_b200 -- C ABI of the B200 (sm_100a) packed groupwise INT2 / INT4 small-M GEMV library.
 *
 * Plain pointers and sizes only: no torch types, no C++ in the signatures.  Every pointer is
 * a CUDA device pointer unless stated otherwise; the caller owns every buffer, including the
 * output and the workspace.  No function here synchronises the device, allocates device
 * memory or aborts; each returns QGEMV_OK (0) or a negative QGEMV_ERR_* code, and
 * qgemv_error_string() describes the most recent failure on the calling thread.
 *
 * Each entry point names the interface of the reference project (ai_accel_lab v5.0.0) that it
 * stands in for, as path:line inside that project.
 */
#ifndef QGEMV_B200_H
#define QGEMV_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QGEMV_ABI_VERSION 1

enum qgemv_status {
    QGEMV_OK = 0,
    QGEMV_ERR_BAD_ARG = -1,      /* null pointer, non-positive size, M outside 1..QGEMV_MAX_M, bad enum */
    QGEMV_ERR_SHAPE = -2,        /* Kpad not a multiple of the group, group not a multiple of the codes per byte, ... */
    QGEMV_ERR_ALIGN = -3,        /* a pointer or leading dimension violates the documented alignment */
    QGEMV_ERR_WORKSPACE = -4,    /* workspace missing or smaller than qgemv_workspace_bytes() */
    QGEMV_ERR_LAUNCH = -5,       /* the CUDA runtime refused the launch (see qgemv_error_string) */
    QGEMV_ERR_TOO_LARGE = -6     /* a size exceeds a stated fixed limit */
};

enum qgemv_act { QGEMV_ACT_NONE = 0, QGEMV_ACT_RELU = 1, QGEMV_ACT_SILU = 2 };
enum qgemv_dtype { QGEMV_F16 = 0, QGEMV_BF16 = 1, QGEMV_F32 = 2 };

/* Which kernel family a call may use.  AUTO picks the tensor-core-assisted streaming kernel
 * when the shape allows it and the CUDA-core kernel otherwise; the other two force a family
 * (used by the tests and by the profiles that justify the choice). */
enum qgemv_kernel { QGEMV_KERNEL_AUTO = 0, QGEMV_KERNEL_SIMT = 1, QGEMV_KERNEL_MMA = 2 };

#define QGEMV_MAX_M 4

/* One fused GEMV:  y[m, n] = act( sum_k x[m,k] * level(code[n,k]) * scale[n, k/group]
 *                               + sum_j x[m, outlier_idx[j]] * outlier_w[n, j]
 *                               + sum_r res_u[n, r] * (sum_k res_v[r, k] * x[m, k])
 *                               + bias[n] )
 * level(c) = (-1, -1/3, 1/3, 1)[c] for bits == 2 and c - 8 for bits == 4.
 *
 * Layouts (all row-major, leading dimensions in ELEMENTS of the tensor's own type):
 *   x          fp16 or bf16 [M, Kpad]     ldx >= Kpad, inner stride 1 (rows may be strided views)
 *   packed     uint8 [N, Kpad*bits/8]     bits == 2: byte b = c(4b) | c(4b+1)<<2 | c(4b+2)<<4 | c(4b+3)<<6
 *                                         bits == 4: byte b = c(2b) | c(2b+1)<<4
 *   scales     fp16 [N, Kpad/group]
 *   bias       fp16 [N] or NULL
 *   outlier_idx int32 [oc] (values < Korig), outlier_w fp16 [N, oc]; oc may be any count >= 0
 *   res_u      fp16 [N, rank], res_v fp16 [rank, Korig]; rank may be 0
 *   y          fp16 or bf16 (same type as x) [M, N]
 *   The weight-side tensors (packed, scales, bias, outlier_*, res_*) must already be final when
 *   the call is issued: the kernel may start reading them before the preceding kernel of the
 *   stream has finished (it waits for that kernel only before it reads x).
 *   workspace  zero-initialised ONCE by the caller, at least qgemv_workspace_bytes() bytes,
 *              256-byte aligned, private to calls that may overlap on the device.  The
 *              kernels leave it ready for the next call (no memset between calls).
 */
typedef struct qgemv_problem {
    int32_t bits;            /* 2 or 4 */
    int32_t m, n;            /* 1 <= m <= QGEMV_MAX_M */
    int32_t k_padded;        /* multiple of group */
    int32_t k_original;      /* <= k_padded; outlier_idx and res_v refer to this range */
    int32_t group;           /* multiple of 4 (bits 2) or 2 (bits 4) */
    int32_t act;             /* enum qgemv_act */
    int32_t x_dtype;         /* QGEMV_F16 or QGEMV_BF16; y has the same type */
    int32_t outliers;        /* oc */
    int32_t rank;            /* residual rank, <= 64 */
    int32_t kernel;          /* enum qgemv_kernel */
    int32_t reserved;
    const void* x;           int64_t ldx;
    const uint8_t* packed;   int64_t ldp;    /* bytes per packed row */
    const void* scales;      int64_t lds;
    const void* bias;
    const int32_t* outlier_idx;
    const void* outlier_w;   int64_t ldow;
    const void* res_u;       int64_t ldu;
    const void* res_v;       int64_t ldv;
    void* y;                 int64_t ldy;
    void* workspace;         size_t workspace_bytes;
} qgemv_problem;

/* Fused small-M GEMV on `stream` (a cudaStream_t).  Capturable in a CUDA graph.
 * Replaces: decode_int2_linear  ai_accel_lab/kernels/decode_int2.py:99-144 (kernel :43-96),
 *           decode_int4_linear  ai_accel_lab/kernels/groupwise_int4.py:110-127 (kernel :85-107),
 *           plus the two residual F.linear launches of ai_accel_lab/optimize/hybrid_int2.py:104-106
 *           and, with group == Kpad, int2_linear of csrc/packed_kernels.cpp:19-23
 *           (packed_dense_kernel<0>, csrc/packed_kernels_cuda.cu:27-83). */
int qgemv_run(const qgemv_problem* p, void* stream);

/* The same fused GEMV for callers that may not allocate device memory (code running under a
 * memory budget fixed at start-up, inside somebody else's allocator-free plugin hook, or in a
 * process whose only device buffers are the ones handed to it): p->workspace and
 * p->workspace_bytes are ignored and a scratch area built into the library is used instead.
 * It has no counterpart in the reference project.
 *
 *  - The scratch is a fixed 328 704-byte array in device memory that every GPU which loads the
 *    library carries until the process exits.  It serves problems with N <= QGEMV_STATIC_MAX_N
 *    and rank <= 64; anything larger is refused with QGEMV_ERR_TOO_LARGE.
 *  - The first call on each device (with that device current) looks up the array's device address
 *    and clears its counters on `stream`; make that first call before starting a stream capture.
 *    Later calls only launch kernels.  No call allocates or frees anything.
 *  - All calls on a device share the one array, and it keeps what the last call left in it.
 *    Calls that can overlap on the GPU (different streams without ordering) would race on it:
 *    serialise them, or use qgemv_run with separate workspaces. */
#define QGEMV_STATIC_MAX_N 262128
int qgemv_run_static(const qgemv_problem* p, void* stream);

/* Bytes of workspace qgemv_run needs for a problem of this shape (never 0; at most a few MB). */
size_t qgemv_workspace_bytes(int bits, int m, int n, int k_padded, int group, int rank);

/* Name of the kernel variant qgemv_run would launch for `p` (static string, host memory), or
 * NULL if the problem is invalid.  No launch happens. */
const char* qgemv_plan_name(const qgemv_problem* p);

/* Number of kernel launches qgemv_run would issue for `p` (1 or 2: the general kernel and a few
 * shapes of the fast one compute the residual projections in a small kernel of their own), or a
 * negative QGEMV_ERR_* if the problem is invalid.  No launch happens. */
int qgemv_plan_launches(const qgemv_problem* p);

/* Dequantise to a dense [N, Korig] matrix of out_dtype (QGEMV_F16 / BF16 / F32), bit-identical to
 * the reference's torch expression `levels.to(dtype)[codes] * scales.to(dtype)[:, k // group]`.
 * Replaces: unpack_groupwise_int2  ai_accel_lab/kernels/groupwise_int2.py:122-130,
 *           unpack_groupwise_int4  ai_accel_lab/kernels/groupwise_int4.py:63-69. */
int qdequant(int bits, const uint8_t* packed, int64_t ldp, const void* scales, int64_t lds,
             int n, int k_padded, int k_original, int group,
             void* out, int64_t ld_out, int out_dtype, void* stream);

/* Expand packed bytes to one uint8 code per weight, [N, Kpad].
 * Replaces the code extraction of ai_accel_lab/kernels/groupwise_int2.py:123-124 and
 * ai_accel_lab/kernels/groupwise_int4.py:64-65. */
int qunpack_codes(int bits, const uint8_t* packed, int64_t ldp, int n, int k_padded,
                  uint8_t* codes, int64_t ld_codes, void* stream);

/* Description of the last error raised on the calling host thread (host memory, never NULL). */
const char* qgemv_error_string(void);

/* QGEMV_ABI_VERSION the library was built with. */
int qgemv_abi_version(void);

/* sizeof(qgemv_problem) as the library sees it, for bindings to cross-check their layout. */
size_t qgemv_sizeof_problem(void);

#ifdef __cplusplus
}
#endif
#endif /* QGEMV_B200_H */
