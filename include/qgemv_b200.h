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

#define QGEMV_ABI_VERSION 4

enum qgemv_status {
    QGEMV_OK = 0,
    QGEMV_ERR_BAD_ARG = -1,      /* null pointer, non-positive size, M outside 1..QGEMV_MAX_M, bad enum */
    QGEMV_ERR_SHAPE = -2,        /* Kpad not a multiple of the group, group not a multiple of the codes per byte, ... */
    QGEMV_ERR_ALIGN = -3,        /* a pointer or leading dimension violates the documented alignment */
    QGEMV_ERR_WORKSPACE = -4,    /* workspace missing or smaller than qgemv_workspace_bytes() */
    QGEMV_ERR_LAUNCH = -5,       /* the CUDA runtime refused the launch (see qgemv_error_string) */
    QGEMV_ERR_TOO_LARGE = -6     /* a size exceeds a stated fixed limit */
};

/* SILU_MUL fuses the gated product of a feed-forward block (act_fn(gate_proj(x)) * up_proj(x)) into the
 * epilogue of ONE launch over both projections.  The N weight rows (N a multiple of 16) come in blocks
 * of 16: 8 rows of the gate projection followed by the 8 matching rows of the up projection, and the
 * output is [M, N/2]:
 *     y[m, 8b + j] = r( r(silu(r(v[m, 16b + j]))) * r(v[m, 16b + 8 + j]) )
 * with v the result before activation (bias included) and r() rounding to the activation type -- the
 * roundings a 16-bit framework makes when it runs the two projections, the activation and the product
 * as separate operators.  ldy >= N/2.  Tensor-core kernels only (QGEMV_ERR_SHAPE where the shape needs
 * the CUDA-core kernel).  No counterpart in the reference, which launches the three operators apart. */
enum qgemv_act { QGEMV_ACT_NONE = 0, QGEMV_ACT_RELU = 1, QGEMV_ACT_SILU = 2, QGEMV_ACT_SILU_MUL = 3 };
enum qgemv_dtype { QGEMV_F16 = 0, QGEMV_BF16 = 1, QGEMV_F32 = 2 };

/* Which kernel a call may use.  AUTO picks the tensor-core-assisted streaming kernel (persistent
 * grid, runs of a tile dealt over all CTAs, one CTA barrier between the streaming phase and the
 * tile phase) when the shape allows it and the CUDA-core kernel otherwise; SIMT and MMA force one
 * of the two.  MMA_PIPE asks for the barrier-free variant of the tensor-core kernel (whole 16-row
 * tiles per CTA, per-tile arrival counters instead of the CTA barrier); it is measured slower than
 * MMA on the benchmark shapes (13.7 against 10.4 us on the headline one) and is kept for A/B
 * measurements and as the base of further work; AUTO takes it only for M = 1 with rows of 14 KB of
 * codes or more, the one case where it measured faster.  A forced kernel that the
 * shape does not allow returns QGEMV_ERR_SHAPE. */
enum qgemv_kernel { QGEMV_KERNEL_AUTO = 0, QGEMV_KERNEL_SIMT = 1, QGEMV_KERNEL_MMA = 2, QGEMV_KERNEL_MMA_PIPE = 3 };

#define QGEMV_MAX_M 4

/* qgemv_problem.debug bits.  DROP_PROJECTIONS makes the CTAs that compute the residual
 * projections of a launch keep them to themselves and shortens the readers' wait to a few
 * microseconds, so a test can watch the wait run out: the launch then finishes with an output
 * that lacks a valid residual term and raises the workspace's status word.  Nothing faults and
 * the workspace stays usable. */
#define QGEMV_DEBUG_DROP_PROJECTIONS 1
/* Tuning aids of the pipelined kernel (benchmarks only): do not announce the weights that follow
 * the ring to L2; smaller or larger ring slots; force the warps per CTA (1..32) or the ring depth per warp (2..4). */
#define QGEMV_DEBUG_NO_L2_HINT 2
#define QGEMV_DEBUG_CHUNK128 4   /* ring slots of 128 packed bytes per row instead of 256 */
#define QGEMV_DEBUG_LATE_TRIGGER 8    /* release the next launch after the x-dependent prologue instead of at kernel entry */
#define QGEMV_DEBUG_CHUNK256 32       /* ring slots of 256 packed bytes per row even where smaller ones would employ more warps */
#define QGEMV_DEBUG_SPLIT_FILL 64     /* before the dependency wait fill only the first ring slot; the rest follows the loads of x */
#define QGEMV_DEBUG_WARPS(n) (((n) & 0xff) << 8)
#define QGEMV_DEBUG_STAGES(n) (((n) & 0xf) << 16)

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
 *              256-byte aligned, private to calls that may overlap on the device (calls on
 *              different streams without ordering need a workspace each).  The kernels leave it
 *              ready for the next call, so no memset is needed between calls: every arrival
 *              counter is back at zero, while three bookkeeping words near the end of the counter
 *              area keep their values on purpose -- the number of launches completed so far (the
 *              tag of the residual projections that CTAs of one launch pass to each other), the
 *              count of CTAs that have finished the current launch (zero between calls) and the
 *              sticky status word that qgemv_workspace_status() reads.
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
    int32_t debug;           /* 0 in production; QGEMV_DEBUG_* bits for the library's own tests */
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
    /* Optional hint: a byte range (16-byte aligned device memory, read-only while the call runs) that
     * the kernel announces to L2 while it works -- typically the packed codes of the GEMV that follows
     * in the stream, which then streams from L2 instead of DRAM.  Weights are static, so the hint can
     * never be wrong, only useless.  NULL / 0: none.  Kernels that cannot use it ignore it. */
    const void* prefetch;    size_t prefetch_bytes;
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

/* Every wait inside the kernels is bounded.  The only one is for the residual projections
 * t = res_v . x that a few CTAs of a launch compute for all the others: a reader that does not see
 * them within its limit (about 30 ms) goes on with whatever value it has and sets the sticky status
 * word of the workspace to 1, so the launch ends and the context stays healthy, but that launch's
 * output is not to be trusted.  This call enqueues, on `stream`, a 4-byte copy of the status word
 * into *host_out (host memory; pinned if the copy is to be asynchronous) followed by a reset of
 * the word to 0.  Synchronise the stream before reading *host_out: 0 = every launch since the
 * last query completed normally, 1 = a wait for residual projections ran out, 2 = a wait for an
 * asynchronous weight copy ran out (never seen; it would mean a lost copy).  `workspace` is the pointer given to qgemv_run, or NULL for the
 * built-in scratch of qgemv_run_static on the current device.  Not capturable in a CUDA graph.
 * It has no counterpart in the reference project (its kernels never wait on each other). */
int qgemv_workspace_status(const void* workspace, void* stream, int32_t* host_out);

/* Bytes of workspace qgemv_run needs for a problem of this shape (never 0; at most a few MB). */
size_t qgemv_workspace_bytes(int bits, int m, int n, int k_padded, int group, int rank);

/* Name of the kernel variant qgemv_run would launch for `p` (static string, host memory), or
 * NULL if the problem is invalid.  No launch happens. */
const char* qgemv_plan_name(const qgemv_problem* p);

/* Number of kernel launches qgemv_run would issue for `p` (1 or 2: the general kernel and a few
 * shapes of the fast one compute the residual projections in a small kernel of their own), or a
 * negative QGEMV_ERR_* if the problem is invalid.  No launch happens. */
int qgemv_plan_launches(const qgemv_problem* p);

/* What qgemv_run would do for `p`, for tests, benchmarks and capacity planning.  No launch happens.
 * Returns QGEMV_OK or a negative QGEMV_ERR_* if the problem is invalid. */
typedef struct qgemv_plan_info {
    int32_t family;          /* QGEMV_KERNEL_SIMT or QGEMV_KERNEL_MMA */
    int32_t variant;         /* MMA family: 1 = barrier-phased kernel, 2 = pipelined kernel; 0 otherwise */
    int32_t launches;        /* as qgemv_plan_launches */
    int32_t grid;            /* CTAs */
    int32_t warps;           /* warps per CTA */
    int32_t smem_bytes;      /* dynamic shared memory per CTA */
    int32_t tile_aligned;    /* 1: every CTA owns whole 16-row tiles; 0: some tiles are shared between CTAs
                                and meet in the workspace (partial sums + arrival counters) */
    int32_t inline_projections;  /* 1: residual projections computed inside the fused kernel */
    int32_t ctas_per_sm;     /* CTAs of this kernel (or of this and the next launch) one SM can hold */
    int32_t stages;          /* MMA family: ring slots per warp */
    int32_t run_chunks;      /* MMA family: chunks (128 or 256 packed bytes per row) per run, the unit of work of a warp */
    int32_t runs_per_tile;
    int32_t epilogue_tiles;  /* pipelined kernel: tiles per CTA whose epilogue operands are prefetched */
    int32_t l2_chunks;       /* pipelined kernel: chunks per warp announced to L2 before the dependency wait */
    int32_t projection_parts;/* K parts of the in-kernel residual projections (0 when they are not inline) */
    int32_t chunk_bytes;     /* MMA family: packed bytes per row per ring slot */
} qgemv_plan_info;
int qgemv_plan_describe(const qgemv_problem* p, qgemv_plan_info* out);

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
