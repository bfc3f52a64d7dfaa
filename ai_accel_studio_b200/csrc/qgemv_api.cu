// C ABI entry points: argument validation, kernel selection, launch.  See include/qgemv_b200.h.
#include <cstdarg>
#include <cstdio>

#include "qgemv_common.cuh"

namespace qgemv {

static thread_local char g_error[512] = "no error";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int check_launch(const char* what) {
    const cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        // Clear the (non-sticky) launch error so that the next call starts clean.
        (void)cudaGetLastError();
        set_error("%s: %s", what, cudaGetErrorString(e));
        return QGEMV_ERR_LAUNCH;
    }
    return QGEMV_OK;
}

namespace {

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Largest load unit (bytes) the CUDA-core kernel may use for this problem.
int simt_unit_bytes(const qgemv_problem& p) {
    const int cpb = 8 / p.bits;
    if (aligned(p.packed, 16) && p.ldp % 16 == 0 && p.group % (16 * cpb) == 0) return 16;
    if (aligned(p.packed, 4) && p.ldp % 4 == 0 && p.group % (4 * cpb) == 0) return 4;
    return 1;
}

int validate(const qgemv_problem* p, size_t need) {
    if (!p) { set_error("qgemv_run: problem is NULL"); return QGEMV_ERR_BAD_ARG; }
    if (p->bits != 2 && p->bits != 4) { set_error("qgemv_run: bits must be 2 or 4 (got %d)", p->bits); return QGEMV_ERR_BAD_ARG; }
    if (p->m < 1 || p->m > QGEMV_MAX_M) { set_error("qgemv_run: M must be 1..%d (got %d); larger batches use the dequantise + GEMM path", QGEMV_MAX_M, p->m); return QGEMV_ERR_BAD_ARG; }
    if (p->n < 1 || p->k_padded < 1 || p->k_original < 1 || p->k_original > p->k_padded) { set_error("qgemv_run: bad N / K (n=%d, k_padded=%d, k_original=%d)", p->n, p->k_padded, p->k_original); return QGEMV_ERR_BAD_ARG; }
    if (!p->x || !p->packed || !p->scales || !p->y) { set_error("qgemv_run: x, packed, scales and y must be non-null"); return QGEMV_ERR_BAD_ARG; }
    if (p->act < QGEMV_ACT_NONE || p->act > QGEMV_ACT_SILU_MUL) { set_error("qgemv_run: unknown activation %d", p->act); return QGEMV_ERR_BAD_ARG; }
    if (p->x_dtype != QGEMV_F16 && p->x_dtype != QGEMV_BF16) { set_error("qgemv_run: activations must be fp16 or bf16"); return QGEMV_ERR_BAD_ARG; }
    if (p->kernel < QGEMV_KERNEL_AUTO || p->kernel > QGEMV_KERNEL_MMA_PIPE) { set_error("qgemv_run: unknown kernel selector %d", p->kernel); return QGEMV_ERR_BAD_ARG; }
    if (p->outliers < 0 || (p->outliers > 0 && (!p->outlier_idx || !p->outlier_w))) { set_error("qgemv_run: outliers=%d needs outlier_idx and outlier_w", p->outliers); return QGEMV_ERR_BAD_ARG; }
    if (p->rank < 0 || (p->rank > 0 && (!p->res_u || !p->res_v))) { set_error("qgemv_run: rank=%d needs res_u and res_v", p->rank); return QGEMV_ERR_BAD_ARG; }
    if (p->rank > kMaxRank) { set_error("qgemv_run: residual rank %d exceeds the limit of %d", p->rank, kMaxRank); return QGEMV_ERR_TOO_LARGE; }
    const int cpb = 8 / p->bits;
    if (p->group < cpb || p->group % cpb || p->k_padded % p->group) { set_error("qgemv_run: group=%d must be a multiple of %d and divide k_padded=%d", p->group, cpb, p->k_padded); return QGEMV_ERR_SHAPE; }
    if (p->act == QGEMV_ACT_SILU_MUL && p->n % 16) { set_error("qgemv_run: the gated-pair activation needs N to be a multiple of 16 (got %d)", p->n); return QGEMV_ERR_SHAPE; }
    if (p->ldx < p->k_padded || p->ldy < (p->act == QGEMV_ACT_SILU_MUL ? p->n / 2 : p->n) || p->ldp < (int64_t)p->k_padded / cpb || p->lds < p->k_padded / p->group) { set_error("qgemv_run: a leading dimension is smaller than its row"); return QGEMV_ERR_SHAPE; }
    if (p->outliers > 0 && p->ldow < p->outliers) { set_error("qgemv_run: ldow < outliers"); return QGEMV_ERR_SHAPE; }
    if (p->rank > 0 && (p->ldu < p->rank || p->ldv < p->k_original)) { set_error("qgemv_run: ldu < rank or ldv < k_original"); return QGEMV_ERR_SHAPE; }
    if (!aligned(p->x, 2) || !aligned(p->y, 2) || !aligned(p->scales, 2)) { set_error("qgemv_run: 16-bit tensors must be 2-byte aligned"); return QGEMV_ERR_ALIGN; }
    if (!p->workspace || p->workspace_bytes < need) { set_error("qgemv_run: workspace of %zu bytes required (got %zu)", need, p->workspace ? p->workspace_bytes : (size_t)0); return QGEMV_ERR_WORKSPACE; }
    if (!aligned(p->workspace, 256)) { set_error("qgemv_run: workspace must be 256-byte aligned"); return QGEMV_ERR_ALIGN; }
    return QGEMV_OK;
}

Args make_args(const qgemv_problem& p, size_t partial_floats) {
    Args a{};
    a.x = p.x; a.ldx = p.ldx;
    a.packed = p.packed; a.ldp = p.ldp;
    a.scales = static_cast<const __half*>(p.scales); a.lds = p.lds;
    a.bias = static_cast<const __half*>(p.bias);
    a.oidx = p.outlier_idx;
    a.ow = static_cast<const __half*>(p.outlier_w); a.ldow = p.ldow;
    a.ru = static_cast<const __half*>(p.res_u); a.ldu = p.ldu;
    a.rv = static_cast<const __half*>(p.res_v); a.ldv = p.ldv;
    a.y = p.y; a.ldy = p.ldy;
    char* ws = static_cast<char*>(p.workspace);
    a.t = reinterpret_cast<float*>(ws + kWsTOff);
    a.counters = reinterpret_cast<int*>(ws + kWsCounterOff);
    a.partial = reinterpret_cast<float*>(ws + kWsPartialOff);
    a.tparts = a.partial + (partial_floats - kTPartFloats);
    a.m = p.m; a.n = p.n; a.kpad = p.k_padded; a.korig = p.k_original; a.group = p.group;
    a.act = p.act; a.oc = p.outliers; a.rank = p.rank;
    a.splits = 1; a.kspan = p.k_padded;
    if (p.prefetch && p.prefetch_bytes >= 16 && reinterpret_cast<uintptr_t>(p.prefetch) % 16 == 0) {
        a.hint = static_cast<const unsigned char*>(p.prefetch);
        // at most 48 MB: two launches' worth of hints must sit in the 126 MB L2 beside what is being streamed
        const size_t cap = (size_t)48 << 20;
        a.hint_bytes = (long long)((p.prefetch_bytes < cap ? p.prefetch_bytes : cap) & ~(size_t)15);
    }
    return a;
}

}  // namespace
}  // namespace qgemv

using namespace qgemv;

extern "C" int qgemv_abi_version(void) { return QGEMV_ABI_VERSION; }

extern "C" const char* qgemv_error_string(void) { return g_error; }

extern "C" size_t qgemv_sizeof_problem(void) { return sizeof(qgemv_problem); }

extern "C" size_t qgemv_workspace_bytes(int bits, int m, int n, int k_padded, int group, int rank) {
    (void)bits; (void)m; (void)n; (void)k_padded; (void)group; (void)rank;
    // Shape independent: residual projections + counters + kMaxPartialFloats split-K partials.
    // The planner never picks a split count whose partial sums would not fit.
    return kWsPartialOff + kMaxPartialFloats * sizeof(float);
}

namespace {

// The kernel a valid problem gets: the phased tensor-core kernel, its barrier-free variant when the
// caller asks for it, or (ok == false) the CUDA-core kernel.  `forced_missing` is set when the caller
// forced a tensor-core kernel and the shape does not allow it.
MmaPlan choose(const qgemv_problem& p, size_t partial_floats, bool* forced_missing) {
    MmaPlan plan{};
    *forced_missing = false;
    const bool needs_mma = p.act == QGEMV_ACT_SILU_MUL;      // the gated-pair epilogue exists in the tensor-core kernels only
    if (p.kernel == QGEMV_KERNEL_SIMT) { *forced_missing = needs_mma; return plan; }
    plan = plan_mma(p, partial_floats);
    if (!plan.ok) {
        *forced_missing = needs_mma || p.kernel == QGEMV_KERNEL_MMA || p.kernel == QGEMV_KERNEL_MMA_PIPE;
        return plan;
    }
    if (p.kernel == QGEMV_KERNEL_MMA_PIPE) {
        const MmaPlan pipe = plan_pipe(p, plan);
        if (!pipe.ok) *forced_missing = true;
        return pipe;
    }
    // Very long rows (14 KB of codes and more, e.g. INT4 with K = 28672) are the one measured case where the
    // barrier-free variant wins (35.1 against 41.7 us on 8192 x 28672 INT4, M = 1; at half that row length it
    // loses again, 14.6 against 11.4 us).  Beside 57 KB of staged activations the phased kernel has room for 12 of
    // its 16 warp rings, the barrier-free one (no run slots, smaller tables) keeps all 16.
    if (p.kernel == QGEMV_KERNEL_AUTO && p.m == 1 && (long long)p.k_padded * p.bits / 8 >= 14336) {
        const MmaPlan pipe = plan_pipe(p, plan);
        if (pipe.ok) return pipe;
    }
    return plan;
}

}  // namespace

extern "C" const char* qgemv_plan_name(const qgemv_problem* p) {
    if (validate(p, qgemv_workspace_bytes(0, 0, 0, 0, 0, 0)) != QGEMV_OK) return nullptr;
    bool missing = false;
    const MmaPlan plan = choose(*p, kMaxPartialFloats, &missing);
    if (plan.ok) return plan.name;
    if (missing) return nullptr;
    return simt_name(p->bits, p->m, simt_unit_bytes(*p));
}

namespace {

// Validate, pick a kernel, launch.  `partial_floats` is the capacity of the partial-sum area of
// the workspace the problem points at.
int run_checked(const qgemv_problem* p, void* stream, size_t need_bytes, size_t partial_floats) {
    const int v = validate(p, need_bytes);
    if (v != QGEMV_OK) return v;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    Args a = make_args(*p, partial_floats);
    const bool bf16 = p->x_dtype == QGEMV_BF16;

    bool missing = false;
    const MmaPlan plan = choose(*p, partial_floats, &missing);
    const bool use_mma = plan.ok;
    {
        if (missing) {
            set_error("qgemv_run: the tensor-core-assisted kernel does not support this shape "
                      "(needs 16-byte aligned x and packed rows, group in {32,64,128} for INT4 or {64,128,256} for INT2, "
                      "at most 256 outlier columns, and M * k_padded small enough for shared memory)");
            return QGEMV_ERR_SHAPE;
        }
    }
    if (a.rank > 0 && !(use_mma && plan.t_inline)) {
        const int r = launch_residual_t(a, bf16, s);
        if (r != QGEMV_OK) return r;
    }
    if (use_mma && plan.variant == 2) return launch_pipe(a, p->bits, bf16, plan, p->debug, s);
    if (use_mma) return launch_mma(a, p->bits, bf16, plan, p->debug, s);
    return launch_simt(a, p->bits, bf16, simt_unit_bytes(*p), s);
}

// ---- scratch for callers that cannot allocate ---------------------------------------------------
// Same layout as a caller-provided workspace, with a smaller partial-sum area: enough for a
// persistent grid of up to 256 CTAs (a B200 has 148 SMs).  Lives in every device that loads the
// library until the process exits; zero-initialised when the module is loaded.
constexpr size_t kStaticPartialFloats = 65536;
constexpr size_t kStaticScratchBytes = kWsPartialOff + kStaticPartialFloats * sizeof(float);   // 328 704 bytes
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void* g_static_scratch_addr[kMaxDevices] = {nullptr};

}  // namespace

extern "C" int qgemv_run_static(const qgemv_problem* p, void* stream) {
    if (!p) { set_error("qgemv_run_static: problem is NULL"); return QGEMV_ERR_BAD_ARG; }
    if ((long long)p->n > (long long)QGEMV_STATIC_MAX_N) {
        set_error("qgemv_run_static: N = %d exceeds the built-in scratch's limit of %d rows; "
                  "use qgemv_run with a caller-provided workspace", p->n, QGEMV_STATIC_MAX_N);
        return QGEMV_ERR_TOO_LARGE;
    }
    if (p->rank > kMaxRank) {
        set_error("qgemv_run_static: residual rank %d exceeds the limit of %d", p->rank, kMaxRank);
        return QGEMV_ERR_TOO_LARGE;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        (void)cudaGetLastError();
        set_error("qgemv_run_static: no current CUDA device (or device ordinal >= %d)", kMaxDevices);
        return QGEMV_ERR_LAUNCH;
    }
    if (!g_static_scratch_addr[dev]) {
        // One-time set-up on this device: the symbol's name is only a host-side handle, the kernels
        // need its device address.  Also puts the arrival counters into their required state.
        void* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr) {
            (void)cudaGetLastError();
            set_error("qgemv_run_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return QGEMV_ERR_LAUNCH;
        }
        const cudaError_t m = cudaMemsetAsync(ptr, 0, kWsPartialOff, static_cast<cudaStream_t>(stream));
        if (m != cudaSuccess) {
            (void)cudaGetLastError();
            set_error("qgemv_run_static: clearing the scratch counters failed: %s", cudaGetErrorString(m));
            return QGEMV_ERR_LAUNCH;
        }
        g_static_scratch_addr[dev] = ptr;
    }
    qgemv_problem q = *p;
    q.workspace = g_static_scratch_addr[dev];
    q.workspace_bytes = kStaticScratchBytes;
    return run_checked(&q, stream, kStaticScratchBytes, kStaticPartialFloats);
}

extern "C" int qgemv_plan_describe(const qgemv_problem* p, qgemv_plan_info* out) {
    if (!out) { set_error("qgemv_plan_describe: out is NULL"); return QGEMV_ERR_BAD_ARG; }
    const int v = validate(p, qgemv_workspace_bytes(0, 0, 0, 0, 0, 0));
    if (v != QGEMV_OK) return v;
    bool missing = false;
    const MmaPlan plan = choose(*p, kMaxPartialFloats, &missing);
    if (missing) { set_error("qgemv_plan_describe: the tensor-core-assisted kernels do not support this shape"); return QGEMV_ERR_SHAPE; }
    *out = qgemv_plan_info{};
    const bool inline_t = plan.ok && plan.t_inline;
    out->launches = (p->rank > 0 && !inline_t) ? 2 : 1;
    if (plan.ok) {
        out->family = QGEMV_KERNEL_MMA;
        out->variant = plan.variant;
        out->grid = plan.grid;
        out->warps = plan.nw;
        out->smem_bytes = plan.smem_bytes;
        out->tile_aligned = plan.tile_aligned;
        out->inline_projections = inline_t ? 1 : 0;
        out->ctas_per_sm = (plan.variant == 2 && 2 * (plan.smem_bytes + 1024) <= 233472) ? 2 : 1;
        out->stages = plan.stages;
        out->run_chunks = plan.rlen;
        out->runs_per_tile = plan.rpt;
        out->epilogue_tiles = plan.variant == 2 ? plan.epi_tiles : 0;
        out->l2_chunks = plan.variant == 2 ? plan.l2_chunks : 0;
        out->projection_parts = inline_t ? plan.t_parts : 0;
        out->chunk_bytes = plan.variant == 2 ? plan.chunk : (plan.gb == 16 ? 128 : 256);
    } else {
        out->family = QGEMV_KERNEL_SIMT;
        out->tile_aligned = 1;
    }
    return QGEMV_OK;
}

extern "C" int qgemv_plan_launches(const qgemv_problem* p) {
    qgemv_plan_info info;
    const int v = qgemv_plan_describe(p, &info);
    return v != QGEMV_OK ? v : info.launches;
}

extern "C" int qgemv_workspace_status(const void* workspace, void* stream, int32_t* host_out) {
    if (!host_out) { set_error("qgemv_workspace_status: host_out is NULL"); return QGEMV_ERR_BAD_ARG; }
    const char* ws = static_cast<const char*>(workspace);
    if (!ws) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices || !g_static_scratch_addr[dev]) {
            (void)cudaGetLastError();
            *host_out = 0;                       // the built-in scratch has not been used on this device yet
            return QGEMV_OK;
        }
        ws = static_cast<const char*>(g_static_scratch_addr[dev]);
    }
    int* word = reinterpret_cast<int*>(const_cast<char*>(ws) + kWsCounterOff) + kWsStatusIdx;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(host_out, word, sizeof(int32_t), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaMemsetAsync(word, 0, sizeof(int32_t), s) != cudaSuccess)
        return check_launch("qgemv_workspace_status");
    return QGEMV_OK;
}

extern "C" int qgemv_run(const qgemv_problem* p, void* stream) {
    return run_checked(p, stream, qgemv_workspace_bytes(0, 0, 0, 0, 0, 0), kMaxPartialFloats);
}
