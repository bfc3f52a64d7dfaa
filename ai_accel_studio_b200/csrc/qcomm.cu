// One-shot all-reduce of small 16-bit vectors over peer memory (self-validating words), and the same
// collective fused with the residual update and RMS norm that follow it: see include/qcomm_b200.h.
#include <cstring>

#include "qgemv_common.cuh"
#include "../../include/qcomm_b200.h"

namespace qgemv {
namespace {

constexpr int kCommThreads = 512;                 // 8 elements (16 bytes) per thread
constexpr int kCommChunk = kCommThreads * 8;      // elements per CTA
constexpr int kDefaultWaitLimit = 1 << 23;        // probes of 64+ ns each: about a second

struct CommArgs {
    unsigned char* slots[QCOMM_MAX_RANKS];
    unsigned* flags[QCOMM_MAX_RANKS];
    unsigned* state;                               // [0] calls completed, [1] CTAs finished, [2] status
    void* data;
    int rank, world, max_elems, elems, wait_limit;
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
// 16-byte load that always goes to L2 (the slot was written by another GPU; never serve it from L1)
__device__ __forceinline__ uint4 ld_cg_u128(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned ld_relaxed_gpu(const unsigned* p) {
    unsigned v; asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}

// One-shot all-reduce, plain data + flags: every rank stores its vector into its slot of every rank's receive
// buffer, makes the stores visible system-wide, raises a flag per rank (release), waits for the others' flags
// (acquire, bounded) and adds the slots in rank order.  One polling thread per peer: the protocol of choice
// from 4 ranks up (70B-shape decode on 8 GPUs: 131 tok/s against 118 with the tagged words below).
template <bool BF16>
__global__ void __launch_bounds__(kCommThreads) qcomm_allreduce_flags_kernel(const CommArgs c) {
    using T = typename Act16<BF16>::T;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int tid = threadIdx.x, b = blockIdx.x;
    const int idx = (b * kCommThreads + tid) * 8;            // first element of this thread
    const bool live = idx < c.elems;
    asm volatile("griddepcontrol.wait;" ::: "memory");      // the producer of `data` has finished
    const unsigned call = ld_relaxed_gpu(c.state);           // calls completed so far: the same on every rank
    const unsigned half = call & 1u, tag = call + 1u;
    const size_t half_elems = (size_t)c.world * c.max_elems;

    // 1. my vector into my slot of every rank's receive buffer
    uint4 mine = make_uint4(0u, 0u, 0u, 0u);
    if (live) {
        mine = *reinterpret_cast<const uint4*>(static_cast<const T*>(c.data) + idx);
        for (int p = 0; p < c.world; ++p) {
            const int peer = (c.rank + p) % c.world;          // start with my own buffer, spread the rest
            T* dst = reinterpret_cast<T*>(c.slots[peer]) + half * half_elems + (size_t)c.rank * c.max_elems + idx;
            *reinterpret_cast<uint4*>(dst) = mine;
        }
    }
    __threadfence_system();                                  // my stores are visible system-wide before the flags
    __syncthreads();
    // 2. raise my flag for this CTA's chunk at every rank, then wait for everybody's flag here
    if (tid < c.world) {
        unsigned* f = c.flags[tid] + (half * c.world + c.rank) * QCOMM_MAX_BLOCKS + b;
        st_release_sys(f, tag);
    }
    if (tid < c.world) {
        const unsigned* f = c.flags[c.rank] + (half * c.world + tid) * QCOMM_MAX_BLOCKS + b;
        int probes = 0;
        while (ld_acquire_sys(f) != tag) {
            if (++probes > c.wait_limit) { atomicExch(c.state + 2, 1u); break; }
            __nanosleep(64);
        }
    }
    __syncthreads();
    // 3. add the slots in rank order: the same order, hence the same bits, on every rank
    if (live) {
        float acc[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] = 0.0f;
        const T* base = reinterpret_cast<const T*>(c.slots[c.rank]) + half * half_elems + idx;
        for (int r = 0; r < c.world; ++r) {
            const uint4 v = ld_cg_u128(base + (size_t)r * c.max_elems);
            const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[q] += Act16<BF16>::to_float(e[q]);
        }
        uint4 out;
        T* o = reinterpret_cast<T*>(&out);
#pragma unroll
        for (int q = 0; q < 8; ++q) o[q] = Act16<BF16>::from_float(acc[q]);
        *reinterpret_cast<uint4*>(static_cast<T*>(c.data) + idx) = out;
    }
    // 4. the last CTA of the launch advances the call counter (every CTA has read it by now)
    __syncthreads();
    if (tid == 0) {
        const unsigned old = atomicAdd(c.state + 1, 1u);
        if (old == gridDim.x - 1) {
            c.state[1] = 0u;
            __threadfence();
            c.state[0] = tag;
        }
    }
}


// Bytes of the plain receive area (used by the fused all-reduce + RMS norm kernel with its flags) and of the
// self-validating area behind it (used by qcomm_allreduce): [2 halves][world][max_elems / 2] words of 8 bytes,
// each {two 16-bit elements, 32-bit call tag}.
__host__ __device__ inline size_t plain_bytes(int world, int max_elems) { return (size_t)2 * world * max_elems * 2; }

__device__ __forceinline__ void st_relaxed_sys_v2(unsigned long long* p, unsigned long long a, unsigned long long b) {
    asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void ld_relaxed_sys_v2(const unsigned long long* p, unsigned long long& a, unsigned long long& b) {
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}

// One-shot all-reduce with self-validating words: every 8-byte word carries 4 bytes of data and the tag of
// the call, and an aligned 8-byte store arrives whole, so a receiver that sees the tag has the data -- no
// fence, no separate flag, no second trip over the link.  A thread owns 8 elements (4 words).
template <bool BF16>
__global__ void __launch_bounds__(kCommThreads) qcomm_allreduce_kernel(const CommArgs c) {
    using T = typename Act16<BF16>::T;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int tid = threadIdx.x, b = blockIdx.x;
    const int idx = (b * kCommThreads + tid) * 8;            // first element of this thread
    const bool live = idx < c.elems;
    asm volatile("griddepcontrol.wait;" ::: "memory");      // the producer of `data` has finished
    const unsigned call = ld_relaxed_gpu(c.state);           // calls completed so far: the same on every rank
    const unsigned half = call & 1u, tag = call + 1u;        // never 0: the buffers start zero-filled
    const size_t rank_words = (size_t)c.max_elems / 2, half_words = (size_t)c.world * rank_words;
    const size_t ll_off = plain_bytes(c.world, c.max_elems);
    if (live) {
        const unsigned long long hi = (unsigned long long)tag << 32;
        const uint4 mine = *reinterpret_cast<const uint4*>(static_cast<const T*>(c.data) + idx);
        for (int p = 0; p < c.world; ++p) {
            const int peer = (c.rank + p) % c.world;          // start with my own buffer, spread the rest
            unsigned long long* dst = reinterpret_cast<unsigned long long*>(c.slots[peer] + ll_off) + half * half_words +
                                      (size_t)c.rank * rank_words + idx / 2;
            st_relaxed_sys_v2(dst, hi | mine.x, hi | mine.y);
            st_relaxed_sys_v2(dst + 2, hi | mine.z, hi | mine.w);
        }
        // collect: the slots of all ranks in rank order (the same order, hence the same bits, on every rank)
        float acc[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] = 0.0f;
        const unsigned long long* base = reinterpret_cast<const unsigned long long*>(c.slots[c.rank] + ll_off) + half * half_words + idx / 2;
        bool gave_up = false;
        for (int r = 0; r < c.world; ++r) {
            const unsigned long long* src = base + (size_t)r * rank_words;
            unsigned long long w[4];
            int probes = 0;
            for (;;) {
                ld_relaxed_sys_v2(src, w[0], w[1]);
                ld_relaxed_sys_v2(src + 2, w[2], w[3]);
                if ((unsigned)(w[0] >> 32) == tag && (unsigned)(w[1] >> 32) == tag && (unsigned)(w[2] >> 32) == tag &&
                    (unsigned)(w[3] >> 32) == tag)
                    break;
                if (++probes > c.wait_limit) { gave_up = true; break; }
                __nanosleep(32);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const unsigned lo = (unsigned)w[q];
                const T* e = reinterpret_cast<const T*>(&lo);
                acc[2 * q] += Act16<BF16>::to_float(e[0]);
                acc[2 * q + 1] += Act16<BF16>::to_float(e[1]);
            }
        }
        if (gave_up) atomicExch(c.state + 2, 1u);
        uint4 out;
        T* o = reinterpret_cast<T*>(&out);
#pragma unroll
        for (int q = 0; q < 8; ++q) o[q] = Act16<BF16>::from_float(acc[q]);
        *reinterpret_cast<uint4*>(static_cast<T*>(c.data) + idx) = out;
    }
    // the last CTA of the launch advances the call counter (every CTA has read it by now)
    __syncthreads();
    if (tid == 0) {
        const unsigned old = atomicAdd(c.state + 1, 1u);
        if (old == gridDim.x - 1) {
            c.state[1] = 0u;
            __threadfence();
            c.state[0] = tag;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// all-reduce + residual update + RMS normalisation: one CTA per row
// ---------------------------------------------------------------------------------------------
constexpr int kFusedThreads = 256;
constexpr int kFusedMaxVec = 8;                   // 8-element vectors per thread: hidden <= 256 * 8 * 8

struct FusedArgs {
    CommArgs c;
    const void* partial; long long ldp;
    void* h; long long ldh;
    const void* weight;
    void* y; long long ldy;
    int hidden;
    float eps;
};

template <bool BF16>
__global__ void __launch_bounds__(kFusedThreads) qcomm_allreduce_rmsnorm_kernel(const FusedArgs a) {
    using T = typename Act16<BF16>::T;
    const CommArgs& c = a.c;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int tid = threadIdx.x, row = blockIdx.x, nvec = a.hidden >> 3;
    asm volatile("griddepcontrol.wait;" ::: "memory");      // the producer of `partial` (and of h) has finished
    const unsigned call = ld_relaxed_gpu(c.state);
    const unsigned half = call & 1u, tag = call + 1u;
    const size_t half_elems = (size_t)c.world * c.max_elems;
    const size_t row_off = (size_t)row * a.hidden;
    __shared__ float red[kFusedThreads / 32];
    __shared__ float total;

    // 1. this rank's partial row into its slot of every rank's receive buffer
    const T* part = static_cast<const T*>(a.partial) + (size_t)row * a.ldp;
#pragma unroll
    for (int i = 0; i < kFusedMaxVec; ++i) {
        const int v = tid + i * kFusedThreads;
        if (v < nvec) {
            const uint4 mine = *reinterpret_cast<const uint4*>(part + v * 8);
            for (int p = 0; p < c.world; ++p) {
                const int peer = (c.rank + p) % c.world;
                T* dst = reinterpret_cast<T*>(c.slots[peer]) + half * half_elems + (size_t)c.rank * c.max_elems + row_off + v * 8;
                *reinterpret_cast<uint4*>(dst) = mine;
            }
        }
    }
    __threadfence_system();
    __syncthreads();
    // 2. flags: raise mine for this row at every rank, wait (bounded) for everybody's here
    if (tid < c.world) {
        st_release_sys(c.flags[tid] + (half * c.world + c.rank) * QCOMM_MAX_BLOCKS + row, tag);
        const unsigned* f = c.flags[c.rank] + (half * c.world + tid) * QCOMM_MAX_BLOCKS + row;
        int probes = 0;
        while (ld_acquire_sys(f) != tag) {
            if (++probes > c.wait_limit) { atomicExch(c.state + 2, 1u); break; }
            __nanosleep(64);
        }
    }
    __syncthreads();
    // 3. sum of the slots in rank order, rounded; residual update; sum of squares
    T* h = static_cast<T*>(a.h) + (size_t)row * a.ldh;
    const T* base = reinterpret_cast<const T*>(c.slots[c.rank]) + half * half_elems + row_off;
    float f[kFusedMaxVec][8];
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < kFusedMaxVec; ++i) {
        const int v = tid + i * kFusedThreads;
        if (v < nvec) {
            float acc[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[q] = 0.0f;
            for (int r = 0; r < c.world; ++r) {
                const uint4 sv = ld_cg_u128(base + (size_t)r * c.max_elems + v * 8);
                const T* e = reinterpret_cast<const T*>(&sv);
#pragma unroll
                for (int q = 0; q < 8; ++q) acc[q] += Act16<BF16>::to_float(e[q]);
            }
            const uint4 hv = *reinterpret_cast<const uint4*>(h + v * 8);
            const T* he = reinterpret_cast<const T*>(&hv);
            uint4 ov;
            T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float d = Act16<BF16>::to_float(Act16<BF16>::from_float(acc[q]));
                oe[q] = Act16<BF16>::from_float(Act16<BF16>::to_float(he[q]) + d);
                f[i][q] = Act16<BF16>::to_float(oe[q]);
                sq = fmaf(f[i][q], f[i][q], sq);
            }
            *reinterpret_cast<uint4*>(h + v * 8) = ov;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    if ((tid & 31) == 0) red[tid >> 5] = sq;
    __syncthreads();
    if (tid == 0) {
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < kFusedThreads / 32; ++i) t += red[i];
        total = rsqrtf(t / (float)a.hidden + a.eps);
        // 5. the last CTA of the launch advances the call counter (every CTA has read it by now)
        const unsigned old = atomicAdd(c.state + 1, 1u);
        if (old == gridDim.x - 1) {
            c.state[1] = 0u;
            __threadfence();
            c.state[0] = tag;
        }
    }
    __syncthreads();
    // 4. normalise
    const float inv = total;
    const T* w = static_cast<const T*>(a.weight);
    T* y = static_cast<T*>(a.y) + (size_t)row * a.ldy;
#pragma unroll
    for (int i = 0; i < kFusedMaxVec; ++i) {
        const int v = tid + i * kFusedThreads;
        if (v < nvec) {
            const uint4 wv = *reinterpret_cast<const uint4*>(w + v * 8);
            const T* we = reinterpret_cast<const T*>(&wv);
            uint4 ov;
            T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
            for (int q = 0; q < 8; ++q)
                oe[q] = Act16<BF16>::from_float(Act16<BF16>::to_float(we[q]) *
                                                Act16<BF16>::to_float(Act16<BF16>::from_float(f[i][q] * inv)));
            *reinterpret_cast<uint4*>(y + v * 8) = ov;
        }
    }
}

// Validate a group and fill the device-side view of it.
int fill_comm_args(const qcomm_group* g, const char* who, CommArgs& c) {
    if (!g) { set_error("%s: group is NULL", who); return QGEMV_ERR_BAD_ARG; }
    if (g->world < 1 || g->world > QCOMM_MAX_RANKS || g->rank < 0 || g->rank >= g->world) {
        set_error("%s: bad rank %d / world %d (at most %d ranks)", who, g->rank, g->world, QCOMM_MAX_RANKS);
        return QGEMV_ERR_BAD_ARG;
    }
    if (g->max_elems % 8) { set_error("%s: max_elems must be a multiple of 8", who); return QGEMV_ERR_SHAPE; }
    if (!g->state) { set_error("%s: state is NULL", who); return QGEMV_ERR_BAD_ARG; }
    for (int r = 0; r < g->world; ++r) {
        if (!g->slots[r] || !g->flags[r]) { set_error("%s: slots / flags of rank %d are NULL", who, r); return QGEMV_ERR_BAD_ARG; }
        c.slots[r] = static_cast<unsigned char*>(g->slots[r]);
        c.flags[r] = static_cast<unsigned*>(g->flags[r]);
    }
    c.state = static_cast<unsigned*>(g->state);
    c.rank = g->rank; c.world = g->world; c.max_elems = g->max_elems;
    c.wait_limit = g->wait_limit > 0 ? g->wait_limit : kDefaultWaitLimit;
    return QGEMV_OK;
}

}  // namespace
}  // namespace qgemv

using namespace qgemv;

extern "C" int qcomm_allreduce_rmsnorm(const qcomm_group* g, const void* partial, int64_t ldp, void* h, int64_t ldh,
                                       const void* weight, void* y, int64_t ldy, int rows, int hidden, float eps,
                                       int dtype, void* stream) {
    FusedArgs a{};
    const int rc = fill_comm_args(g, "qcomm_allreduce_rmsnorm", a.c);
    if (rc != QGEMV_OK) return rc;
    if (!partial || !h || !weight || !y) { set_error("qcomm_allreduce_rmsnorm: null pointer"); return QGEMV_ERR_BAD_ARG; }
    if (dtype != QGEMV_F16 && dtype != QGEMV_BF16) { set_error("qcomm_allreduce_rmsnorm: dtype must be fp16 or bf16"); return QGEMV_ERR_BAD_ARG; }
    if (rows < 1 || rows > QCOMM_MAX_BLOCKS) { set_error("qcomm_allreduce_rmsnorm: 1..%d rows (got %d)", QCOMM_MAX_BLOCKS, rows); return QGEMV_ERR_TOO_LARGE; }
    if (hidden < 8 || hidden % 8 || hidden > kFusedThreads * kFusedMaxVec * 8) { set_error("qcomm_allreduce_rmsnorm: hidden=%d must be a multiple of 8, at most %d", hidden, kFusedThreads * kFusedMaxVec * 8); return QGEMV_ERR_SHAPE; }
    if ((int64_t)rows * hidden > g->max_elems) { set_error("qcomm_allreduce_rmsnorm: %d x %d elements exceed the slot capacity of %d", rows, hidden, g->max_elems); return QGEMV_ERR_TOO_LARGE; }
    if (ldp < hidden || ldh < hidden || ldy < hidden) { set_error("qcomm_allreduce_rmsnorm: a leading dimension is smaller than hidden"); return QGEMV_ERR_SHAPE; }
    if (reinterpret_cast<uintptr_t>(partial) % 16 || reinterpret_cast<uintptr_t>(h) % 16 || reinterpret_cast<uintptr_t>(y) % 16 ||
        reinterpret_cast<uintptr_t>(weight) % 16 || ldp % 8 || ldh % 8 || ldy % 8) {
        set_error("qcomm_allreduce_rmsnorm: rows must be 16-byte aligned");
        return QGEMV_ERR_ALIGN;
    }
    a.partial = partial; a.ldp = ldp; a.h = h; a.ldh = ldh; a.weight = weight; a.y = y; a.ldy = ldy;
    a.hidden = hidden; a.eps = eps;
    a.c.data = nullptr; a.c.elems = rows * hidden;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows);
    cfg.blockDim = dim3(kFusedThreads);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = dtype == QGEMV_BF16 ? cudaLaunchKernelEx(&cfg, qcomm_allreduce_rmsnorm_kernel<true>, a)
                                              : cudaLaunchKernelEx(&cfg, qcomm_allreduce_rmsnorm_kernel<false>, a);
    (void)e;
    return check_launch("qcomm_allreduce_rmsnorm_kernel");
}

extern "C" size_t qcomm_slot_bytes(int world, int max_elems) {
    // the plain area and, behind it, the area of self-validating words (8 bytes per 2 elements)
    return plain_bytes(world, max_elems) + (size_t)2 * world * (max_elems / 2) * 8;
}
extern "C" size_t qcomm_flag_bytes(int world) { return (size_t)2 * world * QCOMM_MAX_BLOCKS * sizeof(unsigned); }
extern "C" size_t qcomm_state_bytes(void) { return 256; }

extern "C" int qcomm_allreduce(const qcomm_group* g, void* data, int64_t elems, int dtype, void* stream) {
    if (!g || !data) { set_error("qcomm_allreduce: group and data must be non-null"); return QGEMV_ERR_BAD_ARG; }
    if (g->world < 1 || g->world > QCOMM_MAX_RANKS || g->rank < 0 || g->rank >= g->world) {
        set_error("qcomm_allreduce: bad rank %d / world %d (at most %d ranks)", g->rank, g->world, QCOMM_MAX_RANKS);
        return QGEMV_ERR_BAD_ARG;
    }
    if (dtype != QGEMV_F16 && dtype != QGEMV_BF16) { set_error("qcomm_allreduce: dtype must be fp16 or bf16"); return QGEMV_ERR_BAD_ARG; }
    if (elems < 8 || elems % 8 || g->max_elems % 8) { set_error("qcomm_allreduce: element counts must be positive multiples of 8 (got %lld)", (long long)elems); return QGEMV_ERR_SHAPE; }
    if (elems > g->max_elems) { set_error("qcomm_allreduce: %lld elements exceed the slot capacity of %d", (long long)elems, g->max_elems); return QGEMV_ERR_TOO_LARGE; }
    const int blocks = (int)((elems + kCommChunk - 1) / kCommChunk);
    if (blocks > QCOMM_MAX_BLOCKS) { set_error("qcomm_allreduce: %lld elements need more than %d CTAs", (long long)elems, QCOMM_MAX_BLOCKS); return QGEMV_ERR_TOO_LARGE; }
    if (reinterpret_cast<uintptr_t>(data) % 16) { set_error("qcomm_allreduce: data must be 16-byte aligned"); return QGEMV_ERR_ALIGN; }
    if (!g->state) { set_error("qcomm_allreduce: state is NULL"); return QGEMV_ERR_BAD_ARG; }
    CommArgs c{};
    for (int r = 0; r < g->world; ++r) {
        if (!g->slots[r] || !g->flags[r]) { set_error("qcomm_allreduce: slots / flags of rank %d are NULL", r); return QGEMV_ERR_BAD_ARG; }
        c.slots[r] = static_cast<unsigned char*>(g->slots[r]);
        c.flags[r] = static_cast<unsigned*>(g->flags[r]);
    }
    c.state = static_cast<unsigned*>(g->state);
    c.data = data;
    c.rank = g->rank; c.world = g->world; c.max_elems = g->max_elems; c.elems = (int)elems;
    c.wait_limit = g->wait_limit > 0 ? g->wait_limit : kDefaultWaitLimit;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(kCommThreads);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // Two ranks: tagged words (one trip over the link; 98.4 against 92.9 tok/s on the 70B-shape decode).  More ranks:
    // plain data + flags (every thread of the tagged version polls every peer, which costs more than the fence it saves).
    const bool tagged = g->world <= 2;
    cudaError_t e;
    if (tagged)
        e = dtype == QGEMV_BF16 ? cudaLaunchKernelEx(&cfg, qcomm_allreduce_kernel<true>, c)
                                : cudaLaunchKernelEx(&cfg, qcomm_allreduce_kernel<false>, c);
    else
        e = dtype == QGEMV_BF16 ? cudaLaunchKernelEx(&cfg, qcomm_allreduce_flags_kernel<true>, c)
                                : cudaLaunchKernelEx(&cfg, qcomm_allreduce_flags_kernel<false>, c);
    (void)e;
    return check_launch("qcomm_allreduce_kernel");
}

extern "C" int qcomm_status(const qcomm_group* g, void* stream, int32_t* host_out) {
    if (!g || !g->state || !host_out) { set_error("qcomm_status: group, state and host_out must be non-null"); return QGEMV_ERR_BAD_ARG; }
    unsigned* word = static_cast<unsigned*>(g->state) + 2;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(host_out, word, sizeof(int32_t), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaMemsetAsync(word, 0, sizeof(int32_t), s) != cudaSuccess)
        return check_launch("qcomm_status");
    return QGEMV_OK;
}

extern "C" int qcomm_alloc(size_t bytes, void** dev_ptr) {
    if (!dev_ptr || bytes == 0) { set_error("qcomm_alloc: bad arguments"); return QGEMV_ERR_BAD_ARG; }
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess || cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
        const int r = check_launch("qcomm_alloc");
        if (p) cudaFree(p);
        return r != QGEMV_OK ? r : QGEMV_ERR_LAUNCH;
    }
    *dev_ptr = p;
    return QGEMV_OK;
}

extern "C" int qcomm_free(void* dev_ptr) {
    if (dev_ptr && cudaFree(dev_ptr) != cudaSuccess) return check_launch("qcomm_free");
    return QGEMV_OK;
}

extern "C" int qcomm_ipc_export(void* dev_ptr, void* handle_out) {
    static_assert(sizeof(cudaIpcMemHandle_t) == QCOMM_IPC_HANDLE_BYTES, "unexpected IPC handle size");
    if (!dev_ptr || !handle_out) { set_error("qcomm_ipc_export: bad arguments"); return QGEMV_ERR_BAD_ARG; }
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, dev_ptr) != cudaSuccess) return check_launch("cudaIpcGetMemHandle");
    memcpy(handle_out, &h, sizeof(h));
    return QGEMV_OK;
}

extern "C" int qcomm_ipc_open(const void* handle, void** dev_ptr) {
    if (!handle || !dev_ptr) { set_error("qcomm_ipc_open: bad arguments"); return QGEMV_ERR_BAD_ARG; }
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return check_launch("cudaIpcOpenMemHandle");
    *dev_ptr = p;
    return QGEMV_OK;
}

extern "C" int qcomm_ipc_close(void* dev_ptr) {
    if (dev_ptr && cudaIpcCloseMemHandle(dev_ptr) != cudaSuccess) return check_launch("cudaIpcCloseMemHandle");
    return QGEMV_OK;
}
