// One-shot all-reduce of small 16-bit vectors over peer memory: see include/qcomm_b200.h.
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

template <bool BF16>
__global__ void __launch_bounds__(kCommThreads) qcomm_allreduce_kernel(const CommArgs c) {
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

}  // namespace
}  // namespace qgemv

using namespace qgemv;

extern "C" size_t qcomm_slot_bytes(int world, int max_elems) { return (size_t)2 * world * max_elems * 2; }
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
    const cudaError_t e = dtype == QGEMV_BF16 ? cudaLaunchKernelEx(&cfg, qcomm_allreduce_kernel<true>, c)
                                              : cudaLaunchKernelEx(&cfg, qcomm_allreduce_kernel<false>, c);
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
