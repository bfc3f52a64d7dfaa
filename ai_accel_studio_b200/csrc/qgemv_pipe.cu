// Pipelined fused GEMV for packed groupwise INT2 / INT4 weights, M <= 4, sm_100a.
//
// Same arithmetic as qgemv_mma.cu (codes used in place as fp16 subnormals, mma.sync.m16n8k16 for the
// dot products, fp32 group combine, fused outlier / residual / bias / activation epilogue); what
// changes is how one launch is laid out in time, because at these sizes (5 - 60 MB of weights, a few
// microseconds at HBM rate) the fixed parts of a launch cost as much as the stream itself:
//
//  * Half an SM per CTA.  One CTA per SM, 8 warps, at most 128 registers per thread and at most
//    113 KB of shared memory, so that the CTA of the NEXT launch in the stream fits on the same SM
//    while this one is still running.  Launches carry the programmatic-stream-serialisation
//    attribute and signal griddepcontrol.launch_dependents first thing.
//  * Weights before the dependency.  Packed codes, scales, outlier-weight rows, residual rows and
//    bias are static, so a CTA fills its whole ring of asynchronous copies (and announces the rest
//    of its share to L2) BEFORE griddepcontrol.wait.  While launch n computes, launch n+1 already
//    has ~60 KB per SM of its weights on chip or in flight: DRAM keeps streaming through the
//    prologue and the tail of every launch, which is where the phased kernel left it idle.
//  * The ring is filled by the tensor-map copy engine (TMA): ONE request per slot for the codes (a
//    16-row x CB-byte box) and one for the scales, completion counted in bytes on an mbarrier per slot.
//    Two other ways were measured first.  Per-thread 16-byte cp.async copies: with two CTAs on an SM
//    the waiting CTA's copies sit in the load/store queues that the running CTA's shared-memory loads
//    also go through; the running launch's main loop took 14 us instead of 3 and a dependent 8-byte
//    load 3 us.  One bulk copy per row per slot (40 requests per 4 KB slot): the copy engine handles
//    roughly one request per ten cycles, so the requests, not the bytes, set the pace (23 us per GEMV).
//    The packed matrix is described to the engine as a 3-D tensor [group bytes][row][group], so the box
//    lands in shared memory as [group][row][group bytes]: the lanes of one shared-memory load then read
//    128 contiguous bytes, and no swizzle is needed.
//  * After the wait only x-dependent work is left: load x (L2 hits), stage it in B-fragment order,
//    gather the outlier activations, one CTA barrier, main loop.
//  * No barrier after the main loop.  A warp that completes a run parks its partial sums and bumps
//    the tile's arrival counter in shared memory; whichever warp arrives last adds the runs in run
//    order (bit-repeatable) and finishes the tile at once -- outlier columns, residual, bias,
//    activation, store -- from operands that were prefetched with the ring.  Epilogues overlap the
//    other warps' streaming.
//  * CTAs always own whole tiles (no hand-over between CTAs through global memory).  Shapes whose
//    balance needs shared tiles stay with the phased kernel.
//
// The residual projections t = V.x are computed by the first rank * parts CTAs right after the
// wait and travel to the others as {value, launch tag} words, exactly as in qgemv_mma.cu; every
// wait on them is bounded and reports through the workspace's status word.
//
// Replaces _decode_gemv (ai_accel_lab/kernels/decode_int2.py:43-96) and _decode_int4_gemv
// (ai_accel_lab/kernels/groupwise_int4.py:85-107) of the reference project.
#include <cuda.h>

#include <type_traits>

#include "qgemv_mma_dev.cuh"

namespace qgemv {

// Tensor maps of one launch (kernel parameter): packed codes, scales, outlier weights, residual rows.
struct PipeMaps {
    CUtensorMap w, s, ow, ru;
};

namespace {

constexpr int kPipeWarps = 8;                 // warps per CTA the kernel is compiled for (128 registers x 256 threads x 2 CTAs = one SM)
constexpr int kPipeMaxStages = 8;             // ring descriptors reserved per warp
#ifndef QGEMV_BATCH_GROUPS
#define QGEMV_BATCH_GROUPS 4
#endif
constexpr int kBatchGroups = QGEMV_BATCH_GROUPS;   // groups whose tensor-core chains a warp keeps in flight together
constexpr int kSmemPerSm = 233472;            // 228 KB of shared memory per SM on sm_100
constexpr int kHalfSmSmem = (kSmemPerSm - 2 * 1024) / 2;   // dynamic bytes that let two CTAs share an SM (1 KB per CTA is reserved)
constexpr int kBarSpinLimit = 1 << 22;        // bound of the wait for a bulk copy (each probe blocks for a while in hardware)
constexpr int kFlagSpinLimit = 1 << 22;       // bound of the in-CTA wait for the table of residual projections
constexpr int kTagSpinLimit = 1 << 20;        // bound of the wait for another CTA's projection (about 30 ms)
constexpr int kTagSpinLimitDebug = 1 << 7;    // ... with QGEMV_DEBUG_DROP_PROJECTIONS (a few microseconds)

// Optional phase trace (build with -DQGEMV_TRACE): lane 0 of every warp stores the global nanosecond
// timer at a few points into the upper half of the partial-sum scratch; bits 24..27 of the debug
// word select one of 12 regions, so that the launches of a chain can be told apart.
#ifdef QGEMV_TRACE
#define PTRACE(slot)                                                                            \
    do {                                                                                        \
        if ((threadIdx.x & 31) == 0) {                                                          \
            unsigned long long t_;                                                              \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_) :: "memory");                  \
            reinterpret_cast<unsigned long long*>(p.a.partial + (kMaxPartialFloats / 2))        \
                [((size_t)((p.debug >> 24) & 15) * 148 * kPipeWarps +                           \
                  (size_t)blockIdx.x * kPipeWarps + (threadIdx.x >> 5)) * 16 + (slot)] = t_;    \
        }                                                                                       \
    } while (0)
#define PTRACE_VAL(slot, value)                                                                 \
    do {                                                                                        \
        if ((threadIdx.x & 31) == 0)                                                            \
            reinterpret_cast<unsigned long long*>(p.a.partial + (kMaxPartialFloats / 2))        \
                [((size_t)((p.debug >> 24) & 15) * 148 * kPipeWarps +                           \
                  (size_t)blockIdx.x * kPipeWarps + (threadIdx.x >> 5)) * 16 + (slot)] = (value); \
    } while (0)
#define PTRACE_NOW(var) unsigned long long var; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(var) :: "memory")
#else
#define PTRACE(slot) do { } while (0)
#define PTRACE_VAL(slot, value) do { } while (0)
#define PTRACE_NOW(var) do { } while (0)
#endif

// Announce `bytes` (multiple of 16) at a 16-byte aligned global address to L2; no data reaches the SM.
__device__ __forceinline__ void l2_prefetch_bulk(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ int ld_volatile_shared(const int* p) {
    int v; asm volatile("ld.volatile.shared.s32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory"); return v;
}
// mbarrier + bulk-copy wrappers (shared::cta addresses are 32-bit shared-window addresses).
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done;
}
// Global -> shared bulk copy of `bytes` (multiple of 16; both addresses 16-byte aligned) whose
// completion is counted, in bytes, on the mbarrier at `bar`.  This CTA's own shared memory only.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// Tiled tensor-map copies of one box into this CTA's shared memory (128-byte aligned), completion on `bar`.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tmap, int c0, int c1, int c2, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(tmap), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_prefetch_3d(const void* tmap, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global [%0, {%1, %2, %3}];" ::"l"(tmap), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_prefetch_2d(const void* tmap, int c0, int c1) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(tmap), "r"(c0), "r"(c1) : "memory");
}
// Orders this thread's earlier generic-proxy accesses to shared memory before later async-proxy ones.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// Activation staging after the dependency wait (whole CTA, no barrier inside; the caller's barrier
// publishes the results): x -> fp16 multiplicands in B-fragment order with the per (group, row)
// offset term and power-of-two normalisation (see qgemv_mma.cu for the number format), the outlier
// activations x[m][outlier_idx[j]] as fp32, and, in the CTAs that carry one, a residual-projection
// job.  Every global load is issued before the first result is needed.
// `cols` holds the outlier column of entries tid, tid + nthr, ... (read before the wait).
// ---------------------------------------------------------------------------------------------
template <int BITS, int GB, int M, bool BF16, bool EX>
__device__ __forceinline__ void pipe_stage_x(const MmaArgs& p, unsigned char* smem, const int (&cols)[4]) {
    using XT = typename Act16<BF16>::T;
    using GE = Geo<BITS, GB>;
    constexpr int EPI = GE::G / 4;          // activations per item (group, row m, quad lane t)
    constexpr int PPI = EPI / 8;            // 16-byte pieces per item
    constexpr int WP = GE::CW / 8;          // pieces per 32-bit code word (INT2: 2, INT4: 1)
    constexpr int RC = PPI <= 4 ? 2 : 1;    // items whose loads one thread keeps in flight together
    constexpr int PVMAX = M == 1 ? 4 : (M == 2 ? 3 : 2);   // pieces of V per thread of a projection job
    const Args& a = p.a;
    const int tid = threadIdx.x, nthr = blockDim.x;
    float* xo = reinterpret_cast<float*>(smem + p.off_xo);
    float2* gx = reinterpret_cast<float2*>(smem + p.off_gx);          // {offset term, accumulator scale} per (group, m)
    uint4* xs16 = reinterpret_cast<uint4*>(smem + p.off_xs);
    const XT* x = static_cast<const XT*>(a.x);
    const int items = p.ng * M * 4;
    const int span = nthr * RC;

    // outlier activations: up to four per thread in flight, the rest (oc * M > 4 * threads) one by one
    const int n_xo = EX ? a.oc * M : 0;
    XT xraw[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int i = tid + r * nthr;
        xraw[r] = Act16<BF16>::from_float(0.0f);
        if (EX && i < n_xo) {
            const int col = cols[r];
            if (col >= 0 && col < a.kpad) xraw[r] = x[(size_t)(i % M) * a.ldx + col];
        }
    }

    uint4 v[RC][PPI];
    int vg[RC], vm[RC], vt[RC];
    auto load_items = [&](int base) {
#pragma unroll
        for (int r = 0; r < RC; ++r) {
            const int item = base + r * nthr + tid;
            if (item < items) {
                vt[r] = item & 3;
                const int gm = item >> 2;
                vg[r] = gm / M;
                vm[r] = gm - vg[r] * M;
                const XT* src = x + (size_t)vm[r] * a.ldx + (size_t)vg[r] * GE::G + vt[r] * EPI;
#pragma unroll
                for (int i = 0; i < PPI; ++i) v[r][i] = reinterpret_cast<const uint4*>(src)[i];
            } else {
                vm[r] = -1; vg[r] = 0; vt[r] = 0;
#pragma unroll
                for (int i = 0; i < PPI; ++i) v[r][i] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };
    load_items(0);

    // Residual projections t[m][c] = sum_k V[c,k] x[m,k]: job j = (column c, K-part) belongs to CTA j.
    const int t_jobs = (EX && p.t_inline) ? a.rank * p.t_parts : 0;
    const bool has_job = (int)blockIdx.x < t_jobs;
    if (has_job) {
        const int c = blockIdx.x % a.rank, part = blockIdx.x / a.rank;
        const int t_cols = nthr * 8 * p.t_pv;
        uint4 tv[PVMAX], tx[PVMAX][M];
#pragma unroll
        for (int pv = 0; pv < PVMAX; ++pv) {
            const int k = part * t_cols + (pv * nthr + tid) * 8;
            const bool live = pv < p.t_pv && k < a.korig;
            tv[pv] = live ? *reinterpret_cast<const uint4*>(a.rv + (size_t)c * a.ldv + k) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int m = 0; m < M; ++m)
                tx[pv][m] = live ? *reinterpret_cast<const uint4*>(x + (size_t)m * a.ldx + k) : make_uint4(0u, 0u, 0u, 0u);
        }
        const int warp_id = tid >> 5, lane_id = tid & 31;
        float ts[M];
#pragma unroll
        for (int m = 0; m < M; ++m) ts[m] = 0.0f;
#pragma unroll
        for (int pv = 0; pv < PVMAX; ++pv) {
            const __half* vh = reinterpret_cast<const __half*>(&tv[pv]);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const XT* xh = reinterpret_cast<const XT*>(&tx[pv][m]);
#pragma unroll
                for (int q = 0; q < 8; ++q) ts[m] = fmaf(__half2float(vh[q]), Act16<BF16>::to_float(xh[q]), ts[m]);
            }
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ts[m] += __shfl_xor_sync(0xffffffffu, ts[m], o);
        }
        float* red = reinterpret_cast<float*>(smem + p.off_red);      // read by warp 0 after the caller's barrier
        if (lane_id == 0) {
#pragma unroll
            for (int m = 0; m < M; ++m) red[warp_id * M + m] = ts[m];
        }
    }

    for (int base = 0; base < items; base += span) {
        if (base) load_items(base);
#pragma unroll
        for (int r = 0; r < RC; ++r) {
            const bool live = vm[r] >= 0;
            const int mrow = live ? vm[r] : 0, grp = vg[r], tq = vt[r];
            float f[EPI];
            float part = 0.0f, big = 0.0f;
#pragma unroll
            for (int i = 0; i < PPI; ++i) {
                const XT* e = reinterpret_cast<const XT*>(&v[r][i]);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    f[i * 8 + q] = Act16<BF16>::to_float(e[q]);
                    part += f[i * 8 + q];
                    big = fmaxf(big, fabsf(f[i * 8 + q]));
                }
            }
            part += __shfl_xor_sync(0xffffffffu, part, 1);
            part += __shfl_xor_sync(0xffffffffu, part, 2);
            big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, 1));
            big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, 2));
            int e2 = 0;
            if (big > 0.0f && big < 3.0e38f) e2 = (int)((__float_as_uint(big) >> 23) & 0xffu) - 127 - 13;   // floor(log2) - 13
            e2 = max(-60, min(100, e2));
            const float down = __int_as_float((127 - e2) << 23);         // 2^-e : multiplier for x
            const float up = __int_as_float((127 + 24 + e2) << 23);      // 2^(24+e): undoes subnormal unit and group scale
            if (live) {
                if (tq == 0) gx[grp * M + mrow] = make_float2(BITS == 2 ? part : 8.0f * part,
                                                              BITS == 2 ? up * (2.0f / 3.0f) : up);
#pragma unroll
                for (int i = 0; i < GE::TW; ++i) {            // one 32-bit code word of this lane
#pragma unroll
                    for (int cp = 0; cp < GE::NCLS / 2; ++cp) {
                        __half2 h2[4];
#pragma unroll
                        for (int hh = 0; hh < 8; hh += 2) {
                            float o[2];
#pragma unroll
                            for (int z = 0; z < 2; ++z) {
                                const int h = hh + z;
                                const int cl = h >> 2, pp = h & 3;
                                const int qq = (pp & 1) * 2 + (pp >> 1);
                                const int c = 2 * cp + cl;
                                const int j = qq * GE::NCLS + c;                       // code index inside the word
                                const float sc = __int_as_float((127 - BITS * c) << 23);   // radix^-c
                                o[z] = f[i * (WP * 8) + j] * down * sc;
                            }
                            h2[hh >> 1] = __floats2half2_rn(o[0], o[1]);
                        }
                        uint4 outv;
                        outv.x = *reinterpret_cast<uint32_t*>(&h2[0]); outv.y = *reinterpret_cast<uint32_t*>(&h2[1]);
                        outv.z = *reinterpret_cast<uint32_t*>(&h2[2]); outv.w = *reinterpret_cast<uint32_t*>(&h2[3]);
                        xs16[(((size_t)(grp * GE::TW + i) * (GE::NCLS / 2) + cp) * M + mrow) * 4 + tq] = outv;
                    }
                }
            }
        }
    }

    if (EX) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int i = tid + r * nthr;
            if (i < n_xo) xo[i] = Act16<BF16>::to_float(xraw[r]);
        }
        for (int i = tid + 4 * nthr; i < n_xo; i += nthr) {
            const int col = a.oidx[i / M];
            xo[i] = (col >= 0 && col < a.kpad) ? Act16<BF16>::to_float(x[(size_t)(i % M) * a.ldx + col]) : 0.0f;
        }
    }
}

// Table of residual projections t[q][m] in shared memory, built by one warp; `early0/1` are the
// words that warp requested one ring slot earlier (entry lane and lane + 32).  A word whose tag is
// not this launch's is read again, a bounded number of times; if the bound is hit the workspace's
// status word is raised and the stale value is used.
template <int M>
__device__ __noinline__ void pipe_build_t_table(const MmaArgs& p, unsigned char* smem, float* scratch, unsigned t_tag,
                                                unsigned long long early0, unsigned long long early1, bool requested) {
    const Args& a = p.a;
    const int lane = threadIdx.x & 31;
    float* tt = reinterpret_cast<float*>(smem + p.off_tt);
    const int RM = a.rank * M;
    if (!p.t_inline) {
        if (!p.wait_for_x) pdl_wait();            // t comes from the kernel launched just before this one
        for (int i = lane; i < RM; i += 32) {
            const int q = i / M, m = i - q * M;
            tt[i] = ld_cg_f32(a.t + m * kMaxRank + q);
        }
        return;
    }
    const int limit = (p.debug & QGEMV_DEBUG_DROP_PROJECTIONS) ? kTagSpinLimitDebug : kTagSpinLimit;
    auto settle = [&](unsigned long long w, const unsigned long long* addr) {
        int spins = 0;
        while ((unsigned)(w >> 32) != t_tag) {
            if (++spins > limit) { atomicExch(a.counters + kWsStatusIdx, 1); break; }
            __nanosleep(32);
            w = ld_relaxed_u64(addr);
        }
        return __uint_as_float((unsigned)w);
    };
    const int entries = p.t_parts * RM;
    if (entries <= 64) {
        const unsigned long long early[2] = {early0, early1};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int idx = lane + 32 * e;
            if (idx < entries) {
                const unsigned long long* addr = t_entry(a, M, idx);
                scratch[idx] = settle(requested ? early[e] : ld_relaxed_u64(addr), addr);
            }
        }
        __syncwarp();
        for (int i = lane; i < RM; i += 32) {
            float v = 0.0f;
            for (int part = 0; part < p.t_parts; ++part) v += scratch[part * RM + i];
            tt[i] = v;
        }
    } else {
        const unsigned long long* src = reinterpret_cast<const unsigned long long*>(a.tparts);
        for (int i = lane; i < RM; i += 32) {
            const int q = i / M, m = i - q * M;
            float v = 0.0f;
            for (int part = 0; part < p.t_parts; ++part) {
                const unsigned long long* addr = src + (part * QGEMV_MAX_M + m) * kMaxRank + q;
                v += settle(ld_relaxed_u64(addr), addr);
            }
            tt[i] = v;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The kernel.  One CTA per SM (at most), blockDim.x = 32 * nw <= 256; every warp is its own producer
// and consumer of a ring of asynchronous copies.
// ---------------------------------------------------------------------------------------------
template <int BITS, int GB, int CB, int M, bool BF16, bool EX>
__global__ void __launch_bounds__(kPipeWarps * 32, 2) qgemv_pipe_kernel(const __grid_constant__ MmaArgs p,
                                                                         const __grid_constant__ PipeMaps tm) {
    using GE = Geo<BITS, GB, CB>;
    constexpr int TT = (M + 1) / 2;                   // quad lanes that hold useful output columns
    constexpr int SLOT_BYTES = 8 * TT * 16;           // one run's partial sums in shared memory
    extern __shared__ __align__(128) unsigned char smem[];
    const Args& a = p.a;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    // The next launch of the stream is released only after this CTA's x-dependent prologue (below):
    // its CTAs then arrive, and pour their ring fills into the memory system, while this launch is
    // in its main loop.  Released at kernel entry they arrive just as this launch reads x, and those
    // few dependent loads -- on the critical path of the whole chain -- queue behind ~60 KB per SM
    // of the newcomer's weight copies (measured: 17.6 instead of 10.4 us per GEMV).
    if (p.debug & QGEMV_DEBUG_EARLY_TRIGGER) pdl_launch_dependents();
    PTRACE(0);

    // This CTA's tiles [T0, T1) and their runs [r0, r1).
    const int grid = gridDim.x, cta = blockIdx.x;
    const int T0 = first_unit(p, cta, grid), T1 = first_unit(p, cta + 1, grid);
    const int r0 = T0 * p.rpt, r1 = T1 * p.rpt;
    const int nstages = p.stages;

    unsigned char* ring = smem + p.off_ring + (size_t)warp * nstages * GE::STAGE_BYTES;
    const uint32_t ring_u32 = smem_u32(ring);
    int4* meta = reinterpret_cast<int4*>(smem + p.off_meta) + warp * kPipeMaxStages;   // per stage: tile, chunk, slot, last
    int* cnt = reinterpret_cast<int*>(smem + p.off_cnt);                               // arrivals per local tile; then the table flag
    const int ntl = T1 - T0;
    int* t_flag = cnt + (p.uq + 1);
    for (int i = tid; i < p.uq + 2; i += blockDim.x) cnt[i] = 0;

    // ---- barriers ---------------------------------------------------------------------------------
    // One mbarrier per ring slot of every warp (one arrival: the lane that announces the bytes), one
    // for the CTA's prefetched epilogue operands.
    const uint32_t bars_u32 = smem_u32(smem + p.off_bar) + warp * kPipeMaxStages * 8;
    const uint32_t epi_bar = smem_u32(smem + p.off_bar) + kPipeWarps * kPipeMaxStages * 8;
    if (lane == 0) {
        for (int s = 0; s < nstages; ++s) mbar_init(bars_u32 + s * 8, 1);
        if (warp == 0) mbar_init(epi_bar, 1);
        fence_mbar_init();
    }
    fence_proxy_async();
    __syncthreads();                                 // barriers and counters initialised before any copy can signal them
    PTRACE(1);

    // ---- producer side --------------------------------------------------------------------------
    const bool t_inline = EX && p.t_inline;
    const bool has_job = t_inline && (int)blockIdx.x < a.rank * p.t_parts;   // this CTA also computes a residual projection
    const int nwk = p.nw;
    // Runs are dealt round-robin: warp w takes runs r0 + w, r0 + w + nw, ...
    int pf_run = r0 + warp, pf_tile = 0, pf_j = 0, pf_ch = 0, pf_end = 0;   // pf_j: run index inside the tile
    if (pf_run < r1) {
        pf_tile = pf_run / p.rpt;
        pf_j = pf_run - pf_tile * p.rpt;
        pf_ch = pf_j * p.rlen;
        pf_end = min(pf_ch + p.rlen, p.nch);
    } else {
        pf_run = -1;
    }
    // A slot holds the codes of one chunk as [group][row][GB bytes] (16 rows, CG groups), followed by
    // 16 bytes of scales per row: the 8 scales of the aligned block of 8 groups that contains the
    // chunk's groups.  Rows past N and groups past the end of a row are zero-filled by the engine.
    // Step the (run, chunk) cursor of this warp to the next chunk it owns; false when there is none.
    auto advance = [&]() {
        if (pf_run >= 0 && pf_ch == pf_end) {          // current run exhausted: step to this warp's next run
            pf_run += nwk;
            pf_j += nwk;
            while (pf_j >= p.rpt) { pf_j -= p.rpt; ++pf_tile; }
            if (pf_run < r1) {
                pf_ch = pf_j * p.rlen;
                pf_end = min(pf_ch + p.rlen, p.nch);
            } else {
                pf_run = -1;
            }
        }
        return pf_run >= 0;
    };
    auto issue_next = [&](int s) {
        if (advance()) {
            const int ngr = min(GE::CG, p.ng - pf_ch * GE::CG);
            const uint32_t sbase = ring_u32 + s * GE::STAGE_BYTES;
            const uint32_t bar = bars_u32 + s * 8;
            const int row0 = pf_tile * kTileRows, g0 = pf_ch * GE::CG;
            fence_proxy_async();                                       // this slot was read with ordinary loads a moment ago
            if (lane == 0) {
                const int code_bytes = p.tma3d ? kTileRows * GE::CB : kTileRows * GB * ngr;
                mbar_arrive_expect_tx(bar, (uint32_t)(code_bytes + (p.scales_async ? kTileRows * 16 : 0)));
                if (p.tma3d) tma_load_3d(sbase, &tm.w, 0, row0, g0, bar);
                if (p.scales_async) tma_load_2d(sbase + GE::SCALE_OFF, &tm.s, g0 & ~7, row0, bar);
            }
            __syncwarp();
            if (!p.tma3d && lane < ngr)                                // one 16-row x GB box per group of the chunk
                tma_load_2d(sbase + lane * (kTileRows * GB), &tm.w, (g0 + lane) * GB, row0, bar);
            if (!p.scales_async && lane < kTileRows) {                 // unaligned scale rows: plain loads, this row's groups of the chunk
                const int row = min(row0 + lane, a.n - 1);
                const __half* src = a.scales + (size_t)row * a.lds + g0;
                __half* d = reinterpret_cast<__half*>(ring + s * GE::STAGE_BYTES + GE::SCALE_OFF + lane * 16) + (g0 & 7);
                for (int i = 0; i < ngr; ++i) d[i] = __ldg(src + i);
            }
            if (lane == 0) meta[s] = make_int4(pf_tile, pf_ch, pf_run - r0, pf_ch + 1 == pf_end);
            ++pf_ch;
        } else if (lane == 0) {
            meta[s] = make_int4(-1, 0, 0, 0);
        }
    };

    // ---- everything that does not depend on the previous kernel -----------------------------------
    // Epilogue operands (outlier-weight rows, residual rows, bias) of the CTA's first tiles: one box
    // each per tile, all counted on one barrier that every thread checks before the prologue ends.
    {
        const int full_tiles = a.n / kTileRows;                       // tiles that lie completely inside N
        const int npre = p.epi_async ? min(min(p.epi_tiles, ntl), max(0, full_tiles - T0)) : 0;
        const int ocb = EX ? p.ocb : 0, rb = EX ? p.rb : 0, bb = a.bias ? 32 : 0;
        if (tid == 0) mbar_arrive_expect_tx(epi_bar, (uint32_t)(npre * (kTileRows * (ocb + rb) + bb)));
        __syncwarp();
        const uint32_t epi_u32 = smem_u32(smem + p.off_epi);
        for (int i = tid; i < npre * 3; i += blockDim.x) {
            const int lt = i / 3, q = i - lt * 3;
            const int row0 = (T0 + lt) * kTileRows;
            const uint32_t dst = epi_u32 + lt * p.epi_bytes;
            if (q == 0) { if (ocb) tma_load_2d(dst, &tm.ow, 0, row0, epi_bar); }
            else if (q == 1) { if (rb) tma_load_2d(dst + kTileRows * ocb, &tm.ru, 0, row0, epi_bar); }
            else if (bb) bulk_g2s(dst + kTileRows * (ocb + rb), a.bias + row0, 32u, epi_bar);
        }
    }
    PTRACE(6);
    for (int s = 0; s < nstages; ++s) issue_next(s);
    PTRACE(7);
    // The chunks that follow the ring are announced to L2 now (one request per chunk), so that the main
    // loop finds them there instead of in DRAM.
    if (p.l2_chunks > 0 && lane == 0) {
        const int s_run = pf_run, s_tile = pf_tile, s_j = pf_j, s_ch = pf_ch, s_end = pf_end;
        for (int i = 0; i < p.l2_chunks && advance(); ++i) {
            if (p.tma3d) tma_prefetch_3d(&tm.w, 0, pf_tile * kTileRows, pf_ch * GE::CG);
            else
                for (int gi = 0; gi < min(GE::CG, p.ng - pf_ch * GE::CG); ++gi)
                    tma_prefetch_2d(&tm.w, (pf_ch * GE::CG + gi) * GB, pf_tile * kTileRows);
            ++pf_ch;
        }
        pf_run = s_run; pf_tile = s_tile; pf_j = s_j; pf_ch = s_ch; pf_end = s_end;
    }
    // outlier columns of the entries this thread will gather (static data)
    int cols[4] = {-1, -1, -1, -1};
    if (EX) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int i = tid + r * (int)blockDim.x;
            if (i < a.oc * M) cols[r] = a.oidx[i / M];
        }
    }
    PTRACE(8);

    // ---- from here on the previous kernel's results are needed ------------------------------------
    if (p.wait_for_x) pdl_wait();
    PTRACE(9);
    // Tag of this launch for the residual projections that travel between CTAs: the workspace holds a
    // launch count that the last CTA of every launch advances.
    const bool t_reader = EX && a.rank > 0 && warp == p.nw - 1;
    unsigned t_tag = 0;
    if (t_inline && (warp == 0 || t_reader)) t_tag = ld_relaxed_u32(a.counters + kWsEpochIdx) + 1u;
    pipe_stage_x<BITS, GB, M, BF16, EX>(p, smem, cols);
    PTRACE(10);
    {                                                 // the epilogue operands have landed (long ago, normally)
        int spins = 0;
        while (!mbar_try_wait(epi_bar, 0)) {
            if (++spins > kBarSpinLimit) { atomicExch(a.counters + kWsStatusIdx, 2); break; }
        }
    }
    __syncthreads();                                  // staged activations, counters and operands visible to every warp
    if (!(p.debug & QGEMV_DEBUG_EARLY_TRIGGER)) pdl_launch_dependents();
    PTRACE(2);
    if (has_job && warp == 0 && !(p.debug & QGEMV_DEBUG_DROP_PROJECTIONS)) {
        // The warps' partial sums were written before the barrier: add them in warp order and publish
        // {sum, launch tag} for every CTA's epilogue with one relaxed 64-bit store.
        const float* red = reinterpret_cast<const float*>(smem + p.off_red);
        if (lane < M) {
            float tot = 0.0f;
            for (int w = 0; w < p.nw; ++w) tot += red[w * M + lane];
            const int c = blockIdx.x % a.rank, part = blockIdx.x / a.rank;
            st_relaxed_u64(reinterpret_cast<unsigned long long*>(a.tparts) + (part * QGEMV_MAX_M + lane) * kMaxRank + c,
                           ((unsigned long long)t_tag << 32) | __float_as_uint(tot));
        }
    }

    // ---- consumer side ----------------------------------------------------------------------------
    unsigned char* slots = smem + p.off_slots;
    const int ma = min(2 * t, M - 1), mb = min(2 * t + 1, M - 1);
    // Lanes g >= M feed B columns whose results are never read: they load row M-1 instead of zeros.
    const uint32_t xs_lane_u32 = smem_u32(smem + p.off_xs) + (min(g, M - 1) * 4 + t) * 16;
    const uint32_t gx_lane_u32 = smem_u32(smem + p.off_gx) + (M % 2 == 0 ? (M >= 2 ? min(2 * t, M - 2) : 0) : 0) * 8;
    const uint32_t gx_a_u32 = smem_u32(smem + p.off_gx) + ma * 8, gx_b_u32 = smem_u32(smem + p.off_gx) + mb * 8;
    const uint32_t slots_u32 = smem_u32(slots) + (g * TT + t) * 16;
    const uint32_t meta_u32 = smem_u32(meta);
    const uint32_t lane_row_u32 = ring_u32 + g * GB + t * GE::TB;   // this lane's bytes of row g, group 0, slot 0 (row g+8: 8 rows further)
    const uint32_t lane_sc_u32 = ring_u32 + GE::SCALE_OFF + g * 16;
    const int ng_total = p.ng;
    constexpr int GSTRIDE = GE::TW * (GE::NCLS / 2) * M * 4 * 16;    // bytes of staged x per group

    // One group of one chunk: G = absolute group index, gi = group inside the chunk.
    auto do_group = [&](uint32_t rowa, uint32_t rowb, int gi, int G, float s0, float s1, float (&yy)[4]) {
        const uint32_t off = (uint32_t)(gi * (kTileRows * GB));       // groups are kTileRows * GB bytes apart in a slot
        uint32_t w0[GE::TW], w1[GE::TW];
        if constexpr (GE::TW == 1) {
            w0[0] = lds32(rowa + off); w1[0] = lds32(rowb + off);
        } else if constexpr (GE::TW == 2) {
            const uint2 v0 = lds64(rowa + off), v1 = lds64(rowb + off);
            w0[0] = v0.x; w0[1] = v0.y; w1[0] = v1.x; w1[1] = v1.y;
        } else {
            const uint4 v0 = lds128(rowa + off), v1 = lds128(rowb + off);
            w0[0] = v0.x; w0[1] = v0.y; w0[2] = v0.z; w0[3] = v0.w;
            w1[0] = v1.x; w1[1] = v1.y; w1[2] = v1.z; w1[3] = v1.w;
        }
        const uint32_t xg = xs_lane_u32 + (uint32_t)G * GSTRIDE;
        uint4 b[GE::TW * (GE::NCLS / 2)];
#pragma unroll
        for (int q = 0; q < GE::TW * (GE::NCLS / 2); ++q) b[q] = lds128(xg + q * (M * 4 * 16));
        float2 ga, gb;
        if constexpr (M % 2 == 0) {
            const float4 gq = lds128f(gx_lane_u32 + (uint32_t)G * (M * 8));
            ga = make_float2(gq.x, gq.y); gb = make_float2(gq.z, gq.w);
        } else {
            ga = lds64f(gx_a_u32 + (uint32_t)G * (M * 8)); gb = lds64f(gx_b_u32 + (uint32_t)G * (M * 8));
        }
        // two independent accumulator chains (the classes alternate between them); the first
        // instruction of each chain takes zero as its addend, so nothing has to be cleared
        float accA[4], accB[4];
#pragma unroll
        for (int i = 0; i < GE::TW; ++i) {
            const uint32_t h0 = w0[i] >> 8, h1 = w1[i] >> 8;
#pragma unroll
            for (int cp = 0; cp < GE::NCLS / 2; ++cp) {
                const uint4 bb = b[i * (GE::NCLS / 2) + cp];
                constexpr uint32_t MK = GE::MASK;
                const uint32_t m0 = MK << (BITS * (2 * cp)), m1 = MK << (BITS * (2 * cp + 1));
                if (i == 0 && cp == 0) {
                    mma_f16_first(accA, w0[i] & m0, w1[i] & m0, h0 & m0, h1 & m0, bb.x, bb.y);
                    mma_f16_first(accB, w0[i] & m1, w1[i] & m1, h0 & m1, h1 & m1, bb.z, bb.w);
                } else {
                    mma_f16(accA, w0[i] & m0, w1[i] & m0, h0 & m0, h1 & m0, bb.x, bb.y);
                    mma_f16(accB, w0[i] & m1, w1[i] & m1, h0 & m1, h1 & m1, bb.z, bb.w);
                }
            }
        }
        yy[0] = fmaf(s0, fmaf(ga.y, accA[0] + accB[0], -ga.x), yy[0]);
        yy[1] = fmaf(s0, fmaf(gb.y, accA[1] + accB[1], -gb.x), yy[1]);
        yy[2] = fmaf(s1, fmaf(ga.y, accA[2] + accB[2], -ga.x), yy[2]);
        yy[3] = fmaf(s1, fmaf(gb.y, accA[3] + accB[3], -gb.x), yy[3]);
    };

    // NB consecutive groups of one chunk, starting at group gi0 of the chunk (absolute group G0 + gi0),
    // with the tensor-core instructions of the NB groups interleaved step by step.  A warp's
    // mma.sync instructions on one accumulator are a dependent chain, and the legacy tensor path has
    // a long latency on this part: group after group (do_group) a warp needs ~600 cycles per group
    // and the kernel is bound by that latency, whatever the number of resident warps (measured: the same
    // 1.2 us per 4 KB chunk per warp with 7 and with 16 warps per SM).  Interleaving keeps 2 * NB
    // independent chains in flight per warp.  Same arithmetic, same order per group as do_group.
    auto do_batch = [&](auto nb_tag, uint32_t rowa, uint32_t rowb, int gi0, int G0, const __half* sc0, const __half* sc1,
                        float (&yy)[4]) {
        constexpr int NB = decltype(nb_tag)::value;
        uint32_t w0[NB][GE::TW], w1[NB][GE::TW];
#pragma unroll
        for (int n = 0; n < NB; ++n) {
            const uint32_t off = (uint32_t)((gi0 + n) * (kTileRows * GB));
            if constexpr (GE::TW == 1) {
                w0[n][0] = lds32(rowa + off); w1[n][0] = lds32(rowb + off);
            } else if constexpr (GE::TW == 2) {
                const uint2 v0 = lds64(rowa + off), v1 = lds64(rowb + off);
                w0[n][0] = v0.x; w0[n][1] = v0.y; w1[n][0] = v1.x; w1[n][1] = v1.y;
            } else {
                const uint4 v0 = lds128(rowa + off), v1 = lds128(rowb + off);
                w0[n][0] = v0.x; w0[n][1] = v0.y; w0[n][2] = v0.z; w0[n][3] = v0.w;
                w1[n][0] = v1.x; w1[n][1] = v1.y; w1[n][2] = v1.z; w1[n][3] = v1.w;
            }
        }
        const uint32_t xg = xs_lane_u32 + (uint32_t)(G0 + gi0) * GSTRIDE;
        float accA[NB][4], accB[NB][4];
#pragma unroll
        for (int i = 0; i < GE::TW; ++i) {
#pragma unroll
            for (int cp = 0; cp < GE::NCLS / 2; ++cp) {
                constexpr uint32_t MK = GE::MASK;
                const uint32_t m0 = MK << (BITS * (2 * cp)), m1 = MK << (BITS * (2 * cp + 1));
#pragma unroll
                for (int n = 0; n < NB; ++n) {
                    const uint4 bb = lds128(xg + (uint32_t)n * GSTRIDE + (i * (GE::NCLS / 2) + cp) * (M * 4 * 16));
                    const uint32_t a0 = w0[n][i], a1 = w1[n][i], h0 = a0 >> 8, h1 = a1 >> 8;
                    if (i == 0 && cp == 0) {
                        mma_f16_first(accA[n], a0 & m0, a1 & m0, h0 & m0, h1 & m0, bb.x, bb.y);
                        mma_f16_first(accB[n], a0 & m1, a1 & m1, h0 & m1, h1 & m1, bb.z, bb.w);
                    } else {
                        mma_f16(accA[n], a0 & m0, a1 & m0, h0 & m0, h1 & m0, bb.x, bb.y);
                        mma_f16(accB[n], a0 & m1, a1 & m1, h0 & m1, h1 & m1, bb.z, bb.w);
                    }
                }
            }
        }
#pragma unroll
        for (int n = 0; n < NB; ++n) {
            const int G = G0 + gi0 + n;
            float2 ga, gb;
            if constexpr (M % 2 == 0) {
                const float4 gq = lds128f(gx_lane_u32 + (uint32_t)G * (M * 8));
                ga = make_float2(gq.x, gq.y); gb = make_float2(gq.z, gq.w);
            } else {
                ga = lds64f(gx_a_u32 + (uint32_t)G * (M * 8)); gb = lds64f(gx_b_u32 + (uint32_t)G * (M * 8));
            }
            const float s0 = __half2float(sc0[gi0 + n]), s1 = __half2float(sc1[gi0 + n]);
            yy[0] = fmaf(s0, fmaf(ga.y, accA[n][0] + accB[n][0], -ga.x), yy[0]);
            yy[1] = fmaf(s0, fmaf(gb.y, accA[n][1] + accB[n][1], -gb.x), yy[1]);
            yy[2] = fmaf(s1, fmaf(ga.y, accA[n][2] + accB[n][2], -ga.x), yy[2]);
            yy[3] = fmaf(s1, fmaf(gb.y, accA[n][3] + accB[n][3], -gb.x), yy[3]);
        }
    };

    // Residual projections computed by other CTAs: the reader warp requests a small table now (the
    // producers publish right after their own barrier) and checks the tags one ring slot later.
    const int t_entries = t_inline ? p.t_parts * a.rank * M : 0;
    unsigned long long t_early[2] = {0ull, 0ull};
    bool t_requested = false;
    bool t_pending = t_reader;                      // this warp still owes the CTA the table of t
    if (t_pending && t_inline && t_entries <= 64) {
        t_requested = true;
#pragma unroll
        for (int e = 0; e < 2; ++e)
            if (lane + 32 * e < t_entries) t_early[e] = ld_relaxed_u64(t_entry(a, M, lane + 32 * e));
    }
    auto publish_table = [&]() {
        pipe_build_t_table<M>(p, smem, reinterpret_cast<float*>(smem + p.off_red) + kPipeWarps * QGEMV_MAX_M, t_tag,
                              t_early[0], t_early[1], t_requested);
        __syncwarp();
        if (lane == 0) { __threadfence_block(); atomicExch(t_flag, 1); }
        t_pending = false;
        PTRACE(12);
    };

    float y[4] = {0.f, 0.f, 0.f, 0.f};
    int stage = 0;
    uint32_t phases = 0;                            // bit s: parity of the next completion of slot s's barrier
    bool first = true;
#ifdef QGEMV_TRACE
    unsigned long long waited_ns = 0, epilogue_ns = 0, iterations = 0;
#endif
    for (;;) {
        __syncwarp();                               // lane 0's descriptor of this slot is visible
        const uint4 mt = lds128(meta_u32 + stage * 16);          // tile, chunk, slot, last-of-run
        if ((int)mt.x < 0) break;
        {                                           // the slot's bytes have landed
            PTRACE_NOW(w0_);
            const uint32_t bar = bars_u32 + stage * 8, parity = (phases >> stage) & 1u;
            int spins = 0;
            while (!mbar_try_wait(bar, parity)) {
                if (++spins > kBarSpinLimit) { atomicExch(a.counters + kWsStatusIdx, 2); break; }
            }
            phases ^= 1u << stage;
#ifdef QGEMV_TRACE
            PTRACE_NOW(w1_);
            waited_ns += w1_ - w0_; ++iterations;
#endif
        }
        if (first) { PTRACE(3); first = false; }
        const int ch = (int)mt.y;
        const uint32_t rowa = lane_row_u32 + stage * GE::STAGE_BYTES, rowb = rowa + 8 * GB;
        const uint32_t sca = lane_sc_u32 + stage * GE::STAGE_BYTES + (((uint32_t)ch * GE::CG) & 7u) * 2, scb = sca + 8 * 16;
        __align__(16) __half sc0[8], sc1[8];
        if constexpr (GE::CG == 8) {
            *reinterpret_cast<uint4*>(sc0) = lds128(sca); *reinterpret_cast<uint4*>(sc1) = lds128(scb);
        } else if constexpr (GE::CG == 4) {
            *reinterpret_cast<uint2*>(sc0) = lds64(sca); *reinterpret_cast<uint2*>(sc1) = lds64(scb);
        } else {
            *reinterpret_cast<uint32_t*>(sc0) = lds32(sca); *reinterpret_cast<uint32_t*>(sc1) = lds32(scb);
        }
        const int G0 = ch * GE::CG;
        if (G0 + GE::CG <= ng_total) {             // full chunk: straight-line code, groups interleaved in batches
            constexpr int NB = GE::CG < kBatchGroups ? GE::CG : kBatchGroups;
#pragma unroll
            for (int gi0 = 0; gi0 < GE::CG; gi0 += NB)
                do_batch(std::integral_constant<int, NB>{}, rowa, rowb, gi0, G0, sc0, sc1, y);
        } else {                                   // last, shorter chunk of a row
#pragma unroll
            for (int gi = 0; gi < GE::CG; ++gi)
                if (G0 + gi < ng_total)
                    do_group(rowa, rowb, gi, G0 + gi, __half2float(sc0[gi]), __half2float(sc1[gi]), y);
        }
        __syncwarp();                               // every lane is done reading the slot before it is refilled
        issue_next(stage);
        stage = stage + 1 == nstages ? 0 : stage + 1;
        if (t_pending) publish_table();             // before this warp could be the one that finishes a tile
        if (mt.w) {                                 // run complete: park its partial sums, count the arrival
            if (t < TT) sts128f(slots_u32 + mt.z * SLOT_BYTES, make_float4(y[0], y[1], y[2], y[3]));
            y[0] = y[1] = y[2] = y[3] = 0.f;
            const int tile = (int)mt.x, lt = tile - T0;
            __syncwarp();
            int old = 0;
            if (lane == 0) { __threadfence_block(); old = atomicAdd(cnt + lt, 1); }
            old = __shfl_sync(0xffffffffu, old, 0);
            if (old == p.rpt - 1) {                 // last run of the tile: add the runs in run order and finish it
                PTRACE_NOW(e0_);
                __threadfence_block();
                float yy[4] = {0.f, 0.f, 0.f, 0.f};
                if (t < TT) {
                    const uint32_t s0 = slots_u32 + (uint32_t)(lt * p.rpt) * SLOT_BYTES;
                    for (int j = 0; j < p.rpt; ++j) {
                        const float4 v = lds128f(s0 + j * SLOT_BYTES);
                        yy[0] += v.x; yy[1] += v.y; yy[2] += v.z; yy[3] += v.w;
                    }
                }
                if (EX && a.rank > 0) {             // the table of t is built by the reader warp early on
                    int spins = 0;
                    while (ld_volatile_shared(t_flag) == 0) {
                        if (++spins > kFlagSpinLimit) { if (lane == 0) atomicExch(a.counters + kWsStatusIdx, 1); break; }
                        __nanosleep(20);
                    }
                    __threadfence_block();
                }
                PTRACE(14);
                const bool pre = p.epi_async && lt < p.epi_tiles && (tile + 1) * kTileRows <= a.n;
                finish_tile<M, BF16, EX>(p, smem, tile, yy, pre ? smem + p.off_epi + (size_t)lt * p.epi_bytes : nullptr);
#ifdef QGEMV_TRACE
                PTRACE_NOW(e1_);
                epilogue_ns += e1_ - e0_;
#endif
            }
        }
    }
    if (t_pending) publish_table();                 // a reader warp without work still owes the table
    PTRACE(5);
#ifdef QGEMV_TRACE
    PTRACE_VAL(11, waited_ns); PTRACE_VAL(13, iterations); PTRACE_VAL(15, epilogue_ns);
#endif
    if (t_inline && a.rank > 0 && tid == 0) {
        // The last CTA to get here advances the launch count (every CTA has read it, and every reader
        // has its projections) and clears the arrival counter for the next launch.
        const int old = atomicAdd(a.counters + kWsDoneIdx, 1);
        if (old == (int)gridDim.x - 1) {
            a.counters[kWsEpochIdx] = (int)t_tag;
            a.counters[kWsDoneIdx] = 0;
        }
    }
}

template <int BITS, int GB, int CB, int M, bool BF16, bool EX>
int pipe_launch_ex(const MmaArgs& p, const PipeMaps& tm, int grid, int smem_bytes, cudaStream_t s) {
    auto kern = qgemv_pipe_kernel<BITS, GB, CB, M, BF16, EX>;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem) != cudaSuccess)
            return check_launch("cudaFuncSetAttribute(qgemv_pipe_kernel)");
        // all of the SM's unified cache as shared memory, so that two CTAs of 113 KB fit
        if (cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess)
            return check_launch("cudaFuncSetAttribute(qgemv_pipe_kernel, carveout)");
        configured[dev] = true;
    }
    // Programmatic dependent launch: the grid may become resident while the previous kernel of the
    // stream is still running; it touches only static operands until its griddepcontrol.wait.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(p.nw * 32);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, p, tm) != cudaSuccess) return check_launch("qgemv_pipe_kernel");
    return check_launch("qgemv_pipe_kernel");
}

template <int BITS, int GB, int CB, int M, bool BF16>
int pipe_launch_one(const MmaArgs& p, const PipeMaps& tm, int grid, int smem_bytes, cudaStream_t s) {
    if (p.a.oc > 0 || p.a.rank > 0) return pipe_launch_ex<BITS, GB, CB, M, BF16, true>(p, tm, grid, smem_bytes, s);
    return pipe_launch_ex<BITS, GB, CB, M, BF16, false>(p, tm, grid, smem_bytes, s);
}
template <int BITS, int GB, int CB, int M>
int pipe_launch_bf(const MmaArgs& p, const PipeMaps& tm, bool bf16, int grid, int smem, cudaStream_t s) {
    return bf16 ? pipe_launch_one<BITS, GB, CB, M, true>(p, tm, grid, smem, s) : pipe_launch_one<BITS, GB, CB, M, false>(p, tm, grid, smem, s);
}
template <int BITS, int GB, int CB>
int pipe_launch_m(const MmaArgs& p, const PipeMaps& tm, bool bf16, int grid, int smem, cudaStream_t s) {
    switch (p.a.m) {
        case 1: return pipe_launch_bf<BITS, GB, CB, 1>(p, tm, bf16, grid, smem, s);
        case 2: return pipe_launch_bf<BITS, GB, CB, 2>(p, tm, bf16, grid, smem, s);
        case 3: return pipe_launch_bf<BITS, GB, CB, 3>(p, tm, bf16, grid, smem, s);
        default: return pipe_launch_bf<BITS, GB, CB, 4>(p, tm, bf16, grid, smem, s);
    }
}
template <int BITS>
int pipe_launch_gb(const MmaArgs& p, const PipeMaps& tm, int gb, int cb, bool bf16, int grid, int smem, cudaStream_t s) {
    if (gb == 16) return pipe_launch_m<BITS, 16, 128>(p, tm, bf16, grid, smem, s);
    if (gb == 32) return cb == 128 ? pipe_launch_m<BITS, 32, 128>(p, tm, bf16, grid, smem, s) : pipe_launch_m<BITS, 32, 256>(p, tm, bf16, grid, smem, s);
    return cb == 128 ? pipe_launch_m<BITS, 64, 128>(p, tm, bf16, grid, smem, s) : pipe_launch_m<BITS, 64, 256>(p, tm, bf16, grid, smem, s);
}

}  // namespace

// One translation unit per bit width keeps the build parallel: QGEMV_INST_BITS selects which
// instantiations (and, for 2, the planner) this compilation provides.
#if !defined(QGEMV_INST_BITS) || QGEMV_INST_BITS == 2
int launch_pipe_int2(const MmaArgs& p, const PipeMaps& tm, int gb, int cb, bool bf16, int grid, int smem, cudaStream_t s) {
    return pipe_launch_gb<2>(p, tm, gb, cb, bf16, grid, smem, s);
}
#endif
#if !defined(QGEMV_INST_BITS) || QGEMV_INST_BITS == 4
int launch_pipe_int4(const MmaArgs& p, const PipeMaps& tm, int gb, int cb, bool bf16, int grid, int smem, cudaStream_t s) {
    return pipe_launch_gb<4>(p, tm, gb, cb, bf16, grid, smem, s);
}
#endif

#if !defined(QGEMV_INST_BITS) || QGEMV_INST_BITS == 2
// Plan of the pipelined kernel, or ok == false when the shape should stay with the phased kernel
// (`base` is that kernel's plan for the same problem).
MmaPlan plan_pipe(const qgemv_problem& p, const MmaPlan& base) {
    MmaPlan pl = base;
    pl.ok = false;
    if (!base.ok || !base.tile_aligned) return pl;
    const int gb = base.gb;
    // Chunk = packed bytes per row per ring slot.  128-byte chunks give a ring of many small slots (more
    // copies in flight per byte of shared memory), 256-byte chunks fewer trips through the loop.
    int cb = gb == 16 ? 128 : 256;
    if (gb != 16 && (p.debug & QGEMV_DEBUG_CHUNK128)) cb = 128;
    const int cg = cb / gb, stage_bytes = kTileRows * cb + kTileRows * 16;
    pl.chunk = cb;
    pl.nch = (pl.ng + cg - 1) / cg;
    {
        auto al0 = [](const void* q, size_t a) { return reinterpret_cast<uintptr_t>(q) % a == 0; };
        // scale rows go through the copy engine in aligned blocks of 8 scales (16 bytes; zero fill past the row's end)
        pl.scales_async = (p.lds % 8 == 0) && al0(p.scales, 16) ? 1 : 0;
    }
    const int sms = sm_count();
    const int grid = pl.nt < sms ? pl.nt : sms;
    const int tiles_max = (pl.nt + grid - 1) / grid, tiles_min = pl.nt / grid;
    const int slot_bytes = 8 * ((p.m + 1) / 2) * 16;
    // Runs: consecutive chunks of one tile; one chunk per run unless the partial sums of a CTA's runs
    // would then need more than 16 KB of shared memory.
    int rlen = 1, rpt = pl.nch;
    for (;; rlen *= 2) {
        rpt = (pl.nch + rlen - 1) / rlen;
        if ((long long)tiles_max * rpt * slot_bytes <= 16384 || rlen >= pl.nch) break;
    }
    const int slot_cap = tiles_max * rpt;
    if ((long long)slot_cap * slot_bytes > 49152) return pl;
    pl.grid = grid; pl.rlen = rlen; pl.rpt = rpt; pl.tile_aligned = 1;

    // warps: as many as the smallest CTA has runs for, at most 8
    int nw_cap = tiles_min * rpt;
    nw_cap = nw_cap < 1 ? 1 : (nw_cap > kPipeWarps ? kPipeWarps : nw_cap);

    // epilogue operands: prefetched for the first tiles of a CTA, up to 12 KB
    // (a tile's operand block is the destination of tensor-map copies: 128-byte aligned)
    const int epi_bytes = align_up(kTileRows * (pl.ocb + pl.rb) + 32, 128);
    int epi_tiles = 0;
    if (pl.epi_async) {
        epi_tiles = 12288 / epi_bytes;
        if (epi_tiles > tiles_max) epi_tiles = tiles_max;
    }

    int off = 64;
    pl.off_cnt = off;   off = align_up(off + (tiles_max + 2) * 4, 16);
    pl.off_red = off;   off = align_up(off + (kPipeWarps * QGEMV_MAX_M + 64) * 4, 16);     // job partial sums + 64 floats of table scratch
    pl.off_tt = off;    off = align_up(off + (p.rank * p.m > 64 ? p.rank * p.m : 64) * 4, 16);
    pl.off_xo = off;    off = align_up(off + p.outliers * p.m * 4, 16);
    pl.off_gx = off;    off = align_up(off + pl.ng * p.m * 8, 16);
    pl.off_slots = off; off = align_up(off + slot_cap * slot_bytes, 128);
    pl.off_xs = off;    off = align_up(off + p.m * p.k_padded * 2, 128);
    pl.off_meta = off;  off += kPipeWarps * kPipeMaxStages * 16;
    pl.off_bar = off;   off = align_up(off + kPipeWarps * kPipeMaxStages * 8 + 8, 128);
    pl.off_epi = off;   off = align_up(off + epi_tiles * epi_bytes, 128);
    pl.off_ring = off;
    pl.epi_bytes = epi_bytes;
    pl.epi_tiles = epi_tiles;

    // Ring.  Warps first (the main loop is bound by instruction issue: two warps per scheduler), then
    // as many slots per warp as fit, up to 4 (8 for 128-byte chunks).  First within half an SM, so that
    // the next launch's CTA fits beside this one; if not even 6 warps (or all the CTA has work for)
    // with 2 slots fit there -- very long K, or M = 4 with a long K -- within a whole SM.
    const int max_stages = cb == 128 ? kPipeMaxStages : 4;
    int nw = 0, stages = 0;
    const int forced_nw = (p.debug >> 8) & 0xff, forced_st = (p.debug >> 16) & 0xf;
    for (int budget_i = 0; budget_i < 2 && !nw; ++budget_i) {
        const int budget = (budget_i == 0 ? kHalfSmSmem : kMaxDynSmem) - off;
        const int w_min = budget_i == 0 ? (nw_cap < 6 ? nw_cap : 6) : 1;
        for (int w = nw_cap; w >= w_min && !nw; --w) {
            if (forced_nw && w != forced_nw) continue;
            int st = budget / (w * stage_bytes);
            if (st > max_stages) st = max_stages;
            if (forced_st) { if (st < forced_st) continue; st = forced_st; }
            if (st >= 2) { nw = w; stages = st; }
        }
    }
    if (!nw) return pl;
    pl.nw = nw; pl.stages = stages;
    pl.smem_bytes = off + nw * stages * stage_bytes;

    // residual projections inside the kernel: K is cut into parts of 8 * threads * pv columns
    const int pvmax = p.m == 1 ? 4 : (p.m == 2 ? 3 : 2);
    int pv = 1, parts = 0;
    for (;; ++pv) {                      // fewest pieces per thread that keep the jobs within the grid
        parts = (p.k_original + nw * 256 * pv - 1) / (nw * 256 * pv);
        if ((parts <= kMaxTParts && p.rank * parts <= grid) || pv >= pvmax) break;
    }
    auto al = [](const void* q, size_t a) { return reinterpret_cast<uintptr_t>(q) % a == 0; };
    pl.t_parts = parts; pl.t_pv = pv;
    pl.t_inline = (p.rank > 0 && p.k_original % 8 == 0 && p.ldv % 8 == 0 && al(p.res_v, 16) && parts <= kMaxTParts &&
                   p.rank * parts <= grid) ? 1 : 0;
    // L2 announcements: every chunk of a warp beyond its ring, as long as the whole problem is at most
    // a quarter of the 126 MB L2 (so that two launches in flight never push each other out).
    const long long weight_bytes = (long long)p.n * p.k_padded * p.bits / 8;
    const int chunks_per_warp = (tiles_max * rpt + nw - 1) / nw * rlen;
    pl.l2_chunks = (weight_bytes <= (32ll << 20) && !(p.debug & QGEMV_DEBUG_NO_L2_HINT)) ? chunks_per_warp : 0;
    static const char* names[2][3] = {{"pipe_int2_g64", "pipe_int2_g128", "pipe_int2_g256"},
                                      {"pipe_int4_g32", "pipe_int4_g64", "pipe_int4_g128"}};
    pl.name = names[p.bits == 2 ? 0 : 1][gb == 16 ? 0 : gb == 32 ? 1 : 2];
    pl.variant = 2;
    pl.ok = true;
    return pl;
}

int launch_pipe_int2(const MmaArgs& p, const PipeMaps& tm, int gb, int cb, bool bf16, int grid, int smem, cudaStream_t s);
int launch_pipe_int4(const MmaArgs& p, const PipeMaps& tm, int gb, int cb, bool bf16, int grid, int smem, cudaStream_t s);

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime (the library does not link against the driver).
EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            (void)cudaGetLastError();
            p = nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// rank-2 or rank-3 map with unit element strides, no interleave, no swizzle, zero fill outside the tensor
bool encode(CUtensorMap* m, CUtensorMapDataType dt, int rank, const void* base, const cuuint64_t* dims,
            const cuuint64_t* strides_bytes, const cuuint32_t* box) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    const cuuint32_t ones[3] = {1, 1, 1};
    return fn(m, dt, (cuuint32_t)rank, const_cast<void*>(base), dims, strides_bytes, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

int launch_pipe(const Args& a, int bits, bool bf16, const MmaPlan& pl, int debug, cudaStream_t s) {
    MmaArgs p{};
    p.a = a;
    p.nt = pl.nt; p.nch = pl.nch; p.ng = pl.ng;
    p.row_bytes = a.kpad * bits / 8;
    p.nw = pl.nw; p.stages = pl.stages;
    p.rlen = pl.rlen; p.rpt = pl.rpt; p.runs = pl.nt * pl.rpt;
    p.uq = pl.nt / pl.grid; p.urem = pl.nt % pl.grid;
    p.scales_async = pl.scales_async; p.epi_async = pl.epi_async; p.ocb = pl.ocb; p.rb = pl.rb;
    p.epi_bytes = pl.epi_bytes; p.epi_tiles = pl.epi_tiles;
    p.off_xo = pl.off_xo; p.off_gx = pl.off_gx; p.off_slots = pl.off_slots; p.off_epi = pl.off_epi;
    p.off_meta = pl.off_meta; p.off_xs = pl.off_xs; p.off_ring = pl.off_ring;
    p.off_cnt = pl.off_cnt; p.off_red = pl.off_red; p.off_tt = pl.off_tt; p.off_bar = pl.off_bar;
    p.t_inline = pl.t_inline; p.t_parts = pl.t_parts; p.t_pv = pl.t_pv;
    p.l2_chunks = pl.l2_chunks;
    p.debug = debug;
    p.wait_for_x = (a.rank > 0 && !pl.t_inline) ? 0 : 1;
    p.tile_aligned = 1;

    // Tensor maps.  Codes: the packed matrix seen as [group bytes][row][group] (strides 1, ldp, GB), box
    // GB x 16 rows x CG groups -> one request per ring slot.  Should the driver refuse that view, the
    // plain [row bytes][row] matrix with one GB x 16 box per group of a chunk serves instead.
    PipeMaps tm{};
    const int gb = pl.gb, cg = pl.chunk / gb;
    {
        const cuuint64_t dims[3] = {(cuuint64_t)gb, (cuuint64_t)a.n, (cuuint64_t)pl.ng};
        const cuuint64_t strides[2] = {(cuuint64_t)a.ldp, (cuuint64_t)gb};
        const cuuint32_t box[3] = {(cuuint32_t)gb, (cuuint32_t)kTileRows, (cuuint32_t)cg};
        p.tma3d = (!(debug & QGEMV_DEBUG_BOX_PER_GROUP) && encode(&tm.w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a.packed, dims, strides, box)) ? 1 : 0;
        if (!p.tma3d) {
            const cuuint64_t dims2[2] = {(cuuint64_t)pl.ng * gb, (cuuint64_t)a.n};
            const cuuint64_t strides2[1] = {(cuuint64_t)a.ldp};
            const cuuint32_t box2[2] = {(cuuint32_t)gb, (cuuint32_t)kTileRows};
            if (!encode(&tm.w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.packed, dims2, strides2, box2)) {
                set_error("qgemv_run: cuTensorMapEncodeTiled failed for the packed matrix");
                return QGEMV_ERR_LAUNCH;
            }
        }
    }
    if (p.scales_async) {
        const cuuint64_t dims[2] = {(cuuint64_t)pl.ng, (cuuint64_t)a.n};
        const cuuint64_t strides[1] = {(cuuint64_t)a.lds * 2};
        const cuuint32_t box[2] = {8, (cuuint32_t)kTileRows};
        if (!encode(&tm.s, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, a.scales, dims, strides, box)) p.scales_async = 0;
    }
    if (p.epi_async && a.oc > 0) {
        const cuuint64_t dims[2] = {(cuuint64_t)a.oc, (cuuint64_t)a.n};
        const cuuint64_t strides[1] = {(cuuint64_t)a.ldow * 2};
        const cuuint32_t box[2] = {(cuuint32_t)a.oc, (cuuint32_t)kTileRows};
        if (!encode(&tm.ow, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, a.ow, dims, strides, box)) p.epi_async = 0;
    }
    if (p.epi_async && a.rank > 0) {
        const cuuint64_t dims[2] = {(cuuint64_t)a.rank, (cuuint64_t)a.n};
        const cuuint64_t strides[1] = {(cuuint64_t)a.ldu * 2};
        const cuuint32_t box[2] = {(cuuint32_t)a.rank, (cuuint32_t)kTileRows};
        if (!encode(&tm.ru, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, a.ru, dims, strides, box)) p.epi_async = 0;
    }
    return bits == 2 ? launch_pipe_int2(p, tm, pl.gb, pl.chunk, bf16, pl.grid, pl.smem_bytes, s)
                     : launch_pipe_int4(p, tm, pl.gb, pl.chunk, bf16, pl.grid, pl.smem_bytes, s);
}
#endif

}  // namespace qgemv
