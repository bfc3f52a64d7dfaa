// Barrier-free fused GEMV for packed groupwise INT2 / INT4 weights, M <= 4, sm_100a.
//
// Same arithmetic and the same per-warp ring of asynchronous copies as qgemv_mma.cu (codes used in
// place as fp16 subnormals, mma.sync.m16n8k16 for the dot products, fp32 group combine, fused outlier /
// residual / bias / activation epilogue).  What changes is how one launch is laid out in time, because
// at these sizes (5 - 60 MB of weights, a few microseconds at HBM rate) the fixed parts of a launch cost
// as much as the stream itself:
//
//  * Weights before the dependency.  Packed codes, scales, outlier-weight rows, residual rows and bias
//    are static, so a CTA fills its ring of asynchronous copies, announces the chunks that follow the
//    ring to L2, and passes on the caller's L2 hint (normally the next GEMV's packed codes) BEFORE
//    griddepcontrol.wait.  Launches carry the programmatic-stream-serialisation attribute and signal
//    griddepcontrol.launch_dependents first thing, so a CTA of the next launch starts on an SM the
//    moment this launch's CTA there has finished, while other SMs are still in their tail.
//  * After the wait only x-dependent work is left: load x (L2 hits), stage it in B-fragment order,
//    gather the outlier activations, one CTA barrier, main loop.
//  * No barrier after the main loop.  A warp that completes a run parks its partial sums and bumps
//    the tile's arrival counter in shared memory; whichever warp arrives last adds the runs in run
//    order (bit-repeatable) and finishes the tile at once -- outlier columns, residual, bias,
//    activation, store -- from operands that were prefetched with the ring.  Epilogues overlap the
//    other warps' streaming, and a CTA is gone as soon as its last tile is.
//  * CTAs always own whole tiles (no hand-over between CTAs through global memory).  Shapes whose
//    balance needs shared tiles stay with the phased kernel.
//
// Measured on B200 (microseconds per GEMV in a chain of 16, INT4 benchmark shape) this kernel takes
// 13.7 with 16 warps and one CTA per SM, the phased kernel 10.4; it is slower on the INT2 shapes too
// (5.9 against 4.2 on the 4096 x 4096 one).  The phase trace shows why: a CTA lives for the whole launch
// (prologue 2.5 us, x staging 3 us, stream 7 us), so the next launch's CTA cannot become resident
// early, and whole tiles per CTA leave the last CTA 5 us behind the median one where the phased
// kernel's dealt runs end together.  The planner therefore never picks this kernel by itself
// (QGEMV_KERNEL_MMA_PIPE asks for it); it stays as the base for a CTA-wide ring.
//
// Variants measured on the way and dropped (same shape and unit):
//   - two CTAs of 8 warps per SM, so that the next launch's CTA sits beside the running one with its
//     ring already full: 17.7.  A warp of this kernel is latency bound (about 1.2 us per 16 x 256-byte
//     chunk whatever else runs), so halving the warps of the running CTA halves its speed; and the
//     waiting CTA's 16-byte copies queue in the load/store path the running CTA's shared-memory loads
//     share (a dependent 8-byte load took 3 us);
//   - the ring filled by the bulk-copy engine instead of per-thread copies: one bulk copy per row per
//     slot 23, one 3-D tensor box [group bytes][16 rows][groups] per slot 17.4, swizzled 2-D boxes of
//     128 bytes x 16 rows 19.6 - 22.8, with 7 to 32 warps per CTA.  The engine keeps only a few
//     requests in flight per SM, and requests of 2 - 4 KB (all a per-warp ring can offer) then move
//     about 20 KB per microsecond per SM, half of what the stream needs.  Large boxes need a ring
//     shared by the whole CTA; that is future work;
//   - 32 warps of 64 registers per CTA: 22.4; 8 or 12 warps: 19.1 / 16.6; ring slots of 128 bytes per
//     row: 18.0; filling only the first slot before the dependency wait: 14.4; no L2 announcements: 13.6.
//
// The residual projections t = V.x are computed by the first rank * parts CTAs right after the
// wait and travel to the others as {value, launch tag} words, exactly as in qgemv_mma.cu; every
// wait on them is bounded and reports through the workspace's status word.
//
// Replaces _decode_gemv (ai_accel_lab/kernels/decode_int2.py:43-96) and _decode_int4_gemv
// (ai_accel_lab/kernels/groupwise_int4.py:85-107) of the reference project.
#include "qgemv_mma_dev.cuh"

namespace qgemv {
namespace {

#ifndef QGEMV_PIPE_WARPS
#define QGEMV_PIPE_WARPS 16
#endif
constexpr int kPipeWarps = QGEMV_PIPE_WARPS;  // warps per CTA the kernel is compiled for (16: 128 registers per thread; 32: 64)
constexpr int kPipeMaxStages = 8;             // ring descriptors reserved per warp
constexpr int kFlagSpinLimit = 1 << 22;       // bound of the in-CTA wait for the table of residual projections
constexpr int kTagSpinLimit = 1 << 20;        // bound of the wait for another CTA's projection (about 30 ms)
constexpr int kTagSpinLimitDebug = 1 << 7;    // ... with QGEMV_DEBUG_DROP_PROJECTIONS (a few microseconds)

// Optional phase trace (build with -DQGEMV_TRACE): lane 0 of every warp stores the global nanosecond
// timer at a few points into the upper half of the partial-sum scratch; bits 24..27 of the debug
// word select one of 12 regions, so that the launches of a chain can be told apart.
#ifdef QGEMV_TRACE
constexpr int kTraceWarps = 8;                // warps of a CTA (the first ones) that record
#define PTRACE(slot)                                                                            \
    do {                                                                                        \
        if ((threadIdx.x & 31) == 0 && threadIdx.x < 32 * kTraceWarps) {                        \
            unsigned long long t_;                                                              \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_) :: "memory");                  \
            reinterpret_cast<unsigned long long*>(p.a.partial + (kMaxPartialFloats / 2))        \
                [((size_t)((p.debug >> 24) & 15) * 148 * kTraceWarps +                          \
                  (size_t)blockIdx.x * kTraceWarps + (threadIdx.x >> 5)) * 16 + (slot)] = t_;   \
        }                                                                                       \
    } while (0)
#else
#define PTRACE(slot) do { } while (0)
#endif

// Announce `bytes` (multiple of 16) at a 16-byte aligned global address to L2; no data reaches the SM.
__device__ __forceinline__ void l2_prefetch_bulk(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ int ld_volatile_shared(const int* p) {
    int v; asm volatile("ld.volatile.shared.s32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory"); return v;
}
// cp.async.wait_group takes an immediate: leave at most `pending` (0..8) groups of this thread in flight.
__device__ __forceinline__ void cp_async_wait_dyn(int pending) {
    switch (pending) {
        case 0: cp_async_wait<0>(); break;
        case 1: cp_async_wait<1>(); break;
        case 2: cp_async_wait<2>(); break;
        case 3: cp_async_wait<3>(); break;
        case 4: cp_async_wait<4>(); break;
        case 5: cp_async_wait<5>(); break;
        case 6: cp_async_wait<6>(); break;
        case 7: cp_async_wait<7>(); break;
        default: cp_async_wait<8>(); break;
    }
}

// ---------------------------------------------------------------------------------------------
// Activation staging after the dependency wait (whole CTA, no barrier inside; the caller's barrier
// publishes the results): x -> fp16 multiplicands in B-fragment order with the per (group, row)
// offset term and power-of-two normalisation (see qgemv_mma.cu for the number format), the outlier
// activations x[m][outlier_idx[j]] as fp32, and, in the CTAs that carry one, a residual-projection
// job.  Every global load is issued before the first result is needed.
// `cols` holds the outlier column of entries tid, tid + nthr, ... (read before the wait).
// ---------------------------------------------------------------------------------------------
template <int BITS, int GB, int M, bool BF16, bool EX, typename AfterLoads>
__device__ __forceinline__ void pipe_stage_x(const MmaArgs& p, unsigned char* smem, const int (&cols)[4], AfterLoads after_loads) {
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
        after_loads();                                               // every load of x is in flight: the caller may queue more copies
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
    } else {
        after_loads();
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
__global__ void __launch_bounds__(kPipeWarps * 32, 1) qgemv_pipe_kernel(const __grid_constant__ MmaArgs p) {
    using GE = Geo<BITS, GB, CB>;
    constexpr int TT = (M + 1) / 2;                   // quad lanes that hold useful output columns
    constexpr int SLOT_BYTES = 8 * TT * 16;           // one run's partial sums in shared memory
    extern __shared__ __align__(128) unsigned char smem[];
    const Args& a = p.a;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    // Release the next launch of the stream at once: its CTAs take the place of this launch's CTAs as
    // they finish and fill their rings while the rest of this launch is still in its tail.
    if (!(p.debug & QGEMV_DEBUG_LATE_TRIGGER)) pdl_launch_dependents();
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

    // ---- producer side --------------------------------------------------------------------------
    constexpr int PPR = GE::CB / 16;                 // 16-byte pieces per row of a full chunk
    constexpr int RPI = 32 / PPR;                    // rows covered by one warp-wide copy instruction
    const int lrow = lane / PPR, lcol = lane % PPR;
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
    constexpr int NIT = kTileRows / RPI;
    const size_t tile_stride = (size_t)kTileRows * a.ldp;
    const size_t it_stride = (size_t)RPI * a.ldp;
    const uint8_t* lane_src = a.packed + (size_t)lrow * a.ldp + lcol * 16;
    uint32_t dst_off[NIT];
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
        const int r = it * RPI + lrow;
        dst_off[it] = r * GE::PITCH + ((lcol ^ GE::swz(r)) << 4);
    }
    const __half* lane_sc = a.scales + (size_t)min(lane, kTileRows - 1) * a.lds;
    const size_t sc_tile_stride = (size_t)kTileRows * a.lds;
    const bool ragged_n = (a.n % kTileRows) != 0;
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
            const bool edge = ragged_n && pf_tile == p.nt - 1;        // rows past N are clamped to the last row
            if (ngr == GE::CG && !edge && p.scales_async) {
                // common case, straight-line: NIT row-group copies by every lane + one scale copy by lanes 0..15
                const uint8_t* src = lane_src + (size_t)pf_tile * tile_stride + (size_t)pf_ch * GE::CB;
#pragma unroll
                for (int it = 0; it < NIT; ++it) { cp_async16(sbase + dst_off[it], src); src += it_stride; }
                const __half* ssrc = lane_sc + (size_t)pf_tile * sc_tile_stride + pf_ch * GE::CG;
                const uint32_t sdst = sbase + GE::SCALE_OFF + lane * 16;
                if (lane < kTileRows) {
                    if constexpr (GE::CG == 8) cp_async16(sdst, ssrc);
                    else if constexpr (GE::CG == 4) cp_async8(sdst, ssrc);
                    else cp_async4(sdst, ssrc);
                }
            } else {
                const int pieces = (ngr * GB) >> 4;
                if (lcol < pieces) {
                    const uint8_t* src = a.packed + (size_t)pf_ch * GE::CB + lcol * 16;
#pragma unroll
                    for (int it = 0; it < NIT; ++it) {
                        const int row = min(pf_tile * kTileRows + it * RPI + lrow, a.n - 1);
                        cp_async16(sbase + dst_off[it], src + (size_t)row * a.ldp);
                    }
                }
                if (lane < kTileRows) {                   // this row's scales for the chunk
                    const __half* src = a.scales + (size_t)min(pf_tile * kTileRows + lane, a.n - 1) * a.lds + pf_ch * GE::CG;
                    if (p.scales_async && ngr == GE::CG) {
                        const uint32_t dst = sbase + GE::SCALE_OFF + lane * 16;
                        if constexpr (GE::CG == 8) cp_async16(dst, src);
                        else if constexpr (GE::CG == 4) cp_async8(dst, src);
                        else cp_async4(dst, src);
                    } else {
                        __half* d = reinterpret_cast<__half*>(ring + s * GE::STAGE_BYTES + GE::SCALE_OFF + lane * 16);
                        for (int i = 0; i < ngr; ++i) d[i] = __ldg(src + i);
                    }
                }
            }
            if (lane == 0) meta[s] = make_int4(pf_tile, pf_ch, pf_run - r0, pf_ch + 1 == pf_end);
            ++pf_ch;
        } else if (lane == 0) {
            meta[s] = make_int4(-1, 0, 0, 0);
        }
        cp_async_commit();
    };

    // ---- everything that does not depend on the previous kernel -----------------------------------
    // Oldest copy group: epilogue operands (outlier-weight rows, residual rows, bias) of the CTA's
    // first tiles, issued by all threads; the barrier that ends the prologue makes them visible.
    {
        const int opieces = EX ? p.ocb >> 4 : 0, upieces = EX ? p.rb >> 4 : 0;
        const int per_tile = kTileRows * (opieces + upieces) + (a.bias ? 2 : 0);
        const int full_tiles = a.n / kTileRows;                       // tiles that lie completely inside N
        const int npre = p.epi_async ? min(min(p.epi_tiles, ntl), max(0, full_tiles - T0)) : 0;
        const uint32_t epi_u32 = smem_u32(smem + p.off_epi);
        for (int i = tid; i < npre * per_tile; i += blockDim.x) {
            const int lt = i / per_tile, q = i - lt * per_tile;
            const int row0 = (T0 + lt) * kTileRows;
            const uint32_t dst = epi_u32 + lt * p.epi_bytes;
            if (q < kTileRows * opieces) {
                const int r = q % kTileRows, c = q / kTileRows;
                cp_async16(dst + r * p.ocb + c * 16, reinterpret_cast<const unsigned char*>(a.ow + (size_t)(row0 + r) * a.ldow) + c * 16);
            } else if (q < kTileRows * (opieces + upieces)) {
                const int qq = q - kTileRows * opieces, r = qq % kTileRows, c = qq / kTileRows;
                cp_async16(dst + kTileRows * p.ocb + r * p.rb + c * 16,
                           reinterpret_cast<const unsigned char*>(a.ru + (size_t)(row0 + r) * a.ldu) + c * 16);
            } else {
                const int c = q - kTileRows * (opieces + upieces);
                cp_async16(dst + kTileRows * (p.ocb + p.rb) + c * 16, reinterpret_cast<const unsigned char*>(a.bias + row0) + c * 16);
            }
        }
        cp_async_commit();
    }
    // The whole ring, or (QGEMV_DEBUG_SPLIT_FILL) only its first slot: loads of x issued behind queued weight
    // copies are served after them, so a ring that is still filling when the wait returns delays the
    // prologue; the remaining slots then go out right behind the loads of x.
    const int first_fill = (p.debug & QGEMV_DEBUG_SPLIT_FILL) ? 1 : nstages;
    for (int s = 0; s < first_fill; ++s) issue_next(s);
    // The chunks that follow the ring go to L2 now (one instruction per chunk: lanes 0..15 take a row
    // each), so that the main loop finds them there instead of in DRAM.
    if (p.l2_chunks > 0 && lane < kTileRows) {
        const int s_run = pf_run, s_tile = pf_tile, s_j = pf_j, s_ch = pf_ch, s_end = pf_end;
        for (int i = 0; i < p.l2_chunks && advance(); ++i) {
            const int row = pf_tile * kTileRows + lane;
            const int ngr = min(GE::CG, p.ng - pf_ch * GE::CG);
            if (row < a.n) l2_prefetch_bulk(a.packed + (size_t)row * a.ldp + (size_t)pf_ch * GE::CB, (uint32_t)(ngr * GB));
            ++pf_ch;
        }
        pf_run = s_run; pf_tile = s_tile; pf_j = s_j; pf_ch = s_ch; pf_end = s_end;
    }
    // The caller's hint (normally the packed codes of the next GEMV of the stream): this CTA announces
    // its 1/grid share to L2 in pieces of 4 KB, one request per piece, spread over the warps.
    if (a.hint_bytes > 0 && lane == 0 && !(p.debug & QGEMV_DEBUG_NO_L2_HINT)) {
        constexpr long long kPiece = 4096;
        const long long pieces = (a.hint_bytes + kPiece - 1) / kPiece;
        const long long per_cta = (pieces + grid - 1) / grid;
        const long long first = (long long)cta * per_cta, last = min(pieces, first + per_cta);
        for (long long i = first + warp; i < last; i += p.nw) {
            const long long off = i * kPiece;
            l2_prefetch_bulk(a.hint + off, (uint32_t)min(kPiece, a.hint_bytes - off));
        }
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
    pipe_stage_x<BITS, GB, M, BF16, EX>(p, smem, cols, [&]() {
        for (int s = first_fill; s < nstages; ++s) issue_next(s);
    });
    cp_async_wait_dyn(nstages);                       // the epilogue operands (oldest group) have landed
    __syncthreads();                                  // staged activations, counters and operands visible to every warp
    if (p.debug & QGEMV_DEBUG_LATE_TRIGGER) pdl_launch_dependents();
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
    const int sw16 = GE::swz(g) << 4;
    const uint32_t lane_row_u32 = ring_u32 + g * GE::PITCH;         // row g of slot 0 (row g+8 is 8 rows further)
    const uint32_t lane_sc_u32 = ring_u32 + GE::SCALE_OFF + g * 16;
    const int ng_total = p.ng;
    constexpr int GSTRIDE = GE::TW * (GE::NCLS / 2) * M * 4 * 16;    // bytes of staged x per group

    // One group of one chunk: G = absolute group index, gi = group inside the chunk.
    auto do_group = [&](uint32_t rowa, uint32_t rowb, int gi, int G, float s0, float s1, float (&yy)[4]) {
        const int lo = gi * GB + t * GE::TB;                          // logical byte offset of this lane's bytes
        const uint32_t off = (uint32_t)(((lo & ~15) ^ sw16) + (lo & 15));
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
    bool first = true;
    for (;;) {
        cp_async_wait_dyn(nstages - 1);         // all but the newest stages-1 groups are done: this slot has landed
        __syncwarp();
        const uint4 mt = lds128(meta_u32 + stage * 16);          // tile, chunk, slot, last-of-run
        if ((int)mt.x < 0) break;
        if (first) { PTRACE(3); first = false; }
        const int ch = (int)mt.y;
        const uint32_t rowa = lane_row_u32 + stage * GE::STAGE_BYTES, rowb = rowa + 8 * GE::PITCH;
        const uint32_t sca = lane_sc_u32 + stage * GE::STAGE_BYTES, scb = sca + 8 * 16;
        __align__(16) __half sc0[8], sc1[8];
        if constexpr (GE::CG == 8) {
            *reinterpret_cast<uint4*>(sc0) = lds128(sca); *reinterpret_cast<uint4*>(sc1) = lds128(scb);
        } else if constexpr (GE::CG == 4) {
            *reinterpret_cast<uint2*>(sc0) = lds64(sca); *reinterpret_cast<uint2*>(sc1) = lds64(scb);
        } else {
            *reinterpret_cast<uint32_t*>(sc0) = lds32(sca); *reinterpret_cast<uint32_t*>(sc1) = lds32(scb);
        }
        const int G0 = ch * GE::CG;
        if (G0 + GE::CG <= ng_total) {             // full chunk: straight-line code
#pragma unroll
            for (int gi = 0; gi < GE::CG; ++gi)
                do_group(rowa, rowb, gi, G0 + gi, __half2float(sc0[gi]), __half2float(sc1[gi]), y);
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
            }
        }
    }
    cp_async_wait<0>();
    if (t_pending) publish_table();                 // a reader warp without work still owes the table
    PTRACE(5);
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
int pipe_launch_ex(const MmaArgs& p, int grid, int smem_bytes, cudaStream_t s) {
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
    if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) return check_launch("qgemv_pipe_kernel");
    return check_launch("qgemv_pipe_kernel");
}

template <int BITS, int GB, int CB, int M, bool BF16>
int pipe_launch_one(const MmaArgs& p, int grid, int smem_bytes, cudaStream_t s) {
    if (p.a.oc > 0 || p.a.rank > 0) return pipe_launch_ex<BITS, GB, CB, M, BF16, true>(p, grid, smem_bytes, s);
    return pipe_launch_ex<BITS, GB, CB, M, BF16, false>(p, grid, smem_bytes, s);
}
template <int BITS, int GB, int CB, int M>
int pipe_launch_bf(const MmaArgs& p, bool bf16, int grid, int smem, cudaStream_t s) {
    return bf16 ? pipe_launch_one<BITS, GB, CB, M, true>(p, grid, smem, s) : pipe_launch_one<BITS, GB, CB, M, false>(p, grid, smem, s);
}
template <int BITS, int GB, int CB>
int pipe_launch_m(const MmaArgs& p, bool bf16, int grid, int smem, cudaStream_t s) {
    switch (p.a.m) {
        case 1: return pipe_launch_bf<BITS, GB, CB, 1>(p, bf16, grid, smem, s);
        case 2: return pipe_launch_bf<BITS, GB, CB, 2>(p, bf16, grid, smem, s);
        case 3: return pipe_launch_bf<BITS, GB, CB, 3>(p, bf16, grid, smem, s);
        default: return pipe_launch_bf<BITS, GB, CB, 4>(p, bf16, grid, smem, s);
    }
}
template <int BITS>
int pipe_launch_gb(const MmaArgs& p, int gb, int cb, bool bf16, int grid, int smem, cudaStream_t s) {
    if (gb == 16) return pipe_launch_m<BITS, 16, 128>(p, bf16, grid, smem, s);
    if (gb == 32) return cb == 128 ? pipe_launch_m<BITS, 32, 128>(p, bf16, grid, smem, s) : pipe_launch_m<BITS, 32, 256>(p, bf16, grid, smem, s);
    return cb == 128 ? pipe_launch_m<BITS, 64, 128>(p, bf16, grid, smem, s) : pipe_launch_m<BITS, 64, 256>(p, bf16, grid, smem, s);
}

}  // namespace

// One translation unit per bit width keeps the build parallel: QGEMV_INST_BITS selects which
// instantiations (and, for 2, the planner) this compilation provides.
#if !defined(QGEMV_INST_BITS) || QGEMV_INST_BITS == 2
int launch_pipe_int2(const MmaArgs& p, int gb, int cb, bool bf16, int grid, int smem, cudaStream_t s) {
    return pipe_launch_gb<2>(p, gb, cb, bf16, grid, smem, s);
}
#endif
#if !defined(QGEMV_INST_BITS) || QGEMV_INST_BITS == 4
int launch_pipe_int4(const MmaArgs& p, int gb, int cb, bool bf16, int grid, int smem, cudaStream_t s) {
    return pipe_launch_gb<4>(p, gb, cb, bf16, grid, smem, s);
}
#endif

#if !defined(QGEMV_INST_BITS) || QGEMV_INST_BITS == 2
namespace {

// Plan for one chunk size (packed bytes per row per ring slot); false if nothing fits.
bool plan_pipe_chunk(const qgemv_problem& p, const MmaPlan& base, int cb, MmaPlan& pl) {
    pl = base;
    pl.ok = false;
    const int gb = base.gb;
    const int cg = cb / gb, stage_bytes = kTileRows * cb + kTileRows * 16;
    pl.chunk = cb;
    pl.nch = (pl.ng + cg - 1) / cg;
    auto al = [](const void* q, size_t a) { return reinterpret_cast<uintptr_t>(q) % a == 0; };
    pl.scales_async = (p.lds % cg == 0) && al(p.scales, (size_t)cg * 2) ? 1 : 0;
    const int sms = sm_count();
    const int grid = pl.nt < sms ? pl.nt : sms;
    const int tiles_max = (pl.nt + grid - 1) / grid, tiles_min = pl.nt / grid;
    const int slot_bytes = 8 * ((p.m + 1) / 2) * 16;
    // Runs: consecutive chunks of one tile; one chunk per run unless the partial sums of a CTA's runs
    // would then need more than 24 KB of shared memory.
    int rlen = 1, rpt = pl.nch;
    for (;; rlen *= 2) {
        rpt = (pl.nch + rlen - 1) / rlen;
        if ((long long)tiles_max * rpt * slot_bytes <= 24576 || rlen >= pl.nch) break;
    }
    const int slot_cap = tiles_max * rpt;
    if ((long long)slot_cap * slot_bytes > 49152) return false;
    pl.grid = grid; pl.rlen = rlen; pl.rpt = rpt; pl.tile_aligned = 1;

    // warps: as many as the smallest CTA has runs for, at most kPipeWarps
    int nw_cap = tiles_min * rpt;
    nw_cap = nw_cap < 1 ? 1 : (nw_cap > kPipeWarps ? kPipeWarps : nw_cap);

    // epilogue operands: prefetched for the first tiles of a CTA, up to 12 KB
    const int epi_bytes = align_up(kTileRows * (pl.ocb + pl.rb) + 32, 16);
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
    pl.off_epi = off;   off = align_up(off + epi_tiles * epi_bytes, 128);
    pl.off_ring = off;
    pl.epi_bytes = epi_bytes;
    pl.epi_tiles = epi_tiles;

    // Ring.  Warps first -- a warp of this kernel is latency bound, the SM's throughput grows with the
    // number of warps -- then as many slots per warp as fit (up to 4, 8 for 128-byte chunks).
    const int budget = kMaxDynSmem - off;
    const int max_stages = cb == 128 ? kPipeMaxStages : 4;
    int nw = 0, stages = 0;
    const int forced_nw = (p.debug >> 8) & 0xff, forced_st = (p.debug >> 16) & 0xf;
    for (int w = nw_cap; w >= 1 && !nw; --w) {
        if (forced_nw && w != forced_nw) continue;
        int st = budget / (w * stage_bytes);
        if (st > max_stages) st = max_stages;
        if (forced_st) { if (st < forced_st) continue; st = forced_st; }
        if (st >= 2) { nw = w; stages = st; }
    }
    if (!nw) return false;
    pl.nw = nw; pl.stages = stages;
    pl.smem_bytes = off + nw * stages * stage_bytes;

    // residual projections inside the kernel: K is cut into parts of 8 * threads * pv columns
    const int pvmax = p.m == 1 ? 4 : (p.m == 2 ? 3 : 2);
    int pv = 1, parts = 0;
    for (;; ++pv) {                      // fewest pieces per thread that keep the jobs within the grid
        parts = (p.k_original + nw * 256 * pv - 1) / (nw * 256 * pv);
        if ((parts <= kMaxTParts && p.rank * parts <= grid) || pv >= pvmax) break;
    }
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
    return true;
}

}  // namespace

// Plan of the barrier-free kernel, or ok == false when the shape should stay with the phased kernel
// (`base` is that kernel's plan for the same problem).  Of the two chunk sizes the one that puts more
// warps to work wins (128-byte chunks: twice the runs per tile and half the ring per warp); on a tie
// the larger chunk (fewer trips through the loop).
MmaPlan plan_pipe(const qgemv_problem& p, const MmaPlan& base) {
    MmaPlan none = base;
    none.ok = false;
    if (!base.ok || !base.tile_aligned) return none;
    const int gb = base.gb;
    const int cands[2] = {256, 128};
    int forced = 0;
    if (p.debug & QGEMV_DEBUG_CHUNK256) forced = 256;
    if (p.debug & QGEMV_DEBUG_CHUNK128) forced = 128;
    MmaPlan best = none;
    for (int cb : cands) {
        if (cb > 8 * gb) continue;                      // 16-byte groups only come with 128-byte chunks
        if (forced && cb != forced) continue;
        MmaPlan cand{};
        if (plan_pipe_chunk(p, base, cb, cand) && (!best.ok || cand.nw > best.nw)) best = cand;
    }
    return best.ok ? best : none;
}

int launch_pipe_int2(const MmaArgs& p, int gb, int cb, bool bf16, int grid, int smem, cudaStream_t s);
int launch_pipe_int4(const MmaArgs& p, int gb, int cb, bool bf16, int grid, int smem, cudaStream_t s);

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
    p.off_cnt = pl.off_cnt; p.off_red = pl.off_red; p.off_tt = pl.off_tt;
    p.t_inline = pl.t_inline; p.t_parts = pl.t_parts; p.t_pv = pl.t_pv;
    p.l2_chunks = pl.l2_chunks;
    p.debug = debug;
    p.wait_for_x = (a.rank > 0 && !pl.t_inline) ? 0 : 1;
    p.tile_aligned = 1;
    return bits == 2 ? launch_pipe_int2(p, pl.gb, pl.chunk, bf16, pl.grid, pl.smem_bytes, s)
                     : launch_pipe_int4(p, pl.gb, pl.chunk, bf16, pl.grid, pl.smem_bytes, s);
}
#endif

}  // namespace qgemv
