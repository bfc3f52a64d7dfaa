// Streaming fused GEMV for packed groupwise INT2 / INT4 weights, M <= 4, sm_100a.
//
// Why this kernel exists: at full HBM rate a B200 SM receives ~24 packed bytes per clock, i.e.
// ~95 INT2 or ~47 INT4 weights, but can issue only 128 thread-instructions per clock.  An
// "unpack + fp32 FMA per weight" loop needs 2 + M instructions per weight and is therefore
// issue bound (qgemv_simt.cu measures that).  Here the per-weight cost is ~0.6 instructions:
//
//  * Packed rows are brought into a per-warp shared-memory ring with 16-byte asynchronous copies
//    (cp.async.cg, 128 contiguous bytes per row per chunk, pieces XOR-swizzled so that every later
//    shared-memory read is conflict free without padding) -- no staging registers, ~100 KB in
//    flight per SM.  (Filling the ring with one cp.async.bulk per row per chunk through the TMA
//    engine measured the same; cp.async needs no mbarriers and allows the swizzle.)
//  * Codes are NOT converted to numbers.  A 32-bit word is AND-ed with a mask that leaves one
//    code in the low mantissa bits of each 16-bit half; read as fp16 that is the subnormal
//    value code * radix^c * 2^-24 (radix = 4 for INT2, 16 for INT4, c = position class).  The
//    activation it will meet was pre-multiplied by radix^-c (exact, power of two) when it was
//    staged, so one AND yields two ready multiplicands.
//  * The dot products run on the legacy tensor-core path, mma.sync.m16n8k16 (fp16 x fp16 ->
//    fp32): 16 weight rows x 16 k x (M <= 8 activation rows) per instruction.  Products of
//    fp16 subnormals are exact and accumulation is fp32, so the result is the exact integer
//    dot product sum(code * x) per group, scaled by a power of two.
//  * Per group the fp32 partial sum is combined with the group scale and the level offset
//    (INT2: level = (2c-3)/3, INT4: level = c-8) using the pre-computed sum of x over the group.
//  * Work is split stream-K style: the (16-row tile, K-run) units are dealt out evenly to the
//    CTAs of a persistent grid (one per SM), so every SM gets the same number of bytes whatever
//    N and K are; inside a CTA the warps pull runs from a shared-memory queue.  Partial sums of
//    a tile meet in shared memory and are added in fixed order.  Only the (at most two) tiles a
//    CTA shares with its neighbours go through global memory, where whichever CTA arrives last
//    adds the contributions in CTA order (no waiting, deterministic).
//  * Everything the kernel needs from DRAM rides the same asynchronous stream as the codes: the
//    group scales sit in the ring beside their chunk, the outlier / residual rows of a warp's
//    first tile are prefetched at kernel start.  A plain load issued while ~100 KB per SM of
//    prefetch is queued would wait behind all of it.
//  * Epilogue in the same kernel: exact fp16 outlier columns, rank-r residual (its projections
//    t = V.x are computed by the first CTAs of the same launch and published through global
//    memory), bias, activation.
//
// Replaces _decode_gemv (ai_accel_lab/kernels/decode_int2.py:43-96) and _decode_int4_gemv
// (ai_accel_lab/kernels/groupwise_int4.py:85-107) of the reference project.
#include "qgemv_mma_dev.cuh"

namespace qgemv {
namespace {



// ---------------------------------------------------------------------------------------------
// Activation staging (whole CTA, one pass, one barrier): x -> fp16 multiplicands in B-fragment
// order, plus per (group, activation row): the offset term and the power-of-two normalisation.
//
// One work item = (group, activation row m, quad lane t): the G/4 consecutive activations that
// lane t of a quad meets in that group.  Items are numbered with (m, t) fastest, which is also
// the order of the 16-byte fragment slots in shared memory, so a warp's stores are contiguous.
// The four lanes of an item quad agree on the group's largest magnitude with two shuffles and
// scale the group so that it sits just below 2^14: fp16 then holds every multiplicand exactly
// (or with an error far below fp32 rounding for elements 2^-20 times smaller than the largest).
// ---------------------------------------------------------------------------------------------
template <int BITS, int GB, int M, bool BF16, bool EX, typename AfterLoads>
__device__ __forceinline__ void stage_activations(const MmaArgs& p, unsigned char* smem, AfterLoads after_loads) {
    using XT = typename Act16<BF16>::T;
    using GE = Geo<BITS, GB>;
    constexpr int EPI = GE::G / 4;          // activations per item
    constexpr int PPI = EPI / 8;            // 16-byte pieces per item
    constexpr int WP = GE::CW / 8;          // pieces per 32-bit code word (INT2: 2, INT4: 1)
    constexpr int RC = PPI <= 4 ? 2 : 1;    // items whose loads one thread keeps in flight together
    const Args& a = p.a;
    const int tid = threadIdx.x, nthr = blockDim.x;
    float* xo = reinterpret_cast<float*>(smem + p.off_xo);
    float2* gx = reinterpret_cast<float2*>(smem + p.off_gx);          // {offset term, accumulator scale} per (group, m)
    uint4* xs16 = reinterpret_cast<uint4*>(smem + p.off_xs);
    const XT* x = static_cast<const XT*>(a.x);
    const int items = p.ng * M * 4;
    const int span = nthr * RC;

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

    // outlier column indices (static data): first round held in a register
    const int n_xo = EX ? a.oc * M : 0;
    int col0 = -1;
    if (EX && tid < n_xo) col0 = a.oidx[tid / M];
    QTRACE(10);
    load_items(0);
    QTRACE(11);
    // Residual projections t[m][c] = sum_k V[c,k] x[m,k], computed in-kernel: job j = (column c,
    // K-part) belongs to CTA j (there are never more jobs than CTAs).  Its loads are issued here,
    // with the activation loads, ahead of the weight prefetch.
    const int t_jobs = (EX && p.t_inline) ? a.rank * p.t_parts : 0;
    const bool has_job = (int)blockIdx.x < t_jobs;
    const int t_part_k = nthr * 8;                 // columns of V one job covers: one 16-byte piece per thread
    uint4 tv = make_uint4(0u, 0u, 0u, 0u), tx[M];
    if (has_job) {
        const int c = blockIdx.x % a.rank, part = blockIdx.x / a.rank;
        const int k = part * t_part_k + tid * 8;
        const bool live = k < a.korig;
        if (live) tv = *reinterpret_cast<const uint4*>(a.rv + (size_t)c * a.ldv + k);
#pragma unroll
        for (int m = 0; m < M; ++m)
            tx[m] = live ? *reinterpret_cast<const uint4*>(x + (size_t)m * a.ldx + k) : make_uint4(0u, 0u, 0u, 0u);
    }
    // Every warp's activation loads are queued before any warp starts the bulk weight prefetch
    // (the barrier waits for the issue of the loads, not for their data).
    __syncthreads();
    after_loads();
    if (has_job) {
        // every warp reduces its 256 columns and hands the M partial sums to warp 0 (see the kernel)
        const int warp_id = tid >> 5, lane_id = tid & 31;
        float ts[M];
        const __half* vh = reinterpret_cast<const __half*>(&tv);
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const XT* xh = reinterpret_cast<const XT*>(&tx[m]);
            ts[m] = 0.0f;
#pragma unroll
            for (int q = 0; q < 8; ++q) ts[m] = fmaf(__half2float(vh[q]), Act16<BF16>::to_float(xh[q]), ts[m]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ts[m] += __shfl_xor_sync(0xffffffffu, ts[m], o);
        }
        float* red = reinterpret_cast<float*>(smem + p.off_tt);   // scratch until the table is built; read after the next barrier
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
            // a warp whose lanes all lie past the last item (the second item slot of a thread when the items
            // just fill the CTA once) skips the slot: warp-uniform, so the shuffles below stay converged
            if (!__any_sync(0xffffffffu, live)) continue;
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
    __syncthreads();
    // Outlier activations, read back from the staged multiplicands (no further global loads of x:
    // they would queue behind the weight stream).  x[m][col] = staged * radix^c * 2^e(group).
    const __half* xs = reinterpret_cast<const __half*>(smem + p.off_xs);
    for (int i = tid; i < n_xo; i += nthr) {
        const int j = i / M, m = i - j * M;
        const int col = i < nthr ? col0 : a.oidx[j];
        float val = 0.0f;
        if (col >= 0 && col < a.kpad) {
            const int grp = col / GE::G, rr = col - grp * GE::G;
            const int wordpos = rr / GE::CW, t = wordpos / GE::TW, ii = wordpos - t * GE::TW;
            const int jj = rr - wordpos * GE::CW;
            const int c = jj % GE::NCLS, qq = jj / GE::NCLS;
            const int pos = (qq & 1) * 2 + (qq >> 1);
            const size_t h = ((((size_t)(grp * GE::TW + ii) * (GE::NCLS / 2) + (c >> 1)) * M + m) * 4 + t) * 8 +
                             (c & 1) * 4 + pos;
            const float up = gx[grp * M + m].y * (BITS == 2 ? 1.5f : 1.0f);      // 2^(24 + e)
            val = __half2float(xs[h]) * __int_as_float((127 - 24 + BITS * c) << 23) * up;
        }
        xo[i] = val;
    }
    QTRACE(6);
    // no barrier here: the table is first read after the CTA-wide barrier that ends the main loop
}


// Table of residual projections t[q][m] in shared memory (one warp).  In-kernel projections arrive
// as {value, launch tag} words from the CTAs that computed them; a small table was requested while
// the warp was still computing (early0/early1, `requested`), so the trip to L2 is hidden, and a
// word whose tag is not this launch's is simply read again (bounded).  `scratch` is idle shared
// memory of the calling warp (64 floats).
template <int M>
__device__ __noinline__ void build_t_table(const MmaArgs& p, unsigned char* smem, float* scratch, unsigned t_tag,
                                           unsigned long long early0, unsigned long long early1, bool requested) {
    const Args& a = p.a;
    const int lane = threadIdx.x & 31;
    float* tt = reinterpret_cast<float*>(smem + p.off_tt);
    const int RM = a.rank * M;
    if (!p.t_inline) {
        pdl_wait();                               // t comes from the kernel launched just before this one
        for (int i = lane; i < RM; i += 32) {
            const int q = i / M, m = i - q * M;
            tt[i] = ld_cg_f32(a.t + m * kMaxRank + q);
        }
        return;
    }
    const unsigned long long* src = reinterpret_cast<const unsigned long long*>(a.tparts);
    auto settle = [&](unsigned long long w, const unsigned long long* addr) {
        int spins = 0;
        // about 30 ms; a few microseconds when a test makes the wait run out on purpose
        const int limit = (p.debug & QGEMV_DEBUG_DROP_PROJECTIONS) ? (1 << 7) : (1 << 20);
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

// A tile whose runs are split between neighbouring CTAs: this CTA parks its sum in global memory
// and counts its arrival; the last CTA to arrive adds the contributions in CTA order and finishes
// the tile.  Out of line: tile-aligned launches never come here.
template <int M, bool BF16, bool EX>
__device__ __noinline__ void shared_tile(const MmaArgs& p, const unsigned char* smem, int tile, float4 sum, int slot) {
    const Args& a = p.a;
    const int lane = threadIdx.x & 31, grid = gridDim.x, cta = blockIdx.x;
    float y[4] = {sum.x, sum.y, sum.z, sum.w};
    float* mine = a.partial + ((size_t)(cta * 2 + slot) * 4) * 32;
#pragma unroll
    for (int i = 0; i < 4; ++i) mine[i * 32 + lane] = y[i];
    __threadfence();
    __syncwarp();
    const int cf = owner_of(p, tile * p.rpt, grid);
    const int cl = owner_of(p, tile * p.rpt + p.rpt - 1, grid);
    int last = 0;
    if (lane == 0) {
        const int old = atomicAdd(&a.counters[tile], 1);
        last = old == cl - cf;
        if (last) a.counters[tile] = 0;          // ready for the next launch
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (!last) return;
    __threadfence();
    y[0] = y[1] = y[2] = y[3] = 0.f;
    for (int cb = cf; cb <= cl; cb += 4) {     // four contributors' loads in flight at a time
        float v[4][4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int c = min(cb + k, cl);
            const int sl = tile == first_unit(p, c, grid) / p.rpt ? 0 : 1;
            const float* src = a.partial + ((size_t)(c * 2 + sl) * 4) * 32;
#pragma unroll
            for (int i = 0; i < 4; ++i) v[k][i] = ld_cg_f32(src + i * 32 + lane);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (cb + k <= cl) {
#pragma unroll
                for (int i = 0; i < 4; ++i) y[i] += v[k][i];
            }
    }
    finish_tile<M, BF16, EX>(p, smem, tile, y, nullptr);
}

// ---------------------------------------------------------------------------------------------
// The kernel.  Persistent grid, blockDim.x = 32 * nw; every warp is its own producer and consumer.
// ---------------------------------------------------------------------------------------------
template <int BITS, int GB, int M, bool BF16, bool EX>
__global__ void __launch_bounds__(kMaxWarps * 32, 1) qgemv_mma_kernel(const __grid_constant__ MmaArgs p) {
    using GE = Geo<BITS, GB>;
    constexpr int TT = (M + 1) / 2;                   // quad lanes that hold useful output columns
    constexpr int SLOT_BYTES = 8 * TT * 16;           // one run's partial sums in shared memory
    extern __shared__ __align__(128) unsigned char smem[];
    const Args& a = p.a;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    pdl_launch_dependents();

    // This CTA's share of the runs, and the tiles they touch.
    const int grid = gridDim.x, cta = blockIdx.x;
    // Whole tiles per CTA when that balances well enough (no tile is then shared between CTAs),
    // otherwise an even split of the runs.
    const int u0 = first_unit(p, cta, grid), u1 = first_unit(p, cta + 1, grid);
    const int r0 = p.tile_aligned ? u0 * p.rpt : u0, r1 = p.tile_aligned ? u1 * p.rpt : u1;
    const int T0 = p.tile_aligned ? u0 : r0 / p.rpt, T1 = p.tile_aligned ? u1 - 1 : (r1 - 1) / p.rpt;

    unsigned char* ring = smem + p.off_ring + (size_t)warp * GE::STAGES * GE::STAGE_BYTES;
    const uint32_t ring_u32 = smem_u32(ring);
    int4* meta = reinterpret_cast<int4*>(smem + p.off_meta) + warp * 4;      // per stage: tile, chunk, slot, last
    unsigned char* epi = smem + p.off_epi + (size_t)warp * p.epi_bytes;
    QTRACE(0);

    // ---- producer side: pull runs from the CTA queue, copy their chunks into the ring ---------
    constexpr int PPR = GE::CB / 16;                 // 16-byte pieces per row of a full chunk
    constexpr int RPI = 32 / PPR;                    // rows covered by one warp-wide copy instruction
    const int lrow = lane / PPR, lcol = lane % PPR;
    // Runs are dealt round-robin: warp w takes runs r0 + w, r0 + w + nw, ...
    const bool t_inline = EX && p.t_inline;
    const bool has_job = t_inline && (int)blockIdx.x < a.rank * p.t_parts;   // this CTA also computes a residual projection
    constexpr int w0 = 0;
    const int nwk = p.nw;
    int pf_run = warp >= w0 ? r0 + warp - w0 : r1, pf_tile = 0, pf_j = 0, pf_ch = 0, pf_end = 0;   // pf_j: run index inside the tile
    if (pf_run < r1) {
        pf_tile = pf_run / p.rpt;
        pf_j = pf_run - pf_tile * p.rpt;
        pf_ch = pf_j * p.rlen;
        pf_end = min(pf_ch + p.rlen, p.nch);
    } else {
        pf_run = -1;
    }
    // Per-lane constants of the copy pattern: one instruction moves RPI rows x 128 bytes.
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
    auto issue_next = [&](int s) {
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
        if (pf_run >= 0) {
            const int ngr = min(GE::CG, p.ng - pf_ch * GE::CG);
            const uint32_t sbase = ring_u32 + s * GE::STAGE_BYTES;
            const bool edge = ragged_n && pf_tile == p.nt - 1;        // rows past N are clamped to the last row
            if (ngr == GE::CG && !edge && p.scales_async) {
                // common case, straight-line: 4 row-group copies by every lane + one scale copy by lanes 0..15
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

    // First copies of this warp: the epilogue operands of the tile it will finish first (oldest
    // group) and its first ring slot.
    // Tiles are finished by the warps in reverse order (warp nw-1 takes the CTA's first tile): the
    // round-robin deal of the runs leaves the high-numbered warps with the fewest runs.
    const int tw = p.nw - 1 - warp;
    const int etile = T0 + tw;
    const bool efull = p.epi_async && etile <= T1 && etile * p.rpt >= r0 && (etile + 1) * p.rpt <= r1 &&
                       (etile + 1) * kTileRows <= a.n;
    auto first_prefetch = [&]() {
        if (efull) {
            const int opieces = EX ? p.ocb >> 4 : 0, upieces = EX ? p.rb >> 4 : 0;
            for (int i = lane; i < kTileRows * opieces; i += 32) {
                const int r = i % kTileRows, c = i / kTileRows;
                cp_async16(smem_u32(epi) + r * p.ocb + c * 16,
                           reinterpret_cast<const unsigned char*>(a.ow + (size_t)(etile * kTileRows + r) * a.ldow) + c * 16);
            }
            for (int i = lane; i < kTileRows * upieces; i += 32) {
                const int r = i % kTileRows, c = i / kTileRows;
                cp_async16(smem_u32(epi) + kTileRows * p.ocb + r * p.rb + c * 16,
                           reinterpret_cast<const unsigned char*>(a.ru + (size_t)(etile * kTileRows + r) * a.ldu) + c * 16);
            }
            if (a.bias && lane < 2)
                cp_async16(smem_u32(epi) + kTileRows * (p.ocb + p.rb) + lane * 16,
                           reinterpret_cast<const unsigned char*>(a.bias + (size_t)etile * kTileRows) + lane * 16);
        }
        cp_async_commit();
        issue_next(0);
    };
    // Activations first, weights second: the activation loads are short and everything waits for
    // them, and loads issued behind the first weight copies are served after those copies.
    QTRACE(8);
    if (p.wait_for_x) pdl_wait();
    QTRACE(9);
    // Tag of this launch for the residual projections that travel between CTAs (see below): the
    // workspace holds a launch count that the last CTA of every launch advances.
    const bool t_reader = t_inline && warp == p.nw - 1;
    unsigned t_tag = 0;
    if (t_inline && (warp == 0 || t_reader)) t_tag = ld_relaxed_u32(a.counters + kWsEpochIdx) + 1u;
    stage_activations<BITS, GB, M, BF16, EX>(p, smem, [&]() {
        QTRACE(7);
        first_prefetch();
        QTRACE(1);
    });
    for (int s = 1; s < GE::STAGES; ++s) issue_next(s);
    __syncthreads();                                  // staged activations visible to every warp
    QTRACE(2);
    if (has_job && warp == 0 && !(p.debug & QGEMV_DEBUG_DROP_PROJECTIONS)) {
        // The warps' partial sums were written before the barrier above: add them in warp order and
        // publish {sum, launch tag} for every CTA's epilogue with one relaxed 64-bit store.
        const float* red = reinterpret_cast<const float*>(smem + p.off_tt);
        if (lane < M) {
            float tot = 0.0f;
            for (int w = 0; w < p.nw; ++w) tot += red[w * M + lane];
            const int c = blockIdx.x % a.rank, part = blockIdx.x / a.rank;
            st_relaxed_u64(reinterpret_cast<unsigned long long*>(a.tparts) + (part * QGEMV_MAX_M + lane) * kMaxRank + c,
                           ((unsigned long long)t_tag << 32) | __float_as_uint(tot));
        }
    }

    const int ma = min(2 * t, M - 1), mb = min(2 * t + 1, M - 1);
    unsigned char* slots = smem + p.off_slots;

    // ---- consumer side ------------------------------------------------------------------------
    // Shared-memory operands are addressed through the 32-bit shared window with explicit
    // ld.shared instructions: the compiler then folds every compile-time offset into the
    // instruction and no 64-bit address arithmetic is left in the loop.
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

    // Residual projections computed by other CTAs: a small table is requested by the reader warp
    // after its second unit (the producers have published by then) and checked after the loop.
    const int t_entries = t_inline ? p.t_parts * a.rank * M : 0;
    unsigned long long t_early[2] = {0ull, 0ull};
    bool t_issued = false;
    int t_request = (t_reader && t_entries <= 64) ? 2 : 0;   // units to finish before the request goes out

    float y[4] = {0.f, 0.f, 0.f, 0.f};
    int stage = 0;
    bool first = true;
    for (;;) {
        cp_async_wait<GE::STAGES - 1>();        // all but the newest STAGES-1 groups are done: this slot has landed
        __syncwarp();
        const uint4 mt = lds128(meta_u32 + stage * 16);          // tile, chunk, slot, last-of-run
        if ((int)mt.x < 0) break;
        if (first) { QTRACE(3); first = false; }
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
#ifdef QGEMV_NOCOMPUTE                              // measurement aid: stream and bookkeeping only
        if (G0 < 0)
#endif
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
        if (mt.w) {                                   // run complete: park its partial sums
            if (t < TT) sts128f(slots_u32 + mt.z * SLOT_BYTES, make_float4(y[0], y[1], y[2], y[3]));
            y[0] = y[1] = y[2] = y[3] = 0.f;
        }
        __syncwarp();                               // every lane is done reading the slot before it is refilled
        issue_next(stage);
        stage = (stage + 1) & (GE::STAGES - 1);
        if (t_request > 0 && --t_request == 0) {
            t_issued = true;
#pragma unroll
            for (int e = 0; e < 2; ++e)
                if (lane + 32 * e < t_entries) t_early[e] = ld_relaxed_u64(t_entry(a, M, lane + 32 * e));
        }
    }
    cp_async_wait<0>();
    QTRACE(4);
    // Table of residual projections t[q][m] in shared memory, built by the last warp of the CTA.
    if (EX && a.rank > 0 && warp == p.nw - 1)
    {
        build_t_table<M>(p, smem, reinterpret_cast<float*>(ring), t_tag, t_early[0], t_early[1], t_issued);
        QTRACE(12);
    }
    __syncthreads();                                  // every run of this CTA is parked, the table is complete
    QTRACE(13);

    // ---- tiles: add the runs in order, finish or hand over --------------------------------------
    for (int tile = T0 + tw; tile <= T1; tile += p.nw) {
        const int lo = max(r0, tile * p.rpt), hi = min(r1, (tile + 1) * p.rpt);
        const bool pre = efull && tile == etile;
        y[0] = y[1] = y[2] = y[3] = 0.f;
        if (t < TT) {
            for (int r = lo; r < hi; ++r) {
                const float4 v = *reinterpret_cast<const float4*>(slots + (size_t)(r - r0) * SLOT_BYTES + (g * TT + t) * 16);
                y[0] += v.x; y[1] += v.y; y[2] += v.z; y[3] += v.w;
            }
        }
        const bool whole = lo == tile * p.rpt && hi == (tile + 1) * p.rpt;
        QTRACE(14);
        if (whole) {
            finish_tile<M, BF16, EX>(p, smem, tile, y, pre ? epi : nullptr);
        } else {
            shared_tile<M, BF16, EX>(p, smem, tile, make_float4(y[0], y[1], y[2], y[3]), tile == T0 ? 0 : 1);
        }
    }
    QTRACE(5);
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

template <int BITS, int GB, int M, bool BF16, bool EX>
int launch_ex(const MmaArgs& p, int grid, int smem_bytes, cudaStream_t s) {
    auto kern = qgemv_mma_kernel<BITS, GB, M, BF16, EX>;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem) != cudaSuccess)
            return check_launch("cudaFuncSetAttribute(qgemv_mma_kernel)");
        configured[dev] = true;
    }
    // Programmatic dependent launch: the grid may become resident while the previous kernel in the
    // stream is still running.  When that kernel is this call's own residual-projection kernel
    // (launched in full stream order), x is already final and only the epilogue waits for it;
    // otherwise the kernel waits for its predecessors before it touches x (p.wait_for_x).
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
    if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) return check_launch("qgemv_mma_kernel");
    return check_launch("qgemv_mma_kernel");
}

// Problems without outlier columns and residual get a kernel that does not contain that code: a
// launch starts with a cold instruction cache, and stepping over unused code is not free.
template <int BITS, int GB, int M, bool BF16>
int launch_one(const MmaArgs& p, int grid, int smem_bytes, cudaStream_t s) {
    if (p.a.oc > 0 || p.a.rank > 0) return launch_ex<BITS, GB, M, BF16, true>(p, grid, smem_bytes, s);
    return launch_ex<BITS, GB, M, BF16, false>(p, grid, smem_bytes, s);
}

template <int BITS, int GB, int M>
int launch_bf(const MmaArgs& p, bool bf16, int grid, int smem, cudaStream_t s) {
    return bf16 ? launch_one<BITS, GB, M, true>(p, grid, smem, s) : launch_one<BITS, GB, M, false>(p, grid, smem, s);
}
template <int BITS, int GB>
int launch_m(const MmaArgs& p, bool bf16, int grid, int smem, cudaStream_t s) {
    switch (p.a.m) {
        case 1: return launch_bf<BITS, GB, 1>(p, bf16, grid, smem, s);
        case 2: return launch_bf<BITS, GB, 2>(p, bf16, grid, smem, s);
        case 3: return launch_bf<BITS, GB, 3>(p, bf16, grid, smem, s);
        default: return launch_bf<BITS, GB, 4>(p, bf16, grid, smem, s);
    }
}
template <int BITS>
int launch_gb(const MmaArgs& p, int gb, bool bf16, int grid, int smem, cudaStream_t s) {
    if (gb == 16) return launch_m<BITS, 16>(p, bf16, grid, smem, s);
    if (gb == 32) return launch_m<BITS, 32>(p, bf16, grid, smem, s);
    return launch_m<BITS, 64>(p, bf16, grid, smem, s);
}

}  // namespace

// One translation unit per bit width keeps the build parallel: QGEMV_INST_BITS selects which
// instantiations (and, for 2, the planner) this compilation provides.
#if !defined(QGEMV_INST_BITS) || QGEMV_INST_BITS == 2
int launch_mma_int2(const MmaArgs& p, int gb, bool bf16, int grid, int smem, cudaStream_t s) {
    return launch_gb<2>(p, gb, bf16, grid, smem, s);
}
#endif
#if !defined(QGEMV_INST_BITS) || QGEMV_INST_BITS == 4
int launch_mma_int4(const MmaArgs& p, int gb, bool bf16, int grid, int smem, cudaStream_t s) {
    return launch_gb<4>(p, gb, bf16, grid, smem, s);
}
#endif

#if !defined(QGEMV_INST_BITS) || QGEMV_INST_BITS == 2
int launch_mma_int2(const MmaArgs& p, int gb, bool bf16, int grid, int smem, cudaStream_t s);
int launch_mma_int4(const MmaArgs& p, int gb, bool bf16, int grid, int smem, cudaStream_t s);

MmaPlan plan_mma(const qgemv_problem& p, size_t partial_floats) {
    MmaPlan pl{};
    pl.ok = false;
    const int gb = p.group * p.bits / 8;
    if (gb != 16 && gb != 32 && gb != 64) return pl;
    if (p.group * p.bits % 8) return pl;
    auto al = [](const void* q, size_t a) { return reinterpret_cast<uintptr_t>(q) % a == 0; };
    if (!al(p.packed, 16) || p.ldp % 16 || !al(p.x, 16) || p.ldx % 8) return pl;
    if (p.outliers > kMaxOutliers || p.rank > kMaxRank) return pl;
    const int cb = gb == 16 ? 128 : 256, cg = cb / gb, stage_bytes = kTileRows * cb + kTileRows * 16;
    pl.gb = gb;
    pl.ng = p.k_padded / p.group;
    pl.nch = (pl.ng + cg - 1) / cg;
    pl.nt = (p.n + kTileRows - 1) / kTileRows;
    if (pl.nt > kWsMaxCounters - 4) return pl;          // the last four counters are status / residual bookkeeping
    if ((long long)pl.nt * pl.nch > 0x3fffffff) return pl;
    const int sms = sm_count();
    // Runs: consecutive chunks of one tile.  One chunk per run unless a CTA would then need more
    // than 32 KB of shared memory for the partial sums of its runs.
    const int slot_bytes = 8 * ((p.m + 1) / 2) * 16;
    // Fewer tiles than SMs: one CTA per tile (its 16 warps split K) instead of a full grid whose
    // CTAs share tiles -- the hand-over through global memory costs ~4 us, more than the idle SMs
    // do as long as one tile's bytes stream in about that time.
    const long long tile_bytes = (long long)kTileRows * p.k_padded * p.bits / 8;
    const int grid_cap = (pl.nt < sms && tile_bytes <= 160 * 1024) ? pl.nt : sms;
    int rlen = 1, rpt = pl.nch, grid = 0, slot_cap = 0;
    for (;; rlen *= 2) {
        rpt = (pl.nch + rlen - 1) / rlen;
        const long long runs = (long long)pl.nt * rpt;
        grid = (int)(runs < grid_cap ? runs : grid_cap);
        slot_cap = (int)((runs + grid - 1) / grid) + 1;
        if (slot_cap * slot_bytes <= 32768 || rlen >= pl.nch) break;
    }
    if (slot_cap * slot_bytes > 65536) return pl;
    pl.rlen = rlen; pl.rpt = rpt; pl.grid = grid;
    // whole tiles per CTA if the busiest CTA then has at most 20 % more than the average, or if it
    // streams so little (<= 160 KB) that the imbalance costs less than sharing tiles would
    pl.tile_aligned = 0;
    if (pl.nt >= grid) {
        const int most = (pl.nt + grid - 1) / grid;
        if ((long long)most * grid * 5 <= (long long)pl.nt * 6 || most * tile_bytes <= 160 * 1024) pl.tile_aligned = 1;
    }
    if (pl.tile_aligned) slot_cap = ((pl.nt + grid - 1) / grid) * rpt;
    if (slot_cap * slot_bytes > 65536) return pl;
    if ((size_t)grid * 2 * 4 * 32 + kTPartFloats > partial_floats) return pl;

    pl.scales_async = (p.lds % cg == 0) && al(p.scales, (size_t)cg * 2) ? 1 : 0;
    pl.ocb = align_up(p.outliers * 2, 16);
    pl.rb = align_up(p.rank * 2, 16);
    bool epi = (p.outliers > 0 || p.rank > 0 || p.bias != nullptr);
    if (p.outliers > 0 && (p.outliers % 8 || p.ldow % 8 || !al(p.outlier_w, 16))) epi = false;
    if (p.rank > 0 && (p.rank % 8 || p.ldu % 8 || !al(p.res_u, 16))) epi = false;
    if (p.bias && !al(p.bias, 16)) epi = false;
    pl.epi_async = epi ? 1 : 0;

    int off = 64;
    pl.off_xo = off;    off = align_up(off + p.outliers * p.m * 4, 16);
    pl.off_gx = off;    off = align_up(off + pl.ng * p.m * 8, 16);
    pl.off_tt = off;    off = align_up(off + (p.rank * p.m > 64 ? p.rank * p.m : 64) * 4, 16);
    pl.off_slots = off; off = align_up(off + slot_cap * slot_bytes, 128);
    pl.off_xs = off;    off = align_up(off + p.m * p.k_padded * 2, 128);
    // per warp: 4 ring descriptors (64 B) + the epilogue prefetch buffer + the ring itself
    const int epi_bytes = align_up(kTileRows * (pl.ocb + pl.rb) + 32, 16);
    const int avail = kMaxDynSmem - off;
    int nw = 0;
    const int stages = cb == 128 ? 4 : 2;
    for (int cand = kMaxWarps; cand >= 4 && !nw; cand -= 4)
        if (avail >= cand * (64 + epi_bytes + stages * stage_bytes)) nw = cand;
    if (!nw) return pl;
    pl.nw = nw; pl.stages = stages;
    pl.t_parts = (p.k_original + nw * 256 - 1) / (nw * 256);
    pl.t_inline = (p.rank > 0 && p.k_original % 8 == 0 && p.ldv % 8 == 0 && al(p.res_v, 16) && pl.t_parts <= kMaxTParts &&
                   p.rank * pl.t_parts <= grid) ? 1 : 0;
    pl.off_meta = off;  off += nw * 64;
    pl.off_epi = off;   off = align_up(off + nw * epi_bytes, 128);
    pl.epi_bytes = epi_bytes;
    pl.off_ring = off;
    pl.smem_bytes = off + nw * stages * stage_bytes;
    static const char* names[2][3] = {{"mma_int2_g64", "mma_int2_g128", "mma_int2_g256"},
                                      {"mma_int4_g32", "mma_int4_g64", "mma_int4_g128"}};
    pl.name = names[p.bits == 2 ? 0 : 1][gb == 16 ? 0 : gb == 32 ? 1 : 2];
    pl.variant = 1;
    pl.ok = true;
    return pl;
}

int launch_mma(const Args& a, int bits, bool bf16, const MmaPlan& pl, int debug, cudaStream_t s) {
    MmaArgs p{};
    p.a = a;
    p.nt = pl.nt; p.nch = pl.nch; p.ng = pl.ng;
    p.row_bytes = a.kpad * bits / 8;
    p.nw = pl.nw; p.stages = pl.stages;
    p.rlen = pl.rlen; p.rpt = pl.rpt; p.runs = pl.nt * pl.rpt;
    const int units = pl.tile_aligned ? pl.nt : p.runs;
    p.uq = units / pl.grid; p.urem = units % pl.grid;
    p.scales_async = pl.scales_async; p.epi_async = pl.epi_async; p.ocb = pl.ocb; p.rb = pl.rb;
    p.epi_bytes = pl.epi_bytes;
    p.off_xo = pl.off_xo; p.off_gx = pl.off_gx; p.off_slots = pl.off_slots; p.off_epi = pl.off_epi;
    p.off_meta = pl.off_meta; p.off_xs = pl.off_xs; p.off_ring = pl.off_ring;
    p.t_inline = pl.t_inline; p.t_parts = pl.t_parts; p.off_tt = pl.off_tt;
    p.wait_for_x = (a.rank > 0 && !pl.t_inline) ? 0 : 1;
    p.debug = debug;
    p.tile_aligned = pl.tile_aligned;
    return bits == 2 ? launch_mma_int2(p, pl.gb, bf16, pl.grid, pl.smem_bytes, s)
                     : launch_mma_int4(p, pl.gb, bf16, pl.grid, pl.smem_bytes, s);
}
#endif

}  // namespace qgemv
