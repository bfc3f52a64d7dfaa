// Streaming fused GEMV for packed groupwise INT2 / INT4 weights, M <= 4, sm_100a.
//
// Why this kernel exists: at full HBM rate a B200 SM receives ~24 packed bytes per clock, i.e.
// ~95 INT2 or ~47 INT4 weights, but can issue only 128 thread-instructions per clock.  An
// "unpack + fp32 FMA per weight" loop needs 2 + M instructions per weight and is therefore
// issue bound (qgemv_simt.cu measures that).  Here the per-weight cost is ~0.6 instructions:
//
//  * Packed rows are brought into a per-warp shared-memory ring with 16-byte asynchronous copies
//    (cp.async.cg, 256 contiguous bytes per row per chunk) -- no staging registers, rows padded
//    so that every later shared-memory read is conflict free, ~100 KB in flight per SM.
//    (One cp.async.bulk per row per chunk was tried first: the TMA engine needed ~110 cycles
//    per 128-256 byte request per SM, 8x too slow for this access pattern.)
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
//  * Work is split stream-K style: the (16-row tile, K-chunk) units are dealt out evenly to
//    all warps of a persistent grid, so every SM gets the same number of bytes whatever N and
//    K are.  A tile finished by one warp goes straight to the epilogue; a tile shared by several
//    warps is summed, in fixed order, by whichever warp arrives last (no waiting, deterministic).
//  * Epilogue in the same kernel: exact fp16 outlier columns, rank-r residual, bias, activation.
//
// Replaces _decode_gemv (ai_accel_lab/kernels/decode_int2.py:43-96) and _decode_int4_gemv
// (ai_accel_lab/kernels/groupwise_int4.py:85-107) of the reference project.
#include "qgemv_common.cuh"

namespace qgemv {
namespace {

constexpr int kTileRows = 16;          // weight rows per mma tile (one warp owns one tile at a time)
constexpr int kMaxOutliers = 256;      // outlier activations staged in shared memory

struct MmaArgs {
    Args a;
    int nt;            // row tiles: ceil(N / 16)
    int nch;           // chunks per tile
    int ng;            // groups per row
    int row_bytes;     // packed bytes per row actually used (Kpad * bits / 8)
    int nw;            // consumer warps per CTA
    int stages;        // ring depth per warp
    int units;         // nt * nch
    int total_warps;   // warps that own work: min(gridDim.x * nw, units)
    // dynamic shared memory layout (byte offsets)
    int off_xo, off_tt, off_sumx, off_xs, off_ring;
};

// ---------------------------------------------------------------------------------------------
// PTX helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Asynchronous 16-byte global -> shared copy (LDGSTS), L2-only caching.  Completion is tracked per
// thread in commit groups; a group counts as done for the whole warp after wait + __syncwarp().
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory"); }
__device__ __forceinline__ void cp_async_wait_dyn(int pending) {
    if (pending >= 3) cp_async_wait<3>();
    else if (pending == 2) cp_async_wait<2>();
    else if (pending == 1) cp_async_wait<1>();
    else cp_async_wait<0>();
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ld_cg_f32(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

// Optional phase trace (build with -DQGEMV_TRACE): lane 0 of every warp stores the global
// nanosecond timer at a few points into the upper half of the partial-sum scratch.
#ifdef QGEMV_TRACE
#define QTRACE(slot)                                                                            \
    do {                                                                                        \
        if ((threadIdx.x & 31) == 0) {                                                          \
            unsigned long long t_;                                                              \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                              \
            reinterpret_cast<unsigned long long*>(p.a.partial + (kMaxPartialFloats / 2))        \
                [((size_t)blockIdx.x * 16 + (threadIdx.x >> 5)) * 8 + (slot)] = t_;             \
        }                                                                                       \
    } while (0)
#else
#define QTRACE(slot) do { } while (0)
#endif

// Compile-time facts per (bits, group bytes).
template <int BITS, int GB>
struct Geo {
    static constexpr int CPB = 8 / BITS;                 // codes per byte
    static constexpr int CW = 32 / BITS;                 // codes per 32-bit word
    static constexpr int NCLS = BITS == 2 ? 4 : 2;       // position classes (codes per 8 mantissa bits)
    static constexpr int G = GB * CPB;                   // group size in codes
    static constexpr int TB = GB / 4;                    // bytes one lane reads per row per group
    static constexpr int TW = TB / 4;                    // ... in 32-bit words
    static constexpr int CG = (256 / GB) > 8 ? 8 : (256 / GB);   // groups per chunk
    static constexpr int CB = CG * GB;                   // chunk bytes per row (128 or 256)
    static constexpr int PITCH = CB + GB;                // shared-memory row pitch: conflict-free for TB-wide reads
    static constexpr int STAGE_BYTES = kTileRows * PITCH;
    static constexpr uint32_t MASK = BITS == 2 ? 0x00030003u : 0x000f000fu;
    // halves of x' per group laid out for the B fragments: [TW][NCLS/2][M][4 lanes t][8 halves]
};


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
template <int BITS, int GB, int M, bool BF16, typename AfterLoads>
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
    float* tt = reinterpret_cast<float*>(smem + p.off_tt);
    float2* gx = reinterpret_cast<float2*>(smem + p.off_sumx);        // {offset term, accumulator scale} per (group, m)
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

    // early loads for the epilogue tables (first round of each held in a register)
    const int n_xo = a.oc * M, n_tt = a.rank * M;
    int col0 = -1;
    if (tid < n_xo) col0 = a.oidx[tid / M];
    float tt0 = 0.0f;
    if (tid < n_tt) { const int q = tid / M, m = tid - q * M; tt0 = a.t[m * kMaxRank + q]; }
    load_items(0);
    // Every warp's activation loads are queued before any warp starts the bulk weight prefetch
    // (the barrier waits for the issue of the loads, not for their data).
    __syncthreads();
    after_loads();
    float xo0 = 0.0f;
    if (tid < n_xo && col0 >= 0 && col0 < a.kpad) xo0 = Act16<BF16>::to_float(x[(size_t)(tid % M) * a.ldx + col0]);

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
    if (tid < n_xo) xo[tid] = xo0;
    if (tid < n_tt) tt[tid] = tt0;
    for (int i = tid + nthr; i < n_xo; i += nthr) {
        const int j = i / M, m = i - j * M;
        const int col = a.oidx[j];
        xo[i] = (col >= 0 && col < a.kpad) ? Act16<BF16>::to_float(x[(size_t)m * a.ldx + col]) : 0.0f;
    }
    for (int i = tid + nthr; i < n_tt; i += nthr) {
        const int q = i / M, m = i - q * M;
        tt[i] = a.t[m * kMaxRank + q];
    }
    QTRACE(6);
    __syncthreads();
}

// ---------------------------------------------------------------------------------------------
// Epilogue of one finished 16-row tile: outlier columns, residual, bias, activation, store.
// Lane (g = lane/4, t = lane%4) holds rows tile*16+g and +8, activation rows 2t and 2t+1.
// ---------------------------------------------------------------------------------------------
template <int M, bool BF16>
__device__ __forceinline__ void finish_tile(const MmaArgs& p, const unsigned char* smem, int tile, float (&y)[4]) {
    using XT = typename Act16<BF16>::T;
    const Args& a = p.a;
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int r0 = tile * kTileRows + g, r1 = r0 + 8;
    const int c0 = min(r0, a.n - 1), c1 = min(r1, a.n - 1);
    if (a.oc > 0 || a.rank > 0) {
        const float* xo = reinterpret_cast<const float*>(smem + p.off_xo);
        const float* tt = reinterpret_cast<const float*>(smem + p.off_tt);
        float e0[M], e1[M];
#pragma unroll
        for (int m = 0; m < M; ++m) { e0[m] = 0.0f; e1[m] = 0.0f; }
        // The four lanes of a quad split the columns; all loads of a batch are issued before use.
        constexpr int JB = 8;
        const __half* ow0 = a.ow + (size_t)c0 * a.ldow;
        const __half* ow1 = a.ow + (size_t)c1 * a.ldow;
        for (int jb = 0; jb < a.oc; jb += 4 * JB) {
            __half w0[JB], w1[JB];
#pragma unroll
            for (int i = 0; i < JB; ++i) {
                const int j = jb + 4 * i + t;
                w0[i] = j < a.oc ? __ldg(ow0 + j) : __half(0.0f);
                w1[i] = j < a.oc ? __ldg(ow1 + j) : __half(0.0f);
            }
#pragma unroll
            for (int i = 0; i < JB; ++i) {
                const int j = min(jb + 4 * i + t, a.oc - 1);
                const float f0 = __half2float(w0[i]), f1 = __half2float(w1[i]);
#pragma unroll
                for (int m = 0; m < M; ++m) { e0[m] = fmaf(f0, xo[j * M + m], e0[m]); e1[m] = fmaf(f1, xo[j * M + m], e1[m]); }
            }
        }
        const __half* ru0 = a.ru + (size_t)c0 * a.ldu;
        const __half* ru1 = a.ru + (size_t)c1 * a.ldu;
        for (int qb = 0; qb < a.rank; qb += 4 * JB) {
            __half w0[JB], w1[JB];
#pragma unroll
            for (int i = 0; i < JB; ++i) {
                const int q = qb + 4 * i + t;
                w0[i] = q < a.rank ? __ldg(ru0 + q) : __half(0.0f);
                w1[i] = q < a.rank ? __ldg(ru1 + q) : __half(0.0f);
            }
#pragma unroll
            for (int i = 0; i < JB; ++i) {
                const int q = min(qb + 4 * i + t, a.rank - 1);
                const float f0 = __half2float(w0[i]), f1 = __half2float(w1[i]);
#pragma unroll
                for (int m = 0; m < M; ++m) { e0[m] = fmaf(f0, tt[q * M + m], e0[m]); e1[m] = fmaf(f1, tt[q * M + m], e1[m]); }
            }
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            e0[m] += __shfl_xor_sync(0xffffffffu, e0[m], 1); e0[m] += __shfl_xor_sync(0xffffffffu, e0[m], 2);
            e1[m] += __shfl_xor_sync(0xffffffffu, e1[m], 1); e1[m] += __shfl_xor_sync(0xffffffffu, e1[m], 2);
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            if (m == 2 * t)     { y[0] += e0[m]; y[2] += e1[m]; }
            if (m == 2 * t + 1) { y[1] += e0[m]; y[3] += e1[m]; }
        }
    }
    XT* out = static_cast<XT*>(a.y);
    const float b0 = a.bias ? __half2float(a.bias[c0]) : 0.0f;
    const float b1 = a.bias ? __half2float(a.bias[c1]) : 0.0f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int m = 2 * t + h;
        if (m < M) {
            if (r0 < a.n) out[(size_t)m * a.ldy + r0] = Act16<BF16>::from_float(apply_act(y[h] + b0, a.act));
            if (r1 < a.n) out[(size_t)m * a.ldy + r1] = Act16<BF16>::from_float(apply_act(y[2 + h] + b1, a.act));
        }
    }
}

// First unit of warp w, and the warp that owns unit u, under the even split of `units` over `warps`.
// (units < 2^31 and warps < 2^16, so the products fit 64 bits; the quotients fit 32.)
__device__ __forceinline__ int first_unit(int w, int units, int warps) {
    return (int)((unsigned long long)w * (unsigned)units / (unsigned)warps);
}
__device__ __forceinline__ int owner_of(int u, int units, int warps) {
    return (int)((((unsigned long long)u + 1) * (unsigned)warps - 1) / (unsigned)units);
}

// ---------------------------------------------------------------------------------------------
// The kernel.  blockDim.x = 32 * nw; every warp is its own producer and consumer.
// ---------------------------------------------------------------------------------------------
template <int BITS, int GB, int M, bool BF16>
__global__ void __launch_bounds__(512, 1) qgemv_mma_kernel(const __grid_constant__ MmaArgs p) {
    using GE = Geo<BITS, GB>;
    extern __shared__ __align__(128) unsigned char smem[];
    const Args& a = p.a;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    // Global warp index, CTA-minor, so that the first W warps are spread over all CTAs.  W never
    // exceeds the number of units: every warp below W owns at least one unit, the rest idle.
    const int W = p.total_warps, U = p.units;
    const int gw = warp * gridDim.x + blockIdx.x;
    const bool active = gw < W;
    const int u0 = active ? first_unit(gw, U, W) : 0, u1 = active ? first_unit(gw + 1, U, W) : 0;

    unsigned char* ring = smem + p.off_ring + (size_t)warp * p.stages * GE::STAGE_BYTES;
    const uint32_t ring_u32 = smem_u32(ring);
    QTRACE(0);

    // Start the copy of the unit (tile, ch) into ring slot s and commit it as one group (every lane
    // commits exactly one group per call, empty or not, so the group arithmetic stays uniform).
    constexpr int PPR = GE::CB / 16;                 // 16-byte pieces per row of a full chunk
    constexpr int RPI = 32 / PPR;                    // rows covered by one warp-wide copy instruction
    const int lrow = lane / PPR, lcol = lane % PPR;
    auto issue = [&](bool valid, int tile, int ch, int s) {
        if (valid) {
            const int pieces = min(GE::CB, p.row_bytes - ch * GE::CB) >> 4;
            if (lcol < pieces) {
                const uint32_t dst = ring_u32 + s * GE::STAGE_BYTES + lcol * 16;
                const uint8_t* src = a.packed + (size_t)ch * GE::CB + lcol * 16;
#pragma unroll
                for (int it = 0; it < kTileRows / RPI; ++it) {
                    const int r = it * RPI + lrow;
                    const int row = min(tile * kTileRows + r, a.n - 1);
                    cp_async16(dst + r * GE::PITCH, src + (size_t)row * a.ldp);
                }
            }
        }
        cp_async_commit();
    };

    // prefetch cursor (pf_*) runs `stages` units ahead of the consume cursor
    int pf = u0, pf_tile = u0 / p.nch, pf_ch = u0 - pf_tile * p.nch;
    auto advance_pf = [&]() { ++pf; if (++pf_ch == p.nch) { pf_ch = 0; ++pf_tile; } };
    stage_activations<BITS, GB, M, BF16>(p, smem, [&]() {
        for (int s = 0; s < p.stages; ++s) { issue(pf < u1, pf_tile, pf_ch, s); advance_pf(); }
        QTRACE(1);
    });                                                   // CTA-wide, ends with __syncthreads()
    QTRACE(2);

    const float2* gx = reinterpret_cast<const float2*>(smem + p.off_sumx);
    const uint4* xs16 = reinterpret_cast<const uint4*>(smem + p.off_xs);
    const int ma = min(2 * t, M - 1), mb = min(2 * t + 1, M - 1);

    // scales of a unit (raw fp16), one per (row g / g+8, group of the chunk), fetched one unit ahead
    __half sc0[GE::CG], sc1[GE::CG];
    auto load_scales = [&](int tile, int ch, __half (&d0)[GE::CG], __half (&d1)[GE::CG]) {
        const int ra = min(tile * kTileRows + g, a.n - 1), rb = min(tile * kTileRows + g + 8, a.n - 1);
        const __half* pa = a.scales + (size_t)ra * a.lds + ch * GE::CG;
        const __half* pb = a.scales + (size_t)rb * a.lds + ch * GE::CG;
        const int ngr = min(GE::CG, p.ng - ch * GE::CG);
#pragma unroll
        for (int i = 0; i < GE::CG; ++i) {
            d0[i] = i < ngr ? __ldg(pa + i) : __half(0.0f);
            d1[i] = i < ngr ? __ldg(pb + i) : __half(0.0f);
        }
    };
    int tile = u0 / p.nch, ch = u0 - tile * p.nch;
    const int my_first_tile = tile;
    if (u0 < u1) load_scales(tile, ch, sc0, sc1);

    float y[4] = {0.f, 0.f, 0.f, 0.f};
    int seg_first_ch = ch;
    int stage = 0;

    for (int u = u0; u < u1; ++u) {
        int ntile = tile, nch_ = ch + 1;
        if (nch_ == p.nch) { nch_ = 0; ++ntile; }
        __half nsc0[GE::CG], nsc1[GE::CG];
        if (u + 1 < u1) load_scales(ntile, nch_, nsc0, nsc1);

        cp_async_wait_dyn(p.stages - 1);        // all but the newest stages-1 groups are done: unit u has landed
        __syncwarp();
        if (u == u0) QTRACE(3);
        const int ngr = min(GE::CG, p.ng - ch * GE::CG);
        const unsigned char* base0 = ring + stage * GE::STAGE_BYTES + g * GE::PITCH + t * GE::TB;
        const unsigned char* base1 = base0 + 8 * GE::PITCH;
#pragma unroll
        for (int gi = 0; gi < GE::CG; ++gi) {
            if (gi < ngr) {
                const int G = ch * GE::CG + gi;
                uint32_t w0[GE::TW], w1[GE::TW];
                if constexpr (GE::TW == 1) {
                    w0[0] = *reinterpret_cast<const uint32_t*>(base0 + gi * GB);
                    w1[0] = *reinterpret_cast<const uint32_t*>(base1 + gi * GB);
                } else if constexpr (GE::TW == 2) {
                    const uint2 v0 = *reinterpret_cast<const uint2*>(base0 + gi * GB);
                    const uint2 v1 = *reinterpret_cast<const uint2*>(base1 + gi * GB);
                    w0[0] = v0.x; w0[1] = v0.y; w1[0] = v1.x; w1[1] = v1.y;
                } else {
                    const uint4 v0 = *reinterpret_cast<const uint4*>(base0 + gi * GB);
                    const uint4 v1 = *reinterpret_cast<const uint4*>(base1 + gi * GB);
                    w0[0] = v0.x; w0[1] = v0.y; w0[2] = v0.z; w0[3] = v0.w;
                    w1[0] = v1.x; w1[1] = v1.y; w1[2] = v1.z; w1[3] = v1.w;
                }
                // two independent accumulator chains (the classes alternate between them)
                float accA[4] = {0.f, 0.f, 0.f, 0.f}, accB[4] = {0.f, 0.f, 0.f, 0.f};
                const uint4* xg = xs16 + ((size_t)(G * GE::TW) * (GE::NCLS / 2) * M + g) * 4 + t;
#pragma unroll
                for (int i = 0; i < GE::TW; ++i) {
                    const uint32_t h0 = w0[i] >> 8, h1 = w1[i] >> 8;
#pragma unroll
                    for (int cp = 0; cp < GE::NCLS / 2; ++cp) {
                        uint4 b = make_uint4(0u, 0u, 0u, 0u);
                        if (g < M) b = xg[(size_t)(i * (GE::NCLS / 2) + cp) * M * 4];
                        constexpr uint32_t MK = GE::MASK;
                        const uint32_t m0 = MK << (BITS * (2 * cp)), m1 = MK << (BITS * (2 * cp + 1));
                        mma_f16(accA, w0[i] & m0, w1[i] & m0, h0 & m0, h1 & m0, b.x, b.y);
                        mma_f16(accB, w0[i] & m1, w1[i] & m1, h0 & m1, h1 & m1, b.z, b.w);
                    }
                }
                const float s0 = __half2float(sc0[gi]), s1 = __half2float(sc1[gi]);
                const float2 ga = gx[G * M + ma], gb = gx[G * M + mb];
                y[0] = fmaf(s0, fmaf(ga.y, accA[0] + accB[0], -ga.x), y[0]);
                y[1] = fmaf(s0, fmaf(gb.y, accA[1] + accB[1], -gb.x), y[1]);
                y[2] = fmaf(s1, fmaf(ga.y, accA[2] + accB[2], -ga.x), y[2]);
                y[3] = fmaf(s1, fmaf(gb.y, accA[3] + accB[3], -gb.x), y[3]);
            }
        }
        __syncwarp();
        issue(pf < u1, pf_tile, pf_ch, stage);
        advance_pf();
        stage = stage + 1 == p.stages ? 0 : stage + 1;
#pragma unroll
        for (int i = 0; i < GE::CG; ++i) { sc0[i] = nsc0[i]; sc1[i] = nsc1[i]; }

        if (u == u1 - 1) QTRACE(4);
        if (ch == p.nch - 1 || u == u1 - 1) {
            if (seg_first_ch == 0 && ch == p.nch - 1) {
                finish_tile<M, BF16>(p, smem, tile, y);
            } else {
                // Partial tile: park the partial sums, count arrivals, last one in adds them up in warp order.
                const int slot = tile == my_first_tile ? 0 : 1;
                float* mine = a.partial + ((size_t)(gw * 2 + slot) * 4) * 32;
#pragma unroll
                for (int i = 0; i < 4; ++i) mine[i * 32 + lane] = y[i];
                __threadfence();
                __syncwarp();
                const int wf = owner_of(tile * p.nch, U, W);
                const int wl = owner_of(tile * p.nch + p.nch - 1, U, W);
                int last = 0;
                if (lane == 0) {
                    const int old = atomicAdd(&a.counters[tile], 1);
                    last = old == wl - wf;
                    if (last) a.counters[tile] = 0;          // ready for the next launch
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence();
                    y[0] = y[1] = y[2] = y[3] = 0.f;
                    for (int wb = wf; wb <= wl; wb += 4) {     // four contributors' loads in flight at a time
                        float v[4][4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int w = min(wb + k, wl);
                            const int s = tile == first_unit(w, U, W) / p.nch ? 0 : 1;
                            const float* src = a.partial + ((size_t)(w * 2 + s) * 4) * 32;
#pragma unroll
                            for (int i = 0; i < 4; ++i) v[k][i] = ld_cg_f32(src + i * 32 + lane);
                        }
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            if (wb + k <= wl) {
#pragma unroll
                                for (int i = 0; i < 4; ++i) y[i] += v[k][i];
                            }
                    }
                    finish_tile<M, BF16>(p, smem, tile, y);
                }
            }
            y[0] = y[1] = y[2] = y[3] = 0.f;
            seg_first_ch = 0;
        }
        tile = ntile; ch = nch_;
    }
    QTRACE(5);
}

constexpr int kMaxDynSmem = 232448;   // 227 KB per CTA on sm_100

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

inline int align_up(int v, int a) { return (v + a - 1) / a * a; }

template <int BITS, int GB, int M, bool BF16>
int launch_one(const MmaArgs& p, int grid, int smem_bytes, cudaStream_t s) {
    auto kern = qgemv_mma_kernel<BITS, GB, M, BF16>;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem) != cudaSuccess)
            return check_launch("cudaFuncSetAttribute(qgemv_mma_kernel)");
        configured[dev] = true;
    }
    kern<<<grid, p.nw * 32, smem_bytes, s>>>(p);
    return check_launch("qgemv_mma_kernel");
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

MmaPlan plan_mma(const qgemv_problem& p) {
    MmaPlan pl{};
    pl.ok = false;
    const int gb = p.group * p.bits / 8;
    if (gb != 16 && gb != 32 && gb != 64) return pl;
    if (p.group * p.bits % 8) return pl;
    auto al = [](const void* q, size_t a) { return reinterpret_cast<uintptr_t>(q) % a == 0; };
    if (!al(p.packed, 16) || p.ldp % 16 || !al(p.x, 16) || p.ldx % 8) return pl;
    if (p.outliers > kMaxOutliers || p.rank > kMaxRank) return pl;
    const int cg = (256 / gb) > 8 ? 8 : (256 / gb);
    const int cb = cg * gb, pitch = cb + gb, stage_bytes = kTileRows * pitch;
    pl.gb = gb;
    pl.ng = p.k_padded / p.group;
    pl.nch = (pl.ng + cg - 1) / cg;
    pl.nt = (p.n + kTileRows - 1) / kTileRows;
    if (pl.nt > kWsMaxCounters - 1) return pl;
    int off = 1024;
    pl.off_xo = off;   off = align_up(off + p.outliers * p.m * 4, 16);
    pl.off_tt = off;   off = align_up(off + p.rank * p.m * 4, 16);
    pl.off_sumx = off; off = align_up(off + pl.ng * p.m * 8, 16);
    pl.off_xs = off;   off = align_up(off + p.m * p.k_padded * 2, 128);
    pl.off_ring = off;
    // Most warps first (latency hiding), at least 3 ring slots each if possible.
    int nw = 0, stages = 0;
    const int avail = kMaxDynSmem - off;
    for (int want = 3; want >= 2 && !nw; --want)
        for (int cand = 16; cand >= 4; cand -= 4)
            if (avail / (cand * stage_bytes) >= want) { nw = cand; stages = avail / (cand * stage_bytes); break; }
    if (!nw) return pl;
    if (stages > 4) stages = 4;
    if ((long long)pl.nt * pl.nch > 0x3fffffff) return pl;
    pl.nw = nw;
    pl.stages = stages;
    pl.off_bar = 0;
    pl.smem_bytes = off + nw * stages * stage_bytes;
    const long long units = (long long)pl.nt * pl.nch;
    const int sms = sm_count();
    pl.grid = (int)(units < sms ? units : sms);
    if ((size_t)pl.grid * nw * 2 * 4 * 32 > kMaxPartialFloats) return pl;
    static const char* names[2][3] = {{"mma_int2_g64", "mma_int2_g128", "mma_int2_g256"},
                                      {"mma_int4_g32", "mma_int4_g64", "mma_int4_g128"}};
    pl.name = names[p.bits == 2 ? 0 : 1][gb == 16 ? 0 : gb == 32 ? 1 : 2];
    pl.ok = true;
    return pl;
}

int launch_mma(const Args& a, int bits, bool bf16, const MmaPlan& pl, cudaStream_t s) {
    MmaArgs p{};
    p.a = a;
    p.nt = pl.nt; p.nch = pl.nch; p.ng = pl.ng;
    p.row_bytes = a.kpad * bits / 8;
    p.nw = pl.nw; p.stages = pl.stages;
    p.units = pl.nt * pl.nch;
    p.total_warps = p.units < pl.grid * pl.nw ? p.units : pl.grid * pl.nw;
    p.off_xo = pl.off_xo; p.off_tt = pl.off_tt; p.off_sumx = pl.off_sumx; p.off_xs = pl.off_xs;
    p.off_ring = pl.off_ring;
    return bits == 2 ? launch_gb<2>(p, pl.gb, bf16, pl.grid, pl.smem_bytes, s)
                     : launch_gb<4>(p, pl.gb, bf16, pl.grid, pl.smem_bytes, s);
}

}  // namespace qgemv
