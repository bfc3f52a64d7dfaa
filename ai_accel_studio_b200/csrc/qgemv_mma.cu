// Streaming fused GEMV for packed groupwise INT2 / INT4 weights, M <= 4, sm_100a.
//
// Why this kernel exists: at full HBM rate a B200 SM receives ~24 packed bytes per clock, i.e.
// ~95 INT2 or ~47 INT4 weights, but can issue only 128 thread-instructions per clock.  An
// "unpack + fp32 FMA per weight" loop needs 2 + M instructions per weight and is therefore
// issue bound (qgemv_simt.cu measures that).  Here the per-weight cost is ~0.6 instructions:
//
//  * Packed rows are brought into shared memory by the TMA engine (cp.async.bulk, one copy per
//    row per chunk, completion on an mbarrier) into a per-warp ring -- no registers, no
//    coalescing constraints, up to 128 KB in flight per SM.
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
constexpr int kWaitPollLimit = 1 << 22;

struct MmaArgs {
    Args a;
    int nt;            // row tiles: ceil(N / 16)
    int nch;           // chunks per tile
    int ng;            // groups per row
    int row_bytes;     // packed bytes per row actually used (Kpad * bits / 8)
    int nw;            // consumer warps per CTA
    int stages;        // ring depth per warp
    long long units;   // nt * nch
    int total_warps;   // warps that own work: min(gridDim.x * nw, units)
    // dynamic shared memory layout (byte offsets)
    int off_xo, off_tt, off_sumx, off_xs, off_ring, off_bar;
};

// ---------------------------------------------------------------------------------------------
// PTX helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after kWaitPollLimit polls and reports through *status.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status) {
    for (int i = 0; i < kWaitPollLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(32);
    }
    atomicExch(status, 1);
    return false;
}
// TMA engine, untiled form: global -> shared, completion counted in bytes on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16.  No multicast.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
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
// Activation staging (whole CTA): x -> fp16 multiplicands in B-fragment order, group sums,
// per-row power-of-two normalisation, outlier activations and residual projections.
// ---------------------------------------------------------------------------------------------
template <int BITS, int GB, int M, bool BF16>
__device__ __forceinline__ void stage_activations(const MmaArgs& p, unsigned char* smem) {
    using XT = typename Act16<BF16>::T;
    using GE = Geo<BITS, GB>;
    const Args& a = p.a;
    const int tid = threadIdx.x, nthr = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarp = nthr >> 5;
    float* hdr = reinterpret_cast<float*>(smem);                      // [0..3] cs[m], [4..7] scratch
    float* red = reinterpret_cast<float*>(smem) + 8;                   // [nwarp][M] absmax scratch (<= 32*4)
    float* xo = reinterpret_cast<float*>(smem + p.off_xo);
    float* tt = reinterpret_cast<float*>(smem + p.off_tt);
    float* sumx = reinterpret_cast<float*>(smem + p.off_sumx);
    __half* xs = reinterpret_cast<__half*>(smem + p.off_xs);
    const XT* x = static_cast<const XT*>(a.x);
    const int k8n = a.kpad >> 3;                                       // 16-byte pieces per row of x

    // pass 1: largest magnitude per activation row
    float mx[M];
#pragma unroll
    for (int m = 0; m < M; ++m) mx[m] = 0.0f;
    for (int i = tid; i < k8n; i += nthr) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)m * a.ldx + (size_t)i * 8);
            const XT* e = reinterpret_cast<const XT*>(&v);
#pragma unroll
            for (int q = 0; q < 8; ++q) mx[m] = fmaxf(mx[m], fabsf(Act16<BF16>::to_float(e[q])));
        }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx[m] = fmaxf(mx[m], __shfl_xor_sync(0xffffffffu, mx[m], o));
        if (lane == 0) red[warp * M + m] = mx[m];
    }
    // outlier activations and residual projections for the epilogue
    for (int i = tid; i < a.oc * M; i += nthr) {
        const int j = i / M, m = i - j * M;
        const int col = a.oidx[j];
        xo[i] = (col >= 0 && col < a.kpad) ? Act16<BF16>::to_float(x[(size_t)m * a.ldx + col]) : 0.0f;
    }
    for (int i = tid; i < a.rank * M; i += nthr) {
        const int q = i / M, m = i - q * M;
        tt[i] = a.t[m * kMaxRank + q];
    }
    __syncthreads();
    if (tid < M) {
        float v = 0.0f;
        for (int w = 0; w < nwarp; ++w) v = fmaxf(v, red[w * M + tid]);
        int e = 0;
        if (v > 0.0f && v < 3.0e38f) e = ilogbf(v) - 13;
        e = max(-60, min(100, e));
        hdr[4 + tid] = __int_as_float((127 - e) << 23);                 // 2^-e : multiplier for x
        const float up = __int_as_float((127 + 24 + e) << 23);          // 2^(24+e): undoes subnormal unit and row scale
        hdr[tid] = BITS == 2 ? up * (2.0f / 3.0f) : up;
    }
    __syncthreads();

    // pass 2: scaled multiplicands in fragment order + per-group sums of x
    constexpr int SEG = GE::G / 8;                                      // lanes that share a group
    const int total = M * k8n;
    const int rounds = (total + nthr - 1) / nthr;
    for (int r = 0; r < rounds; ++r) {
        const int idx = r * nthr + tid;
        const bool live = idx < total;
        const int m = live ? idx / k8n : 0;
        const int i8 = live ? idx - m * k8n : 0;
        float part = 0.0f;
        if (live) {
            const uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)m * a.ldx + (size_t)i8 * 8);
            const XT* e = reinterpret_cast<const XT*>(&v);
            const float down = hdr[4 + m];
            const int k = i8 * 8;
            const int grp = k / GE::G, rr = k - grp * GE::G;
            const int wordpos = rr / GE::CW, t = wordpos / GE::TW, i = wordpos - t * GE::TW;
            const int j0 = rr - wordpos * GE::CW;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float f = Act16<BF16>::to_float(e[q]);
                part += f;
                const int j = j0 + q;
                const int c = j % GE::NCLS, qq = j / GE::NCLS;
                const int pos = (qq & 1) * 2 + (qq >> 1);
                const float sc = __int_as_float((127 - BITS * c) << 23);   // radix^-c
                const size_t h = ((((size_t)(grp * GE::TW + i) * (GE::NCLS / 2) + (c >> 1)) * M + m) * 4 + t) * 8 +
                                 (c & 1) * 4 + pos;
                xs[h] = __float2half_rn(f * down * sc);
            }
        }
#pragma unroll
        for (int o = 1; o < SEG; o <<= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if (live && (lane % SEG) == 0) {
            const int grp = (i8 * 8) / GE::G;
            sumx[grp * M + m] = BITS == 2 ? part : 8.0f * part;
        }
    }
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
        for (int j = t; j < a.oc; j += 4) {
            const float w0 = __half2float(a.ow[(size_t)c0 * a.ldow + j]);
            const float w1 = __half2float(a.ow[(size_t)c1 * a.ldow + j]);
#pragma unroll
            for (int m = 0; m < M; ++m) { e0[m] = fmaf(w0, xo[j * M + m], e0[m]); e1[m] = fmaf(w1, xo[j * M + m], e1[m]); }
        }
        for (int q = t; q < a.rank; q += 4) {
            const float w0 = __half2float(a.ru[(size_t)c0 * a.ldu + q]);
            const float w1 = __half2float(a.ru[(size_t)c1 * a.ldu + q]);
#pragma unroll
            for (int m = 0; m < M; ++m) { e0[m] = fmaf(w0, tt[q * M + m], e0[m]); e1[m] = fmaf(w1, tt[q * M + m], e1[m]); }
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
__device__ __forceinline__ long long first_unit(long long w, long long units, long long warps) { return w * units / warps; }
__device__ __forceinline__ int owner_of(long long u, long long units, long long warps) {
    return (int)(((u + 1) * warps - 1) / units);
}

// ---------------------------------------------------------------------------------------------
// The kernel.  blockDim.x = 32 * nw; every warp is its own producer and consumer.
// ---------------------------------------------------------------------------------------------
template <int BITS, int GB, int M, bool BF16>
__global__ void __launch_bounds__(256, 1) qgemv_mma_kernel(const __grid_constant__ MmaArgs p) {
    using GE = Geo<BITS, GB>;
    extern __shared__ __align__(128) unsigned char smem[];
    const Args& a = p.a;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    // Global warp index, CTA-minor, so that the first W warps are spread over all CTAs.  W never
    // exceeds the number of units: every warp below W owns at least one unit, the rest idle.
    const long long W = p.total_warps;
    const long long gw = (long long)warp * gridDim.x + blockIdx.x;
    const bool active = gw < W;
    const long long u0 = active ? first_unit(gw, p.units, W) : 0, u1 = active ? first_unit(gw + 1, p.units, W) : 0;
    int* status = a.counters + (kWsMaxCounters - 1);

    unsigned char* ring = smem + p.off_ring + (size_t)warp * p.stages * GE::STAGE_BYTES;
    const uint32_t ring_u32 = smem_u32(ring);
    const uint32_t bar_u32 = smem_u32(smem + p.off_bar) + warp * p.stages * 8;

    if (lane == 0) {
        for (int s = 0; s < p.stages; ++s) mbar_init(bar_u32 + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();

    // Start the copy of unit u into ring slot s (all lanes call; lanes 0..15 each move one row).
    auto issue = [&](long long u, int s) {
        const int tile = (int)(u / p.nch), ch = (int)(u - (long long)tile * p.nch);
        const uint32_t bytes = (uint32_t)min(GE::CB, p.row_bytes - ch * GE::CB);
        const uint32_t bar = bar_u32 + s * 8;
        if (lane == 0) mbar_expect_tx(bar, bytes * kTileRows);
        __syncwarp();
        if (lane < kTileRows) {
            const int row = min(tile * kTileRows + lane, a.n - 1);
            bulk_g2s(ring_u32 + s * GE::STAGE_BYTES + lane * GE::PITCH,
                     a.packed + (size_t)row * a.ldp + (size_t)ch * GE::CB, bytes, bar);
        }
    };

    long long pf = u0;
    for (int s = 0; s < p.stages; ++s, ++pf)
        if (pf < u1) issue(pf, s);

    stage_activations<BITS, GB, M, BF16>(p, smem);       // CTA-wide, ends with __syncthreads()

    const float* hdr = reinterpret_cast<const float*>(smem);
    const float* sumx = reinterpret_cast<const float*>(smem + p.off_sumx);
    const uint4* xs16 = reinterpret_cast<const uint4*>(smem + p.off_xs);
    const int ma = min(2 * t, M - 1), mb = min(2 * t + 1, M - 1);
    const float csa = hdr[ma], csb = hdr[mb];

    // scales of the current unit (raw fp16), one per (row g / g+8, group of the chunk)
    __half sc0[GE::CG], sc1[GE::CG];
    auto load_scales = [&](long long u, __half (&d0)[GE::CG], __half (&d1)[GE::CG]) {
        const int tile = (int)(u / p.nch), ch = (int)(u - (long long)tile * p.nch);
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
    if (u0 < u1) load_scales(u0, sc0, sc1);

    float y[4] = {0.f, 0.f, 0.f, 0.f};
    int seg_first_ch = 0, cur_tile = -1;
    const int my_first_tile = (int)(u0 / p.nch);
    uint32_t phases = 0;
    int stage = 0;
    bool healthy = true;

    for (long long u = u0; u < u1; ++u) {
        const int tile = (int)(u / p.nch), ch = (int)(u - (long long)tile * p.nch);
        if (tile != cur_tile) { cur_tile = tile; seg_first_ch = ch; y[0] = y[1] = y[2] = y[3] = 0.f; }
        __half nsc0[GE::CG], nsc1[GE::CG];
        if (u + 1 < u1) load_scales(u + 1, nsc0, nsc1);

        if (healthy) healthy = mbar_wait(bar_u32 + stage * 8, (phases >> stage) & 1u, status);
        phases ^= 1u << stage;
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
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int i = 0; i < GE::TW; ++i) {
                    const uint32_t h0 = w0[i] >> 8, h1 = w1[i] >> 8;
#pragma unroll
                    for (int cp = 0; cp < GE::NCLS / 2; ++cp) {
                        uint4 b = make_uint4(0u, 0u, 0u, 0u);
                        if (g < M) b = xs16[(((size_t)(G * GE::TW + i) * (GE::NCLS / 2) + cp) * M + g) * 4 + t];
                        constexpr uint32_t MK = GE::MASK;
                        const uint32_t m0 = MK << (BITS * (2 * cp)), m1 = MK << (BITS * (2 * cp + 1));
                        mma_f16(acc, w0[i] & m0, w1[i] & m0, h0 & m0, h1 & m0, b.x, b.y);
                        mma_f16(acc, w0[i] & m1, w1[i] & m1, h0 & m1, h1 & m1, b.z, b.w);
                    }
                }
                const float s0 = __half2float(sc0[gi]), s1 = __half2float(sc1[gi]);
                const float xa = sumx[G * M + ma], xb = sumx[G * M + mb];
                y[0] = fmaf(s0, fmaf(csa, acc[0], -xa), y[0]);
                y[1] = fmaf(s0, fmaf(csb, acc[1], -xb), y[1]);
                y[2] = fmaf(s1, fmaf(csa, acc[2], -xa), y[2]);
                y[3] = fmaf(s1, fmaf(csb, acc[3], -xb), y[3]);
            }
        }
        __syncwarp();
        if (pf < u1) issue(pf, stage);
        ++pf;
        stage = stage + 1 == p.stages ? 0 : stage + 1;
#pragma unroll
        for (int i = 0; i < GE::CG; ++i) { sc0[i] = nsc0[i]; sc1[i] = nsc1[i]; }

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
                const int wf = owner_of((long long)tile * p.nch, p.units, W);
                const int wl = owner_of((long long)tile * p.nch + p.nch - 1, p.units, W);
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
                    for (int w = wf; w <= wl; ++w) {
                        const int s = tile == (int)(first_unit(w, p.units, W) / p.nch) ? 0 : 1;
                        const float* src = a.partial + ((size_t)(w * 2 + s) * 4) * 32;
#pragma unroll
                        for (int i = 0; i < 4; ++i) y[i] += ld_cg_f32(src + i * 32 + lane);
                    }
                    finish_tile<M, BF16>(p, smem, tile, y);
                }
            }
        }
    }
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
    pl.off_sumx = off; off = align_up(off + pl.ng * p.m * 4, 16);
    pl.off_xs = off;   off = align_up(off + p.m * p.k_padded * 2, 128);
    pl.off_ring = off;
    int nw = 8, stages = 0;
    for (; nw >= 4; nw -= 4) {
        const int avail = kMaxDynSmem - off - nw * 4 * 8 - 64;
        stages = avail / (nw * stage_bytes);
        if (stages > 4) stages = 4;
        if (stages >= 2) break;
    }
    if (stages < 2) return pl;
    pl.nw = nw;
    pl.stages = stages;
    pl.off_bar = align_up(off + nw * stages * stage_bytes, 16);
    pl.smem_bytes = pl.off_bar + nw * stages * 8;
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
    p.units = (long long)pl.nt * pl.nch;
    p.total_warps = (int)(p.units < (long long)pl.grid * pl.nw ? p.units : (long long)pl.grid * pl.nw);
    p.off_xo = pl.off_xo; p.off_tt = pl.off_tt; p.off_sumx = pl.off_sumx; p.off_xs = pl.off_xs;
    p.off_ring = pl.off_ring; p.off_bar = pl.off_bar;
    return bits == 2 ? launch_gb<2>(p, pl.gb, bf16, pl.grid, pl.smem_bytes, s)
                     : launch_gb<4>(p, pl.gb, bf16, pl.grid, pl.smem_bytes, s);
}

}  // namespace qgemv
