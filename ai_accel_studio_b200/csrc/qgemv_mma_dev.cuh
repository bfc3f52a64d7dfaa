// Device-side building blocks shared by the tensor-core-assisted GEMV kernels (qgemv_mma.cu: the
// barrier-phased kernel, qgemv_pipe.cu: the pipelined kernel): launch parameters, PTX wrappers,
// the compile-time geometry of a (bit width, group bytes) pair, and the tile epilogue.
#pragma once
#include "qgemv_common.cuh"

namespace qgemv {

// Launch parameters of the tensor-core-assisted kernels (one trivially copyable kernel argument).
struct MmaArgs {
    Args a;
    int nt;            // row tiles: ceil(N / 16)
    int nch;           // chunks per tile
    int ng;            // groups per row
    int row_bytes;     // packed bytes per row actually used (Kpad * bits / 8)
    int nw;            // warps per CTA
    int stages;        // ring depth per warp
    int rlen;          // chunks per run (a run = consecutive chunks of one tile, the unit of work)
    int rpt;           // runs per tile
    int runs;          // nt * rpt
    int uq, urem;      // split of the work units (tiles or runs) over the CTAs: see first_unit()
    int scales_async;  // scale rows are aligned for 8/16-byte asynchronous copies
    int epi_async;     // outlier / residual rows are aligned for 16-byte asynchronous copies
    int ocb, rb;       // bytes per prefetched outlier-weight row / residual row (multiples of 16)
    int epi_bytes;     // bytes of one warp's epilogue prefetch buffer
    int wait_for_x;    // 1: the producer of x may still be running when this kernel starts
    int tile_aligned;  // 1: every CTA owns whole tiles
    int t_inline;      // 1: the residual projections t = V.x are computed by the first CTAs of this kernel
    int t_parts;       // K is cut into this many parts of 8 * blockDim.x columns for that
    int off_tt;        // shared-memory table of t
    // dynamic shared memory layout (byte offsets)
    int off_xo, off_gx, off_slots, off_epi, off_meta, off_xs, off_ring;
    // used by the barrier-free kernel only
    int epi_tiles;     // tiles per CTA (its first ones) whose epilogue operands are prefetched into shared memory
    int t_pv;          // 16-byte pieces of res_v per thread of a residual-projection job
    int l2_chunks;     // chunks per warp announced to L2, beyond the ring, before the kernel waits for its predecessor
    int debug;         // qgemv_problem.debug
    int off_cnt;       // per-tile arrival counters of the CTA, followed by the "table of t is ready" flag
    int off_red;       // per-warp partial sums of a residual-projection job
};

namespace {

#ifndef QGEMV_MAX_WARPS
#define QGEMV_MAX_WARPS 16
#endif
constexpr int kMaxWarps = QGEMV_MAX_WARPS;   // warps per CTA the kernel is compiled for (register budget = 65536 / (32 * warps))
constexpr int kTileRows = 16;          // weight rows per mma tile (one warp owns one tile at a time)
constexpr int kMaxOutliers = 256;      // outlier activations staged in shared memory


// ---------------------------------------------------------------------------------------------
// PTX helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Asynchronous 16-byte global -> shared copy (LDGSTS), L2-only caching.  Completion is tracked per
// thread in commit groups; a group counts as done for the whole warp after wait + __syncwarp().
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory"); }

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Same with a zero addend: starts an accumulation chain without clearing registers first.
__device__ __forceinline__ void mma_f16_first(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
// Explicit shared-window loads / stores (32-bit addresses).  volatile: they stay ordered with the
// asynchronous-copy waits, which are volatile too.
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a)); return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v; asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a)); return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v; asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a)); return v;
}
__device__ __forceinline__ float2 lds64f(uint32_t a) {
    float2 v; asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a)); return v;
}
__device__ __forceinline__ float4 lds128f(uint32_t a) {
    float4 v; asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a)); return v;
}
__device__ __forceinline__ void sts128f(uint32_t a, float4 v) {
    asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(a), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
// 64-bit relaxed device-scope accesses: a residual projection travels between CTAs as one aligned
// {value, launch tag} word, so the value needs no separate flag, fence or counter.
__device__ __forceinline__ void st_relaxed_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
    unsigned long long v; asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ unsigned ld_relaxed_u32(const int* p) {
    unsigned v; asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
// Programmatic dependent launch: let the next kernel in the stream begin its prologue now, and
// block until the kernels this one depends on have completed and flushed their writes.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
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
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_) :: "memory");                  \
            reinterpret_cast<unsigned long long*>(p.a.partial + (kMaxPartialFloats / 2))        \
                [((size_t)blockIdx.x * 16 + (threadIdx.x >> 5)) * 16 + (slot)] = t_;            \
        }                                                                                       \
    } while (0)
#else
#define QTRACE(slot) do { } while (0)
#endif

// Compile-time facts per (bits, group bytes, chunk bytes).
template <int BITS, int GB, int CHUNK = (GB == 16 ? 128 : 256)>
struct Geo {
    static constexpr int CPB = 8 / BITS;                 // codes per byte
    static constexpr int CW = 32 / BITS;                 // codes per 32-bit word
    static constexpr int NCLS = BITS == 2 ? 4 : 2;       // position classes (codes per 8 mantissa bits)
    static constexpr int G = GB * CPB;                   // group size in codes
    static constexpr int TB = GB / 4;                    // bytes one lane reads per row per group
    static constexpr int TW = TB / 4;                    // ... in 32-bit words
    static constexpr int CB = CHUNK;                     // chunk bytes per row: one or two 128-byte lines
    static constexpr int CG = CB / GB;                   // groups per chunk (8, 4 or 2)
    static constexpr int STAGES = CB == 128 ? 4 : 2;     // ring slots per warp (about 9 KB of ring per warp either way)
    static constexpr int PITCH = CB;                     // rows are dense in shared memory ...
    // ... and bank conflicts are avoided by storing 16-byte piece c of row r at piece position
    // c ^ swz(r): the rows a shared-memory instruction touches together (2 for 16-byte reads,
    // 4 for 8-byte, 8 for 4-byte reads) land in different 128/R-byte bank groups.
    static constexpr int SWZ_ROWS = 128 / (4 * TB);      // R: 2, 4 or 8
    static constexpr int SWZ_MUL = 8 / SWZ_ROWS;
    static __device__ __forceinline__ int swz(int row) { return (row % SWZ_ROWS) * SWZ_MUL; }
    static constexpr int SCALE_OFF = kTileRows * PITCH;  // 16 bytes of scales per row follow the codes
    static constexpr int STAGE_BYTES = kTileRows * PITCH + kTileRows * 16;
    static constexpr uint32_t MASK = BITS == 2 ? 0x00030003u : 0x000f000fu;
    // halves of x' per group laid out for the B fragments: [TW][NCLS/2][M][4 lanes t][8 halves]
};

// ---------------------------------------------------------------------------------------------
// Epilogue of one finished 16-row tile: outlier columns, residual, bias, activation, store.
// Lane (g = lane/4, t = lane%4) holds rows tile*16+g and +8, activation rows 2t and 2t+1.
// `pre` points at this warp's prefetched copy of the tile's outlier-weight rows, residual rows
// and bias (shared memory), or is null, in which case they are read from global memory.
// ---------------------------------------------------------------------------------------------
// e0[m] += sum_j w0[j] * v[j][m] (same for e1 with w1) over the columns j = t, t+4, ... < cols that
// this lane of the quad owns; v is a shared-memory table [cols][M].  JB columns are loaded before
// they are used.
template <int M, int JB>
__device__ __forceinline__ void epi_dot(const __half* w0, const __half* w1, const float* v, int cols, int t,
                                        float (&e0)[M], float (&e1)[M]) {
    for (int jb = 0; jb < cols; jb += 4 * JB) {
        __half h0[JB], h1[JB];
        float vv[JB][M];
#pragma unroll
        for (int i = 0; i < JB; ++i) {
            const int j = jb + 4 * i + t;
            const int jc = min(j, cols - 1);
            h0[i] = j < cols ? w0[j] : __half(0.0f);
            h1[i] = j < cols ? w1[j] : __half(0.0f);
            if constexpr (M == 4) {
                const float4 q = *reinterpret_cast<const float4*>(v + jc * 4);
                vv[i][0] = q.x; vv[i][1] = q.y; vv[i][2] = q.z; vv[i][3] = q.w;
            } else if constexpr (M == 2) {
                const float2 q = *reinterpret_cast<const float2*>(v + jc * 2);
                vv[i][0] = q.x; vv[i][1] = q.y;
            } else {
#pragma unroll
                for (int m = 0; m < M; ++m) vv[i][m] = v[jc * M + m];
            }
        }
#pragma unroll
        for (int i = 0; i < JB; ++i) {
            const float f0 = __half2float(h0[i]), f1 = __half2float(h1[i]);
#pragma unroll
            for (int m = 0; m < M; ++m) { e0[m] = fmaf(f0, vv[i][m], e0[m]); e1[m] = fmaf(f1, vv[i][m], e1[m]); }
        }
    }
}
// The same for rows held in shared memory (16-byte aligned, cols a multiple of 8): lane t of the
// quad owns columns 8t .. 8t+7 of every block of 32, so a row piece is one 16-byte load.
template <int M>
__device__ __forceinline__ void epi_dot_vec(const unsigned char* w0, const unsigned char* w1, const float* v, int cols, int t,
                                            float (&e0)[M], float (&e1)[M]) {
    for (int jb = 8 * t; jb < cols; jb += 32) {
        const uint4 q0 = *reinterpret_cast<const uint4*>(w0 + jb * 2), q1 = *reinterpret_cast<const uint4*>(w1 + jb * 2);
        const __half2* h0 = reinterpret_cast<const __half2*>(&q0);
        const __half2* h1 = reinterpret_cast<const __half2*>(&q1);
        float vv[8][M];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if constexpr (M == 4) {
                const float4 q = *reinterpret_cast<const float4*>(v + (jb + i) * 4);
                vv[i][0] = q.x; vv[i][1] = q.y; vv[i][2] = q.z; vv[i][3] = q.w;
            } else if constexpr (M == 2) {
                const float2 q = *reinterpret_cast<const float2*>(v + (jb + i) * 2);
                vv[i][0] = q.x; vv[i][1] = q.y;
            } else {
#pragma unroll
                for (int m = 0; m < M; ++m) vv[i][m] = v[(jb + i) * M + m];
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f0 = __half22float2(h0[i]), f1 = __half22float2(h1[i]);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                e0[m] = fmaf(f0.x, vv[2 * i][m], e0[m]); e0[m] = fmaf(f0.y, vv[2 * i + 1][m], e0[m]);
                e1[m] = fmaf(f1.x, vv[2 * i][m], e1[m]); e1[m] = fmaf(f1.y, vv[2 * i + 1][m], e1[m]);
            }
        }
    }
}
template <int M>
__device__ __noinline__ void epi_dot_any(const __half* w0, const __half* w1, const float* v, int cols, int t,
                                            float (&e0)[M], float (&e1)[M]) {
    if (cols <= 8) epi_dot<M, 2>(w0, w1, v, cols, t, e0, e1);
    else if (cols <= 16) epi_dot<M, 4>(w0, w1, v, cols, t, e0, e1);
    else epi_dot<M, 8>(w0, w1, v, cols, t, e0, e1);
}
// Adds the quad's column sums and leaves in y the entries this lane owns (rows g / g+8, activation
// rows 2t and 2t+1).
template <int M>
__device__ __forceinline__ void epi_fold(float (&e0)[M], float (&e1)[M], int t, float (&y)[4]) {
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

// Outlier-column and residual terms of one tile for this lane's four outputs.  Kept out of line:
// a launch starts with a cold instruction cache, and problems without these terms should not
// have to step over their code.
template <int M>
__device__ __forceinline__ float4 tile_extras(const MmaArgs& p, const unsigned char* smem, int tile, const unsigned char* pre,
                                              int row_in_tile = -1) {
    const Args& a = p.a;
    const int lane = threadIdx.x & 31, t = lane & 3;
    const int g = row_in_tile >= 0 ? row_in_tile : lane >> 2;      // tile row of this lane's first output row (second: + 8)
    const int c0 = min(tile * kTileRows + g, a.n - 1), c1 = min(tile * kTileRows + g + 8, a.n - 1);
    float e0[M], e1[M];
#pragma unroll
    for (int m = 0; m < M; ++m) { e0[m] = 0.0f; e1[m] = 0.0f; }
    const float* xo = reinterpret_cast<const float*>(smem + p.off_xo);
    const float* tt = reinterpret_cast<const float*>(smem + p.off_tt);
    if (pre) {                                       // prefetched rows: 16-byte pieces
        if (a.oc > 0) epi_dot_vec<M>(pre + g * p.ocb, pre + (g + 8) * p.ocb, xo, a.oc, t, e0, e1);
        const unsigned char* preu = pre + kTileRows * p.ocb;
        if (a.rank > 0) epi_dot_vec<M>(preu + g * p.rb, preu + (g + 8) * p.rb, tt, a.rank, t, e0, e1);
    } else {
        if (a.oc > 0) epi_dot_any<M>(a.ow + (size_t)c0 * a.ldow, a.ow + (size_t)c1 * a.ldow, xo, a.oc, t, e0, e1);
        if (a.rank > 0) epi_dot_any<M>(a.ru + (size_t)c0 * a.ldu, a.ru + (size_t)c1 * a.ldu, tt, a.rank, t, e0, e1);
    }
    float y[4] = {0.f, 0.f, 0.f, 0.f};
    epi_fold<M>(e0, e1, t, y);
    return make_float4(y[0], y[1], y[2], y[3]);
}

template <int M, bool BF16, bool EX>
__device__ __forceinline__ void finish_tile(const MmaArgs& p, const unsigned char* smem, int tile, float (&y)[4],
                                            const unsigned char* pre, int row_in_tile = -1) {
    using XT = typename Act16<BF16>::T;
    const Args& a = p.a;
    const int lane = threadIdx.x & 31, t = lane & 3;
    const int g = row_in_tile >= 0 ? row_in_tile : lane >> 2;      // tile row of this lane's first output row (second: + 8)
    const int r0 = tile * kTileRows + g, r1 = r0 + 8;
    const int c0 = min(r0, a.n - 1), c1 = min(r1, a.n - 1);
    if constexpr (EX) {
        const float4 e = tile_extras<M>(p, smem, tile, pre, row_in_tile);
        y[0] += e.x; y[1] += e.y; y[2] += e.z; y[3] += e.w;
        QTRACE(15);
    }
    XT* out = static_cast<XT*>(a.y);
    float b0 = 0.0f, b1 = 0.0f;
    if (a.bias) {
        if (pre) {
            const __half* pb = reinterpret_cast<const __half*>(pre + kTileRows * (p.ocb + p.rb));
            b0 = __half2float(pb[g]); b1 = __half2float(pb[g + 8]);
        } else {
            b0 = __half2float(a.bias[c0]); b1 = __half2float(a.bias[c1]);
        }
    }
    if (a.act == QGEMV_ACT_SILU_MUL) {
        // rows g and g + 8 of the tile are a (gate, up) pair, both held by this lane: one output per pair,
        // rounded where separate 16-bit operators would round
        auto r16 = [](float v) { return Act16<BF16>::to_float(Act16<BF16>::from_float(v)); };
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int m = 2 * t + h;
            if (m < M) {
                const float gate = r16(y[h] + b0), up = r16(y[2 + h] + b1);
                const float s = r16(gate / (1.0f + __expf(-gate)));
                out[(size_t)m * a.ldy + tile * (kTileRows / 2) + g] = Act16<BF16>::from_float(s * up);
            }
        }
        return;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int m = 2 * t + h;
        if (m < M) {
            if (r0 < a.n) out[(size_t)m * a.ldy + r0] = Act16<BF16>::from_float(apply_act(y[h] + b0, a.act));
            if (r1 < a.n) out[(size_t)m * a.ldy + r1] = Act16<BF16>::from_float(apply_act(y[2 + h] + b1, a.act));
        }
    }
}

// The work units (whole tiles, or runs) are split over the CTAs on the host: every CTA gets `uq`
// units and the last `urem` CTAs one more (the first CTAs may carry a residual projection on top).
// First unit of CTA c, and the CTA that owns unit u:
__device__ __forceinline__ int first_unit(const MmaArgs& p, int c, int parts) {
    return c * p.uq + max(0, c - (parts - p.urem));
}
__device__ __forceinline__ int owner_of(const MmaArgs& p, int u, int parts) {
    const int plain = parts - p.urem, thr = plain * p.uq;
    return u < thr ? u / p.uq : plain + (u - thr) / (p.uq + 1);
}

// Address of entry idx = (part * rank + q) * M + m of the in-kernel residual projections.
__device__ __forceinline__ const unsigned long long* t_entry(const Args& a, int M, int idx) {
    const int RM = a.rank * M, part = idx / RM, i = idx - part * RM, q = i / M, m = i - q * M;
    return reinterpret_cast<const unsigned long long*>(a.tparts) + (part * QGEMV_MAX_M + m) * kMaxRank + q;
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

}  // namespace
}  // namespace qgemv
