// Shared declarations for the packed groupwise INT2 / INT4 GEMV library (sm_100a).
#pragma once

#include <cstdint>
#include <cstddef>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include "../../include/qgemv_b200.h"

namespace qgemv {

// Workspace layout (bytes from the 256-byte aligned base the caller passes):
//   [0, 1024)            residual projections t[m][r] = sum_k V[r,k] x[m,k], fp32, QGEMV_MAX_M x 64
//   [1024, 1024+4*16384) arrival counters, one int32 per 16-row tile (zero between calls)
//   [kWsPartialOff, ..)   partial sums of tiles shared by several warps, fp32 [warp][2][4][32]
constexpr int    kMaxRank        = 64;
constexpr size_t kWsTOff         = 0;
constexpr size_t kWsCounterOff   = 1024;
constexpr int    kWsMaxCounters  = 16384;          // the last four entries are not tile counters:
constexpr int    kWsStatusIdx    = kWsMaxCounters - 1;   //   wait-timeout status word
constexpr int    kWsDoneIdx      = kWsMaxCounters - 3;   //   CTAs that finished the current launch
constexpr int    kWsEpochIdx     = kWsMaxCounters - 4;   //   launches completed so far (tag of in-kernel residual projections)
constexpr size_t kWsPartialOff   = kWsCounterOff + sizeof(int) * kWsMaxCounters;   // 66560, 256-aligned
constexpr int    kMaxTParts      = 8;              // K-parts of an in-kernel residual projection
// tail of the partial-sum area: {fp32 value, launch tag} per (K-part, m, rank column), in 32-bit words
constexpr int    kTPartFloats    = 2 * kMaxTParts * QGEMV_MAX_M * kMaxRank;
constexpr size_t kMaxPartialFloats = size_t(1) << 20;                             // 4 MiB of fp32 partial sums

// Device-side view of one problem; a trivially copyable kernel parameter.
struct Args {
    const void* x;            long long ldx;
    const uint8_t* packed;    long long ldp;
    const __half* scales;     long long lds;
    const __half* bias;
    const int32_t* oidx;
    const __half* ow;         long long ldow;
    const __half* ru;         long long ldu;
    const __half* rv;         long long ldv;
    void* y;                  long long ldy;
    float* t;                 // residual projections (workspace)
    int* counters;            // split-K counters (workspace)
    float* partial;           // split-K partials (workspace)
    float* tparts;            // per-K-part residual projections, 8-byte {value, tag} words (tail of the partial area)
    int m, n, kpad, korig, group, act, oc, rank;
    const unsigned char* hint; long long hint_bytes;   // optional byte range to announce to L2 (the next GEMV's weights)
    int splits;               // number of K splits (grid.y)
    int kspan;                // codes per K split (multiple of the group)
};

template <bool BF16> struct Act16;
template <> struct Act16<false> {
    using T = __half;
    static __device__ __forceinline__ float to_float(T v) { return __half2float(v); }
    static __device__ __forceinline__ T from_float(float v) { return __float2half_rn(v); }
};
template <> struct Act16<true> {
    using T = __nv_bfloat16;
    static __device__ __forceinline__ float to_float(T v) { return __bfloat162float(v); }
    static __device__ __forceinline__ T from_float(float v) { return __float2bfloat16_rn(v); }
};

__device__ __forceinline__ float apply_act(float v, int act) {
    if (act == QGEMV_ACT_RELU) return fmaxf(v, 0.0f);
    if (act == QGEMV_ACT_SILU) return v / (1.0f + __expf(-v));
    return v;
}

// Host-side error reporting (thread local).
void set_error(const char* fmt, ...);
int  check_launch(const char* what);

// Launchers implemented in the kernel translation units.
int launch_residual_t(const Args& a, bool bf16, cudaStream_t s);
int launch_simt(const Args& a, int bits, bool bf16, int unit_bytes, cudaStream_t s);
const char* simt_name(int bits, int m, int unit_bytes);

struct MmaPlan {
    bool ok;
    int gb;                 // packed bytes per group per row (16, 32 or 64)
    int nw, stages;         // warps per CTA, ring depth per warp
    int grid;               // persistent CTAs
    int nt, nch, ng;        // 16-row tiles, chunks per tile, groups per row
    int rlen, rpt;          // chunks per run, runs per tile
    int tile_aligned;       // CTAs own whole tiles
    int t_inline, t_parts;  // residual projections computed inside the fused kernel; K parts for that
    int off_tt;
    int scales_async, epi_async, ocb, rb, epi_bytes;
    int smem_bytes;         // dynamic shared memory
    int off_xo, off_gx, off_slots, off_epi, off_meta, off_xs, off_ring;
    int variant;            // 1: barrier-phased kernel (qgemv_mma.cu), 2: pipelined kernel (qgemv_pipe.cu)
    int epi_tiles, t_pv, l2_chunks, off_cnt, off_red;   // barrier-free kernel only (see MmaArgs)
    int chunk;              // pipelined kernel: packed bytes per row per ring slot (128 or 256)
    const char* name;
};
MmaPlan plan_mma(const qgemv_problem& p, size_t partial_floats);
int launch_mma(const Args& a, int bits, bool bf16, const MmaPlan& plan, int debug, cudaStream_t s);
// The pipelined kernel takes the shapes whose CTAs own whole tiles; `base` is plan_mma's answer.
MmaPlan plan_pipe(const qgemv_problem& p, const MmaPlan& base);
int launch_pipe(const Args& a, int bits, bool bf16, const MmaPlan& plan, int debug, cudaStream_t s);

}  // namespace qgemv
