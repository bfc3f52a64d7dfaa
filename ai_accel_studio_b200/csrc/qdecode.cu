// The kernels of a decode step between the packed GEMVs: see include/qdecode_b200.h.
//
// All of them are latency-sized (tens of kilobytes to a few megabytes per launch): what matters is
// one launch per step of the layer, coalesced 8 / 16-byte accesses, enough CTAs for the attention
// to spread the cache over the SMs, and no waiting between CTAs (the attention's slices meet through
// an arrival counter: whoever comes last merges).
#include <type_traits>

#include "qgemv_common.cuh"
#include "../../include/qdecode_b200.h"

namespace qgemv {
namespace {

template <bool BF16> __device__ __forceinline__ float r16(float v) {
    return Act16<BF16>::to_float(Act16<BF16>::from_float(v));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------------------------------------
// residual update + RMS normalisation: one CTA per row
// ---------------------------------------------------------------------------------------------
constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 8;                    // 8-element vectors per thread: hidden <= 256 * 8 * 8

template <bool BF16>
__global__ void __launch_bounds__(kNormThreads) rmsnorm_kernel(void* h_, long long ldh, const void* delta_, long long ldd,
                                                               const void* w_, void* y_, long long ldy, int hidden, float eps) {
    using T = typename Act16<BF16>::T;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int row = blockIdx.x, tid = threadIdx.x, nvec = hidden >> 3;
    T* h = static_cast<T*>(h_) + (size_t)row * ldh;
    const T* delta = delta_ ? static_cast<const T*>(delta_) + (size_t)row * ldd : nullptr;
    const T* w = static_cast<const T*>(w_);
    T* y = static_cast<T*>(y_) + (size_t)row * ldy;
    __shared__ float red[kNormThreads / 32];
    __shared__ float total;

    float f[kNormMaxVec][8];
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
        const int v = tid + i * kNormThreads;
        if (v < nvec) {
            uint4 hv = *reinterpret_cast<const uint4*>(h + v * 8);
            const T* he = reinterpret_cast<const T*>(&hv);
            if (delta) {
                const uint4 dv = *reinterpret_cast<const uint4*>(delta + v * 8);
                const T* de = reinterpret_cast<const T*>(&dv);
                uint4 ov;
                T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    oe[q] = Act16<BF16>::from_float(Act16<BF16>::to_float(he[q]) + Act16<BF16>::to_float(de[q]));
                    f[i][q] = Act16<BF16>::to_float(oe[q]);
                }
                *reinterpret_cast<uint4*>(h + v * 8) = ov;
            } else {
#pragma unroll
                for (int q = 0; q < 8; ++q) f[i][q] = Act16<BF16>::to_float(he[q]);
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) sq = fmaf(f[i][q], f[i][q], sq);
        }
    }
    sq = warp_sum(sq);
    if ((tid & 31) == 0) red[tid >> 5] = sq;
    __syncthreads();
    if (tid == 0) {
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < kNormThreads / 32; ++i) t += red[i];
        total = rsqrtf(t / (float)hidden + eps);
    }
    __syncthreads();
    const float inv = total;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
        const int v = tid + i * kNormThreads;
        if (v < nvec) {
            const uint4 wv = *reinterpret_cast<const uint4*>(w + v * 8);
            const T* we = reinterpret_cast<const T*>(&wv);
            uint4 ov;
            T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
            for (int q = 0; q < 8; ++q)
                oe[q] = Act16<BF16>::from_float(Act16<BF16>::to_float(we[q]) * r16<BF16>(f[i][q] * inv));
            *reinterpret_cast<uint4*>(y + v * 8) = ov;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// rotary embedding + cache append: one CTA per (head, sequence); heads = q heads, k heads, v heads
// ---------------------------------------------------------------------------------------------
template <bool BF16>
__global__ void __launch_bounds__(128) rope_append_kernel(void* q_, long long ldq, const void* k_, long long ldk,
                                                          const void* v_, long long ldv, const void* cos_, const void* sin_,
                                                          int table_rows, const long long* pos_, void* kc_, void* vc_,
                                                          int hq, int hkv, int d, int max_len, int* status) {
    using T = typename Act16<BF16>::T;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const long long pos = *pos_;
    if (pos < 0 || pos >= max_len || pos >= table_rows) {
        if (status && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) atomicExch(status, 1);
        return;
    }
    const int head = blockIdx.x, b = blockIdx.y, j = threadIdx.x, half = d >> 1;
    if (j >= half) return;
    const T* cs = static_cast<const T*>(cos_) + (size_t)pos * d;
    const T* sn = static_cast<const T*>(sin_) + (size_t)pos * d;
    auto rotate = [&](const T* src, T* dst) {
        const float lo = Act16<BF16>::to_float(src[j]), hi = Act16<BF16>::to_float(src[j + half]);
        // out[j] = r(r(x[j] cos[j]) + r(-x[j + d/2] sin[j])),  out[j + d/2] = r(r(x[j + d/2] cos[j + d/2]) + r(x[j] sin[j + d/2]))
        const float a = r16<BF16>(lo * Act16<BF16>::to_float(cs[j])) + r16<BF16>(-hi * Act16<BF16>::to_float(sn[j]));
        const float c = r16<BF16>(hi * Act16<BF16>::to_float(cs[j + half])) + r16<BF16>(lo * Act16<BF16>::to_float(sn[j + half]));
        dst[j] = Act16<BF16>::from_float(a);
        dst[j + half] = Act16<BF16>::from_float(c);
    };
    if (head < hq) {
        T* q = static_cast<T*>(q_) + (size_t)b * ldq + (size_t)head * d;
        rotate(q, q);
    } else if (head < hq + hkv) {
        const int kh = head - hq;
        const T* k = static_cast<const T*>(k_) + (size_t)b * ldk + (size_t)kh * d;
        T* dst = static_cast<T*>(kc_) + (((size_t)b * hkv + kh) * max_len + (size_t)pos) * d;
        rotate(k, dst);
    } else {
        const int vh = head - hq - hkv;
        const T* v = static_cast<const T*>(v_) + (size_t)b * ldv + (size_t)vh * d;
        T* dst = static_cast<T*>(vc_) + (((size_t)b * hkv + vh) * max_len + (size_t)pos) * d;
        dst[j] = v[j];
        dst[j + half] = v[j + half];
    }
}

// ---------------------------------------------------------------------------------------------
// attention of one query token per sequence: grid (slice, kv head, sequence), 8 warps per CTA
// ---------------------------------------------------------------------------------------------
constexpr int kAttWarps = 8;
constexpr int kAttMaxSlices = 16;
constexpr int kAttMinSlice = 16;                 // positions: shorter slices are not worth a CTA

// Slices the sequence axis is cut into: enough CTAs to cover the SMs, at most kAttMaxSlices.
inline int attention_slices(int batch, int kv_heads, int max_len) {
    const int ctas = batch * kv_heads;
    int s = (148 + ctas - 1) / ctas;
    s = s < 1 ? 1 : s > kAttMaxSlices ? kAttMaxSlices : s;
    const int by_len = max_len / kAttMinSlice;
    if (s > by_len) s = by_len < 1 ? 1 : by_len;
    return s;
}

// One slice's result per (query head of the group): running maximum, sum of exponentials, weighted values.
template <int D> struct alignas(8) Partial { float m, l, o[D]; };

template <int D, int G, bool BF16>
__global__ void __launch_bounds__(kAttWarps * 32) attention_kernel(const void* q_, long long ldq, const void* kc_, const void* vc_,
                                                                   const long long* pos_, void* out_, long long ldo, int hq, int hkv,
                                                                   int max_len, float scale, float* parts, int* counters) {
    using T = typename Act16<BF16>::T;
    constexpr int E = D / 32;                     // elements per lane
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int slice = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, slices = gridDim.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    long long len = *pos_ + 1;
    len = len < 0 ? 0 : len > max_len ? max_len : len;
    const int per = (int)((len + slices - 1) / slices);
    const int s0 = slice * per, s1 = (int)min((long long)(s0 + per), len);

    float qv[G][E];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const T* q = static_cast<const T*>(q_) + (size_t)b * ldq + (size_t)(kvh * G + g) * D + lane * E;
#pragma unroll
        for (int e = 0; e < E; ++e) qv[g][e] = Act16<BF16>::to_float(q[e]) * scale;
    }
    const T* kbase = static_cast<const T*>(kc_) + ((size_t)b * hkv + kvh) * (size_t)max_len * D + lane * E;
    const T* vbase = static_cast<const T*>(vc_) + ((size_t)b * hkv + kvh) * (size_t)max_len * D + lane * E;

    float m[G], l[G], o[G][E];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -1.0e30f; l[g] = 0.0f;
#pragma unroll
        for (int e = 0; e < E; ++e) o[g][e] = 0.0f;
    }
    // Raw 4 / 8-byte pieces of a cache row; converted only when their turn comes, so that the loads of the
    // next pair of positions stay in flight while this pair is processed (a warp issues in order: the
    // first instruction that needs a pending load stalls everything behind it).
    using Raw = typename std::conditional<E == 4, uint2, uint32_t>::type;
    auto widen = [&](const Raw& raw, float (&dst)[E]) {
        const T* el = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int e = 0; e < E; ++e) dst[e] = Act16<BF16>::to_float(el[e]);
    };
    constexpr int STEP = kAttWarps * 2;           // two positions per warp and iteration: independent reductions overlap
    int p0 = s0 + warp * 2;
    Raw rk0 = {}, rv0 = {}, rk1 = {}, rv1 = {};
    auto fetch = [&](int p, Raw& a, Raw& b, Raw& c, Raw& d) {
        const size_t pa = (size_t)min(p, s1 - 1) * D, pb = (size_t)min(p + 1, s1 - 1) * D;
        a = *reinterpret_cast<const Raw*>(kbase + pa);
        b = *reinterpret_cast<const Raw*>(vbase + pa);
        c = *reinterpret_cast<const Raw*>(kbase + pb);
        d = *reinterpret_cast<const Raw*>(vbase + pb);
    };
    if (p0 < s1) fetch(p0, rk0, rv0, rk1, rv1);
    for (; p0 < s1; p0 += STEP) {
        Raw nk0, nv0, nk1, nv1;
        fetch(p0 + STEP, nk0, nv0, nk1, nv1);       // clamped to the slice: the last iteration re-reads its final row
        const bool two = p0 + 1 < s1;
        float k0[E], k1[E], v0[E], v1[E];
        widen(rk0, k0); widen(rv0, v0); widen(rk1, k1); widen(rv1, v1);
        float sc0[G], sc1[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float a = 0.0f, c = 0.0f;
#pragma unroll
            for (int e = 0; e < E; ++e) { a = fmaf(qv[g][e], k0[e], a); c = fmaf(qv[g][e], k1[e], c); }
            sc0[g] = a; sc1[g] = c;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                sc0[g] += __shfl_xor_sync(0xffffffffu, sc0[g], off);
                sc1[g] += __shfl_xor_sync(0xffffffffu, sc1[g], off);
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float second = two ? sc1[g] : -1.0e30f;
            const float mn = fmaxf(m[g], fmaxf(sc0[g], second));
            const float alpha = __expf(m[g] - mn), p0w = __expf(sc0[g] - mn), p1w = two ? __expf(second - mn) : 0.0f;
            m[g] = mn;
            l[g] = l[g] * alpha + p0w + p1w;
#pragma unroll
            for (int e = 0; e < E; ++e) o[g][e] = fmaf(p1w, v1[e], fmaf(p0w, v0[e], o[g][e] * alpha));
        }
        rk0 = nk0; rv0 = nv0; rk1 = nk1; rv1 = nv1;
    }

    // the CTA's warps meet in shared memory
    __shared__ float sm_m[kAttWarps][G], sm_l[kAttWarps][G];
    __shared__ float sm_o[kAttWarps][G][D];
    __shared__ int is_last;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (lane == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
#pragma unroll
        for (int e = 0; e < E; ++e) sm_o[warp][g][lane * E + e] = o[g][e];
    }
    __syncthreads();
    constexpr int STRIDE = D + 4;                 // floats per (slice, head): m, l, two unused, o[D] (16-byte aligned)
    float* mine = parts + ((((size_t)b * hkv + kvh) * slices + slice) * G) * STRIDE;
    for (int i = tid; i < G * D; i += kAttWarps * 32) {
        const int g = i / D, dd = i - g * D;
        float mm = sm_m[0][g];
#pragma unroll
        for (int w = 1; w < kAttWarps; ++w) mm = fmaxf(mm, sm_m[w][g]);
        float acc = 0.0f, ll = 0.0f;
#pragma unroll
        for (int w = 0; w < kAttWarps; ++w) {
            const float f = __expf(sm_m[w][g] - mm);
            acc = fmaf(sm_o[w][g][dd], f, acc);
            ll = fmaf(sm_l[w][g], f, ll);
        }
        mine[g * STRIDE + 4 + dd] = acc;
        if (dd == 0) { mine[g * STRIDE] = mm; mine[g * STRIDE + 1] = ll; }
    }
    // arrival: the last CTA of this (sequence, kv head) merges the slices; nobody waits
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int old = atomicAdd(counters + b * hkv + kvh, 1);
        is_last = old == slices - 1;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // Every load of the merge is independent of the others and issued before the first use: one
    // trip to L2 per head instead of one per slice.  A warp takes a head; a lane takes 4 output elements.
    const float* all = parts + (((size_t)b * hkv + kvh) * slices) * G * STRIDE;
    T* out = static_cast<T*>(out_) + (size_t)b * ldo + (size_t)kvh * G * D;
    const bool has_o = lane * 4 < D;
    for (int g = warp; g < G; g += kAttWarps) {
        float mv[kAttMaxSlices], lv[kAttMaxSlices];
        float4 ov[kAttMaxSlices];
#pragma unroll
        for (int s = 0; s < kAttMaxSlices; ++s) {
            mv[s] = -1.0e30f; lv[s] = 0.0f; ov[s] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (s < slices) {
                const float* pp = all + ((size_t)s * G + g) * STRIDE;
                const float2 ml = __ldcg(reinterpret_cast<const float2*>(pp));
                mv[s] = ml.x; lv[s] = ml.y;
                if (has_o) ov[s] = __ldcg(reinterpret_cast<const float4*>(pp + 4) + lane);
            }
        }
        float mm = -1.0e30f;
#pragma unroll
        for (int s = 0; s < kAttMaxSlices; ++s) mm = fmaxf(mm, mv[s]);
        float ll = 0.0f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < kAttMaxSlices; ++s) {
            const float f = __expf(mv[s] - mm);
            ll = fmaf(lv[s], f, ll);
            acc.x = fmaf(ov[s].x, f, acc.x); acc.y = fmaf(ov[s].y, f, acc.y);
            acc.z = fmaf(ov[s].z, f, acc.z); acc.w = fmaf(ov[s].w, f, acc.w);
        }
        if (has_o) {
            const float inv = ll > 0.0f ? 1.0f / ll : 0.0f;
            uint2 packed;
            T* pe = reinterpret_cast<T*>(&packed);
            pe[0] = Act16<BF16>::from_float(acc.x * inv); pe[1] = Act16<BF16>::from_float(acc.y * inv);
            pe[2] = Act16<BF16>::from_float(acc.z * inv); pe[3] = Act16<BF16>::from_float(acc.w * inv);
            *reinterpret_cast<uint2*>(out + g * D + lane * 4) = packed;
        }
    }
    if (tid == 0) counters[b * hkv + kvh] = 0;       // ready for the next launch (stream order makes it visible)
}

// ---------------------------------------------------------------------------------------------
// silu(gate) * up
// ---------------------------------------------------------------------------------------------
template <bool BF16>
__global__ void __launch_bounds__(256) silu_mul_kernel(const void* g_, long long ldg, const void* u_, long long ldu, void* y_,
                                                       long long ldy, int width, bool vec) {
    using T = typename Act16<BF16>::T;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int row = blockIdx.y;
    const T* g = static_cast<const T*>(g_) + (size_t)row * ldg;
    const T* u = static_cast<const T*>(u_) + (size_t)row * ldu;
    T* y = static_cast<T*>(y_) + (size_t)row * ldy;
    auto one = [](T gv, T uv) {
        const float gf = Act16<BF16>::to_float(gv);
        return Act16<BF16>::from_float(r16<BF16>(gf / (1.0f + __expf(-gf))) * Act16<BF16>::to_float(uv));
    };
    if (vec) {
        for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < (width >> 3); v += gridDim.x * blockDim.x) {
            const uint4 gv = *reinterpret_cast<const uint4*>(g + v * 8), uv = *reinterpret_cast<const uint4*>(u + v * 8);
            const T* ge = reinterpret_cast<const T*>(&gv);
            const T* ue = reinterpret_cast<const T*>(&uv);
            uint4 ov;
            T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
            for (int q = 0; q < 8; ++q) oe[q] = one(ge[q], ue[q]);
            *reinterpret_cast<uint4*>(y + v * 8) = ov;
        }
    } else {
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < width; i += gridDim.x * blockDim.x) y[i] = one(g[i], u[i]);
    }
}

bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

// Launch with the programmatic-stream-serialisation attribute: the kernels above release their
// successor at entry and wait for their predecessor before they touch memory.
template <typename... KArgs, typename... Args>
int launch_pdl(const char* what, void (*kern)(KArgs...), dim3 grid, dim3 block, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    (void)cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
    return check_launch(what);
}

template <int D, bool BF16>
int launch_attention(int group, dim3 grid, cudaStream_t s, const void* q, long long ldq, const void* kc, const void* vc,
                     const long long* pos, void* out, long long ldo, int hq, int hkv, int max_len, float scale, float* parts,
                     int* counters) {
    const dim3 block(kAttWarps * 32);
#define QDEC_ATT(GG)                                                                                                    \
    case GG: return launch_pdl("attention_kernel", attention_kernel<D, GG, BF16>, grid, block, s, q, ldq, kc, vc, pos, out, ldo, \
                               hq, hkv, max_len, scale, parts, counters)
    switch (group) {
        QDEC_ATT(1); QDEC_ATT(2); QDEC_ATT(3); QDEC_ATT(4); QDEC_ATT(5); QDEC_ATT(6); QDEC_ATT(7); QDEC_ATT(8);
        default: break;
    }
#undef QDEC_ATT
    set_error("qdec_attention: %d query heads per kv head (1..8 supported)", group);
    return QGEMV_ERR_SHAPE;
}

size_t attention_parts_floats(int batch, int q_heads, int kv_heads, int head_dim, int max_len) {
    const int slices = attention_slices(batch, kv_heads, max_len);
    return (size_t)batch * q_heads * slices * (head_dim + 4);
}

}  // namespace
}  // namespace qgemv

using namespace qgemv;

extern "C" int qdec_rmsnorm(void* h, int64_t ldh, const void* delta, int64_t ldd, const void* weight, void* y, int64_t ldy,
                            int rows, int hidden, float eps, int dtype, void* stream) {
    if (!h || !weight || !y || rows < 1 || hidden < 8) { set_error("qdec_rmsnorm: null pointer or non-positive size"); return QGEMV_ERR_BAD_ARG; }
    if (dtype != QGEMV_F16 && dtype != QGEMV_BF16) { set_error("qdec_rmsnorm: dtype must be fp16 or bf16"); return QGEMV_ERR_BAD_ARG; }
    if (hidden % 8 || hidden > kNormThreads * kNormMaxVec * 8) { set_error("qdec_rmsnorm: hidden=%d must be a multiple of 8, at most %d", hidden, kNormThreads * kNormMaxVec * 8); return QGEMV_ERR_SHAPE; }
    if (ldh < hidden || ldy < hidden || (delta && ldd < hidden)) { set_error("qdec_rmsnorm: a leading dimension is smaller than hidden"); return QGEMV_ERR_SHAPE; }
    if (!aligned16(h) || !aligned16(y) || !aligned16(weight) || (delta && !aligned16(delta)) || ldh % 8 || ldy % 8 || (delta && ldd % 8)) {
        set_error("qdec_rmsnorm: rows must be 16-byte aligned");
        return QGEMV_ERR_ALIGN;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == QGEMV_BF16)
        return launch_pdl("rmsnorm_kernel", rmsnorm_kernel<true>, dim3(rows), dim3(kNormThreads), s, h, (long long)ldh, delta, (long long)ldd, weight, y, (long long)ldy, hidden, eps);
    return launch_pdl("rmsnorm_kernel", rmsnorm_kernel<false>, dim3(rows), dim3(kNormThreads), s, h, (long long)ldh, delta, (long long)ldd, weight, y, (long long)ldy, hidden, eps);
}

extern "C" int qdec_rope_append(void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv,
                                const void* cos_table, const void* sin_table, int table_rows, const int64_t* pos,
                                void* kcache, void* vcache, int batch, int q_heads, int kv_heads, int head_dim, int max_len,
                                int32_t* status, int dtype, void* stream) {
    if (!q || !k || !v || !cos_table || !sin_table || !pos || !kcache || !vcache) { set_error("qdec_rope_append: null pointer"); return QGEMV_ERR_BAD_ARG; }
    if (batch < 1 || q_heads < 1 || kv_heads < 1 || max_len < 1 || table_rows < 1) { set_error("qdec_rope_append: non-positive size"); return QGEMV_ERR_BAD_ARG; }
    if (dtype != QGEMV_F16 && dtype != QGEMV_BF16) { set_error("qdec_rope_append: dtype must be fp16 or bf16"); return QGEMV_ERR_BAD_ARG; }
    if (head_dim < 2 || head_dim % 2 || head_dim > 256) { set_error("qdec_rope_append: head_dim=%d must be even, at most 256", head_dim); return QGEMV_ERR_SHAPE; }
    if (ldq < (int64_t)q_heads * head_dim || ldk < (int64_t)kv_heads * head_dim || ldv < (int64_t)kv_heads * head_dim) { set_error("qdec_rope_append: a leading dimension is smaller than its row"); return QGEMV_ERR_SHAPE; }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const dim3 grid(q_heads + 2 * kv_heads, batch), block(128);
    const long long* p = reinterpret_cast<const long long*>(pos);
    if (dtype == QGEMV_BF16)
        return launch_pdl("rope_append_kernel", rope_append_kernel<true>, grid, block, s, q, (long long)ldq, k, (long long)ldk, v, (long long)ldv,
                          cos_table, sin_table, table_rows, p, kcache, vcache, q_heads, kv_heads, head_dim, max_len, status);
    return launch_pdl("rope_append_kernel", rope_append_kernel<false>, grid, block, s, q, (long long)ldq, k, (long long)ldk, v, (long long)ldv,
                      cos_table, sin_table, table_rows, p, kcache, vcache, q_heads, kv_heads, head_dim, max_len, status);
}

extern "C" size_t qdec_attention_workspace_bytes(int batch, int q_heads, int kv_heads, int head_dim, int max_len) {
    if (batch < 1 || q_heads < 1 || kv_heads < 1 || head_dim < 1 || max_len < 1) return 0;
    const size_t parts = attention_parts_floats(batch, q_heads, kv_heads, head_dim, max_len) * sizeof(float);
    const size_t counters = ((size_t)batch * kv_heads * sizeof(int) + 255) / 256 * 256;
    return counters + (parts + 255) / 256 * 256;
}

extern "C" int qdec_attention(const void* q, int64_t ldq, const void* kcache, const void* vcache, const int64_t* pos,
                              void* out, int64_t ldo, int batch, int q_heads, int kv_heads, int head_dim, int max_len,
                              float scale, void* workspace, size_t workspace_bytes, int dtype, void* stream) {
    if (!q || !kcache || !vcache || !pos || !out || !workspace) { set_error("qdec_attention: null pointer"); return QGEMV_ERR_BAD_ARG; }
    if (batch < 1 || q_heads < 1 || kv_heads < 1 || max_len < 1) { set_error("qdec_attention: non-positive size"); return QGEMV_ERR_BAD_ARG; }
    if (dtype != QGEMV_F16 && dtype != QGEMV_BF16) { set_error("qdec_attention: dtype must be fp16 or bf16"); return QGEMV_ERR_BAD_ARG; }
    if (head_dim != 64 && head_dim != 128) { set_error("qdec_attention: head_dim=%d (64 and 128 are built)", head_dim); return QGEMV_ERR_SHAPE; }
    if (q_heads % kv_heads || q_heads / kv_heads > 8) { set_error("qdec_attention: %d query heads over %d kv heads (a group of 1..8 is built)", q_heads, kv_heads); return QGEMV_ERR_SHAPE; }
    if (ldq < (int64_t)q_heads * head_dim || ldo < (int64_t)q_heads * head_dim) { set_error("qdec_attention: a leading dimension is smaller than its row"); return QGEMV_ERR_SHAPE; }
    if (batch > 65535 || kv_heads > 65535) { set_error("qdec_attention: batch and kv_heads are grid dimensions (at most 65535)"); return QGEMV_ERR_TOO_LARGE; }
    const size_t need = qdec_attention_workspace_bytes(batch, q_heads, kv_heads, head_dim, max_len);
    if (workspace_bytes < need) { set_error("qdec_attention: workspace of %zu bytes required (got %zu)", need, workspace_bytes); return QGEMV_ERR_WORKSPACE; }
    if (reinterpret_cast<uintptr_t>(workspace) % 256 || reinterpret_cast<uintptr_t>(q) % 8 || reinterpret_cast<uintptr_t>(kcache) % 8 ||
        reinterpret_cast<uintptr_t>(vcache) % 8 || (ldq * 2) % 8 || reinterpret_cast<uintptr_t>(out) % 8 || (ldo * 2) % 8) {
        set_error("qdec_attention: workspace must be 256-byte aligned, q, out and the caches 8-byte aligned");
        return QGEMV_ERR_ALIGN;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int* counters = static_cast<int*>(workspace);
    float* parts = reinterpret_cast<float*>(static_cast<char*>(workspace) + ((size_t)batch * kv_heads * sizeof(int) + 255) / 256 * 256);
    const dim3 grid(attention_slices(batch, kv_heads, max_len), kv_heads, batch);
    const int group = q_heads / kv_heads;
    const long long* p = reinterpret_cast<const long long*>(pos);
    const bool bf16 = dtype == QGEMV_BF16;
    if (head_dim == 64)
        return bf16 ? launch_attention<64, true>(group, grid, s, q, ldq, kcache, vcache, p, out, ldo, q_heads, kv_heads, max_len, scale, parts, counters)
                    : launch_attention<64, false>(group, grid, s, q, ldq, kcache, vcache, p, out, ldo, q_heads, kv_heads, max_len, scale, parts, counters);
    return bf16 ? launch_attention<128, true>(group, grid, s, q, ldq, kcache, vcache, p, out, ldo, q_heads, kv_heads, max_len, scale, parts, counters)
                : launch_attention<128, false>(group, grid, s, q, ldq, kcache, vcache, p, out, ldo, q_heads, kv_heads, max_len, scale, parts, counters);
}

extern "C" int qdec_silu_mul(const void* gate, int64_t ldg, const void* up, int64_t ldu, void* y, int64_t ldy,
                             int rows, int width, int dtype, void* stream) {
    if (!gate || !up || !y || rows < 1 || width < 1) { set_error("qdec_silu_mul: null pointer or non-positive size"); return QGEMV_ERR_BAD_ARG; }
    if (dtype != QGEMV_F16 && dtype != QGEMV_BF16) { set_error("qdec_silu_mul: dtype must be fp16 or bf16"); return QGEMV_ERR_BAD_ARG; }
    if (ldg < width || ldu < width || ldy < width) { set_error("qdec_silu_mul: a leading dimension is smaller than width"); return QGEMV_ERR_SHAPE; }
    if (rows > 65535) { set_error("qdec_silu_mul: at most 65535 rows"); return QGEMV_ERR_TOO_LARGE; }
    const bool vec = width % 8 == 0 && aligned16(gate) && aligned16(up) && aligned16(y) && ldg % 8 == 0 && ldu % 8 == 0 && ldy % 8 == 0;
    const int units = vec ? width / 8 : width;
    int blocks = (units + 255) / 256;
    blocks = blocks < 1 ? 1 : blocks > 148 * 4 ? 148 * 4 : blocks;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const dim3 grid(blocks, rows), block(256);
    if (dtype == QGEMV_BF16)
        return launch_pdl("silu_mul_kernel", silu_mul_kernel<true>, grid, block, s, gate, (long long)ldg, up, (long long)ldu, y, (long long)ldy, width, vec);
    return launch_pdl("silu_mul_kernel", silu_mul_kernel<false>, grid, block, s, gate, (long long)ldg, up, (long long)ldu, y, (long long)ldy, width, vec);
}
