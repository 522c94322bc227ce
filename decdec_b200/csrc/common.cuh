// Shared device/host definitions for the DecDEC decode hot path on sm_100a.
//
// Output protocol used by every kernel in this library: partial results are added with fp32
// reductions into a zero-initialised accumulator `acc[N]`; each CTA then "arrives" on the tickets of
// the output tiles it touched, and the CTA that arrives last on a tile adds the accumulator to the
// caller's output in one rounding step, and clears accumulator and ticket for the next launch.
// No CTA ever waits for another one, so no co-residency is required.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace dd {

enum : int { FP32 = 0, FP16 = 1, BF16 = 2 };

constexpr int kThreads = 256;          // every kernel here runs 256-thread CTAs
constexpr int kChunk = 1024;           // selection chunk (reference: macros.h:8)
constexpr int kBuckets = 32;           // reference: macros.h:18

template <int DT> struct Tr;
template <> struct Tr<FP32> {
    using T = float;
    static __device__ __forceinline__ float to_f(float v) { return v; }
    static __device__ __forceinline__ float from_f(float v) { return v; }
    static __device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
    static __device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
};
template <> struct Tr<FP16> {
    using T = __half;
    static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
    static __device__ __forceinline__ __half add(__half a, __half b) { return __hadd(a, b); }
    static __device__ __forceinline__ __half sub(__half a, __half b) { return __hsub(a, b); }
};
template <> struct Tr<BF16> {
    using T = __nv_bfloat16;
    static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
    static __device__ __forceinline__ __nv_bfloat16 add(__nv_bfloat16 a, __nv_bfloat16 b) { return __hadd(a, b); }
    static __device__ __forceinline__ __nv_bfloat16 sub(__nv_bfloat16 a, __nv_bfloat16 b) { return __hsub(a, b); }
};

// Output tiling and the accumulate/finalize state shared by the roles of one launch.
struct FinParams {
    float* acc;            // [>= N] fp32, all zero between launches
    unsigned* tickets;     // [>= n_tiles], all zero between launches
    unsigned* err;         // device error word of the workspace (0 = fine)
    float* acc2;           // [>= N] fp32 accumulator of the UNSCALED compensation sums (null: no compensation role)
    const void* scales;    // [N] reordered residual scales, applied when a tile is finalized (layout [nibble][N/8])
    void* y;               // caller's output [N], accumulated into
    uint32_t N;
    uint32_t tile_units;   // outputs per tile = 32 * tile_units
    uint32_t n_tiles;
    uint32_t expected;     // arrivals per tile before it is finalized
};

// Arguments of the compensation (DEC) role.
struct DecParams {
    const uint32_t* cheat;     // [K, N/8] packed 4-bit residual, usually mapped pinned host memory
    const void* scales;        // [N] reordered scales (device copy), layout [nibble][N/8]
    const void* x;             // [K] activations
    int* sel_rows;             // context buffer, >= k entries
    void* sel_acts;            // context buffer, >= k entries
    float thr_a, thr_b;        // thresholds[0], thresholds[k-1] (exact values of the activation dtype)
    uint32_t K, N;
    uint32_t k_chunk;
    uint32_t k_total;          // k_chunk * K / 1024
    uint32_t n_rowparts;       // CTAs along the selected-row dimension
    uint32_t n_colparts;       // CTAs along the output dimension
    uint32_t n_cta;            // n_rowparts * n_colparts (0 = role absent)
    uint32_t fused_select;     // 1: select rows from x; 0: rows are given in sel_rows
};

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_stream(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may
// start while the previous kernel of the stream is still draining.  `pdl_trigger` lets the NEXT
// kernel's CTAs be scheduled early; `pdl_wait` blocks until the PREVIOUS kernel has completed and its
// writes are visible - it must precede every access to data a previous kernel may have written
// (activations, outputs, accumulator, tickets, selection buffers).  Both are no-ops for plain launches.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// The error word of a workspace lives in mapped host memory (the host reads it before every call without a copy):
// a plain store plus a system-scope fence, never an atomic.
__device__ __forceinline__ void raise_error(unsigned* err, unsigned code) {
    *reinterpret_cast<volatile unsigned*>(err) = code;
    __threadfence_system();
}

// explicit shared-window load (the table lookups must not degrade to generic loads)
__device__ __forceinline__ float lds_f32(uint32_t saddr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(saddr));
    return v;
}

// Packed accumulator word (launches without tickets): bits 0..7 arrivals, 8..15 arrivals whose partial sum was not
// finite, 16..63 the sum as signed fixed point with 20 fractional bits (finite partial sums are clamped to +-2^22).
__device__ __forceinline__ unsigned long long pack_partial(float v) {
    const bool finite = fabsf(v) <= 3.0e38f;      // false for inf and NaN
    const float c = fminf(fmaxf(finite ? v : 0.0f, -4194304.0f), 4194304.0f);
    const long long q = __float2ll_rn(c * 1048576.0f);
    return ((unsigned long long)q << 16) + (finite ? 1ull : 0x101ull);
}

// The atomic of output n returned `old` when `mine` was added: if that was the last of `expected` arrivals, the
// complete sum goes into y (y0 = the output's value read earlier) and the word is cleared for the next launch.
template <int DT>
__device__ __forceinline__ void finish_packed(unsigned long long old, unsigned long long mine, unsigned expected,
                                              unsigned long long* word, typename Tr<DT>::T* yp, float y0) {
    const unsigned long long now = old + mine;
    if ((unsigned)(now & 0xffull) != expected) return;
    const float sum = __ll2float_rn((long long)now >> 16) * (1.0f / 1048576.0f);
    const float out = ((now >> 8) & 0xffull) ? __int_as_float(0x7fc00000) : y0 + sum;
    *yp = Tr<DT>::from_f(out);
    __stcg(word, 0ull);
}

// Fold accumulator entries [n0, n1) into y (single rounding) and re-zero them.  n0 is a multiple of 32.
// Four outputs per thread with all loads issued before the first use: the finalizing CTA sits at the
// very end of a launch, so its dependent-load round trips are not hidden by anything.
template <int DT>
__device__ __forceinline__ void finalize_span(const FinParams& f, uint32_t n0, uint32_t n1, uint32_t nthreads) {
    using T = typename Tr<DT>::T;
    T* y = reinterpret_cast<T*>(f.y);
    const T* sc = reinterpret_cast<const T*>(f.scales);
    const uint32_t wpr = f.N / 8;
    const bool vec = ((f.N & 3u) == 0u) && ((reinterpret_cast<uintptr_t>(f.y) & (4u * sizeof(T) - 1u)) == 0u);
    if (vec) {
        constexpr int U = 2;      // groups of four outputs per thread and pass, loads of all groups issued first
        for (uint32_t nb = n0 + 4u * threadIdx.x; nb < n1; nb += 4u * nthreads * U) {
            float4 v[U], r[U];
            float s4[U][4];
            float yo[U][4];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint32_t n = nb + 4u * nthreads * u;
                r[u] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int i = 0; i < 4; ++i) s4[u][i] = 0.f;
                if (n >= n1) continue;
                v[u] = __ldcg(reinterpret_cast<const float4*>(f.acc + n));
                if (f.acc2) {
                    // compensation sums are kept unscaled so that the scale loads sit here, beside the
                    // accumulator loads, and not on the critical path of the fetch
                    r[u] = __ldcg(reinterpret_cast<const float4*>(f.acc2 + n));
                    const uint32_t w = n >> 3, nib = n & 7u;   // nib is 0 or 4
#pragma unroll
                    for (int i = 0; i < 4; ++i) s4[u][i] = Tr<DT>::to_f(sc[(size_t)(nib + i) * wpr + w]);
                }
                if constexpr (DT == FP32) {
                    const float4 yy = *reinterpret_cast<const float4*>(y + n);
                    yo[u][0] = yy.x; yo[u][1] = yy.y; yo[u][2] = yy.z; yo[u][3] = yy.w;
                } else {
                    const uint2 raw = *reinterpret_cast<const uint2*>(y + n);
                    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
                    for (int i = 0; i < 4; ++i) yo[u][i] = Tr<DT>::to_f(e[i]);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint32_t n = nb + 4u * nthreads * u;
                if (n >= n1) continue;
                __stcg(reinterpret_cast<float4*>(f.acc + n), make_float4(0.f, 0.f, 0.f, 0.f));
                if (f.acc2) __stcg(reinterpret_cast<float4*>(f.acc2 + n), make_float4(0.f, 0.f, 0.f, 0.f));
                yo[u][0] += fmaf(r[u].x, s4[u][0], v[u].x);
                yo[u][1] += fmaf(r[u].y, s4[u][1], v[u].y);
                yo[u][2] += fmaf(r[u].z, s4[u][2], v[u].z);
                yo[u][3] += fmaf(r[u].w, s4[u][3], v[u].w);
                if constexpr (DT == FP32) {
                    *reinterpret_cast<float4*>(y + n) = make_float4(yo[u][0], yo[u][1], yo[u][2], yo[u][3]);
                } else {
                    uint2 raw;
                    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
                    for (int i = 0; i < 4; ++i) e[i] = Tr<DT>::from_f(yo[u][i]);
                    *reinterpret_cast<uint2*>(y + n) = raw;
                }
            }
        }
    } else {
        for (uint32_t n = n0 + threadIdx.x; n < n1; n += nthreads) {
            float v = __ldcg(&f.acc[n]);
            __stcg(&f.acc[n], 0.0f);
            if (f.acc2) {
                const float r = __ldcg(&f.acc2[n]);
                __stcg(&f.acc2[n], 0.0f);
                v = fmaf(r, Tr<DT>::to_f(sc[(size_t)(n & 7u) * wpr + (n >> 3)]), v);
            }
            y[n] = Tr<DT>::from_f(Tr<DT>::to_f(y[n]) + v);
        }
    }
}

// Arrive on tiles [t0, t1); the last arriver of a tile folds the accumulator into y.
// Must be called by all threads of the CTA, after all its reductions into the accumulators were issued.
// `nthreads` = number of threads of the CTA that take part (threads beyond it must have exited; the
// first warp always takes part).  The tickets of up to 32 tiles are taken by one warp in parallel, so a
// CTA that covers many tiles pays one atomic round trip, not one per tile.
template <int DT>
__device__ __forceinline__ void arrive_and_finalize(const FinParams& f, uint32_t t0, uint32_t t1, unsigned* s_flag,
                                                    uint32_t nthreads = kThreads) {
    __threadfence();
    __syncthreads();
    for (uint32_t tb = t0; tb < t1; tb += 32u) {
        if (threadIdx.x < 32u) {
            const uint32_t t = tb + threadIdx.x;
            bool last = false;
            if (t < t1) last = (atomicAdd(&f.tickets[t], 1u) + 1u == f.expected);
            const unsigned m = __ballot_sync(0xffffffffu, last);
            if (threadIdx.x == 0) *s_flag = m;
        }
        __syncthreads();
        unsigned m = *s_flag;
        if (m) {
            __threadfence();
            while (m) {
                // a run of consecutive finished tiles is folded as one span, so all threads have work
                const uint32_t b0 = (uint32_t)(__ffs(m) - 1);
                const unsigned rest = ~(m >> b0);
                const uint32_t run = rest ? (uint32_t)(__ffs(rest) - 1) : 32u - b0;
                m = (b0 + run >= 32u) ? 0u : (m & (0xffffffffu << (b0 + run)));
                const uint32_t t = tb + b0;
                const uint32_t n0 = t * f.tile_units * 32u;
                const uint32_t n1 = min(f.N, n0 + run * f.tile_units * 32u);
                finalize_span<DT>(f, n0, n1, nthreads);
                if (threadIdx.x < run) f.tickets[t + threadIdx.x] = 0u;
            }
        }
        __syncthreads();
    }
}

}  // namespace dd
