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

// explicit shared-window load (the table lookups must not degrade to generic loads)
__device__ __forceinline__ float lds_f32(uint32_t saddr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(saddr));
    return v;
}

// Arrive on tiles [t0, t1); the last arriver of a tile folds the accumulator into y.
// Must be called by all threads of the CTA, after all its reductions into `acc` were issued.
// `nthreads` = number of threads of the CTA that take part (threads beyond it must have exited).
template <int DT>
__device__ __forceinline__ void arrive_and_finalize(const FinParams& f, uint32_t t0, uint32_t t1, unsigned* s_flag,
                                                    uint32_t nthreads = kThreads) {
    using T = typename Tr<DT>::T;
    __threadfence();
    __syncthreads();
    for (uint32_t t = t0; t < t1; ++t) {
        if (threadIdx.x == 0) {
            unsigned old = atomicAdd(&f.tickets[t], 1u);
            *s_flag = (old + 1u == f.expected) ? 1u : 0u;
        }
        __syncthreads();
        if (*s_flag) {
            __threadfence();
            const uint32_t n0 = t * f.tile_units * 32u;
            const uint32_t n1 = min(f.N, n0 + f.tile_units * 32u);
            T* y = reinterpret_cast<T*>(f.y);
            for (uint32_t n = n0 + threadIdx.x; n < n1; n += nthreads) {
                float v = __ldcg(&f.acc[n]);
                __stcg(&f.acc[n], 0.0f);
                y[n] = Tr<DT>::from_f(Tr<DT>::to_f(y[n]) + v);
            }
            if (threadIdx.x == 0) f.tickets[t] = 0u;
        }
        __syncthreads();
    }
}

}  // namespace dd
