// Compensation (DEC) role: bucket-threshold channel selection, zero-copy fetch of the selected
// 4-bit residual rows, residual GEMV, fp32 reduction into the shared accumulator.
//
// Replaces `fused_dec_kernel` / `dec_kernel` of the reference (decdec_extension/dec.cu:26-280,
// :284-426).  Differences in structure, not in result:
//  * a CTA is (row part, column part).  In fused-select mode a row part is a set of 1024-channel
//    chunks and every CTA of that row part repeats the (cheap) selection of its chunks, so no grid
//    barrier and no cooperative launch is needed;
//  * inside a bucket rows are ranked by ascending channel index with warp ballots (the reference
//    ranks by atomic arrival order, dec.cu:146-154), so the selection is reproducible;
//  * residual rows are fetched with 16-byte streaming loads, eight rows in flight per thread;
//  * the dot products are accumulated in fp32 and scaled once per output.
#pragma once
#include "common.cuh"

namespace dd {

// Dynamic shared memory carve-up of the DEC role (bytes).
struct DecSmem {
    static constexpr int kXf = 0;                         // float  xf[1024]     signed activations of the chunk
    static constexpr int kBall = kXf + 4096;              // u32    ball[32][32] ballots  [virtual warp][bucket]
    static constexpr int kPre = kBall + 4096;             // u32    pre[32][32]  exclusive counts before a virtual warp
    static constexpr int kFloor = kPre + 4096;            // float  floors[32], ceils[32]
    static constexpr int kOff = kFloor + 256;             // u32    off[32] + filled
    static constexpr int kRow = kOff + 256;               // int    srow[1024]
    static constexpr int kAct = kRow + 4096;              // float  sact[1024]
    static constexpr int kRed = kAct + 4096;              // float  red[4096]
    static constexpr int kFlag = kRed + 16384;            // u32 flag
    static constexpr int kBytes = kFlag + 16;
};

// Bucket lower bounds in the activation dtype, bit-for-bit the reference recipe (dec.cu:117-130):
// L < 16: a + DT(float(DT(b - a)) * L / 15);  L >= 16: DT(float(b) * (31 - L) / 16).
template <int DT>
__device__ __forceinline__ float bucket_floor(float a_f, float b_f, int L) {
    using T = typename Tr<DT>::T;
    const T a = Tr<DT>::from_f(a_f), b = Tr<DT>::from_f(b_f);
    if (L < 16) {
        const float d = Tr<DT>::to_f(Tr<DT>::sub(b, a));
        const float t = __fdiv_rn(__fmul_rn(d, (float)L), 15.0f);
        return Tr<DT>::to_f(Tr<DT>::add(a, Tr<DT>::from_f(t)));
    }
    const float t = __fdiv_rn(__fmul_rn(b_f, (float)(31 - L)), 16.0f);
    return Tr<DT>::to_f(Tr<DT>::from_f(t));
}

// Select kq rows of chunk `c` into srow/sact (shared).  Returns nothing; all threads participate.
template <int DT>
__device__ void dec_select_chunk(const DecParams& p, uint32_t c, uint32_t kq, bool publish, unsigned char* sm) {
    using T = typename Tr<DT>::T;
    float* xf = reinterpret_cast<float*>(sm + DecSmem::kXf);
    uint32_t* ball = reinterpret_cast<uint32_t*>(sm + DecSmem::kBall);
    uint32_t* pre = reinterpret_cast<uint32_t*>(sm + DecSmem::kPre);
    float* floors = reinterpret_cast<float*>(sm + DecSmem::kFloor);
    uint32_t* off = reinterpret_cast<uint32_t*>(sm + DecSmem::kOff);
    int* srow = reinterpret_cast<int*>(sm + DecSmem::kRow);
    float* sact = reinterpret_cast<float*>(sm + DecSmem::kAct);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t s = c * kChunk;
    const uint32_t len = min((uint32_t)kChunk, p.K - s);
    const T* x = reinterpret_cast<const T*>(p.x);

    if (tid < kBuckets) {
        floors[tid] = bucket_floor<DT>(p.thr_a, p.thr_b, tid);
    }
    float xv[4];
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const uint32_t e = it * kThreads + tid;
        xv[it] = (e < len) ? Tr<DT>::to_f(x[s + e]) : __int_as_float(0x7fc00000);  // NaN = member of no bucket
        xf[e] = xv[it];
    }
    __syncthreads();
    if (tid < kBuckets) floors[32 + tid] = (tid == 0) ? __int_as_float(0x7f800000) : floors[tid - 1];
    __syncthreads();

    // membership masks (normally one bit; the exact per-bucket test of dec.cu:145 is kept so that
    // degenerate thresholds behave like the reference)
    uint32_t mem[4];
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const float ax = fabsf(xv[it]);
        uint32_t m = 0;
#pragma unroll 8
        for (int L = 0; L < kBuckets; ++L) {
            const bool in = (ax >= floors[L]) && (ax < floors[32 + L]);
            m |= (in ? 1u : 0u) << L;
        }
        mem[it] = m;
    }
    // ballots: virtual warp vw = it*8 + warp holds elements 32*vw .. 32*vw+31
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int vw = it * 8 + warp;
        uint32_t mine = 0;
#pragma unroll
        for (int L = 0; L < kBuckets; ++L) {
            const uint32_t b = __ballot_sync(0xffffffffu, (mem[it] >> L) & 1u);
            if (lane == L) mine = b;
        }
        ball[vw * 32 + lane] = mine;
    }
    __syncthreads();
    if (warp == 0) {
        // lane = bucket: exclusive prefix over virtual warps, then exclusive scan over buckets
        uint32_t run = 0;
        for (int vw = 0; vw < 32; ++vw) {
            pre[vw * 32 + lane] = run;
            run += __popc(ball[vw * 32 + lane]);
        }
        uint32_t inc = run;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t o = __shfl_up_sync(0xffffffffu, inc, d);
            if (lane >= d) inc += o;
        }
        off[lane] = inc - run;
        if (lane == 31) off[32] = min(inc, kq);  // number of slots that get a real row
    }
    __syncthreads();
    const uint32_t lt = (1u << lane) - 1u;
    int* g_rows = p.sel_rows + (size_t)c * p.k_chunk;
    T* g_acts = reinterpret_cast<T*>(p.sel_acts) + (size_t)c * p.k_chunk;
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int vw = it * 8 + warp;
        uint32_t m = mem[it];
        while (m) {
            const int L = __ffs(m) - 1;
            m &= m - 1;
            const uint32_t r = off[L] + pre[vw * 32 + L] + __popc(ball[vw * 32 + L] & lt);
            if (r < kq) {
                const int row = (int)(s + it * kThreads + tid);
                srow[r] = row;
                sact[r] = xv[it];
                if (publish) { g_rows[r] = row; g_acts[r] = Tr<DT>::from_f(xv[it]); }
            }
        }
    }
    // fewer than kq finite members (NaN/inf activations): pad with a harmless (row, 0) pair.
    // The reference aborts with a device assert here (dec.cu:178).
    const uint32_t filled = off[32];
    for (uint32_t r = filled + tid; r < kq; r += kThreads) {
        srow[r] = (int)s;
        sact[r] = 0.0f;
        if (publish) { g_rows[r] = (int)s; g_acts[r] = Tr<DT>::from_f(0.0f); }
    }
    __syncthreads();
}

__device__ __forceinline__ void dec_decode_word(uint32_t w, float a, float* acc) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        // 0x4B000000 | nib is the float 2^23 + nib; subtracting 2^23 + 8 leaves nib - 8 exactly
        const float f = __uint_as_float(0x4B000000u | ((w >> (4 * i)) & 0xFu)) - 8388616.0f;
        acc[i] = fmaf(f, a, acc[i]);
    }
}

// Fetch rows srow[0..nrows) x packed columns [w0, w1) and add scale * sum into acc_g.
// VW = words per load (4: 16-byte loads, needs N % 32 == 0; 1: scalar fallback).
template <int DT, int VW>
__device__ void dec_fetch(const DecParams& p, float* acc_g, uint32_t nrows, uint32_t w0, uint32_t w1, unsigned char* sm) {
    using T = typename Tr<DT>::T;
    const int* srow = reinterpret_cast<const int*>(sm + DecSmem::kRow);
    const float* sact = reinterpret_cast<const float*>(sm + DecSmem::kAct);
    float* red = reinterpret_cast<float*>(sm + DecSmem::kRed);
    const T* scales = reinterpret_cast<const T*>(p.scales);
    const uint32_t wpr = p.N / 8;  // words per residual row
    const int tid = threadIdx.x;
    constexpr uint32_t kBlockWords = 128 * VW;  // at most 128 loads wide, so at least 2 row groups
    constexpr int UN = 8;                       // rows in flight per thread

    for (uint32_t cb = w0; cb < w1; cb += kBlockWords) {
        const uint32_t nw = min(kBlockWords, w1 - cb);
        const uint32_t tv = (nw + VW - 1) / VW;
        const uint32_t R = kThreads / tv;
        for (uint32_t o = tid; o < nw * 8; o += kThreads) red[o] = 0.0f;
        __syncthreads();
        const uint32_t v = tid % tv, rg = tid / tv;
        if (rg < R) {
            float a[VW * 8];
#pragma unroll
            for (int i = 0; i < VW * 8; ++i) a[i] = 0.0f;
            const uint32_t col = cb + v * VW;
            for (uint32_t i0 = rg; i0 < nrows; i0 += R * UN) {
                if constexpr (VW == 4) {
                    uint4 q[UN];
                    float xa[UN];
#pragma unroll
                    for (int b = 0; b < UN; ++b) {
                        const uint32_t i = i0 + b * R;
                        if (i < nrows) {
                            q[b] = ldg_stream(reinterpret_cast<const uint4*>(p.cheat + (size_t)srow[i] * wpr + col));
                            xa[b] = sact[i];
                        } else {
                            q[b] = make_uint4(0, 0, 0, 0);
                            xa[b] = 0.0f;
                        }
                    }
#pragma unroll
                    for (int b = 0; b < UN; ++b) {
                        dec_decode_word(q[b].x, xa[b], a + 0);
                        dec_decode_word(q[b].y, xa[b], a + 8);
                        dec_decode_word(q[b].z, xa[b], a + 16);
                        dec_decode_word(q[b].w, xa[b], a + 24);
                    }
                } else {
                    uint32_t q[UN];
                    float xa[UN];
#pragma unroll
                    for (int b = 0; b < UN; ++b) {
                        const uint32_t i = i0 + b * R;
                        if (i < nrows) {
                            q[b] = ldg_stream(p.cheat + (size_t)srow[i] * wpr + col);
                            xa[b] = sact[i];
                        } else {
                            q[b] = 0;
                            xa[b] = 0.0f;
                        }
                    }
#pragma unroll
                    for (int b = 0; b < UN; ++b) dec_decode_word(q[b], xa[b], a);
                }
            }
#pragma unroll
            for (int i = 0; i < VW * 8; ++i) atomicAdd(&red[v * VW * 8 + i], a[i]);
        }
        __syncthreads();
        for (uint32_t o = tid; o < nw * 8; o += kThreads) {
            const uint32_t n = cb * 8 + o;
            const float sc = Tr<DT>::to_f(scales[(size_t)(n & 7u) * wpr + (n >> 3)]);
            atomicAdd(&acc_g[n], red[o] * sc);
        }
        __syncthreads();
    }
}

// One DEC CTA.  `cta` in [0, p.n_cta).
template <int DT>
__device__ void dec_role(const DecParams& p, const FinParams& f, uint32_t cta, unsigned char* sm) {
    using T = typename Tr<DT>::T;
    const uint32_t rp = cta % p.n_rowparts;
    const uint32_t cp = cta / p.n_rowparts;
    // column part = a contiguous range of output tiles
    const uint32_t t0 = (uint32_t)(((uint64_t)cp * f.n_tiles) / p.n_colparts);
    const uint32_t t1 = (uint32_t)(((uint64_t)(cp + 1) * f.n_tiles) / p.n_colparts);
    const uint32_t wpr = p.N / 8;
    const uint32_t w0 = min(wpr, t0 * f.tile_units * 4u);
    const uint32_t w1 = min(wpr, t1 * f.tile_units * 4u);
    const bool vec = (p.N % 32u) == 0u;
    int* srow = reinterpret_cast<int*>(sm + DecSmem::kRow);
    float* sact = reinterpret_cast<float*>(sm + DecSmem::kAct);

    if (p.fused_select) {
        const uint32_t num_chunks = (p.K + kChunk - 1) / kChunk;
        for (uint32_t c = rp; c < num_chunks; c += p.n_rowparts) {
            const uint32_t len = min((uint32_t)kChunk, p.K - c * kChunk);
            const uint32_t kq = p.k_chunk * len / kChunk;
            if (kq == 0) continue;
            dec_select_chunk<DT>(p, c, kq, cp == 0, sm);
            if (w1 > w0) {
                if (vec) dec_fetch<DT, 4>(p, f.acc, kq, w0, w1, sm);
                else dec_fetch<DT, 1>(p, f.acc, kq, w0, w1, sm);
            }
        }
    } else {
        // rows supplied by the caller (context buffer); activation gathered as x[row] (dec.cu:346)
        const T* x = reinterpret_cast<const T*>(p.x);
        const uint32_t r0 = (uint32_t)(((uint64_t)rp * p.k_total) / p.n_rowparts);
        const uint32_t r1 = (uint32_t)(((uint64_t)(rp + 1) * p.k_total) / p.n_rowparts);
        for (uint32_t b0 = r0; b0 < r1; b0 += kChunk) {
            const uint32_t nb = min((uint32_t)kChunk, r1 - b0);
            for (uint32_t i = threadIdx.x; i < nb; i += kThreads) {
                const int row = p.sel_rows[b0 + i];
                const bool ok = row >= 0 && (uint32_t)row < p.K;   // out-of-range rows contribute nothing
                srow[i] = ok ? row : 0;
                sact[i] = ok ? Tr<DT>::to_f(x[row]) : 0.0f;
            }
            __syncthreads();
            if (w1 > w0) {
                if (vec) dec_fetch<DT, 4>(p, f.acc, nb, w0, w1, sm);
                else dec_fetch<DT, 1>(p, f.acc, nb, w0, w1, sm);
            }
        }
    }
    arrive_and_finalize<DT>(f, t0, t1, reinterpret_cast<unsigned*>(sm + DecSmem::kFlag));
}

}  // namespace dd
