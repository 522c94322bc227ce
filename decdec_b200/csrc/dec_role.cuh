// Compensation (DEC) role: bucket-threshold channel selection, zero-copy fetch of the selected
// 4-bit residual rows, residual GEMV, fp32 reduction into the shared accumulator.
//
// Replaces `fused_dec_kernel` / `dec_kernel` of the reference (decdec_extension/dec.cu:26-280,
// :284-426).  Differences in structure, not in result:
//  * a CTA is (row part, column part).  In fused-select mode a row part is a set of 1024-channel
//    chunks and every CTA of that row part repeats the (cheap) selection of its chunks, so no grid
//    barrier and no cooperative launch is needed;
//  * the bucket that overflows the quota gives its lowest channel indices (the reference takes
//    whichever rows arrive first at a shared-memory atomic, dec.cu:146-154), and the published order
//    is reproducible; ranks come from warp ballots and bit-matrix transposes, not atomics;
//  * residual rows are fetched with 16-byte streaming loads, up to eight rows in flight per thread, in
//    one of two forms chosen by the width of the CTA's column range: `dec_fetch_direct` (all threads of
//    the CTA, sums added with 16-byte vector reductions, no barrier) and `dec_fetch` (256 threads, row
//    groups combined through shared memory);
//  * the dot products are accumulated in fp32 and go UNSCALED into their own accumulator; the output
//    scale is applied once per output by the CTA that finalizes the tile (common.cuh).
#pragma once
#include "common.cuh"

namespace dd {


// Barrier of the first kThreads threads of the CTA (selection and the grouped fetch run on those; a launch
// shared with a wider GEMV role has more threads, which only join the CTA-wide phases).
__device__ __forceinline__ void dec_bar() { asm volatile("bar.sync 2, %0;" :: "n"(kThreads) : "memory"); }

// Dynamic shared memory carve-up of the DEC role (bytes).
struct DecSmem {
    static constexpr int kXf = 0;                         // float  xf[1024]     signed activations of the chunk
    static constexpr int kBall = kXf + 4096;              // u32    ball[32][32] ballots  [virtual warp][bucket]
    static constexpr int kPre = kBall + 4096;             // u32    pre[32][32]  exclusive counts before a virtual warp
    static constexpr int kFloor = kPre + 4096;            // float  floors[32], ceils[32]
    static constexpr int kOff = kFloor + 256;             // u32    off[32], filled, totals[32] at +40
    static constexpr int kRow = kOff + 512;               // int    srow[1024]
    static constexpr int kAct = kRow + 4096;              // float  sact[1024]
    static constexpr int kRed = kAct + 4096;              // float  red[32][257] per-thread partials, [value][thread]
    static constexpr int kFlag = kRed + 32 * 257 * 4;     // u32 flag
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

// Select kq rows of chunk `c` into srow/sact (shared); the first kThreads threads participate.
//
// Rule (same set as the reference, dec.cu:117-177, made reproducible):
//   bucket(e)  = the lowest L with floor[L] <= |x_e|   (NaN and inf belong to no bucket);
//   buckets are drained in order 0,1,2,... until kq channels are taken; the bucket that overflows
//   the quota gives its lowest channel indices.
// Output order: channels of the fully taken buckets by ascending index, then the picks of the
// boundary bucket by ascending index.  (The reference order depends on atomic arrival.)
template <int DT>
__device__ void dec_select_chunk(const DecParams& p, uint32_t c, uint32_t kq, bool publish, unsigned char* sm) {
    using T = typename Tr<DT>::T;
    float* floors = reinterpret_cast<float*>(sm + DecSmem::kFloor);
    uint32_t* cum = reinterpret_cast<uint32_t*>(sm + DecSmem::kOff);        // [32] cumulative bucket counts
    uint32_t* cnt = cum + 32;                                               // [32] per virtual warp (A | B << 16)
    int* srow = reinterpret_cast<int*>(sm + DecSmem::kRow);
    float* sact = reinterpret_cast<float*>(sm + DecSmem::kAct);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t s = c * kChunk;
    const uint32_t len = min((uint32_t)kChunk, p.K - s);
    const T* x = reinterpret_cast<const T*>(p.x);

    float xv[4];
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const uint32_t e = it * kThreads + tid;
        xv[it] = (e < len) ? Tr<DT>::to_f(x[s + e]) : __int_as_float(0x7fc00000);  // NaN = no bucket
    }
    if (tid < kBuckets) {
        floors[tid] = bucket_floor<DT>(p.thr_a, p.thr_b, tid);
        cum[tid] = 0u;
    }
    dec_bar();

    // G bit L = (|x| >= floor[L]); bucket = lowest set bit
    uint32_t G[4] = {0u, 0u, 0u, 0u};
    {
        float ax[4];
#pragma unroll
        for (int it = 0; it < 4; ++it) ax[it] = fabsf(xv[it]);
        const float4* fl4 = reinterpret_cast<const float4*>(floors);
#pragma unroll
        for (int L4 = 0; L4 < 8; ++L4) {
            const float4 fl = fl4[L4];
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                uint32_t m = (ax[it] >= fl.x) ? 1u : 0u;
                m |= (ax[it] >= fl.y) ? 2u : 0u;
                m |= (ax[it] >= fl.z) ? 4u : 0u;
                m |= (ax[it] >= fl.w) ? 8u : 0u;
                G[it] |= m << (4 * L4);
            }
        }
    }
    int bk[4];
    uint32_t C[4];   // bit L = (bucket <= L)
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const bool finite = fabsf(xv[it]) < __int_as_float(0x7f800000);   // false for inf and NaN
        bk[it] = (finite && G[it]) ? (__ffs(G[it]) - 1) : 32;
        C[it] = (bk[it] < 32) ? (0xffffffffu << bk[it]) : 0u;
    }
    // 32x32 bit transposes: lane L gets, per virtual warp, the ballot of (bucket <= L)
    uint32_t below = 0;
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        uint32_t v = C[it];
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) {
            const uint32_t msk = (d == 16) ? 0x0000ffffu : (d == 8) ? 0x00ff00ffu : (d == 4) ? 0x0f0f0f0fu
                                : (d == 2) ? 0x33333333u : 0x55555555u;
            const bool up = (lane & d) != 0;
            const uint32_t send = up ? (v << d) : (v >> d);
            const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, d);
            v = up ? ((v & ~msk) | (recv & msk)) : ((v & msk) | (recv & ~msk));
        }
        below += __popc(v);
    }
    atomicAdd(&cum[lane], below);
    dec_bar();

    // boundary bucket: first L with cum[L] >= kq (32 if the chunk has fewer than kq finite values)
    const uint32_t cl = cum[lane];
    const uint32_t ge = __ballot_sync(0xffffffffu, cl >= kq);
    const int Lb = ge ? (__ffs(ge) - 1) : 32;
    const uint32_t cprev = (Lb == 0) ? 0u : __shfl_sync(0xffffffffu, cl, (Lb - 1) & 31);
    const uint32_t total = __shfl_sync(0xffffffffu, cl, 31);
    const uint32_t quota = (Lb < 32) ? (kq - cprev) : 0u;

    uint32_t balA[4], balB[4];
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        balA[it] = __ballot_sync(0xffffffffu, bk[it] < Lb);
        balB[it] = __ballot_sync(0xffffffffu, bk[it] == Lb && Lb < 32);
        if (lane == 0) cnt[it * 8 + warp] = __popc(balA[it]) | (__popc(balB[it]) << 16);
    }
    dec_bar();
    uint32_t inc = cnt[lane];
    const uint32_t own = inc;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t o = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += o;
    }
    const uint32_t excl = inc - own;   // packed exclusive prefix for virtual warp = lane
    const uint32_t lt = (1u << lane) - 1u;
    int* g_rows = p.sel_rows + (size_t)c * p.k_chunk;
    T* g_acts = reinterpret_cast<T*>(p.sel_acts) + (size_t)c * p.k_chunk;
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const uint32_t pre = __shfl_sync(0xffffffffu, excl, it * 8 + warp);
        uint32_t r = 0xffffffffu;
        if (bk[it] < Lb) {
            r = (pre & 0xffffu) + __popc(balA[it] & lt);
        } else if (bk[it] == Lb && Lb < 32) {
            const uint32_t rb = (pre >> 16) + __popc(balB[it] & lt);
            if (rb < quota) r = cprev + rb;
        }
        if (r < kq) {
            const int row = (int)(s + it * kThreads + tid);
            srow[r] = row;
            sact[r] = xv[it];
            if (publish) { g_rows[r] = row; g_acts[r] = Tr<DT>::from_f(xv[it]); }
        }
    }
    // fewer than kq finite values (NaN/inf activations): pad with a harmless (row, 0) pair.
    // The reference aborts with a device assert here (dec.cu:178).
    const uint32_t filled = min(total, kq);
    for (uint32_t r = filled + tid; r < kq; r += kThreads) {
        srow[r] = (int)s;
        sact[r] = 0.0f;
        if (publish) { g_rows[r] = (int)s; g_acts[r] = Tr<DT>::from_f(0.0f); }
    }
    dec_bar();
}

__device__ __forceinline__ void dec_decode_word(uint32_t w, float a, float* acc) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        // 0x4B000000 | nib is the float 2^23 + nib; subtracting 2^23 + 8 leaves nib - 8 exactly
        const float f = __uint_as_float(0x4B000000u | ((w >> (4 * i)) & 0xFu)) - 8388616.0f;
        acc[i] = fmaf(f, a, acc[i]);
    }
}

// Fetch rows srow[0..nrows) x packed columns [w0, w1) and add the unscaled sums into acc_g.
// Grouped form, run by the first kThreads threads: a block of columns is covered by R row groups of
// threads whose partial sums meet in shared memory - the right shape when the CTA's column range is
// narrow (many compensation CTAs).
// VW = words per load (4: 16-byte loads, needs N % 32 == 0; 1: scalar fallback).
template <int DT, int VW>
__device__ void dec_fetch(const DecParams& p, float* acc_g, uint32_t nrows, uint32_t w0, uint32_t w1, unsigned char* sm) {
    using T = typename Tr<DT>::T;
    const int* srow = reinterpret_cast<const int*>(sm + DecSmem::kRow);
    const float* sact = reinterpret_cast<const float*>(sm + DecSmem::kAct);
    float* red = reinterpret_cast<float*>(sm + DecSmem::kRed);
    const uint32_t wpr = p.N / 8;  // words per residual row
    const int tid = threadIdx.x;
    constexpr uint32_t kBlockWords = 128 * VW;  // at most 128 loads wide, so at least 2 row groups
    constexpr int UN = 8;                       // rows in flight per thread

    for (uint32_t cb = w0; cb < w1; cb += kBlockWords) {
        const uint32_t nw = min(kBlockWords, w1 - cb);
        const uint32_t tv = (nw + VW - 1) / VW;
        const uint32_t R = kThreads / tv;
        const uint32_t v = tid % tv, rg = tid / tv;
        float a[VW * 8];
#pragma unroll
        for (int i = 0; i < VW * 8; ++i) a[i] = 0.0f;
        if (rg < R) {
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
                        if (i0 + b * R < nrows) {      // nothing to decode for the slots beyond the last row
                            dec_decode_word(q[b].x, xa[b], a + 0);
                            dec_decode_word(q[b].y, xa[b], a + 8);
                            dec_decode_word(q[b].z, xa[b], a + 16);
                            dec_decode_word(q[b].w, xa[b], a + 24);
                        }
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
                    for (int b = 0; b < UN; ++b)
                        if (i0 + b * R < nrows) dec_decode_word(q[b], xa[b], a);
                }
            }
        }
        // per-thread partials -> red[value][thread] (pitch 257: conflict-free both ways), then each
        // output sums its R row groups
#pragma unroll
        for (int i = 0; i < VW * 8; ++i) red[i * 257 + tid] = a[i];
        dec_bar();
        for (uint32_t o = tid; o < nw * 8; o += kThreads) {
            const uint32_t vv = o / (VW * 8), i = o % (VW * 8);
            float sum = 0.0f;
            for (uint32_t r = 0; r < R; ++r) sum += red[i * 257 + r * tv + vv];
            atomicAdd(&acc_g[cb * 8 + o], sum);      // unscaled: the scale is applied when the tile is finalized
        }
        dec_bar();
    }
}

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" :: "l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Direct form, run by all `nthr` threads of the CTA: a thread owns a 16-byte column vector (32 outputs) and
// every R-th selected row of it (R = thread groups that fit beside each other on the column range), keeps
// up to eight row loads in flight, and adds its sums with 16-byte vector reductions.  No shared-memory
// exchange and no barrier, so warps drift apart and keep the link busy; the right shape when the CTA's
// column range is wide (few compensation CTAs).  The 32 sums are formed in two halves of 16 so that the
// eight loaded vectors stay in registers under the register cap of the widest GEMV launch.
// Needs N % 32 == 0 (w0, w1 are then multiples of 4 words).
template <int DT>
__device__ void dec_fetch_direct(const DecParams& p, float* acc_g, uint32_t nrows, uint32_t w0, uint32_t w1,
                                 const unsigned char* sm, uint32_t nthr) {
    const int* srow = reinterpret_cast<const int*>(sm + DecSmem::kRow);
    const float* sact = reinterpret_cast<const float*>(sm + DecSmem::kAct);
    const uint32_t wpr = p.N / 8;
    const uint32_t nvec = (w1 - w0) / 4u;
    uint32_t R = nthr / nvec;                       // row groups side by side (1..32 by the caller's choice of form)
    if (R == 0) R = 1;
    // R == 1: threads stride over the column vectors; R > 1: one sweep, thread -> (vector, row group)
    const uint32_t stride = R > 1 ? nvec * R : nthr;
    constexpr int UN = 8;
    for (uint32_t t = threadIdx.x; t < nvec * R; t += stride) {
        const uint32_t v = t % nvec;
        const uint32_t rg = t / nvec;
        const uint32_t col = w0 + 4u * v;
        float* dst = acc_g + (size_t)col * 8;
        for (uint32_t i0 = rg; i0 < nrows; i0 += R * UN) {
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
            for (int h = 0; h < 2; ++h) {
                float a[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) a[i] = 0.0f;
#pragma unroll
                for (int b = 0; b < UN; ++b) {
                    if (i0 + b * R < nrows) {
                        dec_decode_word(h ? q[b].z : q[b].x, xa[b], a + 0);
                        dec_decode_word(h ? q[b].w : q[b].y, xa[b], a + 8);
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    red_add_v4(dst + 16 * h + 4 * j, a[4 * j], a[4 * j + 1], a[4 * j + 2], a[4 * j + 3]);
            }
        }
    }
}

// One DEC CTA.  `cta` in [0, p.n_cta).  Called by all threads of the CTA (blockDim.x >= kThreads).
template <int DT>
__device__ void dec_role(const DecParams& p, const FinParams& f, uint32_t cta, unsigned char* sm) {
    using T = typename Tr<DT>::T;
    const uint32_t nthr = blockDim.x;
    const bool first = threadIdx.x < kThreads;
    pdl_trigger();
    pdl_wait();                             // everything below reads activations / writes shared state
    const uint32_t rp = cta % p.n_rowparts;
    const uint32_t cp = cta / p.n_rowparts;
    // column part = a contiguous range of output tiles
    const uint32_t t0 = (uint32_t)(((uint64_t)cp * f.n_tiles) / p.n_colparts);
    const uint32_t t1 = (uint32_t)(((uint64_t)(cp + 1) * f.n_tiles) / p.n_colparts);
    const uint32_t wpr = p.N / 8;
    const uint32_t w0 = min(wpr, t0 * f.tile_units * 4u);
    const uint32_t w1 = min(wpr, t1 * f.tile_units * 4u);
    const bool vec = (p.N % 32u) == 0u;
    // wide column range: at most sixteen thread groups share a column vector - or up to thirty-two when so few
    // rows are selected per chunk that every group gets one row and one load (small k_chunk on the narrow layers)
    const bool direct = vec && ((w1 - w0) * 4u >= nthr || ((w1 - w0) * 8u >= nthr && p.k_chunk <= 16u));
    int* srow = reinterpret_cast<int*>(sm + DecSmem::kRow);
    float* sact = reinterpret_cast<float*>(sm + DecSmem::kAct);

    if (p.fused_select) {
        const uint32_t num_chunks = (p.K + kChunk - 1) / kChunk;
        for (uint32_t c = rp; c < num_chunks; c += p.n_rowparts) {
            const uint32_t len = min((uint32_t)kChunk, p.K - c * kChunk);
            const uint32_t kq = p.k_chunk * len / kChunk;
            if (kq == 0) continue;
            if (first) dec_select_chunk<DT>(p, c, kq, cp == 0, sm);
            __syncthreads();
            if (w1 > w0) {
                if (direct) dec_fetch_direct<DT>(p, f.acc2, kq, w0, w1, sm, nthr);
                else if (first) {
                    if (vec) dec_fetch<DT, 4>(p, f.acc2, kq, w0, w1, sm);
                    else dec_fetch<DT, 1>(p, f.acc2, kq, w0, w1, sm);
                }
            }
            __syncthreads();                // the next chunk's selection overwrites srow/sact
        }
    } else {
        // rows supplied by the caller (context buffer); activation gathered as x[row] (dec.cu:346)
        const T* x = reinterpret_cast<const T*>(p.x);
        const uint32_t r0 = (uint32_t)(((uint64_t)rp * p.k_total) / p.n_rowparts);
        const uint32_t r1 = (uint32_t)(((uint64_t)(rp + 1) * p.k_total) / p.n_rowparts);
        for (uint32_t b0 = r0; b0 < r1; b0 += kChunk) {
            const uint32_t nb = min((uint32_t)kChunk, r1 - b0);
            for (uint32_t i = threadIdx.x; i < nb; i += nthr) {
                const int row = p.sel_rows[b0 + i];
                const bool ok = row >= 0 && (uint32_t)row < p.K;   // out-of-range rows contribute nothing
                srow[i] = ok ? row : 0;
                sact[i] = ok ? Tr<DT>::to_f(x[row]) : 0.0f;
            }
            __syncthreads();
            if (w1 > w0) {
                if (direct) dec_fetch_direct<DT>(p, f.acc2, nb, w0, w1, sm, nthr);
                else if (first) {
                    if (vec) dec_fetch<DT, 4>(p, f.acc2, nb, w0, w1, sm);
                    else dec_fetch<DT, 1>(p, f.acc2, nb, w0, w1, sm);
                }
            }
            __syncthreads();
        }
    }
    arrive_and_finalize<DT>(f, t0, t1, reinterpret_cast<unsigned*>(sm + DecSmem::kFlag), nthr);
}

// ---- compensation role of launches without tickets (packed accumulator words, common.cuh) -------------------------
// The CTA keeps its sums to itself until the end: every thread adds what it fetched into PRIVATE fp32 cells in shared
// memory (cell (i, slot) at i * stride + slot with an ODD stride: neighbouring lanes hit neighbouring banks both when
// lanes are slots, in the fetch, and when lanes are the 32 elements i of a vector, in the last pass), over all chunks
// of the CTA's row part; then one barrier, one pass that adds the row groups of an output, scales it, and makes ONE arrival per
// output with a 64-bit atomic.  The thread whose atomic returns the last arrival count writes y.  No global partial
// sums, no fence, no ticket; the residual scales are loaded before the wait for the previous kernel.
// Needs N % 32 == 0 and fused selection.  Shared memory: DecSmem followed by 32 * (nslots | 1) floats.
constexpr int kDecPrivOff = (DecSmem::kBytes + 127) & ~127;

// slots a CTA needs for a column range of `nvec` 16-byte vectors when `nthr` threads take part
__host__ __device__ inline uint32_t dec_private_slots(uint32_t nvec, uint32_t nthr) {
    const uint32_t R = nvec ? nthr / nvec : 0u;
    return R ? nvec * R : nvec;
}

template <int DT>
__device__ void dec_fetch_private(const DecParams& p, float* cells, uint32_t nslots, uint32_t stride, uint32_t nrows, uint32_t w0,
                                  uint32_t nvec, const unsigned char* sm, uint32_t nthr) {
    const int* srow = reinterpret_cast<const int*>(sm + DecSmem::kRow);
    const float* sact = reinterpret_cast<const float*>(sm + DecSmem::kAct);
    const uint32_t wpr = p.N / 8;
    const uint32_t R = nthr / nvec;                 // row groups side by side; 0: fewer threads than vectors
    const uint32_t Ruse = R ? R : 1u;
    constexpr int UN = 8;
    for (uint32_t t = threadIdx.x; t < nslots; t += nthr) {      // one sweep when R >= 1
        const uint32_t v = R ? t % nvec : t;
        const uint32_t rg = R ? t / nvec : 0u;
        const uint32_t col = w0 + 4u * v;
        float* cell = cells + t;
        for (uint32_t i0 = rg; i0 < nrows; i0 += Ruse * UN) {
            uint4 q[UN];
            float xa[UN];
#pragma unroll
            for (int b = 0; b < UN; ++b) {
                const uint32_t i = i0 + b * Ruse;
                if (i < nrows) {
                    q[b] = ldg_stream(reinterpret_cast<const uint4*>(p.cheat + (size_t)srow[i] * wpr + col));
                    xa[b] = sact[i];
                } else {
                    q[b] = make_uint4(0, 0, 0, 0);
                    xa[b] = 0.0f;
                }
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float a[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) a[i] = 0.0f;
#pragma unroll
                for (int b = 0; b < UN; ++b) {
                    if (i0 + b * Ruse < nrows) {
                        dec_decode_word(h ? q[b].z : q[b].x, xa[b], a + 0);
                        dec_decode_word(h ? q[b].w : q[b].y, xa[b], a + 8);
                    }
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) cell[(size_t)(16 * h + i) * stride] += a[i];
            }
        }
    }
}

template <int DT>
__device__ void dec_role_packed(const DecParams& p, const FinParams& f, uint32_t cta, unsigned char* sm, uint32_t arrivals) {
    using T = typename Tr<DT>::T;
    const uint32_t nthr = blockDim.x;
    const bool first = threadIdx.x < kThreads;
    pdl_trigger();
    const uint32_t rp = cta % p.n_rowparts;
    const uint32_t cp = cta / p.n_rowparts;
    const uint32_t t0 = (uint32_t)(((uint64_t)cp * f.n_tiles) / p.n_colparts);
    const uint32_t t1 = (uint32_t)(((uint64_t)(cp + 1) * f.n_tiles) / p.n_colparts);
    const uint32_t wpr = p.N / 8;
    const uint32_t w0 = min(wpr, t0 * f.tile_units * 4u);
    const uint32_t w1 = min(wpr, t1 * f.tile_units * 4u);
    const uint32_t nvec = (w1 - w0) / 4u;
    const uint32_t nslots = dec_private_slots(nvec, nthr);
    const uint32_t stride = nslots | 1u;
    float* cells = reinterpret_cast<float*>(sm + kDecPrivOff);
    for (uint32_t i = threadIdx.x; i < 32u * stride; i += nthr) cells[i] = 0.0f;
    pdl_wait();                             // everything below reads activations / writes shared state
    const uint32_t num_chunks = (p.K + kChunk - 1) / kChunk;
    for (uint32_t c = rp; c < num_chunks; c += p.n_rowparts) {
        const uint32_t len = min((uint32_t)kChunk, p.K - c * kChunk);
        const uint32_t kq = p.k_chunk * len / kChunk;
        if (kq == 0) continue;
        if (first) dec_select_chunk<DT>(p, c, kq, cp == 0, sm);
        __syncthreads();
        if (nvec) dec_fetch_private<DT>(p, cells, nslots, stride, kq, w0, nvec, sm, nthr);
        __syncthreads();                // the next chunk's selection overwrites srow/sact
    }
    __syncthreads();
    // one arrival per output of the column range; lanes take CONSECUTIVE outputs, so the accesses to y, to the
    // accumulator words and (four lanes per sector) to the scales coalesce
    const uint32_t R = nthr / max(nvec, 1u);
    const uint32_t Ruse = R ? R : 1u;
    T* y = reinterpret_cast<T*>(f.y);
    const T* sc = reinterpret_cast<const T*>(f.scales);
    unsigned long long* words = reinterpret_cast<unsigned long long*>(f.acc);
    const uint32_t nbase = w0 * 8u;
    // eight outputs per thread and pass: their loads travel together, then their atomics travel together
    constexpr int U = 8;
    for (uint32_t ob = threadIdx.x; ob < 32u * nvec; ob += nthr * U) {
        unsigned long long mine[U], old[U];
        float y0[U];
        uint32_t nn[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t o = ob + u * nthr;
            nn[u] = 0xffffffffu;
            if (o >= 32u * nvec) continue;
            const uint32_t v = o >> 5, i = o & 31u;
            float tot = 0.0f;
            for (uint32_t rg = 0; rg < Ruse; ++rg) tot += cells[(size_t)i * stride + v + nvec * rg];
            const uint32_t n = nbase + o;
            nn[u] = n;
            y0[u] = Tr<DT>::to_f(y[n]);
            mine[u] = pack_partial(tot * Tr<DT>::to_f(sc[(size_t)(n & 7u) * wpr + (n >> 3)]));
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (nn[u] != 0xffffffffu) old[u] = atomicAdd(words + nn[u], mine[u]);
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (nn[u] != 0xffffffffu) finish_packed<DT>(old[u], mine[u], arrivals, words + nn[u], y + nn[u], y0[u]);
    }
}

}  // namespace dd
