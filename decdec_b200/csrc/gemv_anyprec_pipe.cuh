// Any-precision GEMV role for 3 to 8 bits, bulk-copy pipelined variant.
//
// In the tensor [plane][row][K/32] consecutive rows of one plane are contiguous, so a stage of R rows is one
// contiguous run per plane plus the R LUT rows.  A producer thread moves them with 1-D bulk asynchronous
// copies (cp.async.bulk, completion counted on an mbarrier) several stages ahead of the consumer warps;
// a warp's work item is (row of the stage, 4096-channel segment of that row).
// Two decoders.  The 3-bit byte-permute decoder has the arithmetic of gemv_anyprec.cuh:ap3_role (register-
// resident byte tables, activations staged in pair order).  The lookup decoder serves every width: the plane
// words of 32 channels are regrouped into 4-bit fields with a handful of logic operations, each code indexes
// the row's LUT where the bulk copy landed it in shared memory (a row of up to 64 entries spans at most 32 banks
// and equal entries broadcast, so a warp's lookup is one wavefront), and the product goes into one of four fp32
// sums with a mixed-precision multiply-add (16-bit factors, fp32 accumulator): no 16-bit partial sums.
// A CTA owns its rows completely (all of K), so the row sums meet in a small shared-memory buffer and the
// CTA folds them into y itself: GEMV-only launches use no global accumulator, ticket or fence.  Fused
// launches store the sums into the workspace accumulator and arrive on the tile's ticket, where they meet
// the compensation CTAs.
// Requirements: K % 128 == 0, K <= 32768.  Every mbarrier wait is bounded.
#pragma once
#include "gemv_anyprec.cuh"
#include "gemv_bcq_pipe.cuh"

namespace dd {

constexpr int kApPipeThreads = 544;   // 16 consumer warps + 1 producer warp

struct ApPipeGeom {
    uint32_t rows_per_stage;   // R
    uint32_t segs;             // ceil(K / 4096): warps per row
    uint32_t stages;           // pipeline depth
    uint32_t stage_bytes;
    uint32_t lookup;           // 1: lookup decoder, 0: byte-permute decoder (3 bits only)
    uint32_t x_bytes;          // staged activations (rounded to 128)
    uint32_t rows_per_cta;     // multiple of R
    uint32_t part_bytes;       // row sums of the CTA (fp32, rounded to 128 bytes)
    uint32_t smem_bytes;
    uint32_t direct;           // 1: fold into y; 0: store into the accumulator and take the tile's ticket
    uint32_t wait_ns;          // limit of one mbarrier wait (DECDEC_PIPE_WAIT_NS)
};

constexpr int kApPipeHdr = 256;   // [abort, flag][full barriers 8][empty barriers 8]

// 4-bit fields from up to four plane words: field t (bits 4t..4t+3) of result ph holds, most significant plane
// first, the bits that planes P[0..B-1] carry at position 4t + ph.
template <int B>
__device__ __forceinline__ void ap_fields(const uint32_t* P, uint32_t (&V)[4]) {
    uint32_t R[B];
#pragma unroll
    for (int i = 0; i < B; ++i) R[i] = i ? __funnelshift_r(P[i], P[i], i) : P[0];
#pragma unroll
    for (int ph = 0; ph < 4; ++ph) {
        uint32_t m = 0u;
#pragma unroll
        for (int i = 0; i < B; ++i) m |= R[i] & (0x11111111u << ((ph - i) & 3));
        const int rot = (B - 1 - ph) & 31;
        V[ph] = rot ? __funnelshift_l(m, m, rot) : m;
    }
}

// d += a * b with 16-bit factors (raw bits of the element type) and an fp32 accumulator
template <int DT>
__device__ __forceinline__ void ap_mixed_fma(float& d, uint16_t a, uint16_t b) {
    if constexpr (DT == FP16) asm("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(d) : "h"(a), "h"(b));
    else asm("fma.rn.f32.bf16 %0, %1, %2, %0;" : "+f"(d) : "h"(a), "h"(b));
}

// One plane-word position (32 channels) of one row through the lookup decoder.  `lutrow` is the row's LUT where the
// bulk copy landed it; X[j] holds the activations of channels 8 * E * j + (0..7) of the word's group.
template <int DT, int BITS>
__device__ __forceinline__ void ap_lookup_word(const uint32_t* q, const unsigned char* lutrow, const uint4 (&X)[4], float (&acc)[4]) {
    constexpr int BH = BITS < 4 ? BITS : 4, BL = BITS - BH;
    uint32_t Vh[4], Vl[4] = {0u, 0u, 0u, 0u};
    ap_fields<BH>(q, Vh);
    if constexpr (BL > 0) ap_fields<BL>(q + 4, Vl);
#pragma unroll
    for (int ph = 0; ph < 4; ++ph) {
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            const int pos = 31 - (4 * t + ph);          // channel = 8 * E * (pos / 8) + pos % 8 inside the word's group
            const int jj = pos >> 3, r = pos & 7;
            uint32_t off;                                // byte offset of the code's entry: 2 * code
            if constexpr (BL == 0) {
                off = t ? ((Vh[ph] >> (4 * t - 1)) & 0x1eu) : ((Vh[ph] << 1) & 0x1eu);
            } else {
                constexpr uint32_t mh = 0xfu << (BL + 1), ml = ((1u << BL) - 1u) << 1;
                const int sh = 4 * t - BL - 1;
                off = (sh >= 0) ? ((Vh[ph] >> (sh & 31)) & mh) : ((Vh[ph] << ((-sh) & 31)) & mh);
                off |= t ? ((Vl[ph] >> (4 * t - 1)) & ml) : ((Vl[ph] << 1) & ml);
            }
            const uint16_t w = *reinterpret_cast<const uint16_t*>(lutrow + off);
            const uint32_t xw = (&X[jj].x)[r >> 1];
            const uint16_t xv = (r & 1) ? (uint16_t)(xw >> 16) : (uint16_t)(xw & 0xffffu);
            ap_mixed_fma<DT>(acc[t & 3], w, xv);
        }
    }
}

// BITS planes; LOOKUP selects the decoder (the byte-permute decoder exists for 3 bits only)
template <int DT, int BITS, bool LOOKUP>
__device__ void ap_pipe_role(const ApParams& p, const FinParams& f, const ApPipeGeom& geo, uint32_t cta, unsigned char* sm) {
    static_assert(LOOKUP || BITS == 3, "the byte-permute decoder is 3-bit");
    constexpr uint32_t kLutRow = 2u << BITS;             // bytes of one row's LUT
    constexpr int NW = 16;                               // consumer warps; warp NW is the producer
    constexpr int NT = (NW + 1) * 32;
    using T = typename Tr<DT>::T;
    static_assert(DT != FP32, "any-precision kernels take fp16/bf16 only");
    volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(sm);
    unsigned* s_flag = reinterpret_cast<unsigned*>(sm + 4);
    const uint32_t bar_full = smem_u32(sm + 64);
    const uint32_t bar_empty = bar_full + 64;
    T* sx = reinterpret_cast<T*>(sm + kApPipeHdr);
    float* part = reinterpret_cast<float*>(sm + kApPipeHdr + geo.x_bytes);
    unsigned char* stage0 = sm + kApPipeHdr + geo.x_bytes + geo.part_bytes;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t nwords = p.K / 32;
    const uint32_t rowbytes = nwords * 4;
    const uint32_t R = geo.rows_per_stage, S = geo.stages;
    const uint32_t r0 = cta * geo.rows_per_cta;
    const uint32_t r1 = min(p.N, r0 + geo.rows_per_cta);
    const uint32_t nst = (r1 - r0 + R - 1) / R;
    const uint32_t lut_off = BITS * R * rowbytes;       // LUT rows sit after the plane runs

    pdl_trigger();
    if (tid == 0) {
        *s_abort = 0u;
        for (uint32_t s = 0; s < S; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, NW);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (uint32_t i = tid; i < geo.rows_per_cta; i += NT) part[i] = 0.0f;
    __syncthreads();

    if (warp == NW) {
        // ------------------------------ producer (one elected lane) -----------------------------
        if (lane == 0) {
            const size_t plane_stride = (size_t)p.N * nwords;
            const unsigned char* lutb = reinterpret_cast<const unsigned char*>(p.lut);
            uint32_t issued = 0;
            for (uint32_t i = 0; i < nst; ++i) {
                const uint32_t s = i % S, use = i / S;
                if (use > 0) {
                    // slots free only after the consumers' wait for the previous kernel: resolve the dependency before
                    // the first bounded wait (every slot is full by now, so no copy is delayed)
                    if (use == 1 && s == 0) pdl_wait();
                    if (!mbar_wait(bar_empty + 8 * s, (use - 1) & 1u, s_abort, geo.wait_ns)) break;
                }
                const uint32_t n0 = r0 + i * R;
                const uint32_t rows = min(R, r1 - n0);
                const uint32_t full = bar_full + 8 * s;
                mbar_expect_tx(full, rows * (BITS * rowbytes + kLutRow));
                const uint32_t dst = smem_u32(stage0 + (size_t)s * geo.stage_bytes);
#pragma unroll
                for (int pl = 0; pl < BITS; ++pl)
                    bulk_g2s(dst + pl * R * rowbytes, p.qweight + pl * plane_stride + (size_t)n0 * nwords, rows * rowbytes, full);
                bulk_g2s(dst + lut_off, lutb + (size_t)n0 * kLutRow, rows * kLutRow, full);
                issued = i + 1;
            }
            if (*s_abort) {
                const uint32_t first = issued > S ? issued - S : 0;
                for (uint32_t i = first; i < issued; ++i) {
                    volatile uint32_t never = 0;
                    mbar_wait(bar_full + 8 * (i % S), (i / S) & 1u, &never, 1000000000u);
                }
            }
        }
    } else if constexpr (LOOKUP) {
        // ------------------------------ consumers, lookup decoder -------------------------------
        pdl_wait();     // weights are already streaming (producer warp); activations come from earlier kernels
        const T* x = reinterpret_cast<const T*>(p.x);
        for (uint32_t k = tid; k < p.K; k += 512) sx[k] = x[k];
        asm volatile("bar.sync 1, 512;" ::: "memory");

        const uint32_t tailE = nwords & 31u, nfull = nwords >> 5;
        const uint32_t row_in_stage = warp / geo.segs, seg = warp % geo.segs;
        const bool has_item = row_in_stage < R;
        const uint32_t wi0 = seg * 128 + lane;            // the lane's words: wi0 + 32 * u, u = 0..3
        const bool lane_active = has_item && wi0 < nwords;

        for (uint32_t i = 0; i < nst; ++i) {
            const uint32_t s = i % S;
            if (!mbar_wait(bar_full + 8 * s, (i / S) & 1u, s_abort, geo.wait_ns)) break;
            const unsigned char* st = stage0 + (size_t)s * geo.stage_bytes;
            const uint32_t n = r0 + i * R + row_in_stage;
            float facc = 0.0f;
            if (lane_active && n < r1) {
                const unsigned char* lutrow = st + lut_off + row_in_stage * kLutRow;
                const uint32_t* rowp = reinterpret_cast<const uint32_t*>(st + (size_t)row_in_stage * rowbytes) + wi0;
                uint32_t q[4][BITS];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const bool ok = wi0 + 32 * u < nwords;
#pragma unroll
                    for (int pl = 0; pl < BITS; ++pl) q[u][pl] = ok ? rowp[32 * u + pl * R * nwords] : 0u;
                }
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t wi = wi0 + 32 * u;
                    if (wi >= nwords) break;
                    const uint32_t blk = wi >> 5, t = wi & 31u;
                    const uint32_t E = (blk == nfull) ? tailE : 32u;
                    const T* xb = sx + blk * 1024u + 8u * t;
                    uint4 X[4];
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) X[jj] = *reinterpret_cast<const uint4*>(xb + 8u * E * jj);
                    ap_lookup_word<DT, BITS>(q[u], lutrow, X, acc);
                }
                facc = (acc[0] + acc[1]) + (acc[2] + acc[3]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * s);      // the stage (plane words and LUT row) is no longer read
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) facc += __shfl_xor_sync(0xffffffffu, facc, d);
            if (lane == 0 && has_item && n < r1) {
                if (geo.segs == 1) part[n - r0] = facc;           // one warp per row: nobody else writes it
                else atomicAdd(&part[n - r0], facc);              // the K segments of a row meet here
            }
        }
    } else {
        // ------------------------------ consumers, byte-permute decoder -------------------------
        pdl_wait();     // weights are already streaming (producer warp); activations come from earlier kernels
        const T* x = reinterpret_cast<const T*>(p.x);
        for (uint32_t k = tid; k < p.K; k += 512) sx[(k & ~7u) | ap_perm(k & 7u)] = x[k];
        asm volatile("bar.sync 1, 512;" ::: "memory");

        const uint32_t tailE = nwords & 31u, nfull = nwords >> 5;
        const uint32_t row_in_stage = warp / geo.segs, seg = warp % geo.segs;
        const bool has_item = row_in_stage < R;
        // lane handles words seg*128 + 32*u + lane (u = 0..3): consecutive lanes read consecutive words and
        // consecutive 16-byte activation groups, so neither shared load has bank conflicts
        const uint32_t wi0 = seg * 128 + lane;
        const bool lane_active = has_item && wi0 < nwords;

        for (uint32_t i = 0; i < nst; ++i) {
            const uint32_t s = i % S;
            if (!mbar_wait(bar_full + 8 * s, (i / S) & 1u, s_abort, geo.wait_ns)) break;
            const unsigned char* st = stage0 + (size_t)s * geo.stage_bytes;
            const uint32_t n = r0 + i * R + row_in_stage;
            float facc = 0.0f;
            if (lane_active && n < r1) {
                const uint4 L = *reinterpret_cast<const uint4*>(st + lut_off + row_in_stage * 16);
                const uint32_t lo01 = __byte_perm(L.x, L.y, 0x6420), lo23 = __byte_perm(L.z, L.w, 0x6420);
                const uint32_t hi01 = __byte_perm(L.x, L.y, 0x7531), hi23 = __byte_perm(L.z, L.w, 0x7531);
                const uint32_t* rowp = reinterpret_cast<const uint32_t*>(st + (size_t)row_in_stage * rowbytes) + wi0;
                uint32_t aw[4], bw[4], cw[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const bool ok = wi0 + 32 * u < nwords;
                    aw[u] = ok ? rowp[32 * u] : 0u;
                    bw[u] = ok ? rowp[32 * u + R * nwords] : 0u;
                    cw[u] = ok ? rowp[32 * u + 2 * R * nwords] : 0u;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t wi = wi0 + 32 * u;
                    if (wi >= nwords) break;
                    const uint32_t blk = wi >> 5, t = wi & 31u;
                    const uint32_t E = (blk == nfull) ? tailE : 32u;
                    const T* xb = sx + blk * 1024u + 8u * t;
                    uint4 X[4];
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) X[jj] = *reinterpret_cast<const uint4*>(xb + 8u * E * jj);
                    const uint32_t a = aw[u];
                    const uint32_t b = __funnelshift_r(bw[u], bw[u], 1);
                    const uint32_t c = __funnelshift_r(cw[u], cw[u], 2);
                    uint32_t V[4];
                    V[0] = (a & 0x11111111u) | (b & 0x88888888u) | (c & 0x44444444u);
                    V[0] = __funnelshift_l(V[0], V[0], 2);
                    V[1] = (a & 0x22222222u) | (b & 0x11111111u) | (c & 0x88888888u);
                    V[1] = __funnelshift_l(V[1], V[1], 1);
                    V[2] = (a & 0x44444444u) | (b & 0x22222222u) | (c & 0x11111111u);
                    V[3] = ((a & 0x88888888u) | (b & 0x44444444u) | (c & 0x22222222u)) >> 1;
                    uint32_t hacc[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                    for (int ph = 0; ph < 4; ++ph) {
                        const uint32_t v = V[ph];
                        const uint32_t vh = v >> 16;
                        const uint32_t l0 = __byte_perm(lo01, lo23, v), h0 = __byte_perm(hi01, hi23, v);
                        const uint32_t l1 = __byte_perm(lo01, lo23, vh), h1 = __byte_perm(hi01, hi23, vh);
                        const uint32_t w3 = __byte_perm(l0, h0, 0x5140), w2 = __byte_perm(l0, h0, 0x7362);
                        const uint32_t w1 = __byte_perm(l1, h1, 0x5140), w0 = __byte_perm(l1, h1, 0x7362);
                        const uint32_t x3 = (&X[3].x)[ph], x2 = (&X[2].x)[ph], x1 = (&X[1].x)[ph], x0 = (&X[0].x)[ph];
                        ap_fma<DT>(w3, x3, hacc[3], facc);
                        ap_fma<DT>(w2, x2, hacc[2], facc);
                        ap_fma<DT>(w1, x1, hacc[1], facc);
                        ap_fma<DT>(w0, x0, hacc[0], facc);
                    }
                    if constexpr (DT == FP16) {
                        facc += ap_sum2<DT>(hacc[0]) + ap_sum2<DT>(hacc[1]);
                        facc += ap_sum2<DT>(hacc[2]) + ap_sum2<DT>(hacc[3]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * s);      // stage words are in registers
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) facc += __shfl_xor_sync(0xffffffffu, facc, d);
            if (lane == 0 && has_item && n < r1) {
                if (geo.segs == 1) part[n - r0] = facc;           // one warp per row: nobody else writes it
                else atomicAdd(&part[n - r0], facc);              // the K segments of a row meet here
            }
        }
    }
    if (warp == NW) pdl_wait();     // the producer warp touches the accumulator and y only from here on
    // fold the CTA's rows: four consecutive outputs per thread; y is read before the barrier so that the
    // load overlaps the last warps' work
    T* y = reinterpret_cast<T*>(f.y);
    const uint32_t nrows = r1 - r0;
    const bool yvec = geo.direct && (nrows & 3u) == 0u && (r0 & 3u) == 0u &&
                      (reinterpret_cast<uintptr_t>(f.y) & (4u * sizeof(T) - 1u)) == 0u;
    float y0[4] = {0.f, 0.f, 0.f, 0.f};
    const bool pre = yvec && 4u * (uint32_t)tid < nrows;
    if (pre) {
        const uint2 raw = *reinterpret_cast<const uint2*>(y + r0 + 4u * tid);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) y0[i] = Tr<DT>::to_f(e[i]);
    }
    __syncthreads();
    if (*s_abort && tid == 0) raise_error(f.err, 1u);
    if (geo.direct) {
        if (!*s_abort) {            // an unfinished launch leaves y alone
            if (yvec) {
                for (uint32_t i = 4u * tid; i < nrows; i += 4u * NT) {
                    const float4 v = *reinterpret_cast<const float4*>(part + i);
                    float o[4];
                    if (pre && i == 4u * (uint32_t)tid) { o[0] = y0[0]; o[1] = y0[1]; o[2] = y0[2]; o[3] = y0[3]; }
                    else {
                        const uint2 raw = *reinterpret_cast<const uint2*>(y + r0 + i);
                        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
                        for (int q = 0; q < 4; ++q) o[q] = Tr<DT>::to_f(e[q]);
                    }
                    o[0] += v.x; o[1] += v.y; o[2] += v.z; o[3] += v.w;
                    uint2 raw;
                    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
                    for (int q = 0; q < 4; ++q) e[q] = Tr<DT>::from_f(o[q]);
                    *reinterpret_cast<uint2*>(y + r0 + i) = raw;
                }
            } else {
                for (uint32_t i = tid; i < nrows; i += NT)
                    y[r0 + i] = Tr<DT>::from_f(Tr<DT>::to_f(y[r0 + i]) + part[i]);
            }
        }
        return;
    }
    // fused launch: the sums go to the accumulator (this CTA is their only GEMV writer) and the CTA arrives on its
    // tile even after a failed wait, so that the workspace stays consistent
    for (uint32_t i = tid; i < nrows; i += NT) __stcg(f.acc + r0 + i, part[i]);
    arrive_and_finalize<DT>(f, cta, cta + 1, s_flag, NT);
}

}  // namespace dd
