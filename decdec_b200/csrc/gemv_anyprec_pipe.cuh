// Any-precision 3-bit GEMV role, bulk-copy pipelined variant.
//
// Arithmetic of gemv_anyprec.cuh:ap3_role (register-resident byte tables, byte-permute lookups,
// activations staged in pair order), fed differently: in the tensor [plane][row][K/32] consecutive
// rows of one plane are contiguous, so a stage of R rows is three contiguous runs (one per plane) plus
// the R LUT rows.  A producer thread moves them with four 1-D bulk asynchronous copies
// (cp.async.bulk, 6-8 KB each, completion counted on an mbarrier) several stages ahead of sixteen
// consumer warps; a warp's work item is (row of the stage, 4096-channel segment of that row).
// A CTA owns its rows completely (all of K), so the row sums meet in a small shared-memory buffer and the
// CTA folds them into y itself: GEMV-only launches use no global accumulator, ticket or fence.  Fused
// launches store the sums into the workspace accumulator and arrive on the tile's ticket, where they meet
// the compensation CTAs.
// Requirements: bits == 3, K % 128 == 0, K <= 32768.  Every mbarrier wait is bounded.
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
    uint32_t x_bytes;          // staged activations (rounded to 128)
    uint32_t rows_per_cta;     // multiple of R
    uint32_t part_bytes;       // row sums of the CTA (fp32, rounded to 128 bytes)
    uint32_t smem_bytes;
    uint32_t direct;           // 1: fold into y; 0: store into the accumulator and take the tile's ticket
    uint32_t wait_ns;          // limit of one mbarrier wait (DECDEC_PIPE_WAIT_NS)
};

constexpr int kApPipeHdr = 256;   // [abort, flag][full barriers 8][empty barriers 8]

template <int DT>
__device__ void ap3_pipe_role(const ApParams& p, const FinParams& f, const ApPipeGeom& geo, uint32_t cta, unsigned char* sm) {
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
    const uint32_t lut_off = 3 * R * rowbytes;          // LUT rows sit after the three plane runs

    pdl_trigger();
    if (tid == 0) {
        *s_abort = 0u;
        for (uint32_t s = 0; s < S; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 16);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (uint32_t i = tid; i < geo.rows_per_cta; i += kApPipeThreads) part[i] = 0.0f;
    __syncthreads();

    if (warp == 16) {
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
                mbar_expect_tx(full, rows * (3 * rowbytes + 16));
                const uint32_t dst = smem_u32(stage0 + (size_t)s * geo.stage_bytes);
#pragma unroll
                for (int pl = 0; pl < 3; ++pl)
                    bulk_g2s(dst + pl * R * rowbytes, p.qweight + pl * plane_stride + (size_t)n0 * nwords, rows * rowbytes, full);
                bulk_g2s(dst + lut_off, lutb + (size_t)n0 * 16, rows * 16, full);
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
    } else {
        // ------------------------------ consumers ----------------------------------------------
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
    if (warp == 16) pdl_wait();     // the producer warp touches the accumulator and y only from here on
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
                for (uint32_t i = 4u * tid; i < nrows; i += 4u * kApPipeThreads) {
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
                for (uint32_t i = tid; i < nrows; i += kApPipeThreads)
                    y[r0 + i] = Tr<DT>::from_f(Tr<DT>::to_f(y[r0 + i]) + part[i]);
            }
        }
        return;
    }
    // fused launch: the sums go to the accumulator (this CTA is their only GEMV writer) and the CTA arrives on its
    // tile even after a failed wait, so that the workspace stays consistent
    for (uint32_t i = tid; i < nrows; i += kApPipeThreads) __stcg(f.acc + r0 + i, part[i]);
    arrive_and_finalize<DT>(f, cta, cta + 1, s_flag, kApPipeThreads);
}

}  // namespace dd
