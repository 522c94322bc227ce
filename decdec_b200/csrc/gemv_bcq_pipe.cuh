// Binary-coded (LUT-GEMM) GEMV role, TMA-pipelined variant for the common shapes.
//
// Same arithmetic and table trick as gemv_bcq.cuh (signed-subset-sum tables of the activations,
// byte-permute addressing, bank-conflict-free lane layout), but the weight stream no longer passes
// through registers: a producer thread moves a tile of [16 k-rows x bits planes] x 128 outputs (+ the
// alpha and q_bias rows that go with them) per stage from HBM to shared memory with three tiled TMA
// copies (cp.async.bulk.tensor.2d, completion counted on an mbarrier), several stages ahead of the
// consumer warps (three groups of eight, taking stages round-robin).  HBM latency is then covered by
// bytes in flight (about 29 KB per stage, up to 5 stages per SM) instead of by occupancy.  The tile
// lands densely (512-byte lines); the lanes of a warp read it in a skewed order (k-row j reads the
// 16-byte groups (j + c) mod 8 and +4), so every 128-bit shared load of a quarter warp touches eight
// different bank groups.
//
// Split of the work.  The K dimension is cut into 512-channel slices (one 64 KB table block each); a CTA is
// (K slice, output tile) and the CTAs of a tile are neighbours in the grid.  After every stage a lane adds its
// 32-channel-row total into the fp32 accumulator of the workspace (red.global, fire and forget).  How a tile is
// finished depends on the launch:
//  * GEMV-only launches: the accumulator holds one 64-bit word per output = {fixed-point sum (48 bits, 2^-20),
//    arrivals that were not finite (8 bits), arrivals (8 bits; two per CTA, one per k half)}.  A lane adds its partial sum and one arrival with
//    ONE atomic; the lane whose atomic returns the last arrival count holds the complete sum, writes y (single
//    rounding) and clears the word.  No fence, no ticket, no second pass over the accumulator; integer addition
//    also makes the result independent of the arrival order.  The atomic's result is only looked at after the
//    next stage has been computed, so its round trip is hidden except for the last stage.
//  * fused launches (compensation CTAs in the same grid, which finish late): every CTA takes a ticket and the last
//    arriver folds (common.cuh), so no CTA spins while the host link is busy.
// Measured dead ends for this split: a designated finalizer per tile that polls a counter (no faster than tickets),
// and thread-block clusters with a reduction through distributed shared memory: only 15 clusters of 8 CTAs with this shared-memory footprint are resident at once (120 of 148 SMs),
// cluster placement delays the early start that programmatic dependent launch gives, and walking several K slices
// per CTA costs about 1.5 us per table rebuild.
//
// Requirements (otherwise the register-staged kernel of gemv_bcq.cuh runs): N % 128 == 0,
// K % 512 == 0, group size one of 32..512 dividing 512, at least two stages fit in shared memory.
// Every wait (mbarrier, tile counter) is bounded; on expiry the CTA raises the error word of the workspace, still
// takes part in the counter / ticket protocol (so that the workspace stays consistent) and the caller reads the
// error through decdec_stream_status.
#pragma once
#include "common.cuh"
#include "gemv_bcq.cuh"
#include <cuda.h>
#include "dec_role.cuh"

namespace dd {

constexpr int kPipeStageN = 128;            // outputs per stage
constexpr int kPipeLine = 512;              // bytes of one [k-row, plane] line of a stage (128 outputs)
constexpr int kPipeGroups = 3;              // consumer groups of 8 warps, taking stages round-robin
constexpr int kPipeThreads = kPipeGroups * 256 + 32;   // + 1 producer warp
constexpr uint32_t kPipeSuspendNs = 20000u;      // a poll may sleep this long in hardware (wakes early on completion)

struct PipeGeom {
    uint32_t stages;         // pipeline depth S
    uint32_t stage_bytes;    // bytes of one stage in shared memory
    uint32_t w_bytes;        // weight part of a stage
    uint32_t a_bytes;        // alpha part of a stage
    uint32_t tile_stages;    // stages (128 outputs each) per output tile
    uint32_t smem_bytes;     // dynamic shared memory of the launch
    uint32_t packed;         // 1: sums and arrival counts travel in one 64-bit atomic per output (no tickets)
    uint32_t arrivals;       // packed: arrivals that complete an output = 2 per K slice + 1 per compensation row part
    uint32_t wait_ns;        // limit of one bounded wait (DECDEC_PIPE_WAIT_NS)
    uint32_t test_skip_last; // test hook: the producer withholds its last stage, so that a wait runs out
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(kPipeSuspendNs) : "memory");
    return ok != 0;
}
// bounded wait: false if the barrier did not flip within about `limit_ns` or another thread of the CTA gave up.
// The bound is kept on the SM's own cycle counter (cheap to read; two cycles per nanosecond at the top clock).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    const long long limit = 2ll * (long long)limit_ns;
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > limit) break;
    }
    *abort_flag = 1u;
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void tma_2d_g2s(uint32_t dst, const CUtensorMap* map, uint32_t x, uint32_t y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

struct PipeMaps {
    CUtensorMap w;      // qweight as 2-D uint32 [K/32 * bits, N], box [16 * bits, 128]
    CUtensorMap a;      // alpha   as 2-D       [K/group * bits, N], box [512/group * bits, 128]
    CUtensorMap b;      // q_bias  as 2-D       [K/group, N], box [512/group, 128]
};

template <int DT>
__device__ __forceinline__ void lds4f(const unsigned char* base, uint32_t elem, float* o) {
    if constexpr (DT == FP32) {
        const float4 v = *reinterpret_cast<const float4*>(base + elem * 4);
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    } else if constexpr (DT == FP16) {
        const uint2 v = *reinterpret_cast<const uint2*>(base + elem * 2);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
        o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
    } else {
        const uint2 v = *reinterpret_cast<const uint2*>(base + elem * 2);
        o[0] = __uint_as_float(v.x << 16); o[1] = __uint_as_float(v.x & 0xffff0000u);
        o[2] = __uint_as_float(v.y << 16); o[3] = __uint_as_float(v.y & 0xffff0000u);
    }
}

// Shared memory.  The 64 KB of tables start at the first shared-window address that is a multiple of
// 64 KB, so that a lookup address {entry byte, slot offset} is complete after ONE byte-permute (bits
// 16.. of the address come from two constant bytes); the pipeline stages fill the space before and after:
//   [header 256 B: row sums, flags, 8 full + 8 empty barriers][stages ...][tables @ 64 KB multiple][stages ...]
constexpr int kPipeHdr = 256;
constexpr uint32_t kPipeTblOffAssumed = 65536 - 1024;   // dynamic shared memory normally starts 1 KB into the window

// stages that fit before the tables when these start `tbl_off` bytes into dynamic shared memory
__host__ __device__ inline uint32_t pipe_stages_before(uint32_t tbl_off, uint32_t stage_bytes) {
    return tbl_off > (uint32_t)kPipeHdr ? (tbl_off - kPipeHdr) / stage_bytes : 0u;
}

// activations of one (k-row, byte) table slot: 8 consecutive channels
template <int DT>
__device__ __forceinline__ void pipe_load_x8(const void* xbase, uint32_t k0, bool vec, float* xv) {
    using T = typename Tr<DT>::T;
    const T* x = reinterpret_cast<const T*>(xbase);
    if (vec) {
        if constexpr (DT == FP32) {
            const float4 a = *reinterpret_cast<const float4*>(x + k0);
            const float4 b = *reinterpret_cast<const float4*>(x + k0 + 4);
            xv[0] = a.x; xv[1] = a.y; xv[2] = a.z; xv[3] = a.w; xv[4] = b.x; xv[5] = b.y; xv[6] = b.z; xv[7] = b.w;
        } else {
            const uint4 raw = *reinterpret_cast<const uint4*>(x + k0);
            const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int i = 0; i < 8; ++i) xv[i] = Tr<DT>::to_f(e[i]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) xv[i] = Tr<DT>::to_f(x[k0 + i]);
    }
}

template <int DT, int BITS>
__device__ void bcq_pipe_role(const BcqParams& p, const FinParams& f, const PipeGeom& geo, const PipeMaps& maps,
                              uint32_t cta, unsigned char* sm) {
    using T = typename Tr<DT>::T;
    constexpr uint32_t ESZ = (DT == FP32) ? 4u : 2u;
    constexpr uint32_t NCONS = kPipeGroups * 256;
    const uint32_t sm_base = smem_u32(sm);
    const uint32_t tbl_off = (65536u - (sm_base & 65535u)) & 65535u;     // tables at a 64 KB multiple of the window
    float* tbl = reinterpret_cast<float*>(sm + tbl_off);
    float* rowsum = reinterpret_cast<float*>(sm);
    volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(sm + 64);
    unsigned* s_flag = reinterpret_cast<unsigned*>(sm + 64 + 4);
    const uint32_t bar_full = smem_u32(sm + 80);
    const uint32_t bar_empty = bar_full + 64;
    const uint32_t n_before = pipe_stages_before(tbl_off, geo.stage_bytes);
    auto stage_ptr = [&](uint32_t s) -> unsigned char* {
        return s < n_before ? sm + kPipeHdr + (size_t)s * geo.stage_bytes
                            : sm + tbl_off + kBcqTableBytes + (size_t)(s - n_before) * geo.stage_bytes;
    };

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_trigger();
    const uint32_t ks = cta % p.n_kslices;
    const uint32_t tile = cta / p.n_kslices;
    const uint32_t kbase = ks * kBcqSlice;
    const uint32_t nst_total = p.N / kPipeStageN;
    const uint32_t st0 = tile * geo.tile_stages;
    const uint32_t nst = min(geo.tile_stages, nst_total - st0);
    const uint32_t S = geo.stages;
    const uint32_t groups = kBcqSlice / p.group;        // scale groups inside the K slice

    if (tid == 0) {
        // the host sized the launch for the usual window offset; never run past the allocation
        uint32_t dyn;
        asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
        const uint32_t after = S > n_before ? S - n_before : 0u;
        const bool bad = tbl_off + kBcqTableBytes + after * geo.stage_bytes > dyn || (tbl_off & 127u);
        *s_abort = bad ? 2u : 0u;
        for (uint32_t s = 0; s < S; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 8);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kPipeGroups * 8) {
        // ------------------------------ producer warp (one elected lane) -------------------------
        if (lane == 0 && !*s_abort) {
            const uint32_t tx = geo.w_bytes + geo.a_bytes + groups * kPipeStageN * ESZ;
            const uint32_t n_issue = (geo.test_skip_last && nst) ? nst - 1u : nst;
            uint32_t issued = 0;
            tma_prefetch_desc(&maps.w);
            tma_prefetch_desc(&maps.a);
            tma_prefetch_desc(&maps.b);
            for (uint32_t i = 0; i < n_issue; ++i) {
                const uint32_t s = i % S, use = i / S;
                if (use > 0) {
                    // A slot frees only after the consumers have passed their own wait for the previous kernel, which
                    // may itself be waiting for another GPU: the bounded wait must not run during that time.  Every
                    // slot is full at this point, so waiting for the dependency here delays no copy.
                    if (use == 1 && s == 0) pdl_wait();
                    if (!mbar_wait(bar_empty + 8 * s, (use - 1) & 1u, s_abort, geo.wait_ns)) break;
                }
                const uint32_t full = bar_full + 8 * s;
                mbar_expect_tx(full, tx);
                const uint32_t n0 = (st0 + i) * kPipeStageN;
                const uint32_t dst = smem_u32(stage_ptr(s));
                tma_2d_g2s(dst, &maps.w, n0, (kbase / 32) * BITS, full);
                tma_2d_g2s(dst + geo.w_bytes, &maps.a, n0, (kbase / p.group) * BITS, full);
                tma_2d_g2s(dst + geo.w_bytes + geo.a_bytes, &maps.b, n0, kbase / p.group, full);
                issued = i + 1;
            }
            if (*s_abort) {
                // drain: never leave the CTA with copies still landing in shared memory
                const uint32_t first = issued > S ? issued - S : 0;
                for (uint32_t i = first; i < issued; ++i) {
                    volatile uint32_t never = 0;
                    mbar_wait(bar_full + 8 * (i % S), (i / S) & 1u, &never, 1000000000u);
                }
            }
        }
        pdl_wait();
    } else {
        // ------------------------------ consumer warps (3 groups of 8) ---------------------------
        // Everything that does not depend on memory is prepared before the wait for the previous kernel.
        // table slot = (krow / 8) * 32 + (krow % 8) * 4 + byte; a building thread fills the 32 entries whose
        // bits 5..7 equal warp / 2, for its slot
        const bool builder = warp < 16;
        const uint32_t slot = (warp & 1) * 32 + lane;
        const uint32_t qe = warp >> 1;
        const uint32_t krow_b = (slot >> 5) * 8 + ((slot & 31) >> 2);
        const uint32_t koff = 32 * krow_b + 8 * (slot & 3);
        const bool xvec = (reinterpret_cast<uintptr_t>(p.x) & 15u) == 0u;
        // main loop: warp = (k half, 32-output block); lane = (k-row j, c).  Row j reads the 16-byte groups
        // tA = (j + c) & 7 and tB = tA ^ 4 of the block's 128-byte line segment.
        const uint32_t j = lane & 7, c = lane >> 3;
        const uint32_t grp = warp >> 3;
        const uint32_t blk = warp & 3, khalf = (warp >> 2) & 1;
        const uint32_t krow = khalf * 8 + j;
        const uint32_t tA = (j + c) & 7, tB = tA ^ 4;
        uint32_t sel[4], lb[4];
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            const uint32_t byte = (s + c) & 3;
            sel[s] = 0x6504u | (byte << 4);                // result bytes = {lb.b0, word.byte[byte], lb.b1, lb.b2}
            // b0 = slot offset inside a 256-byte entry row, b1 and b2 = bits 16..31 of the tables' window address
            lb[s] = (khalf * 128 + (4 * j + byte) * 4) | (((smem_u32(tbl) >> 16) & 0xffffu) << 8);
        }
        const uint32_t g = (32 * krow) / p.group;          // scale group of this lane's k-row inside the slice
        const uint32_t nA = blk * 32 + 4 * tA, nB = blk * 32 + 4 * tB;
        // partner lanes of the reduction over k-rows (lanes sharing (j + c) & 3 hold the same two groups)
        const uint32_t p4 = lane ^ 4, p2 = lane ^ 18;
        const uint32_t p1 = (j ^ 1) + 8 * (((j & 1) ? c + 1 : c + 3) & 3);
        const bool swapAB = (tA & 4) != 0;                  // after the swap X = group r, Y = group r + 4, r = tA & 3
        const uint32_t r4 = tA & 3;
        const uint32_t n_out = blk * 32 + ((j & 4) ? 16 : 0) + 4 * r4 + (j & 3);
        float* acc_lane = f.acc + (size_t)st0 * kPipeStageN + n_out;
        bool pending = false;
        unsigned long long p_old = 0, p_mine = 0;
        unsigned long long* p_word = nullptr;
        T* p_y = nullptr;
        float p_y0 = 0.0f;

        pdl_wait();     // weights are already streaming (producer warp); activations come from earlier kernels
        if (builder && !*s_abort) {
            float xv[8];
            pipe_load_x8<DT>(p.x, kbase + koff, xvec, xv);
            float lo[8], hi[4];
#pragma unroll
            for (int e = 0; e < 8; ++e)
                lo[e] = ((e & 1) ? xv[0] : -xv[0]) + ((e & 2) ? xv[1] : -xv[1]) + ((e & 4) ? xv[2] : -xv[2]);
#pragma unroll
            for (int e = 0; e < 4; ++e) hi[e] = ((e & 1) ? xv[3] : -xv[3]) + ((e & 2) ? xv[4] : -xv[4]);
            const float top = ((qe & 1) ? xv[5] : -xv[5]) + ((qe & 2) ? xv[6] : -xv[6]) + ((qe & 4) ? xv[7] : -xv[7]);
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                const float th = top + hi[h];
#pragma unroll
                for (int l = 0; l < 8; ++l) tbl[(qe * 32 + h * 8 + l) * 64 + slot] = th + lo[l];
            }
            // sum of the 32 activations of a k-row (for the q_bias term): four byte slots side by side
            float rs = ((xv[0] + xv[1]) + (xv[2] + xv[3])) + ((xv[4] + xv[5]) + (xv[6] + xv[7]));
            rs += __shfl_xor_sync(0xffffffffu, rs, 1);
            rs += __shfl_xor_sync(0xffffffffu, rs, 2);
            if (qe == 0 && (lane & 3) == 0) rowsum[krow_b] = rs;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(NCONS) : "memory");
        const float sx = rowsum[krow];

        for (uint32_t i = grp; i < nst && !*s_abort; i += kPipeGroups) {
            const uint32_t s = i % S;
            if (!mbar_wait(bar_full + 8 * s, (i / S) & 1u, s_abort, geo.wait_ns)) break;
            const unsigned char* st = stage_ptr(s);
            const unsigned char* wl = st + krow * (BITS * kPipeLine);
            const unsigned char* al = st + geo.w_bytes + (g * BITS) * (kPipeStageN * ESZ);
            const unsigned char* bl = st + geo.w_bytes + geo.a_bytes + g * (kPipeStageN * ESZ);
            float y8[8];
            lds4f<DT>(bl, nA, y8);
            lds4f<DT>(bl, nB, y8 + 4);
#pragma unroll
            for (int q = 0; q < 8; ++q) y8[q] *= sx;
#pragma unroll
            for (int pl = 0; pl < BITS; ++pl) {
                const uint4 wA = *reinterpret_cast<const uint4*>(wl + pl * kPipeLine + nA * 4);
                const uint4 wB = *reinterpret_cast<const uint4*>(wl + pl * kPipeLine + nB * 4);
                float a8[8];
                lds4f<DT>(al + pl * (kPipeStageN * ESZ), nA, a8);
                lds4f<DT>(al + pl * (kPipeStageN * ESZ), nB, a8 + 4);
                const uint32_t wq[8] = {wA.x, wA.y, wA.z, wA.w, wB.x, wB.y, wB.z, wB.w};
                float v[32];
#pragma unroll
                for (int q = 0; q < 8; ++q)
#pragma unroll
                    for (int ss = 0; ss < 4; ++ss) v[q * 4 + ss] = lds_f32(__byte_perm(wq[q], lb[ss], sel[ss]));
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    y8[q] = fmaf(a8[q], (v[q * 4] + v[q * 4 + 1]) + (v[q * 4 + 2] + v[q * 4 + 3]), y8[q]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * s);      // all shared reads of the stage are done
            // X = values of group r, Y = values of group r + 4; reduce over the 8 k-row lanes, halving
            float y4[4], y2[2], y1;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float X = swapAB ? y8[q + 4] : y8[q];
                const float Y = swapAB ? y8[q] : y8[q + 4];
                const float send = (j & 4) ? X : Y;
                const float keep = (j & 4) ? Y : X;
                y4[q] = keep + __shfl_sync(0xffffffffu, send, p4);
            }
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const float send = (j & 2) ? y4[q] : y4[q + 2];
                const float keep = (j & 2) ? y4[q + 2] : y4[q];
                y2[q] = keep + __shfl_sync(0xffffffffu, send, p2);
            }
            {
                const float send = (j & 1) ? y2[0] : y2[1];
                const float keep = (j & 1) ? y2[1] : y2[0];
                y1 = keep + __shfl_sync(0xffffffffu, send, p1);
            }
            if (!geo.packed) {
                atomicAdd(acc_lane + i * kPipeStageN, y1);
            } else {
                // the previous stage's atomic has long returned: settle it, then send this stage's
                if (pending) finish_packed<DT>(p_old, p_mine, geo.arrivals, p_word, p_y, p_y0);
                const uint32_t n = (st0 + i) * kPipeStageN + n_out;
                p_word = reinterpret_cast<unsigned long long*>(f.acc) + n;
                p_y = reinterpret_cast<T*>(f.y) + n;
                p_y0 = Tr<DT>::to_f(*p_y);
                p_mine = pack_partial(y1);
                p_old = atomicAdd(p_word, p_mine);
                pending = true;
            }
        }
        if (pending) finish_packed<DT>(p_old, p_mine, geo.arrivals, p_word, p_y, p_y0);
    }
    if (geo.packed) {
        // nothing to hand over: every output was settled by the lane that made its last arrival.  A wait that ran out
        // leaves the words of the unfinished outputs dirty (their y untouched) until decdec_stream_reset.
        __syncthreads();
        if (*s_abort && tid == 0) raise_error(f.err, *s_abort);
        return;
    }
    // Fused launch: whatever happened above, the CTA takes a ticket on its tile, so that accumulator and tickets are
    // clean for the next launch; a wait that ran out is reported through the error word.
    __syncthreads();
    if (*s_abort && tid == 0) raise_error(f.err, *s_abort);
    arrive_and_finalize<DT>(f, tile, tile + 1, s_flag, kPipeThreads);
}

}  // namespace dd
