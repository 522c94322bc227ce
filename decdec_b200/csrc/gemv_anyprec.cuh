// Any-precision (bit-plane, per-output-row LUT) GEMV role and dequantizer.
//
// Replaces `matmul_kbit_32<1,bits,...>` and `dequant_kbit_store` of the reference
// (decdec_extension/anyprec.cu:344-514, :261-331).  Tensor layout (given by the caller):
// qweight[plane][n][K/32]; a row is cut into blocks of 32 words (tail block: E = (K mod 1024)/32
// words); bit 31-8j-r of word t of a block holds channel block_start + 8*E*j + 8*t + r; plane 0 is
// the most significant code bit.
//
// 3-bit fast path: one warp per output row, coalesced loads of four plane words per lane; the 8-entry
// fp16 LUT of the row lives in four registers split into a low-byte and a high-byte table, codes are
// turned into byte-permute selectors (three logic ops per 8 codes) and each permute looks up four
// table bytes at once - no shared-memory LUT, hence no bank conflicts.  Activations are staged in
// shared memory once per CTA in the pair order the lookups produce.  Products are summed in half2
// over 8 weights, then in fp32.
// Generic path (any width, any K multiple of 32): one word per lane, LUT in shared memory.
// Both roles of this file are the fallback for shapes the pipelined kernel (gemv_anyprec_pipe.cuh) does not take
// (K not a multiple of 128 or above 32768, or the pipeline switched off); common layers run there.
#pragma once
#include "common.cuh"

namespace dd {

struct ApParams {
    const uint32_t* qweight;   // [planes, N, K/32]
    const void* lut;           // [N, 2^bits]
    const void* x;             // [K]
    uint32_t K, N, bits;
    uint32_t n_cta;            // = n_tiles
    uint32_t direct;           // 1: no other role adds to y in this launch -> write y directly
};

// position of channel r (0..7) inside its group of 8 in the staged activation vector:
// stored order [r7, r3, r6, r2, r5, r1, r4, r0]
__device__ __forceinline__ uint32_t ap_perm(uint32_t r) { return (r >= 4) ? 2 * (7 - r) : 2 * (3 - r) + 1; }

template <int DT>
__device__ __forceinline__ float ap_sum2(uint32_t h2) {
    if constexpr (DT == FP16) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
        return f.x + f.y;
    } else {
        return __uint_as_float(h2 << 16) + __uint_as_float(h2 & 0xffff0000u);
    }
}

// multiply-accumulate one half2/bf162 pair of weights with a pair of activations
template <int DT>
__device__ __forceinline__ void ap_fma(uint32_t w2, uint32_t x2, uint32_t& hacc, float& facc) {
    if constexpr (DT == FP16) {
        __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&w2), *reinterpret_cast<const __half2*>(&x2),
                            *reinterpret_cast<const __half2*>(&hacc));
        hacc = *reinterpret_cast<uint32_t*>(&r);
    } else {
        facc = fmaf(__uint_as_float(w2 << 16), __uint_as_float(x2 << 16), facc);
        facc = fmaf(__uint_as_float(w2 & 0xffff0000u), __uint_as_float(x2 & 0xffff0000u), facc);
    }
}

template <int DT>
__device__ __forceinline__ void ap_emit(const FinParams& f, uint32_t direct, uint32_t n, float v) {
    using T = typename Tr<DT>::T;
    if (direct) {
        T* y = reinterpret_cast<T*>(f.y);
        y[n] = Tr<DT>::from_f(Tr<DT>::to_f(y[n]) + v);
    } else {
        atomicAdd(&f.acc[n], v);
    }
}

// ---- 3-bit fast path ---------------------------------------------------------------------------
template <int DT>
__device__ void ap3_role(const ApParams& p, const FinParams& f, uint32_t cta, unsigned char* sm) {
    using T = typename Tr<DT>::T;
    static_assert(DT != FP32, "any-precision kernels take fp16/bf16 only");
    T* sx = reinterpret_cast<T*>(sm);
    unsigned* s_flag = reinterpret_cast<unsigned*>(sm + ((p.K * 2 + 15) & ~15u));
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const T* x = reinterpret_cast<const T*>(p.x);
    for (uint32_t k = tid; k < p.K; k += kThreads) sx[(k & ~7u) | ap_perm(k & 7u)] = x[k];
    __syncthreads();

    const uint32_t nwords = p.K / 32;
    const uint32_t tailE = nwords & 31u;
    const uint32_t nfull = nwords >> 5;
    const uint32_t r0 = cta * f.tile_units * 32u;
    const uint32_t r1 = min(p.N, r0 + f.tile_units * 32u);
    const size_t plane_stride = (size_t)p.N * nwords;
    const uint4* lutv = reinterpret_cast<const uint4*>(p.lut);

    for (uint32_t n = r0 + warp; n < r1; n += 8) {
        const uint4 L = __ldg(lutv + n);
        const uint32_t lo01 = __byte_perm(L.x, L.y, 0x6420), lo23 = __byte_perm(L.z, L.w, 0x6420);
        const uint32_t hi01 = __byte_perm(L.x, L.y, 0x7531), hi23 = __byte_perm(L.z, L.w, 0x7531);
        const uint32_t* row = p.qweight + (size_t)n * nwords;
        float facc = 0.0f;
        for (uint32_t wb = 0; wb < nwords; wb += 128) {
            // lane handles words wb + 32*u + lane: coalesced 128-byte loads per plane, and consecutive
            // lanes read consecutive 16-byte activation groups (no shared-memory bank conflicts)
            const uint32_t wi0 = wb + lane;
            if (wi0 >= nwords) continue;
            uint32_t aw[4], bw[4], cw[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const bool ok = wi0 + 32 * u < nwords;
                aw[u] = ok ? ldg_stream(row + wi0 + 32 * u) : 0u;
                bw[u] = ok ? ldg_stream(row + plane_stride + wi0 + 32 * u) : 0u;
                cw[u] = ok ? ldg_stream(row + 2 * plane_stride + wi0 + 32 * u) : 0u;
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
                    // nibbles 0,1 -> byte 0 of the word (j = 3); 2,3 -> j = 2; 4,5 -> j = 1; 6,7 -> j = 0
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
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) facc += __shfl_xor_sync(0xffffffffu, facc, d);
        if (lane == 0) ap_emit<DT>(f, p.direct, n, facc);
    }
    if (!p.direct) arrive_and_finalize<DT>(f, cta, cta + 1, s_flag);
}

// ---- generic path: any bit width 3..8, any K multiple of 32 -------------------------------------
template <int DT>
__device__ void apg_role(const ApParams& p, const FinParams& f, uint32_t cta, unsigned char* sm) {
    using T = typename Tr<DT>::T;
    T* sx = reinterpret_cast<T*>(sm);                                   // natural order
    const uint32_t xbytes = (p.K * 2 + 15) & ~15u;
    T* slut = reinterpret_cast<T*>(sm + xbytes);                        // [8 warps][256]
    unsigned* s_flag = reinterpret_cast<unsigned*>(sm + xbytes + 8 * 256 * 2);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const T* x = reinterpret_cast<const T*>(p.x);
    for (uint32_t k = tid; k < p.K; k += kThreads) sx[k] = x[k];
    __syncthreads();
    const uint32_t nwords = p.K / 32, nfull = nwords >> 5, tailE = nwords & 31u;
    const uint32_t ncent = 1u << p.bits;
    const uint32_t r0 = cta * f.tile_units * 32u;
    const uint32_t r1 = min(p.N, r0 + f.tile_units * 32u);
    const size_t plane_stride = (size_t)p.N * nwords;
    const T* lut = reinterpret_cast<const T*>(p.lut);
    T* wl = slut + warp * 256;
    for (uint32_t n = r0 + warp; n < r1; n += 8) {
        __syncwarp();
        for (uint32_t e = lane; e < ncent; e += 32) wl[e] = lut[(size_t)n * ncent + e];
        __syncwarp();
        const uint32_t* row = p.qweight + (size_t)n * nwords;
        float facc = 0.0f;
        for (uint32_t wi = lane; wi < nwords; wi += 32) {
            uint32_t q[8];
            for (uint32_t pl = 0; pl < p.bits; ++pl) q[pl] = ldg_stream(row + pl * plane_stride + wi);
            const uint32_t blk = wi >> 5, t = wi & 31u;
            const uint32_t E = (blk == nfull) ? tailE : 32u;
            const T* xb = sx + blk * 1024u + 8u * t;
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    const int bit = 31 - 8 * jj - r;
                    uint32_t code = 0;
                    for (uint32_t pl = 0; pl < p.bits; ++pl) code = (code << 1) | ((q[pl] >> bit) & 1u);
                    facc = fmaf(Tr<DT>::to_f(wl[code]), Tr<DT>::to_f(xb[8u * E * jj + r]), facc);
                }
            }
        }
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) facc += __shfl_xor_sync(0xffffffffu, facc, d);
        if (lane == 0) ap_emit<DT>(f, p.direct, n, facc);
    }
    if (!p.direct) arrive_and_finalize<DT>(f, cta, cta + 1, s_flag);
}

// ---- dequantizer: bit planes -> dense [N, K] ------------------------------------------------------
// One thread per (row, word): 32 codes, written as four 16-byte groups of 8 consecutive channels.
template <int DT>
__global__ void __launch_bounds__(kThreads) ap_dequant_kernel(const uint32_t* __restrict__ qweight, const void* __restrict__ lut_,
                                                             void* __restrict__ out_, uint32_t N, uint32_t K, uint32_t bits) {
    using T = typename Tr<DT>::T;
    const T* lut = reinterpret_cast<const T*>(lut_);
    T* out = reinterpret_cast<T*>(out_);
    const uint32_t nwords = K / 32, nfull = nwords >> 5, tailE = nwords & 31u;
    const size_t total = (size_t)N * nwords;
    const size_t plane_stride = total;
    const uint32_t ncent = 1u << bits;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const uint32_t n = (uint32_t)(idx / nwords), wi = (uint32_t)(idx % nwords);
        uint32_t q[8];
        for (uint32_t pl = 0; pl < bits; ++pl) q[pl] = qweight[pl * plane_stride + idx];
        const uint32_t blk = wi >> 5, t = wi & 31u;
        const uint32_t E = (blk == nfull) ? tailE : 32u;
        const T* l = lut + (size_t)n * ncent;
        T* o = out + (size_t)n * K + blk * 1024u + 8u * t;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            alignas(16) T v[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const int bit = 31 - 8 * jj - r;
                uint32_t code = 0;
                for (uint32_t pl = 0; pl < bits; ++pl) code = (code << 1) | ((q[pl] >> bit) & 1u);
                v[r] = l[code];
            }
            *reinterpret_cast<uint4*>(o + 8u * E * jj) = *reinterpret_cast<const uint4*>(v);
        }
    }
}

}  // namespace dd
