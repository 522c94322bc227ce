// SqueezeLLM (dense-packed codes, per-output-column LUT) GEMV role.
//
// Replaces `VecQuant3MatMulKernelNUQPerChannel` / `VecQuant4MatMulKernelNUQPerChannel` of the
// reference (decdec_extension/sqllm.cu:28-116, :119-169).  Layout (given by the caller):
// qweight[K*bits/32][N]; 4-bit: word r holds channels 8r..8r+7 at bit 4i; 3-bit: three consecutive
// word rows hold 32 channels as a 96-bit little-endian string of 3-bit codes.
//
// A CTA owns 32 output columns for the whole of K: lane = column (128-byte coalesced word rows),
// warp = K slice.  The column LUTs sit in shared memory as fp32 [code][column], so lane l always hits
// bank l.  Sums are fp32; the eight K slices are combined in shared memory, so no cross-CTA
// reduction is needed.
#pragma once
#include "common.cuh"

namespace dd {

struct SqParams {
    const uint32_t* qweight;   // [K*bits/32, N]
    const void* lut;           // [N, 2^bits]
    const void* x;             // [K]
    uint32_t K, N, bits;
    uint32_t n_cta;            // ceil(N / 32)
    uint32_t direct;
};

template <int DT>
__device__ void sq_role(const SqParams& p, const FinParams& f, uint32_t cta, unsigned char* sm) {
    using T = typename Tr<DT>::T;
    float* sx = reinterpret_cast<float*>(sm);                                   // [K] fp32
    const uint32_t xbytes = (p.K * 4 + 15) & ~15u;
    float* slut = reinterpret_cast<float*>(sm + xbytes);                        // [16][32]
    float* part = slut + 16 * 32;                                               // [8][32]
    unsigned* s_flag = reinterpret_cast<unsigned*>(part + 8 * 32);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const T* x = reinterpret_cast<const T*>(p.x);
    const T* lut = reinterpret_cast<const T*>(p.lut);
    for (uint32_t k = tid; k < p.K; k += kThreads) sx[k] = Tr<DT>::to_f(x[k]);
    const uint32_t n = cta * 32 + lane;
    const bool nv = n < p.N;
    const uint32_t ncent = 1u << p.bits;
    for (uint32_t e = warp; e < ncent; e += 8) slut[e * 32 + lane] = nv ? Tr<DT>::to_f(lut[(size_t)n * ncent + e]) : 0.0f;
    __syncthreads();

    float acc = 0.0f;
    const uint32_t ngroups = p.K / 32;                 // 32-channel groups
    const uint32_t g0 = (uint32_t)(((uint64_t)warp * ngroups) / 8), g1 = (uint32_t)(((uint64_t)(warp + 1) * ngroups) / 8);
    const uint32_t* col = p.qweight + n;
    // Word rows are fetched for several 32-channel groups at once (all loads before the first use): a warp
    // then has 1.5-2 KB in flight instead of 384-512 bytes, which is what hides the DRAM latency here.
    constexpr uint32_t GB = 4;                         // groups per batch
    const unsigned char* lbase = reinterpret_cast<const unsigned char*>(slut + lane);   // + code * 128
    auto lut_at = [&](uint32_t byte_off) { return *reinterpret_cast<const float*>(lbase + byte_off); };
    if (p.bits == 4) {
        auto consume = [&](const uint32_t* w, const float* xg) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 xa = *reinterpret_cast<const float4*>(xg + 8 * i);
                const float4 xb = *reinterpret_cast<const float4*>(xg + 8 * i + 4);
                const float xs[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    // code * 128 taken straight out of the word: bits [4c, 4c+4) moved to bit 7
                    const uint32_t off = (4 * c >= 7 ? (w[i] >> (4 * c - 7)) : (w[i] << (7 - 4 * c))) & 0x780u;
                    acc = fmaf(lut_at(off), xs[c], acc);
                }
            }
        };
        uint32_t g = g0;
        for (; g + GB <= g1; g += GB) {
            uint32_t w[GB][4];
#pragma unroll
            for (uint32_t b = 0; b < GB; ++b)
#pragma unroll
                for (int i = 0; i < 4; ++i) w[b][i] = nv ? ldg_stream(col + (size_t)(4 * (g + b) + i) * p.N) : 0u;
#pragma unroll
            for (uint32_t b = 0; b < GB; ++b) consume(w[b], sx + 32 * (g + b));
        }
        for (; g < g1; ++g) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) w[i] = nv ? ldg_stream(col + (size_t)(4 * g + i) * p.N) : 0u;
            consume(w, sx + 32 * g);
        }
    } else {
        auto consume = [&](uint32_t w0, uint32_t w1, uint32_t w2, const float* xg) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float4 xv = *reinterpret_cast<const float4*>(xg + 4 * q);
                const float xs[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int c = 4 * q + j, bit = 3 * c;          // code c sits at bits [3c, 3c+3) of the 96-bit string
                    // 32-bit window that starts at `bit` (funnel shift over the word pair that holds it)
                    uint32_t v;
                    if (bit < 32) v = __funnelshift_r(w0, w1, bit);
                    else if (bit < 64) v = __funnelshift_r(w1, w2, bit - 32);
                    else v = w2 >> (bit - 64);
                    acc = fmaf(lut_at((v & 7u) << 7), xs[j], acc);
                }
            }
        };
        uint32_t g = g0;
        for (; g + GB <= g1; g += GB) {
            uint32_t w[GB][3];
#pragma unroll
            for (uint32_t b = 0; b < GB; ++b)
#pragma unroll
                for (int i = 0; i < 3; ++i) w[b][i] = nv ? ldg_stream(col + (size_t)(3 * (g + b) + i) * p.N) : 0u;
#pragma unroll
            for (uint32_t b = 0; b < GB; ++b) consume(w[b][0], w[b][1], w[b][2], sx + 32 * (g + b));
        }
        for (; g < g1; ++g) {
            const uint32_t w0 = nv ? ldg_stream(col + (size_t)(3 * g) * p.N) : 0u;
            const uint32_t w1 = nv ? ldg_stream(col + (size_t)(3 * g + 1) * p.N) : 0u;
            const uint32_t w2 = nv ? ldg_stream(col + (size_t)(3 * g + 2) * p.N) : 0u;
            consume(w0, w1, w2, sx + 32 * g);
        }
    }
    part[warp * 32 + lane] = acc;
    __syncthreads();
    if (warp == 0) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) v += part[w * 32 + lane];
        if (nv) {
            if (p.direct) {
                T* y = reinterpret_cast<T*>(f.y);
                y[n] = Tr<DT>::from_f(Tr<DT>::to_f(y[n]) + v);
            } else {
                atomicAdd(&f.acc[n], v);
            }
        }
    }
    if (!p.direct) arrive_and_finalize<DT>(f, cta, cta + 1, s_flag);   // launched with one 32-column unit per tile
}

}  // namespace dd
