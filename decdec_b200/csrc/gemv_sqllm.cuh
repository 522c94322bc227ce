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
    if (p.bits == 4) {
        for (uint32_t g = g0; g < g1; ++g) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) w[i] = nv ? ldg_stream(col + (size_t)(4 * g + i) * p.N) : 0u;
            const float* xg = sx + 32 * g;
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int c = 0; c < 8; ++c) acc = fmaf(slut[((w[i] >> (4 * c)) & 15u) * 32 + lane], xg[8 * i + c], acc);
        }
    } else {
        for (uint32_t g = g0; g < g1; ++g) {
            const uint32_t w0 = nv ? ldg_stream(col + (size_t)(3 * g) * p.N) : 0u;
            const uint32_t w1 = nv ? ldg_stream(col + (size_t)(3 * g + 1) * p.N) : 0u;
            const uint32_t w2 = nv ? ldg_stream(col + (size_t)(3 * g + 2) * p.N) : 0u;
            const unsigned long long lo = (unsigned long long)w0 | ((unsigned long long)w1 << 32);
            const float* xg = sx + 32 * g;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                uint32_t code;
                if (3 * c + 3 <= 64) code = (uint32_t)(lo >> (3 * c)) & 7u;
                else if (3 * c >= 64) code = (w2 >> (3 * c - 64)) & 7u;
                else code = ((uint32_t)(lo >> (3 * c)) | (w2 << (64 - 3 * c))) & 7u;
                acc = fmaf(slut[code * 32 + lane], xg[c], acc);
            }
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
