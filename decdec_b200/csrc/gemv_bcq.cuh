// Binary-coded (LUT-GEMM) GEMV role:  y[n] += sum_g ( q_bias[g][n]*sum_{k in g} x[k]
//                                              + sum_p alpha[g][p][n] * sum_{k in g} (2*bit_p(k,n)-1) x[k] ).
//
// Replaces `nqmv_bias` of the reference (decdec_extension/lutgemm.cu:25-150), which gives one CTA a
// 32-channel K tile, lets all lanes of a warp index the same 256-entry table (bank conflicts) and
// merges K/32 partial sums per output with half atomics.  Here:
//  * a CTA owns a 512-channel K slice and a tile of outputs; it builds the 64 signed-subset-sum
//    tables of its slice once (fp32, 256 entries per 8 channels);
//  * tables are interleaved so that entry e of table slot s sits at byte e*256 + s*4: the byte
//    address of a lookup is ONE byte-permute of the weight word, and the 32 lanes of a warp always
//    hit 32 different banks (lane = (k-row j, output group c) walks the 4 bytes of its word in the
//    rotated order (s + c) mod 4);
//  * weight words are read with 16-byte loads, 64 contiguous bytes per k-row per instruction;
//  * partial sums stay in fp32 and reach the accumulator with one reduction per output per K slice.
#pragma once
#include "common.cuh"

namespace dd {

struct BcqParams {
    const uint32_t* qweight;   // [K/32, bits, N]
    const void* alpha;         // [K/group, bits, N]
    const void* q_bias;        // [K/group, N]
    const void* x;             // [K]
    uint32_t K, N, bits, group;
    uint32_t n_kslices;        // ceil(K / 512)
    uint32_t n_cta;            // n_kslices * n_tiles
};

constexpr int kBcqSlice = 512;                   // channels per K slice
constexpr int kBcqTableBytes = 256 * 64 * 4;     // 64 tables x 256 entries x fp32
constexpr int kBcqSmemBytes = kBcqTableBytes + 64 + 16;

template <int DT>
__device__ __forceinline__ void load4f(const void* base, size_t idx, float* o) {
    if constexpr (DT == FP32) {
        const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx);
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    } else if constexpr (DT == FP16) {
        const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(base) + idx);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
        o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
    } else {
        const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(base) + idx);
        o[0] = __uint_as_float(v.x << 16); o[1] = __uint_as_float(v.x & 0xffff0000u);
        o[2] = __uint_as_float(v.y << 16); o[3] = __uint_as_float(v.y & 0xffff0000u);
    }
}

// BITS > 0: plane loop fully unrolled; BITS == 0: runtime plane count (1..8).
template <int DT, int BITS>
__device__ void bcq_role(const BcqParams& p, const FinParams& f, uint32_t cta, unsigned char* sm) {
    using T = typename Tr<DT>::T;
    float* tbl = reinterpret_cast<float*>(sm);
    float* rowsum = reinterpret_cast<float*>(sm + kBcqTableBytes);       // [16] sum of x per 32-channel k-row
    unsigned* s_flag = reinterpret_cast<unsigned*>(sm + kBcqTableBytes + 64);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t ks = cta % p.n_kslices;
    const uint32_t tile = cta / p.n_kslices;
    const uint32_t kbase = ks * kBcqSlice;
    const T* x = reinterpret_cast<const T*>(p.x);
    const uint32_t nbits = BITS > 0 ? (uint32_t)BITS : p.bits;

    // ---- build the 64 subset-sum tables of this K slice --------------------------------------
    // slot = it*32 + 4*j + byte  <->  k-row (2*j + it) of the slice, byte `byte` of its words.
    {
        const uint32_t slot = (warp & 1) * 32 + lane;
        const uint32_t qe = warp >> 1;   // entries [64*qe, 64*qe + 64)
        const uint32_t krow = 2 * ((slot & 31) >> 2) + (slot >> 5);
        const uint32_t k0 = kbase + 32 * krow + 8 * (slot & 3);
        float xv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) xv[i] = (k0 + i < p.K) ? Tr<DT>::to_f(x[k0 + i]) : 0.0f;
        float lo[8], hi[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            lo[e] = ((e & 1) ? xv[0] : -xv[0]) + ((e & 2) ? xv[1] : -xv[1]) + ((e & 4) ? xv[2] : -xv[2]);
            hi[e] = ((e & 1) ? xv[3] : -xv[3]) + ((e & 2) ? xv[4] : -xv[4]) + ((e & 4) ? xv[5] : -xv[5]);
        }
        const float top = ((qe & 1) ? xv[6] : -xv[6]) + ((qe & 2) ? xv[7] : -xv[7]);
#pragma unroll
        for (int h = 0; h < 8; ++h) {
            const float th = top + hi[h];
#pragma unroll
            for (int l = 0; l < 8; ++l) tbl[(qe * 64 + h * 8 + l) * 64 + slot] = th + lo[l];
        }
    }
    __syncthreads();
    if (tid < 16) {
        const uint32_t base = (tid & 1) * 32 + (tid >> 1) * 4;
        rowsum[tid] = tbl[255 * 64 + base] + tbl[255 * 64 + base + 1] + tbl[255 * 64 + base + 2] + tbl[255 * 64 + base + 3];
    }
    __syncthreads();

    // ---- stream the weights -------------------------------------------------------------------
    const uint32_t j = lane & 7, c = lane >> 3;
    uint32_t sel[4], lb[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        const uint32_t byte = (s + c) & 3;
        sel[s] = 0x6504u | (byte << 4);        // result = {lb.byte0, word.byte[byte], 0, 0}
        lb[s] = (4 * j + byte) * 4;            // low part of the slot's byte offset (< 128)
    }
    const unsigned char* tb = reinterpret_cast<const unsigned char*>(tbl);
    const uint32_t nwordrows = p.K / 32;
    const uint32_t u0 = tile * f.tile_units;
    const uint32_t u1 = min(u0 + f.tile_units, (p.N + 31) / 32);
    const bool merge = (p.group % 64u) == 0u;   // both k-rows of a lane lie in one scale group

    for (uint32_t u = u0 + warp; u < u1; u += 8) {
        const uint32_t nA = u * 32 + 4 * c, nB = nA + 16;
        const bool vA = nA < p.N, vB = nB < p.N;
        float y8[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) y8[q] = 0.0f;

#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const uint32_t krow = 2 * j + it;
            const uint32_t kw = kbase / 32 + krow;
            if (kw >= nwordrows) continue;
            const uint32_t g = (kw * 32) / p.group;
            const uint32_t* wrow = p.qweight + (size_t)kw * nbits * p.N;
            const uint32_t tbi_s = (uint32_t)__cvta_generic_to_shared(tb) + it * 128;
            auto plane = [&](uint32_t pl, uint4 wa, uint4 wb) {
                float al[8];
                const size_t ai = ((size_t)g * nbits + pl) * p.N;
                if (vA) load4f<DT>(p.alpha, ai + nA, al); else { al[0] = al[1] = al[2] = al[3] = 0.f; }
                if (vB) load4f<DT>(p.alpha, ai + nB, al + 4); else { al[4] = al[5] = al[6] = al[7] = 0.f; }
                const uint32_t w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    float a = 0.0f;
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
                        const uint32_t addr = __byte_perm(w[q], lb[s], sel[s]);
                        a += lds_f32(tbi_s + addr);
                    }
                    y8[q] = fmaf(al[q], a, y8[q]);
                }
            };
            if constexpr (BITS > 0) {
                uint4 wa[BITS], wb[BITS];
#pragma unroll
                for (int pl = 0; pl < BITS; ++pl) {
                    wa[pl] = vA ? __ldg(reinterpret_cast<const uint4*>(wrow + (size_t)pl * p.N + nA)) : make_uint4(0, 0, 0, 0);
                    wb[pl] = vB ? __ldg(reinterpret_cast<const uint4*>(wrow + (size_t)pl * p.N + nB)) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int pl = 0; pl < BITS; ++pl) plane(pl, wa[pl], wb[pl]);
            } else {
                for (uint32_t pl = 0; pl < nbits; ++pl) {
                    const uint4 wa = vA ? __ldg(reinterpret_cast<const uint4*>(wrow + (size_t)pl * p.N + nA)) : make_uint4(0, 0, 0, 0);
                    const uint4 wb = vB ? __ldg(reinterpret_cast<const uint4*>(wrow + (size_t)pl * p.N + nB)) : make_uint4(0, 0, 0, 0);
                    plane(pl, wa, wb);
                }
            }
            // q_bias term: once per lane when both k-rows share the group, else per k-row
            float sx;
            bool do_bias;
            if (merge) {
                do_bias = (it == 0);
                sx = rowsum[2 * j] + ((kw + 1 < nwordrows) ? rowsum[2 * j + 1] : 0.0f);
            } else {
                do_bias = true;
                sx = rowsum[krow];
            }
            if (do_bias) {
                float bq[8];
                const size_t bi = (size_t)g * p.N;
                if (vA) load4f<DT>(p.q_bias, bi + nA, bq); else { bq[0] = bq[1] = bq[2] = bq[3] = 0.f; }
                if (vB) load4f<DT>(p.q_bias, bi + nB, bq + 4); else { bq[4] = bq[5] = bq[6] = bq[7] = 0.f; }
#pragma unroll
                for (int q = 0; q < 8; ++q) y8[q] = fmaf(bq[q], sx, y8[q]);
            }
        }

        // reduce over the 8 k-row lanes (lane bits 0..2); lane j ends with the total of value q = j
        float y4[4], y2[2], y1;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float send = (j & 4) ? y8[i] : y8[i + 4];
            const float keep = (j & 4) ? y8[i + 4] : y8[i];
            y4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float send = (j & 2) ? y4[i] : y4[i + 2];
            const float keep = (j & 2) ? y4[i + 2] : y4[i];
            y2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
        }
        {
            const float send = (j & 1) ? y2[0] : y2[1];
            const float keep = (j & 1) ? y2[1] : y2[0];
            y1 = keep + __shfl_xor_sync(0xffffffffu, send, 1);
        }
        const uint32_t n = (j < 4) ? (nA + j) : (nB + j - 4);
        if (n < p.N) atomicAdd(&f.acc[n], y1);
    }
    arrive_and_finalize<DT>(f, tile, tile + 1, s_flag);
}

// ---- dequantizer: binary-coded planes -> dense [K, N] (the operand of the prefill GEMM) -----------------
// W[k][n] = DT( DT( sum_p (2*bit_p(k,n) - 1) * alpha[g][p][n] ) + q_bias[g][n] ): the same two roundings as the
// reference's tensor expression (end-to-end/LUTGEMMLinear.py:41-82: plane sum in the layer dtype, then + q_bias).
// Thread = (word row kw, output pair): reads the planes' words of two neighbouring outputs, writes 32 rows of
// 2 x DT (4 or 8 bytes), so a warp writes 128-256 contiguous bytes per row.  Needs N % 2 == 0.
template <int DT>
__global__ void __launch_bounds__(kThreads) bcq_dequant_kernel(const uint32_t* __restrict__ qweight, const void* __restrict__ alpha_,
                                                              const void* __restrict__ qbias_, void* __restrict__ out_, uint32_t N,
                                                              uint32_t K, uint32_t bits, uint32_t group) {
    using T = typename Tr<DT>::T;
    const T* alpha = reinterpret_cast<const T*>(alpha_);
    const T* qbias = reinterpret_cast<const T*>(qbias_);
    T* out = reinterpret_cast<T*>(out_);
    const uint32_t npair = N / 2;
    const size_t total = (size_t)(K / 32) * npair;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const uint32_t kw = (uint32_t)(idx / npair), n = 2u * (uint32_t)(idx % npair);
        const uint32_t g = (kw * 32u) / group;
        uint2 w[8];
        float a0[8], a1[8];
        for (uint32_t pl = 0; pl < bits; ++pl) {
            w[pl] = *reinterpret_cast<const uint2*>(qweight + ((size_t)kw * bits + pl) * N + n);
            a0[pl] = Tr<DT>::to_f(alpha[((size_t)g * bits + pl) * N + n]);
            a1[pl] = Tr<DT>::to_f(alpha[((size_t)g * bits + pl) * N + n + 1]);
        }
        const T b0 = qbias[(size_t)g * N + n], b1 = qbias[(size_t)g * N + n + 1];
        for (uint32_t j = 0; j < 32; ++j) {
            float s0 = 0.0f, s1 = 0.0f;
            for (uint32_t pl = 0; pl < bits; ++pl) {
                s0 += ((w[pl].x >> j) & 1u) ? a0[pl] : -a0[pl];
                s1 += ((w[pl].y >> j) & 1u) ? a1[pl] : -a1[pl];
            }
            T o[2];
            if constexpr (DT == FP32) {
                o[0] = s0 + b0; o[1] = s1 + b1;
            } else {
                o[0] = Tr<DT>::add(Tr<DT>::from_f(s0), b0);
                o[1] = Tr<DT>::add(Tr<DT>::from_f(s1), b1);
            }
            T* dst = out + (size_t)(kw * 32u + j) * N + n;
            dst[0] = o[0]; dst[1] = o[1];
        }
    }
}

}  // namespace dd
