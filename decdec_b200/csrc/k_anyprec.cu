// Any-precision launches (entry points `anyprec_gemv`, `dec_anyprec`, `anyprec_dequant`).
#include "internal.h"
#include "dec_role.cuh"

namespace dd {

template <int DT, bool FAST3>
__global__ void __launch_bounds__(kThreads)
k_anyprec(const __grid_constant__ ApParams g, const __grid_constant__ DecParams d, const __grid_constant__ FinParams f) {
    extern __shared__ __align__(16) unsigned char sm[];
    if (blockIdx.x < d.n_cta) dec_role<DT>(d, f, blockIdx.x, sm);
    else if constexpr (FAST3) ap3_role<DT>(g, f, blockIdx.x - d.n_cta, sm);
    else apg_role<DT>(g, f, blockIdx.x - d.n_cta, sm);
}

size_t anyprec_smem(uint32_t K, bool fast3) {
    const size_t xb = ((size_t)K * 2 + 15) & ~(size_t)15;
    return fast3 ? xb + 16 : xb + 8 * 256 * 2 + 16;
}

template <int DT, bool FAST3>
static cudaError_t go(const ApParams& g, const DecParams& d, const FinParams& f, cudaStream_t s) {
    size_t smem = anyprec_smem(g.K, FAST3);
    if (d.n_cta && smem < (size_t)DecSmem::kBytes) smem = DecSmem::kBytes;
    static size_t configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && dev < 64 && configured[dev] < smem) {
        cudaError_t e = cudaFuncSetAttribute(k_anyprec<DT, FAST3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured[dev] = smem;
    }
    k_anyprec<DT, FAST3><<<d.n_cta + g.n_cta, kThreads, smem, s>>>(g, d, f);
    return cudaGetLastError();
}

cudaError_t launch_anyprec(int dt, const ApParams& g, const DecParams& d, const FinParams& f, cudaStream_t s) {
    const bool fast3 = g.bits == 3 && (g.K % 128u) == 0u;
    if (dt == FP16) return fast3 ? go<FP16, true>(g, d, f, s) : go<FP16, false>(g, d, f, s);
    return fast3 ? go<BF16, true>(g, d, f, s) : go<BF16, false>(g, d, f, s);
}

cudaError_t launch_ap_dequant(int dt, const uint32_t* qweight, const void* lut, void* out, uint32_t N, uint32_t K,
                              uint32_t bits, cudaStream_t s) {
    const size_t total = (size_t)N * (K / 32);
    const int blocks = (int)((total + kThreads - 1) / kThreads < 148 * 16 ? (total + kThreads - 1) / kThreads : 148 * 16);
    if (blocks == 0) return cudaSuccess;
    if (dt == FP16) ap_dequant_kernel<FP16><<<blocks, kThreads, 0, s>>>(qweight, lut, out, N, K, bits);
    else ap_dequant_kernel<BF16><<<blocks, kThreads, 0, s>>>(qweight, lut, out, N, K, bits);
    return cudaGetLastError();
}

}  // namespace dd
