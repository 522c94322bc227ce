// SqueezeLLM launches (entry points `sqllm_gemv`, `dec_sqllm`).
#include "internal.h"
#include "dec_role.cuh"

namespace dd {

template <int DT>
__global__ void __launch_bounds__(kThreads, 3)
k_sqllm(const __grid_constant__ SqParams g, const __grid_constant__ DecParams d, const __grid_constant__ FinParams f) {
    extern __shared__ __align__(128) unsigned char sm[];
    if (blockIdx.x < d.n_cta) dec_role<DT>(d, f, blockIdx.x, sm);
    else sq_role<DT>(g, f, blockIdx.x - d.n_cta, sm);
}

size_t sqllm_smem(uint32_t K) { return (((size_t)K * 4 + 15) & ~(size_t)15) + (16 * 32 + 8 * 32) * 4 + 16; }

template <int DT>
static cudaError_t go(const SqParams& g, const DecParams& d, const FinParams& f, cudaStream_t s) {
    size_t smem = sqllm_smem(g.K);
    if (d.n_cta && smem < (size_t)DecSmem::kBytes) smem = DecSmem::kBytes;
    static size_t configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && dev < 64 && configured[dev] < smem) {
        cudaError_t e = cudaFuncSetAttribute(k_sqllm<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured[dev] = smem;
    }
    k_sqllm<DT><<<d.n_cta + g.n_cta, kThreads, smem, s>>>(g, d, f);
    return cudaGetLastError();
}

cudaError_t launch_sqllm(int dt, const SqParams& g, const DecParams& d, const FinParams& f, cudaStream_t s) {
    switch (dt) {
        case FP32: return go<FP32>(g, d, f, s);
        case FP16: return go<FP16>(g, d, f, s);
        default: return go<BF16>(g, d, f, s);
    }
}

}  // namespace dd
