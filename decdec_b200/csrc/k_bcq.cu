// Binary-coded GEMV launches (entry points `lutgemm_gemv`, `dec_lutgemm`).
#include "internal.h"
#include "dec_role.cuh"

namespace dd {

template <int DT, int BITS>
__global__ void __launch_bounds__(kThreads, 2)
k_bcq(const __grid_constant__ BcqParams g, const __grid_constant__ DecParams d, const __grid_constant__ FinParams f) {
    extern __shared__ __align__(16) unsigned char sm[];
    if (blockIdx.x < d.n_cta) dec_role<DT>(d, f, blockIdx.x, sm);
    else bcq_role<DT, BITS>(g, f, blockIdx.x - d.n_cta, sm);
}

template <int DT, int BITS>
static cudaError_t go(const BcqParams& g, const DecParams& d, const FinParams& f, cudaStream_t s) {
    const size_t smem = kBcqSmemBytes > DecSmem::kBytes ? kBcqSmemBytes : DecSmem::kBytes;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_bcq<DT, BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    k_bcq<DT, BITS><<<d.n_cta + g.n_cta, kThreads, smem, s>>>(g, d, f);
    return cudaGetLastError();
}

template <int DT>
static cudaError_t by_bits(const BcqParams& g, const DecParams& d, const FinParams& f, cudaStream_t s) {
    switch (g.bits) {
        case 3: return go<DT, 3>(g, d, f, s);
        case 4: return go<DT, 4>(g, d, f, s);
        default: return go<DT, 0>(g, d, f, s);
    }
}

cudaError_t launch_bcq(int dt, const BcqParams& g, const DecParams& d, const FinParams& f, cudaStream_t s) {
    switch (dt) {
        case FP32: return by_bits<FP32>(g, d, f, s);
        case FP16: return by_bits<FP16>(g, d, f, s);
        default: return by_bits<BF16>(g, d, f, s);
    }
}

}  // namespace dd
