// Any-precision launches (entry points `anyprec_gemv`, `dec_anyprec`, `anyprec_dequant`).
#include "internal.h"
#include <cstdlib>
#include "dec_role.cuh"
#include "gemv_anyprec_pipe.cuh"

namespace dd {

template <int DT, bool FAST3>
__global__ void __launch_bounds__(kThreads)
k_anyprec(const __grid_constant__ ApParams g, const __grid_constant__ DecParams d, const __grid_constant__ FinParams f) {
    extern __shared__ __align__(128) unsigned char sm[];
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

template <int DT>
__global__ void __launch_bounds__(kApPipeThreads, 1)
k_anyprec_pipe(const __grid_constant__ ApParams g, const __grid_constant__ DecParams d, const __grid_constant__ FinParams f,
               const __grid_constant__ ApPipeGeom geo) {
    extern __shared__ __align__(128) unsigned char sm[];
    if (blockIdx.x < d.n_cta) dec_role<DT>(d, f, blockIdx.x, sm);
    else ap3_pipe_role<DT>(g, f, geo, blockIdx.x - d.n_cta, sm);
}

// Stage geometry of the pipelined 3-bit kernel; false if the shape is not eligible.
bool anyprec_pipe_geometry(uint32_t N, uint32_t K, uint32_t bits, ApPipeGeom* geo, uint32_t sm_budget) {
    if (bits != 3 || K % 128u || K > 32768u || N == 0) return false;
    const uint32_t rowbytes = K / 8;
    geo->segs = (K + 4095) / 4096;
    uint32_t R = 16 / geo->segs;
    if (R == 0) return false;
    while (R & (R - 1)) R &= R - 1;                      // largest power of two <= 16 / segs
    geo->rows_per_stage = R;
    geo->x_bytes = (K * 2 + 127u) & ~127u;
    geo->stage_bytes = (R * (3 * rowbytes + 16) + 127u) & ~127u;
    if (sm_budget == 0) sm_budget = 1;
    uint32_t rows = (N + sm_budget - 1) / sm_budget;
    rows = ((rows + 31) / 32) * 32;
    geo->rows_per_cta = rows;
    geo->part_bytes = (rows * 4u + 127u) & ~127u;
    if (kApPipeHdr + geo->x_bytes + geo->part_bytes + 2u * geo->stage_bytes > 227u * 1024u) return false;
    const uint32_t budget = 227 * 1024 - kApPipeHdr - geo->x_bytes - geo->part_bytes;
    uint32_t smax = budget / geo->stage_bytes;
    if (smax > 8) smax = 8;
    if (smax < 2) return false;
    const uint32_t nst = rows / R;
    geo->stages = nst < smax ? nst : smax;
    geo->smem_bytes = kApPipeHdr + geo->x_bytes + geo->part_bytes + geo->stages * geo->stage_bytes;
    geo->direct = 0;        // set by the caller
    {
        const char* w = getenv("DECDEC_PIPE_WAIT_NS");
        geo->wait_ns = (w && *w) ? (uint32_t)strtoul(w, nullptr, 10) : 50u * 1000u * 1000u;
    }
    if (geo->smem_bytes < (uint32_t)DecSmem::kBytes) geo->smem_bytes = DecSmem::kBytes;
    return true;
}

cudaError_t launch_anyprec_pipe(int dt, const ApParams& g, const DecParams& d, const FinParams& f, const ApPipeGeom& geo, cudaStream_t s) {
    static bool configured[64][2] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const int di = dt == FP16 ? 0 : 1;
    if (dev < 64 && !configured[dev][di]) {
        cudaError_t e = dt == FP16
            ? cudaFuncSetAttribute(k_anyprec_pipe<FP16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024)
            : cudaFuncSetAttribute(k_anyprec_pipe<BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        configured[dev][di] = true;
    }
    // programmatic dependent launch: thread blocks may become resident (and prefetch weights) while the
    // previous kernel of the stream drains; the kernel waits for it before touching activations or outputs
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(d.n_cta + g.n_cta);
    cfg.blockDim = dim3(kApPipeThreads);
    cfg.dynamicSmemBytes = geo.smem_bytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    const char* e = getenv("DECDEC_PDL");
    attr[0].val.programmaticStreamSerializationAllowed = (e && *e == '0') ? 0 : 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (dt == FP16) return cudaLaunchKernelEx(&cfg, k_anyprec_pipe<FP16>, g, d, f, geo);
    return cudaLaunchKernelEx(&cfg, k_anyprec_pipe<BF16>, g, d, f, geo);
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
