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

template <int DT, int BITS, bool LOOKUP>
__global__ void __launch_bounds__(kApPipeThreads, 1)
k_anyprec_pipe(const __grid_constant__ ApParams g, const __grid_constant__ DecParams d, const __grid_constant__ FinParams f,
               const __grid_constant__ ApPipeGeom geo) {
    extern __shared__ __align__(128) unsigned char sm[];
    if (blockIdx.x < d.n_cta) dec_role<DT>(d, f, blockIdx.x, sm);
    else ap_pipe_role<DT, BITS, LOOKUP>(g, f, geo, blockIdx.x - d.n_cta, sm);
}

// Which decoder a 3-bit launch takes: the register-table one unless DECDEC_AP3_DECODER=lookup.
static bool ap_lookup_decoder(uint32_t bits) {
    if (bits != 3) return true;
    const char* v = getenv("DECDEC_AP3_DECODER");
    return v && *v == 'l';
}

// Stage geometry of the pipelined kernel (3 to 8 bits); false if the shape is not eligible.  A CTA's rows are a whole
// number of 32-output finalizer tiles when a compensation role may share the launch; a GEMV-only launch (no config)
// has no finalizer and cuts the rows in multiples of 16, which fills the SMs more evenly (6144 rows: 128 CTAs of 48
// instead of 96 of 64).
bool anyprec_pipe_geometry(uint32_t N, uint32_t K, uint32_t bits, ApPipeGeom* geo, uint32_t sm_budget, bool gemv_only) {
    if (bits < 3 || bits > 8 || K % 128u || K > 32768u || N == 0) return false;
    const bool lookup = ap_lookup_decoder(bits);
    const uint32_t rowbytes = K / 8;
    const uint32_t per_row = bits * rowbytes + (2u << bits);      // plane words and the LUT row
    geo->segs = (K + 4095) / 4096;
    uint32_t R = 16 / geo->segs;
    if (R == 0) return false;
    while (R & (R - 1)) R &= R - 1;                      // largest power of two <= 16 / segs
    geo->lookup = lookup ? 1u : 0u;
    geo->x_bytes = (K * 2 + 127u) & ~127u;
    if (sm_budget == 0) sm_budget = 1;
    uint32_t rows = (N + sm_budget - 1) / sm_budget;
    const uint32_t gran = gemv_only ? 16u : 32u;
    rows = ((rows + gran - 1) / gran) * gran;
    geo->rows_per_cta = rows;
    geo->part_bytes = (rows * 4u + 127u) & ~127u;
    const uint32_t fixed = kApPipeHdr + geo->x_bytes + geo->part_bytes;
    if (fixed >= 227u * 1024u) return false;
    const uint32_t budget = 227 * 1024 - fixed;
    // wide rows: fewer rows per stage until two stages fit (some consumer warps then have no work item)
    while (R > 1 && 2u * ((R * per_row + 127u) & ~127u) > budget) R >>= 1;
    geo->rows_per_stage = R;
    geo->stage_bytes = (R * per_row + 127u) & ~127u;
    uint32_t smax = budget / geo->stage_bytes;
    if (smax > 8) smax = 8;
    if (smax < 2) return false;
    const uint32_t nst = rows / R;
    geo->stages = nst < smax ? nst : smax;
    geo->smem_bytes = fixed + geo->stages * geo->stage_bytes;
    geo->direct = 0;        // set by the caller
    {
        const char* w = getenv("DECDEC_PIPE_WAIT_NS");
        geo->wait_ns = (w && *w) ? (uint32_t)strtoul(w, nullptr, 10) : 50u * 1000u * 1000u;
    }
    if (geo->smem_bytes < (uint32_t)DecSmem::kBytes) geo->smem_bytes = DecSmem::kBytes;
    return true;
}

template <int DT, int BITS, bool LOOKUP>
static cudaError_t go_pipe(const ApParams& g, const DecParams& d, const FinParams& f, const ApPipeGeom& geo, cudaStream_t s) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_anyprec_pipe<DT, BITS, LOOKUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
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
    return cudaLaunchKernelEx(&cfg, k_anyprec_pipe<DT, BITS, LOOKUP>, g, d, f, geo);
}

template <int DT>
static cudaError_t pipe_by_bits(const ApParams& g, const DecParams& d, const FinParams& f, const ApPipeGeom& geo, cudaStream_t s) {
    switch (g.bits) {
        case 3: return geo.lookup ? go_pipe<DT, 3, true>(g, d, f, geo, s) : go_pipe<DT, 3, false>(g, d, f, geo, s);
        case 4: return go_pipe<DT, 4, true>(g, d, f, geo, s);
        case 5: return go_pipe<DT, 5, true>(g, d, f, geo, s);
        case 6: return go_pipe<DT, 6, true>(g, d, f, geo, s);
        case 7: return go_pipe<DT, 7, true>(g, d, f, geo, s);
        case 8: return go_pipe<DT, 8, true>(g, d, f, geo, s);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_anyprec_pipe(int dt, const ApParams& g, const DecParams& d, const FinParams& f, const ApPipeGeom& geo, cudaStream_t s) {
    return dt == FP16 ? pipe_by_bits<FP16>(g, d, f, geo, s) : pipe_by_bits<BF16>(g, d, f, geo, s);
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
