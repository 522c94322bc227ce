// Binary-coded GEMV launches (entry points `lutgemm_gemv`, `dec_lutgemm`).
#include "internal.h"
#include <cstdlib>
#include "dec_role.cuh"
#include "gemv_bcq_pipe.cuh"

namespace dd {

template <int DT, int BITS>
__global__ void __launch_bounds__(kThreads, 2)
k_bcq(const __grid_constant__ BcqParams g, const __grid_constant__ DecParams d, const __grid_constant__ FinParams f) {
    extern __shared__ __align__(128) unsigned char sm[];
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

template <int DT, int BITS>
__global__ void __launch_bounds__(kPipeThreads, 1)
k_bcq_pipe(const __grid_constant__ BcqParams g, const __grid_constant__ DecParams d, const __grid_constant__ FinParams f,
           const __grid_constant__ PipeGeom geo, const __grid_constant__ PipeMaps maps) {
    extern __shared__ __align__(128) unsigned char sm[];
    if (blockIdx.x < d.n_cta) {
        if (geo.packed) dec_role_packed<DT>(d, f, blockIdx.x, sm, geo.arrivals);
        else dec_role<DT>(d, f, blockIdx.x, sm);
    } else {
        bcq_pipe_role<DT, BITS>(g, f, geo, maps, blockIdx.x - d.n_cta, sm);
    }
}

// DECDEC_PDL: 0 = never, 1 = launches without a compensation role, 2 (default) = every launch
static int pdl_mode() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("DECDEC_PDL"); v = (e && *e >= '0' && *e <= '2') ? (*e - '0') : 2; }
    return v;
}

template <int DT, int BITS>
static cudaError_t go_pipe(const BcqParams& g, const DecParams& d, const FinParams& f, const PipeGeom& geo, const PipeMaps& maps,
                           cudaStream_t s) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_bcq_pipe<DT, BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    // programmatic dependent launch: CTAs may become resident (and prefetch weights) while the previous
    // kernel of the stream drains; the kernel waits for it before touching activations or outputs
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(d.n_cta + g.n_cta);
    cfg.blockDim = dim3(kPipeThreads);
    cfg.dynamicSmemBytes = geo.smem_bytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = (pdl_mode() == 2 || (pdl_mode() == 1 && d.n_cta == 0)) ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, k_bcq_pipe<DT, BITS>, g, d, f, geo, maps);
}

template <int DT>
static cudaError_t pipe_by_bits(const BcqParams& g, const DecParams& d, const FinParams& f, const PipeGeom& geo,
                                const PipeMaps& maps, cudaStream_t s) {
    switch (g.bits) {
        case 2: return go_pipe<DT, 2>(g, d, f, geo, maps, s);
        case 3: return go_pipe<DT, 3>(g, d, f, geo, maps, s);
        default: return go_pipe<DT, 4>(g, d, f, geo, maps, s);
    }
}

// cuTensorMapEncodeTiled is fetched from the driver at run time (no link-time dependency on libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

static bool encode_2d(CUtensorMap* m, const void* base, int dt_bytes, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * (uint64_t)dt_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapDataType t = dt_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16;
    return fn(m, t, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

cudaError_t launch_bcq_pipe(int dt, const BcqParams& g, const DecParams& d, const FinParams& f, const PipeGeom& geo, cudaStream_t s) {
    PipeMaps maps;
    const int esz = dt == FP32 ? 4 : 2;
    const uint32_t groups = kBcqSlice / g.group;
    if (!encode_2d(&maps.w, g.qweight, 4, (uint64_t)(g.K / 32) * g.bits, g.N, 16 * g.bits, kPipeStageN) ||
        !encode_2d(&maps.a, g.alpha, esz, (uint64_t)(g.K / g.group) * g.bits, g.N, groups * g.bits, kPipeStageN) ||
        !encode_2d(&maps.b, g.q_bias, esz, (uint64_t)(g.K / g.group), g.N, groups, kPipeStageN))
        return cudaErrorInvalidValue;
    switch (dt) {
        case FP32: return pipe_by_bits<FP32>(g, d, f, geo, maps, s);
        case FP16: return pipe_by_bits<FP16>(g, d, f, geo, maps, s);
        default: return pipe_by_bits<BF16>(g, d, f, geo, maps, s);
    }
}

static uint32_t env_u32_k(const char* name, uint32_t dflt) {
    const char* v = getenv(name);
    return (v && *v) ? (uint32_t)strtoul(v, nullptr, 10) : dflt;
}

// Stage geometry of the pipelined kernel; returns false if the shape is not eligible.
// sm_budget = SMs the GEMV CTAs may fill in one wave.
bool bcq_pipe_geometry(uint32_t N, uint32_t K, uint32_t bits, uint32_t group, int dt, uint32_t n_kslices, PipeGeom* geo,
                       uint32_t sm_budget) {
    if (N % kPipeStageN || K % kBcqSlice || bits < 2 || bits > 4) return false;
    if (group < 32 || group > (uint32_t)kBcqSlice || kBcqSlice % group) return false;
    // the table block sits at the first 64 KB multiple of the shared window; dynamic shared memory starts right
    // after the bytes the system reserves per CTA (this kernel has no static shared memory)
    int dev = 0, reserved = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&reserved, cudaDevAttrReservedSharedMemoryPerBlock, dev) != cudaSuccess) { cudaGetLastError(); return false; }
    if ((uint32_t)reserved != 65536u - kPipeTblOffAssumed) return false;
    const uint32_t esz = dt == FP32 ? 4 : 2;
    const uint32_t groups = kBcqSlice / group;
    geo->w_bytes = 16 * bits * kPipeLine;
    geo->a_bytes = groups * bits * kPipeStageN * esz;
    geo->stage_bytes = (geo->w_bytes + geo->a_bytes + groups * kPipeStageN * esz + 127u) & ~127u;
    // stages sit before and after the 64 KB table block (see gemv_bcq_pipe.cuh)
    const uint32_t n_before = pipe_stages_before(kPipeTblOffAssumed, geo->stage_bytes);
    const uint32_t room_after = 227 * 1024 - (kPipeTblOffAssumed + kBcqTableBytes);
    uint32_t smax = n_before + room_after / geo->stage_bytes;
    if (smax > 8) smax = 8;
    if (smax < 2) return false;
    const uint32_t nst_total = N / kPipeStageN;
    // one CTA per SM; tiles sized so that the grid is at most one wave
    uint32_t per1 = sm_budget / n_kslices; if (per1 == 0) per1 = 1;
    geo->tile_stages = (nst_total + per1 - 1) / per1;
    geo->stages = geo->tile_stages < smax ? geo->tile_stages : smax;
    const uint32_t after = geo->stages > n_before ? geo->stages - n_before : 0;
    geo->smem_bytes = kPipeTblOffAssumed + kBcqTableBytes + after * geo->stage_bytes;
    if (geo->smem_bytes < (uint32_t)DecSmem::kBytes) geo->smem_bytes = DecSmem::kBytes;
    geo->packed = 0;                // set by the caller
    geo->arrivals = 0;
    geo->wait_ns = env_u32_k("DECDEC_PIPE_WAIT_NS", 50u * 1000u * 1000u);
    geo->test_skip_last = env_u32_k("DECDEC_TEST_WITHHOLD_STAGE", 0) ? 1u : 0u;
    return true;
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

cudaError_t launch_bcq_dequant(int dt, const uint32_t* qweight, const void* alpha, const void* q_bias, void* out, uint32_t N,
                               uint32_t K, uint32_t bits, uint32_t group, cudaStream_t s) {
    const size_t total = (size_t)(K / 32) * (N / 2);
    const size_t want = (total + kThreads - 1) / kThreads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (blocks == 0) return cudaSuccess;
    switch (dt) {
        case FP32: bcq_dequant_kernel<FP32><<<blocks, kThreads, 0, s>>>(qweight, alpha, q_bias, out, N, K, bits, group); break;
        case FP16: bcq_dequant_kernel<FP16><<<blocks, kThreads, 0, s>>>(qweight, alpha, q_bias, out, N, K, bits, group); break;
        default: bcq_dequant_kernel<BF16><<<blocks, kThreads, 0, s>>>(qweight, alpha, q_bias, out, N, K, bits, group); break;
    }
    return cudaGetLastError();
}

}  // namespace dd
