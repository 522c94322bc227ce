// decdec_lutgemm_gemv_noalloc: the binary-coded GEMV for callers that must not allocate.
//
// The ordinary entry points keep their fp32 accumulator and tile tickets in a workspace that the
// library obtains with cudaMalloc on first use of a (device, stream).  Some hosts cannot take that
// path: real-time loops that forbid calls which may synchronise the device or touch the driver's
// heap, and embedders whose device memory is handed out up front by their own arena and who
// therefore ban cudaMalloc in plug-ins.
// For them this file carries the same scratch as a fixed array inside the library image.  The
// array exists once per GPU that loads the library, for the life of the process, whether or not
// this entry point is ever called; that is why it is kept modest (kMaxN outputs).
//
// Rules that follow from sharing one array:
//  * every call clears the slice it is about to use (stream-ordered memsets), so a previous call
//    that was cut short cannot poison it;
//  * two calls that are in flight on the same GPU at the same time (different streams, or two
//    host threads) write the same scratch and corrupt each other - serialise them;
//  * the first call on a device looks up the array's device address (cudaGetSymbolAddress); make
//    that first call before starting any stream capture.
#include "internal.h"
#include "../../include/decdec_b200.h"

#include <cstdio>
#include <mutex>

namespace {

using namespace dd;

constexpr uint32_t kMaxN = 32768;       // outputs per call
constexpr uint32_t kMaxTiles = 1024;    // output tiles per call
constexpr size_t kAccBytes = (size_t)kMaxN * sizeof(float);
constexpr size_t kTicketBytes = (size_t)(kMaxTiles + 4) * sizeof(unsigned);

// Scratch shared by all calls on a device: [fp32 accumulator][tile tickets][error word].
// In host code this name is only a handle for cudaGetSymbolAddress, never a pointer to pass on.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kAccBytes + kTicketBytes];

std::mutex g_mu;
unsigned char* g_addr[64] = {};   // device address of the array, per device ordinal

int scratch_for_current_device(unsigned char** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return set_last_error(DECDEC_E_CUDA, cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return set_last_error(DECDEC_E_UNSUPPORTED, "device ordinal out of range for the static scratch table");
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);     // address on the CURRENT device
        if (e != cudaSuccess || !p) {
            char msg[160];
            snprintf(msg, sizeof(msg), "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
            return set_last_error(DECDEC_E_CUDA, msg);
        }
        g_addr[dev] = static_cast<unsigned char*>(p);
    }
    *out = g_addr[dev];
    return 0;
}

uint32_t cdiv(uint32_t a, uint32_t b) { return (a + b - 1) / b; }

}  // namespace

extern "C" int decdec_lutgemm_gemv_noalloc(const void* x, void* y, const int32_t* qw, const void* alpha, const void* q_bias,
                                           uint32_t N, uint32_t K, int bits, int group, int dtype, void* stream) {
    if (!x || !y || !qw || !alpha || !q_bias) return set_last_error(DECDEC_E_INVALID, "null pointer argument");
    if (dtype != FP32 && dtype != FP16 && dtype != BF16) return set_last_error(DECDEC_E_INVALID, "Unsupported data type.");
    if (bits < 1 || bits > 8) return set_last_error(DECDEC_E_INVALID, "Bitwidth must be between 1 and 8.");
    if (N == 0 || K == 0 || K % 32u || N % 8u) return set_last_error(DECDEC_E_INVALID, "need in_features % 32 == 0 and out_features % 8 == 0");
    if (group <= 0 || group % 32 || K % (uint32_t)group) return set_last_error(DECDEC_E_INVALID, "group_size must be a multiple of 32 that divides in_features");
    if ((reinterpret_cast<uintptr_t>(qw) | reinterpret_cast<uintptr_t>(alpha) | reinterpret_cast<uintptr_t>(q_bias)) & 15u)
        return set_last_error(DECDEC_E_INVALID, "lutgemm: q_weight/alpha/q_bias must be 16-byte aligned");
    if (N > kMaxN) {
        char msg[160];
        snprintf(msg, sizeof(msg), "decdec_lutgemm_gemv_noalloc: out_features %u exceeds the static scratch limit of %u outputs", N, kMaxN);
        return set_last_error(DECDEC_E_UNSUPPORTED, msg);
    }
    unsigned char* scratch = nullptr;
    if (int r = scratch_for_current_device(&scratch)) return r;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);

    BcqParams g;
    g.qweight = reinterpret_cast<const uint32_t*>(qw);
    g.alpha = alpha;
    g.q_bias = q_bias;
    g.x = x;
    g.K = K; g.N = N; g.bits = (uint32_t)bits; g.group = (uint32_t)group;
    g.n_kslices = cdiv(K, kBcqSlice);
    PipeGeom geo;
    const bool pipe = bcq_pipe_geometry(N, K, g.bits, g.group, dtype, g.n_kslices, &geo, device_sms());
    uint32_t tile_units;
    if (pipe) {
        tile_units = geo.tile_stages * (kPipeStageN / 32);
    } else {
        uint32_t tiles_target = 296 / g.n_kslices;
        if (tiles_target == 0) tiles_target = 1;
        tile_units = cdiv(cdiv(cdiv(N, 32), tiles_target), 8) * 8;
    }
    FinParams f;
    f.acc = reinterpret_cast<float*>(scratch);
    f.tickets = reinterpret_cast<unsigned*>(scratch + kAccBytes);
    f.err = f.tickets + kMaxTiles;
    f.acc2 = nullptr;       // no compensation role on this path
    f.scales = nullptr;
    f.y = y;
    f.N = N;
    f.tile_units = tile_units;
    f.n_tiles = cdiv(cdiv(N, 32), tile_units);
    f.expected = g.n_kslices;
    if (f.n_tiles > kMaxTiles) return set_last_error(DECDEC_E_UNSUPPORTED, "too many output tiles for the static scratch");
    g.n_cta = f.expected * f.n_tiles;
    DecParams d = {};

    // the array keeps whatever the last call left: clear what this call needs to start at zero
    cudaError_t e = cudaMemsetAsync(f.acc, 0, (size_t)N * sizeof(float), s);
    if (e == cudaSuccess) e = cudaMemsetAsync(f.tickets, 0, (size_t)(f.n_tiles) * sizeof(unsigned), s);
    if (e == cudaSuccess) e = cudaMemsetAsync(f.err, 0, sizeof(unsigned), s);
    if (e == cudaSuccess) e = pipe ? launch_bcq_pipe(dtype, g, d, f, geo, s) : launch_bcq(dtype, g, d, f, s);
    if (e != cudaSuccess) return set_last_error(DECDEC_E_CUDA, cudaGetErrorString(e));
    return 0;
}
