// Host side of the C ABI: handles (context / config), workspace management, argument checks,
// launch geometry.  Mirrors the host launchers of the reference (decdec_extension/decdec.cu,
// dec_config.cu, dec_context.cu) behind plain-C entry points; no torch types.
#include "internal.h"
#include "../../include/decdec_b200.h"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <vector>
#include <mutex>
#include <utility>

namespace dd {
uint32_t device_sms() {
    static uint32_t sms[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!sms[dev]) {
        int n = 0;
        sms[dev] = (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? (uint32_t)n : 148u;
    }
    return sms[dev];
}

}  // namespace dd

namespace {

using namespace dd;

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

#define DD_CUDA(call)                                                                                  \
    do {                                                                                               \
        cudaError_t e__ = (call);                                                                      \
        if (e__ != cudaSuccess) return fail(DECDEC_E_CUDA, "%s failed: %s", #call, cudaGetErrorString(e__)); \
    } while (0)

constexpr uint32_t kAccCap = 1u << 18;      // outputs per call supported by the accumulator
constexpr uint32_t kTicketCap = 1u << 13;

struct Workspace {
    float* acc = nullptr;
    unsigned* tickets = nullptr;
    unsigned* err = nullptr;          // device-visible address of the error word (mapped pinned host memory)
    volatile unsigned* err_host = nullptr;   // the same word as the host sees it: read before every launch, no copy needed
    float* acc2 = nullptr;            // second half of the accumulator allocation (compensation sums)
};

std::mutex g_mu;
std::map<std::pair<int, cudaStream_t>, Workspace> g_ws;
std::map<int, Workspace> g_ws_first;                       // first workspace of a device: capture fallback
std::map<int, std::vector<Workspace>> g_ws_spare;          // set aside for streams first seen while capturing
constexpr int kSpareWorkspaces = 16;
std::map<int, std::pair<cudaStream_t, std::pair<cudaEvent_t, cudaEvent_t>>> g_side;   // dummy_* side stream

// A launch that gave up on a wait left its code in the workspace's error word: every later call on that stream
// fails until decdec_stream_reset, instead of computing on top of an unfinished result.
int check_ws(const Workspace& w) {
    const unsigned code = w.err_host ? *w.err_host : 0u;
    if (code)
        return fail(DECDEC_E_DEVICE, "an earlier launch on this stream gave up waiting (device code %u); read it with "
                                     "decdec_stream_status and clear it with decdec_stream_reset", code);
    return 0;
}

// Allocates and clears one workspace (never called while a stream of the device is capturing).
static int alloc_workspace(Workspace* out) {
    Workspace w;
    if (cudaMalloc(&w.acc, 2 * kAccCap * sizeof(float)) != cudaSuccess) return fail(DECDEC_E_NOMEM, "cudaMalloc(accumulator) failed");
    if (cudaMalloc(&w.tickets, (kTicketCap + 4) * sizeof(unsigned)) != cudaSuccess) { cudaFree(w.acc); return fail(DECDEC_E_NOMEM, "cudaMalloc(tickets) failed"); }
    DD_CUDA(cudaMemset(w.acc, 0, 2 * kAccCap * sizeof(float)));
    w.acc2 = w.acc + kAccCap;
    DD_CUDA(cudaMemset(w.tickets, 0, (kTicketCap + 4) * sizeof(unsigned)));
    {
        // the error word lives in mapped pinned host memory: a kernel that gives up stores into it, and the
        // host sees it at the next call without a copy or a synchronisation
        void* h = nullptr;
        void* d = nullptr;
        if (cudaHostAlloc(&h, 64, cudaHostAllocMapped) != cudaSuccess || cudaHostGetDevicePointer(&d, h, 0) != cudaSuccess) {
            cudaGetLastError();
            cudaFree(w.acc); cudaFree(w.tickets);
            return fail(DECDEC_E_NOMEM, "cudaHostAlloc(error word) failed");
        }
        memset(h, 0, 64);
        w.err = reinterpret_cast<unsigned*>(d);
        w.err_host = reinterpret_cast<volatile unsigned*>(h);
    }
    *out = w;
    return 0;
}

int get_workspace(cudaStream_t stream, Workspace* out) {
    int dev = 0;
    DD_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_ws.find({dev, stream});
    if (it != g_ws.end()) { *out = it->second; return check_ws(*out); }
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    DD_CUDA(cudaStreamIsCapturing(stream, &cs));
    if (cs != cudaStreamCaptureStatusNone) {
        // no allocation while capturing.  A stream first seen during capture (frameworks capture on streams of their
        // own) gets one of the spare workspaces set aside at the device's first call, so that graphs captured on
        // different streams do not share accumulators; when the spares are used up it shares the device's first
        // workspace (then that graph must not run concurrently with work on the owning stream).
        auto sp = g_ws_spare.find(dev);
        if (sp != g_ws_spare.end() && !sp->second.empty()) {
            *out = sp->second.back();
            sp->second.pop_back();
            g_ws[{dev, stream}] = *out;
            return check_ws(*out);
        }
        auto f = g_ws_first.find(dev);
        if (f == g_ws_first.end())
            return fail(DECDEC_E_INVALID, "first call on a device must happen outside stream capture (workspace allocation)");
        *out = f->second;
        return check_ws(*out);
    }
    Workspace w;
    if (int r = alloc_workspace(&w)) return r;
    if (!g_ws_first.count(dev)) {
        g_ws_first[dev] = w;
        for (int i = 0; i < kSpareWorkspaces; ++i) {
            Workspace sw;
            if (alloc_workspace(&sw)) break;            // fewer spares: later captures share the first workspace
            g_ws_spare[dev].push_back(sw);
        }
    }
    DD_CUDA(cudaDeviceSynchronize());
    g_ws[{dev, stream}] = w;
    *out = w;
    return 0;
}

size_t dtype_size(int dt) { return dt == FP32 ? 4 : 2; }

float host_to_float(const void* p, size_t idx, int dt) {
    if (dt == FP32) return reinterpret_cast<const float*>(p)[idx];
    uint16_t h = reinterpret_cast<const uint16_t*>(p)[idx];
    if (dt == BF16) {
        uint32_t u = (uint32_t)h << 16;
        float f;
        memcpy(&f, &u, 4);
        return f;
    }
    __half_raw r;
    r.x = h;
    return __half2float(__half(r));
}

struct Context {
    int dtype;
    int device;
    uint32_t num_tb;
    uint32_t buffer_size;
    int32_t* rows;
    void* acts;
};

struct Config {
    int dtype;
    Context* ctx;
    const uint32_t* cheat_dev;    // device-visible pointer used by kernels
    void* cheat_host_owned;       // pinned mapped allocation (or null)
    void* scales_dev_owned;       // cudaMalloc'd copy
    const void* thresholds_host;  // borrowed
    uint32_t K, N, k_chunk;
};

bool valid_dtype(int dt) { return dt == FP32 || dt == FP16 || dt == BF16; }

uint32_t cdiv(uint32_t a, uint32_t b) { return (a + b - 1) / b; }

// DEC launch geometry.  Fused selection: row parts = chunks (at most num_tb of them), the remaining
// thread blocks split the outputs.  Rows given: rows are cut evenly.
void dec_geometry(const Config* c, bool fused_select, uint32_t n_tiles, DecParams* d) {
    const uint32_t num_chunks = cdiv(c->K, kChunk);
    const uint32_t k_total = (uint32_t)(((uint64_t)c->k_chunk * c->K) / kChunk);
    const uint32_t n_tb = c->ctx->num_tb ? c->ctx->num_tb : 1;
    uint32_t rp = fused_select ? num_chunks : cdiv(k_total, 32u);
    if (rp > n_tb) rp = n_tb;
    if (rp == 0) rp = 1;
    uint32_t cp = n_tb / rp;
    if (cp == 0) cp = 1;
    if (cp > n_tiles) cp = n_tiles;
    d->K = c->K;
    d->N = c->N;
    d->k_chunk = c->k_chunk;
    d->k_total = k_total;
    d->n_rowparts = rp;
    d->n_colparts = cp;
    d->n_cta = k_total ? rp * cp : 0;
    d->fused_select = fused_select ? 1u : 0u;
}

int fill_dec(const Config* c, const void* x, bool fused_select, uint32_t n_tiles, DecParams* d) {
    memset(d, 0, sizeof(*d));
    dec_geometry(c, fused_select, n_tiles, d);
    d->cheat = c->cheat_dev;
    d->scales = c->scales_dev_owned;
    d->x = x;
    d->sel_rows = c->ctx->rows;
    d->sel_acts = c->ctx->acts;
    if (d->k_total) {
        if (d->k_total > c->ctx->buffer_size)
            return fail(DECDEC_E_INVALID, "DECContext buffer size is too small for the given k_chunk.");
        d->thr_a = host_to_float(c->thresholds_host, 0, c->dtype);
        d->thr_b = host_to_float(c->thresholds_host, d->k_total - 1, c->dtype);
    }
    return 0;
}

// SMs left to the GEMV thread blocks of a fused launch.  A few compensation thread blocks take their SMs
// out of the GEMV's single wave (the GEMV grid shrinks accordingly); many of them mean the launch is bound
// by the host link anyway, and the GEMV keeps its full grid and runs in the gaps.
uint32_t gemv_sm_budget(const Config* c, bool fused_select) {
    const uint32_t sms = device_sms();
    if (!c) return sms;
    DecParams d;
    memset(&d, 0, sizeof(d));
    dec_geometry(c, fused_select, 1u << 20, &d);
    return d.n_cta <= sms / 4 + 3 ? sms - d.n_cta : sms;      // up to 40 compensation blocks on a 148-SM part
}

int check_cfg_call(const Config* c, const void* x, void* y, uint32_t K, uint32_t N, int dtype) {
    if (!c) return fail(DECDEC_E_INVALID, "null DECConfig handle");
    if (!x || !y) return fail(DECDEC_E_INVALID, "null input/output pointer");
    if (dtype != c->dtype) return fail(DECDEC_E_INVALID, "Mismatched data types between input tensor and DECConfig.");
    if (K != c->K) return fail(DECDEC_E_INVALID, "input tensor size does not match with DECConfig: input size: %u, DECConfig size: %u", K, c->K);
    if (N != c->N) return fail(DECDEC_E_INVALID, "output tensor size does not match with DECConfig: output size: %u, DECConfig size: %u", N, c->N);
    return 0;
}

uint32_t env_u32(const char* name, uint32_t dflt) {
    const char* v = getenv(name);
    return (v && *v) ? (uint32_t)strtoul(v, nullptr, 10) : dflt;
}

// ---- per-format argument checks and GEMV geometry ---------------------------------------------------

int setup_fin(FinParams* f, const Workspace& ws, void* y, uint32_t N, uint32_t tile_units, uint32_t expected) {
    if (N > kAccCap) return fail(DECDEC_E_UNSUPPORTED, "out_features %u exceeds the accumulator capacity %u", N, kAccCap);
    f->acc = ws.acc;
    f->tickets = ws.tickets;
    f->err = ws.err;
    f->acc2 = nullptr;          // set by the callers that add a compensation role
    f->scales = nullptr;
    f->y = y;
    f->N = N;
    f->tile_units = tile_units;
    f->n_tiles = cdiv(cdiv(N, 32), tile_units);
    f->expected = expected;
    if (f->n_tiles > kTicketCap) return fail(DECDEC_E_UNSUPPORTED, "too many output tiles (%u)", f->n_tiles);
    return 0;
}

int run_dec_only(uintptr_t cfg_h, const void* x, void* y, uint32_t K, uint32_t N, int dtype, void* stream, bool fused_select) {
    Config* c = reinterpret_cast<Config*>(cfg_h);
    if (int r = check_cfg_call(c, x, y, K, N, dtype)) return r;
    const uint32_t k_total = (uint32_t)(((uint64_t)c->k_chunk * K) / kChunk);
    if (k_total == 0) return 0;   // reference: decdec.cu:52-54
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    Workspace ws;
    if (int r = get_workspace(s, &ws)) return r;
    // tiles = column parts
    const uint32_t units = cdiv(N, 32);
    DecParams d;
    {
        // first pass to learn the column-part count for "as many tiles as column parts"
        if (int r = fill_dec(c, x, fused_select, units, &d)) return r;
    }
    const uint32_t tile_units = cdiv(units, d.n_colparts);
    FinParams f;
    if (int r = setup_fin(&f, ws, y, N, tile_units, 0)) return r;
    if (int r = fill_dec(c, x, fused_select, f.n_tiles, &d)) return r;
    f.expected = d.n_rowparts;
    f.acc2 = ws.acc2;
    f.scales = d.scales;
    DD_CUDA(launch_dec_only(dtype, d, f, s));
    return 0;
}

int check_gemv_common(const void* x, void* y, const void* qw, uint32_t N, uint32_t K, int dtype) {
    if (!x || !y || !qw) return fail(DECDEC_E_INVALID, "null pointer argument");
    if (!valid_dtype(dtype)) return fail(DECDEC_E_INVALID, "Unsupported data type.");
    if (N == 0 || K == 0) return fail(DECDEC_E_INVALID, "empty layer (N=%u, K=%u)", N, K);
    if (K % 32u) return fail(DECDEC_E_INVALID, "in_features must be a multiple of 32, got %u", K);
    return 0;
}

int run_bcq(Config* c, const void* x, void* y, const int32_t* qw, const void* alpha, const void* q_bias, uint32_t N,
            uint32_t K, int bits, int group, int dtype, cudaStream_t s) {
    if (int r = check_gemv_common(x, y, qw, N, K, dtype)) return r;
    if (!alpha || !q_bias) return fail(DECDEC_E_INVALID, "null alpha/q_bias");
    if (bits < 1 || bits > 8) return fail(DECDEC_E_INVALID, "Bitwidth must be between 1 and 8.");
    if (group <= 0 || group % 32 || K % (uint32_t)group) return fail(DECDEC_E_INVALID, "group_size must be a multiple of 32 that divides in_features (got %d)", group);
    if (N % 8u) return fail(DECDEC_E_UNSUPPORTED, "lutgemm: out_features must be a multiple of 8, got %u", N);
    if ((reinterpret_cast<uintptr_t>(qw) | reinterpret_cast<uintptr_t>(alpha) | reinterpret_cast<uintptr_t>(q_bias)) & 15u)
        return fail(DECDEC_E_INVALID, "lutgemm: q_weight/alpha/q_bias must be 16-byte aligned");
    Workspace ws;
    if (int r = get_workspace(s, &ws)) return r;
    BcqParams g;
    g.qweight = reinterpret_cast<const uint32_t*>(qw);
    g.alpha = alpha;
    g.q_bias = q_bias;
    g.x = x;
    g.K = K; g.N = N; g.bits = (uint32_t)bits; g.group = (uint32_t)group;
    g.n_kslices = cdiv(K, kBcqSlice);
    const uint32_t units = cdiv(N, 32);
    // tile size: about `target` GEMV thread blocks in total, 8 warps x one 32-output unit each at least
    const uint32_t target = env_u32("DECDEC_BCQ_CTAS", 296);
    uint32_t tiles_target = target / g.n_kslices;
    if (tiles_target == 0) tiles_target = 1;
    uint32_t tile_units = cdiv(units, tiles_target);
    tile_units = cdiv(tile_units, 8) * 8;
    tile_units = env_u32("DECDEC_BCQ_TILE_UNITS", tile_units);
    PipeGeom geo;
    const bool pipe = env_u32("DECDEC_BCQ_PIPE", 1) && bcq_pipe_geometry(N, K, g.bits, g.group, dtype, g.n_kslices, &geo, gemv_sm_budget(c, true));
    FinParams f;
    if (pipe) tile_units = geo.tile_stages * (kPipeStageN / 32);
    if (int r = setup_fin(&f, ws, y, N, tile_units, g.n_kslices)) return r;
    g.n_cta = g.n_kslices * f.n_tiles;
    DecParams d;
    memset(&d, 0, sizeof(d));
    if (c) {
        if (int r = fill_dec(c, x, true, f.n_tiles, &d)) return r;
        if (d.n_cta) { f.expected += d.n_rowparts; f.acc2 = ws.acc2; f.scales = d.scales; }
    }
    // Launches of the pipelined kernel carry sums and arrival counts in one 64-bit atomic per output (the accumulator
    // allocation holds kAccCap such words) instead of tickets; DECDEC_BCQ_PACKED=0 keeps the ticket protocol.  With a
    // compensation role the CTA's private cells must fit in shared memory beside the selection state.
    if (pipe && env_u32("DECDEC_BCQ_PACKED", 1)) {
        const uint32_t arrivals = 2u * g.n_kslices + (d.n_cta ? d.n_rowparts : 0u);
        bool ok = arrivals <= 255u;
        if (ok && d.n_cta) {
            const uint32_t tiles_max = cdiv(f.n_tiles, d.n_colparts);
            const uint32_t nvec_max = cdiv(tiles_max * tile_units * 32u, 32u);
            const uint32_t slots = nvec_max > (uint32_t)kPipeThreads ? nvec_max : (uint32_t)kPipeThreads;
            const uint32_t need = (uint32_t)kDecPrivOff + (slots | 1u) * 128u;
            // every output of a compensation CTA's column range costs it one atomic, and one SM issues about one per
            // clock: beyond ~2048 outputs per CTA (few, wide compensation CTAs) the ticket protocol is faster
            ok = (N % 32u) == 0u && need <= 227u * 1024u && nvec_max * 32u <= env_u32("DECDEC_PACKED_MAX_RANGE", 2048);
            if (ok && geo.smem_bytes < need) geo.smem_bytes = need;
        }
        if (ok) { geo.packed = 1u; geo.arrivals = arrivals; }
    }
    if (pipe) DD_CUDA(launch_bcq_pipe(dtype, g, d, f, geo, s));
    else DD_CUDA(launch_bcq(dtype, g, d, f, s));
    return 0;
}

int run_anyprec(Config* c, const void* x, void* y, const int32_t* qw, uint32_t planes, const void* lut, uint32_t N,
                uint32_t K, int bits, int dtype, cudaStream_t s) {
    if (int r = check_gemv_common(x, y, qw, N, K, dtype)) return r;
    if (!lut) return fail(DECDEC_E_INVALID, "null lut");
    if (bits < 3 || bits > 8) return fail(DECDEC_E_INVALID, "Bitwidth must be between 3 and 8.");
    if (dtype == FP32) return fail(DECDEC_E_INVALID, "Any-Precision GEMV does not support float data type. Please use half or bfloat16.");
    if (planes < (uint32_t)bits) return fail(DECDEC_E_INVALID, "qweight tensor must have at least bitwidth planes (got %u < %d)", planes, bits);
    if ((reinterpret_cast<uintptr_t>(qw) | reinterpret_cast<uintptr_t>(lut)) & 15u)
        return fail(DECDEC_E_INVALID, "anyprec: qweight/lut must be 16-byte aligned");
    Workspace ws;
    if (int r = get_workspace(s, &ws)) return r;
    ApParams g;
    g.qweight = reinterpret_cast<const uint32_t*>(qw);
    g.lut = lut;
    g.x = x;
    g.K = K; g.N = N; g.bits = (uint32_t)bits;
    const uint32_t units = cdiv(N, 32);
    const uint32_t target = env_u32("DECDEC_AP_CTAS", 592);
    uint32_t tile_units = cdiv(units, target);
    tile_units = env_u32("DECDEC_AP_TILE_UNITS", tile_units);
    ApPipeGeom pgeo;
    uint32_t budget = gemv_sm_budget(c, true);
    if (c) {
        // many compensation thread blocks (the launch is bound by the host link): the GEMV runs in the SMs they leave
        // free and takes over the rest as they retire, which it does more evenly in thread blocks a third the size
        DecParams dg;
        memset(&dg, 0, sizeof(dg));
        dec_geometry(c, true, 1u << 20, &dg);
        if (dg.n_cta > device_sms() / 4 + 3) budget *= env_u32("DECDEC_AP_FUSED_SPLIT", 3);
    }
    const bool pipe = env_u32("DECDEC_AP_PIPE", 1) && anyprec_pipe_geometry(N, K, g.bits, &pgeo, budget, c == nullptr);
    if (pipe) tile_units = cdiv(pgeo.rows_per_cta, 32);
    FinParams f;
    if (int r = setup_fin(&f, ws, y, N, tile_units, 1)) return r;
    g.n_cta = (pipe && c == nullptr) ? cdiv(N, pgeo.rows_per_cta) : f.n_tiles;   // no finalizer tiles in a GEMV-only launch
    DecParams d;
    memset(&d, 0, sizeof(d));
    if (c) {
        if (int r = fill_dec(c, x, true, f.n_tiles, &d)) return r;
        if (d.n_cta) { f.expected += d.n_rowparts; f.acc2 = ws.acc2; f.scales = d.scales; }
    }
    g.direct = d.n_cta ? 0u : 1u;
    if (pipe) {
        pgeo.direct = g.direct;
        g.direct = 0u;
        DD_CUDA(launch_anyprec_pipe(dtype, g, d, f, pgeo, s));
        return 0;
    }
    const bool fast3 = bits == 3 && (K % 128u) == 0u;
    if (anyprec_smem(K, fast3) > 200 * 1024) return fail(DECDEC_E_UNSUPPORTED, "anyprec: in_features %u too large for shared-memory staging", K);
    DD_CUDA(launch_anyprec(dtype, g, d, f, s));
    return 0;
}

int run_sqllm(Config* c, const void* x, void* y, const int32_t* qw, const void* lut, uint32_t N, uint32_t K, int bits,
              int dtype, cudaStream_t s) {
    if (int r = check_gemv_common(x, y, qw, N, K, dtype)) return r;
    if (!lut) return fail(DECDEC_E_INVALID, "null lut");
    if (bits != 3 && bits != 4) return fail(DECDEC_E_INVALID, "Bitwidth must be 3 or 4.");
    if (sqllm_smem(K) > 200 * 1024) return fail(DECDEC_E_UNSUPPORTED, "sqllm: in_features %u too large for shared-memory staging", K);
    Workspace ws;
    if (int r = get_workspace(s, &ws)) return r;
    SqParams g;
    g.qweight = reinterpret_cast<const uint32_t*>(qw);
    g.lut = lut;
    g.x = x;
    g.K = K; g.N = N; g.bits = (uint32_t)bits;
    FinParams f;
    if (int r = setup_fin(&f, ws, y, N, 1, 1)) return r;
    g.n_cta = f.n_tiles;
    DecParams d;
    memset(&d, 0, sizeof(d));
    if (c) {
        if (int r = fill_dec(c, x, true, f.n_tiles, &d)) return r;
        if (d.n_cta) { f.expected += d.n_rowparts; f.acc2 = ws.acc2; f.scales = d.scales; }
    }
    g.direct = d.n_cta ? 0u : 1u;
    DD_CUDA(launch_sqllm(dtype, g, d, f, s));
    return 0;
}

// side stream + events for the dummy_* entry points, one set per device
int side_stream(cudaStream_t* s, cudaEvent_t* e1, cudaEvent_t* e2) {
    int dev = 0;
    DD_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_side.find(dev);
    if (it == g_side.end()) {
        cudaStream_t st;
        cudaEvent_t a, b;
        DD_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
        DD_CUDA(cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
        DD_CUDA(cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
        it = g_side.insert({dev, {st, {a, b}}}).first;
    }
    *s = it->second.first;
    *e1 = it->second.second.first;
    *e2 = it->second.second.second;
    return 0;
}

template <typename F>
int run_dummy(int dummy_sm, long long iters, void* stream, F gemv) {
    cudaStream_t main_s = reinterpret_cast<cudaStream_t>(stream), sub;
    cudaEvent_t e1, e2;
    if (int r = side_stream(&sub, &e1, &e2)) return r;
    DD_CUDA(cudaEventRecord(e1, main_s));
    DD_CUDA(launch_burner(dummy_sm, iters, main_s));
    DD_CUDA(cudaStreamWaitEvent(sub, e1, 0));
    if (int r = gemv(sub)) return r;
    DD_CUDA(cudaEventRecord(e2, sub));
    DD_CUDA(cudaStreamWaitEvent(main_s, e2, 0));
    return 0;
}

}  // namespace

namespace dd {
// lets other translation units of the library record the message returned by decdec_last_error()
int set_last_error(int code, const char* msg) { return fail(code, "%s", msg); }
}  // namespace dd

extern "C" {

const char* decdec_last_error(void) { return g_err; }

int decdec_compiled_arch(void) { return 100; }

int decdec_stream_status(void* stream, uint32_t* error_out) {
    if (!error_out) return fail(DECDEC_E_INVALID, "null output pointer");
    int dev = 0;
    DD_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_ws.find({dev, reinterpret_cast<cudaStream_t>(stream)});
    *error_out = (it != g_ws.end() && it->second.err_host) ? *it->second.err_host : 0u;
    return 0;
}


int decdec_stream_reset(void* stream) {
    int dev = 0;
    DD_CUDA(cudaGetDevice(&dev));
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    Workspace w;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = g_ws.find({dev, s});
        if (it == g_ws.end()) return 0;
        w = it->second;
    }
    DD_CUDA(cudaStreamSynchronize(s));
    DD_CUDA(cudaMemsetAsync(w.acc, 0, 2 * kAccCap * sizeof(float), s));
    DD_CUDA(cudaMemsetAsync(w.tickets, 0, (kTicketCap + 4) * sizeof(unsigned), s));
    DD_CUDA(cudaStreamSynchronize(s));
    if (w.err_host) *w.err_host = 0u;
    return 0;
}

int decdec_create_context(uint32_t num_tb, int32_t* rows, void* acts, uint32_t buffer_size, int dtype, uintptr_t* out) {
    if (!out) return fail(DECDEC_E_INVALID, "null output handle");
    if (!rows || !acts) return fail(DECDEC_E_INVALID, "selected_rows_buffer and selected_activations_buffer must be on GPU.");
    if (!valid_dtype(dtype)) return fail(DECDEC_E_INVALID, "Unsupported data type.");
    Context* c = new Context();
    c->dtype = dtype;
    c->num_tb = num_tb;
    c->buffer_size = buffer_size;
    c->rows = rows;
    c->acts = acts;
    c->device = 0;
    cudaGetDevice(&c->device);
    *out = reinterpret_cast<uintptr_t>(c);
    return 0;
}

int decdec_destroy_context(uintptr_t ctx) {
    delete reinterpret_cast<Context*>(ctx);
    return 0;
}

int decdec_create_config(uintptr_t ctx_h, uint32_t k_chunk, const int32_t* q_residual, int q_on_device, uint32_t K,
                         uint32_t N, const void* scales, int scales_on_device, const void* thresholds_host, int dtype,
                         uintptr_t* out) {
    Context* ctx = reinterpret_cast<Context*>(ctx_h);
    if (!out) return fail(DECDEC_E_INVALID, "null output handle");
    if (!ctx) return fail(DECDEC_E_INVALID, "null DECContext handle");
    if (!q_residual || !scales || !thresholds_host) return fail(DECDEC_E_INVALID, "null tensor pointer");
    if (!valid_dtype(dtype)) return fail(DECDEC_E_INVALID, "Unsupported data type in create_dec_config.");
    if (dtype != ctx->dtype) return fail(DECDEC_E_INVALID, "Data type mismatch between DECConfig and DECContext.");
    if (N == 0 || K == 0 || N % 8u) return fail(DECDEC_E_INVALID, "q_residual must be [K, N/8] with N a multiple of 8 (K=%u, N=%u)", K, N);
    if (k_chunk > (uint32_t)kChunk) return fail(DECDEC_E_INVALID, "k_chunk %u exceeds the chunk size 1024", k_chunk);
    Config* c = new Config();
    memset(c, 0, sizeof(*c));
    c->dtype = dtype;
    c->ctx = ctx;
    c->K = K;
    c->N = N;
    c->k_chunk = k_chunk;
    c->thresholds_host = thresholds_host;
    const size_t rbytes = (size_t)K * (N / 8) * sizeof(uint32_t);
    if (!q_on_device) {
        unsigned flags = cudaHostAllocMapped;
        if (env_u32("DECDEC_HOST_WC", 0)) flags |= cudaHostAllocWriteCombined;
        void* h = nullptr;
        if (cudaHostAlloc(&h, rbytes, flags) != cudaSuccess) {
            delete c;
            cudaGetLastError();
            return fail(DECDEC_E_NOMEM, "cudaHostAlloc(%zu bytes, mapped) for q_residual failed", rbytes);
        }
        memcpy(h, q_residual, rbytes);
        void* d = nullptr;
        if (cudaHostGetDevicePointer(&d, h, 0) != cudaSuccess) {
            cudaFreeHost(h);
            delete c;
            return fail(DECDEC_E_CUDA, "cudaHostGetDevicePointer failed");
        }
        c->cheat_host_owned = h;
        c->cheat_dev = reinterpret_cast<const uint32_t*>(d);
    } else {
        c->cheat_dev = reinterpret_cast<const uint32_t*>(q_residual);
    }
    if (reinterpret_cast<uintptr_t>(c->cheat_dev) & 15u) {
        if (c->cheat_host_owned) cudaFreeHost(c->cheat_host_owned);
        delete c;
        return fail(DECDEC_E_INVALID, "q_residual must be 16-byte aligned");
    }
    const size_t sbytes = (size_t)N * dtype_size(dtype);
    if (cudaMalloc(&c->scales_dev_owned, sbytes) != cudaSuccess) {
        if (c->cheat_host_owned) cudaFreeHost(c->cheat_host_owned);
        delete c;
        cudaGetLastError();
        return fail(DECDEC_E_NOMEM, "cudaMalloc(scales) failed");
    }
    cudaError_t e = cudaMemcpy(c->scales_dev_owned, scales, sbytes, scales_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        cudaFree(c->scales_dev_owned);
        if (c->cheat_host_owned) cudaFreeHost(c->cheat_host_owned);
        delete c;
        return fail(DECDEC_E_CUDA, "copy of reordered_scales failed: %s", cudaGetErrorString(e));
    }
    const uint32_t k_total = (uint32_t)(((uint64_t)k_chunk * K) / kChunk);
    if (k_total > ctx->buffer_size) {
        cudaFree(c->scales_dev_owned);
        if (c->cheat_host_owned) cudaFreeHost(c->cheat_host_owned);
        delete c;
        return fail(DECDEC_E_INVALID, "DECContext buffer size is too small for the given k_chunk.");
    }
    *out = reinterpret_cast<uintptr_t>(c);
    return 0;
}

int decdec_update_config(uintptr_t cfg_h, uintptr_t new_ctx_h, uint32_t k_chunk) {
    Config* c = reinterpret_cast<Config*>(cfg_h);
    Context* ctx = reinterpret_cast<Context*>(new_ctx_h);
    if (!c || !ctx) return fail(DECDEC_E_INVALID, "null handle");
    if (ctx->dtype != c->dtype) return fail(DECDEC_E_INVALID, "Data type mismatch between DECConfig and DECContext.");
    if (k_chunk > (uint32_t)kChunk) return fail(DECDEC_E_INVALID, "k_chunk %u exceeds the chunk size 1024", k_chunk);
    const uint32_t k_total = (uint32_t)(((uint64_t)k_chunk * c->K) / kChunk);
    if (k_total > ctx->buffer_size) return fail(DECDEC_E_INVALID, "DECContext buffer size is too small for the given k_chunk.");
    c->ctx = ctx;
    c->k_chunk = k_chunk;
    return 0;
}

int decdec_destroy_config(uintptr_t cfg_h) {
    Config* c = reinterpret_cast<Config*>(cfg_h);
    if (!c) return 0;
    if (c->cheat_host_owned) cudaFreeHost(c->cheat_host_owned);
    if (c->scales_dev_owned) cudaFree(c->scales_dev_owned);
    delete c;
    return 0;
}

int decdec_read_config(uintptr_t cfg_h, decdec_config_info* out) {
    Config* c = reinterpret_cast<Config*>(cfg_h);
    if (!c || !out) return fail(DECDEC_E_INVALID, "null handle");
    DecParams d;
    memset(&d, 0, sizeof(d));
    const uint32_t units = cdiv(c->N, 32);
    dec_geometry(c, true, units, &d);
    const uint32_t tile_units = cdiv(units, d.n_colparts);
    dec_geometry(c, true, cdiv(units, tile_units), &d);
    out->num_chunks = (int32_t)cdiv(c->K, kChunk);
    out->chunk_size = kChunk;
    out->k_chunk = (int32_t)c->k_chunk;
    out->channels_per_tb = (int32_t)(tile_units * 4u);
    out->n_tb = (int32_t)(d.n_rowparts * d.n_colparts);
    out->block_dim_x = kThreads;
    out->block_dim_y = 1;
    out->shared_memory_size = (int32_t)dec_only_smem();
    out->reduced_shared_memory = 0;
    return 0;
}

int decdec_dec(uintptr_t cfg, const void* x, void* y, uint32_t K, uint32_t N, int dtype, void* stream) {
    return run_dec_only(cfg, x, y, K, N, dtype, stream, true);
}

int decdec_unfused_dec(uintptr_t cfg, const void* x, void* y, uint32_t K, uint32_t N, int dtype, void* stream) {
    return run_dec_only(cfg, x, y, K, N, dtype, stream, false);
}

int decdec_anyprec_gemv(const void* x, void* y, const int32_t* qw, uint32_t planes, const void* lut, uint32_t N, uint32_t K,
                        int bits, int dtype, void* stream) {
    return run_anyprec(nullptr, x, y, qw, planes, lut, N, K, bits, dtype, reinterpret_cast<cudaStream_t>(stream));
}

int decdec_lutgemm_gemv(const void* x, void* y, const int32_t* qw, const void* alpha, const void* q_bias, uint32_t N,
                        uint32_t K, int bits, int group, int dtype, void* stream) {
    return run_bcq(nullptr, x, y, qw, alpha, q_bias, N, K, bits, group, dtype, reinterpret_cast<cudaStream_t>(stream));
}

int decdec_sqllm_gemv(const void* x, void* y, const int32_t* qw, const void* lut, uint32_t N, uint32_t K, int bits,
                      int dtype, void* stream) {
    return run_sqllm(nullptr, x, y, qw, lut, N, K, bits, dtype, reinterpret_cast<cudaStream_t>(stream));
}

int decdec_anyprec_dequant(const int32_t* qw, const void* lut, void* out, uint32_t N, uint32_t K, int bits, int dtype,
                           void* stream) {
    if (!qw || !lut || !out) return fail(DECDEC_E_INVALID, "null pointer argument");
    if (dtype == FP32) return fail(DECDEC_E_INVALID, "Any-Precision Dequantization does not support float data type. Please use half or bfloat16.");
    if (!valid_dtype(dtype)) return fail(DECDEC_E_INVALID, "Unsupported data type.");
    if (bits < 3 || bits > 8) return fail(DECDEC_E_INVALID, "Bitwidth must be between 3 and 8.");
    if (K % 32u) return fail(DECDEC_E_INVALID, "in_features must be a multiple of 32, got %u", K);
    DD_CUDA(launch_ap_dequant(dtype, reinterpret_cast<const uint32_t*>(qw), lut, out, N, K, (uint32_t)bits,
                              reinterpret_cast<cudaStream_t>(stream)));
    return 0;
}

int decdec_lutgemm_dequant(const int32_t* qw, const void* alpha, const void* q_bias, void* out, uint32_t N, uint32_t K, int bits,
                           int group, int dtype, void* stream) {
    if (!qw || !alpha || !q_bias || !out) return fail(DECDEC_E_INVALID, "null pointer argument");
    if (!valid_dtype(dtype)) return fail(DECDEC_E_INVALID, "Unsupported data type.");
    if (bits < 1 || bits > 8) return fail(DECDEC_E_INVALID, "Bitwidth must be between 1 and 8.");
    if (N == 0 || K == 0) return fail(DECDEC_E_INVALID, "empty layer (N=%u, K=%u)", N, K);
    if (K % 32u) return fail(DECDEC_E_INVALID, "in_features must be a multiple of 32, got %u", K);
    if (group <= 0 || group % 32 || K % (uint32_t)group) return fail(DECDEC_E_INVALID, "group_size must be a multiple of 32 that divides in_features (got %d)", group);
    if (N % 2u) return fail(DECDEC_E_UNSUPPORTED, "lutgemm dequant: out_features must be even, got %u", N);
    if (reinterpret_cast<uintptr_t>(qw) & 7u) return fail(DECDEC_E_INVALID, "lutgemm dequant: q_weight must be 8-byte aligned");
    DD_CUDA(launch_bcq_dequant(dtype, reinterpret_cast<const uint32_t*>(qw), alpha, q_bias, out, N, K, (uint32_t)bits,
                               (uint32_t)group, reinterpret_cast<cudaStream_t>(stream)));
    return 0;
}

int decdec_dec_anyprec(uintptr_t cfg, const void* x, void* y, const int32_t* qw, uint32_t planes, const void* lut,
                       uint32_t N, uint32_t K, int bits, int dtype, void* stream) {
    Config* c = reinterpret_cast<Config*>(cfg);
    if (int r = check_cfg_call(c, x, y, K, N, dtype)) return r;
    return run_anyprec(c, x, y, qw, planes, lut, N, K, bits, dtype, reinterpret_cast<cudaStream_t>(stream));
}

int decdec_dec_lutgemm(uintptr_t cfg, const void* x, void* y, const int32_t* qw, const void* alpha, const void* q_bias,
                       uint32_t N, uint32_t K, int bits, int group, int dtype, void* stream) {
    Config* c = reinterpret_cast<Config*>(cfg);
    if (int r = check_cfg_call(c, x, y, K, N, dtype)) return r;
    return run_bcq(c, x, y, qw, alpha, q_bias, N, K, bits, group, dtype, reinterpret_cast<cudaStream_t>(stream));
}

int decdec_dec_sqllm(uintptr_t cfg, const void* x, void* y, const int32_t* qw, const void* lut, uint32_t N, uint32_t K,
                     int bits, int dtype, void* stream) {
    Config* c = reinterpret_cast<Config*>(cfg);
    if (int r = check_cfg_call(c, x, y, K, N, dtype)) return r;
    return run_sqllm(c, x, y, qw, lut, N, K, bits, dtype, reinterpret_cast<cudaStream_t>(stream));
}

int decdec_dummy_anyprec(const void* x, void* y, const int32_t* qw, uint32_t planes, const void* lut, uint32_t N,
                         uint32_t K, int bits, int dtype, int dummy_sm, long long iters, void* stream) {
    return run_dummy(dummy_sm, iters, stream, [&](cudaStream_t sub) {
        return run_anyprec(nullptr, x, y, qw, planes, lut, N, K, bits, dtype, sub);
    });
}

int decdec_dummy_lutgemm(const void* x, void* y, const int32_t* qw, const void* alpha, const void* q_bias, uint32_t N,
                         uint32_t K, int bits, int group, int dtype, int dummy_sm, long long iters, void* stream) {
    return run_dummy(dummy_sm, iters, stream, [&](cudaStream_t sub) {
        return run_bcq(nullptr, x, y, qw, alpha, q_bias, N, K, bits, group, dtype, sub);
    });
}

int decdec_dummy_sqllm(const void* x, void* y, const int32_t* qw, const void* lut, uint32_t N, uint32_t K, int bits,
                       int dtype, int dummy_sm, long long iters, void* stream) {
    return run_dummy(dummy_sm, iters, stream, [&](cudaStream_t sub) {
        return run_sqllm(nullptr, x, y, qw, lut, N, K, bits, dtype, sub);
    });
}

}  // extern "C"
