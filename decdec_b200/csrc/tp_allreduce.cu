// One-shot push all-reduce for the row-parallel projections of a tensor-parallel layer.
//
// After a row-parallel GEMV every rank holds a partial output [N]; the sum has to reach every rank.  At
// N = 4096-8192 that is 8-16 KB: a latency problem, not a bandwidth problem.  One kernel per rank:
//   1. push   : the rank stores its partial vector into a slot of every peer's buffer over NVLink.  The
//               slot is made of 16-byte lines {data, flag, data, flag}: every 8-byte half carries the call
//               number next to its 4 bytes of payload, so a line validates itself wherever the fabric
//               splits it - no fence and no separate flag after the data;
//   2. wait   : each thread polls the lines of its own 16 bytes of output from every peer until both flags
//               show this call.  The wait is bounded; on expiry the block records an error and leaves y as is;
//   3. reduce : the thread sums the world's values in rank order in fp32 (identical on every rank) and
//               writes y.
// Slots alternate between two halves by call parity: a peer can be at most one call ahead (it needs
// this rank's lines of call e to finish e), so half (e & 1) is never overwritten while it is still
// being read, and what an older call left there carries an older flag.  The call number lives in device
// memory, one counter per thread block of the (fixed) grid, advanced by the kernel itself, which makes the
// call replayable inside CUDA graphs.  No multicast, no multimem: plain peer stores and local polls.
// The reference has no tensor parallelism; this file has no counterpart there.
#include "internal.h"
#include "../../include/decdec_b200.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace {

using namespace dd;

constexpr uint32_t kTpMaxWorld = 8;
constexpr uint32_t kTpMaxCta = 64;
constexpr uint32_t kTpThreads = 256;
constexpr size_t kTpHdr = 256;                                     // [epoch, ticket, err, pad]

struct TpLayout {
    size_t flags_off, slots_off, bytes;
    uint32_t slot_stride;                                          // bytes per (half, source rank)
};

TpLayout tp_layout(uint32_t world, uint32_t max_n) {
    TpLayout L;
    L.flags_off = kTpHdr;                                          // call counters, one per thread block of the grid
    L.slots_off = (L.flags_off + (size_t)world * kTpMaxCta * sizeof(uint32_t) + 255) & ~(size_t)255;
    L.slot_stride = (uint32_t)(((size_t)max_n * 8 + 255) & ~(size_t)255);     // 8 bytes of line per 4 bytes of payload (fp32 worst case)
    L.bytes = L.slots_off + 2 * (size_t)world * L.slot_stride;
    return L;
}

struct TpComm {
    uint32_t world, rank, max_n;
    int device;
    unsigned char* local;            // this rank's buffer (cudaMalloc)
    unsigned char* peers[kTpMaxWorld];
    bool opened[kTpMaxWorld];        // peers[i] came from cudaIpcOpenMemHandle
    bool connected;
    uint32_t wait_polls;
    uint32_t grid;                   // thread blocks of every launch: enough for max_n fp32 values
    TpLayout L;
};

struct TpArgs {
    unsigned char* peers[kTpMaxWorld];
    uint32_t world, rank, n;
    uint32_t flags_off, slots_off, slot_stride;
    uint32_t wait_polls;
};

__device__ __forceinline__ void st_line(unsigned char* p, uint32_t d0, uint32_t d1, uint32_t flag) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" :: "l"(p), "r"(d0), "r"(flag), "r"(d1), "r"(flag) : "memory");
}
__device__ __forceinline__ uint4 ld_line(const unsigned char* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// A thread owns 16 bytes of y = four 32-bit payload words = two lines of a slot.
template <int DT>
__global__ void __launch_bounds__(kTpThreads) k_tp_allreduce(const __grid_constant__ TpArgs a, void* y_) {
    using T = typename Tr<DT>::T;
    constexpr uint32_t EPT = 16 / sizeof(T);                       // elements per 16-byte vector
    __shared__ uint32_t s_bad;
    pdl_trigger();                 // the next kernel of the stream may become resident while this one exchanges
    unsigned char* mine = a.peers[a.rank];
    uint32_t* hdr = reinterpret_cast<uint32_t*>(mine);
    uint32_t* counter = reinterpret_cast<uint32_t*>(mine + a.flags_off) + blockIdx.x;
    if (threadIdx.x == 0) s_bad = 0u;
    pdl_wait();                    // y comes from the previous kernel; so does this block's call counter
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(counter) + 1u, half = e & 1u;
    __syncthreads();               // everybody has read the counter before thread 0 advances it
    const uint32_t vec = blockIdx.x * kTpThreads + threadIdx.x;              // index of this thread's 16 bytes
    const uint32_t idx = vec * EPT;
    const bool act = idx < a.n;
    T* y = reinterpret_cast<T*>(y_);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (act) v = *reinterpret_cast<const uint4*>(y + idx);

    // 1. push: two self-validating lines per peer
    const size_t line0 = (size_t)a.slots_off + ((size_t)half * a.world + a.rank) * a.slot_stride + (size_t)vec * 32u;
    if (act)
        for (uint32_t s = 0; s < a.world; ++s)
            if (s != a.rank) {
                st_line(a.peers[s] + line0, v.x, v.y, e);
                st_line(a.peers[s] + line0 + 16, v.z, v.w, e);
            }

    // 2. wait (bounded) and 3. reduce in rank order
    float acc[EPT];
#pragma unroll
    for (uint32_t i = 0; i < EPT; ++i) acc[i] = 0.0f;
    if (act) {
        bool bad = false;
        for (uint32_t s = 0; s < a.world && !bad; ++s) {
            uint4 q = v;
            if (s != a.rank) {
                const unsigned char* src = mine + (size_t)a.slots_off + ((size_t)half * a.world + s) * a.slot_stride + (size_t)vec * 32u;
                uint4 l0 = ld_line(src), l1 = ld_line(src + 16);
                uint32_t polls = 0;
                while (l0.y != e || l0.w != e || l1.y != e || l1.w != e) {
                    if (++polls >= a.wait_polls) { bad = true; break; }
                    __nanosleep(32);
                    l0 = ld_line(src);
                    l1 = ld_line(src + 16);
                }
                q = make_uint4(l0.x, l0.z, l1.x, l1.z);
            }
            const T* e4 = reinterpret_cast<const T*>(&q);
#pragma unroll
            for (uint32_t i = 0; i < EPT; ++i) acc[i] += Tr<DT>::to_f(e4[i]);
        }
        if (bad) atomicExch(&s_bad, 1u);
    }
    __syncthreads();
    if (act && !s_bad) {           // if any wait of the block ran out, the block leaves its part of y as it was
        uint4 o;
        T* o4 = reinterpret_cast<T*>(&o);
#pragma unroll
        for (uint32_t i = 0; i < EPT; ++i) o4[i] = Tr<DT>::from_f(acc[i]);
        *reinterpret_cast<uint4*>(y + idx) = o;
    }
    if (threadIdx.x == 0) {
        if (s_bad) atomicExch(hdr + 2, 1u);
        *reinterpret_cast<volatile uint32_t*>(counter) = e;
        if (blockIdx.x == 0) *reinterpret_cast<volatile uint32_t*>(hdr) = e;     // calls completed, read by decdec_tp_status
    }
}

int tp_fail(int code, const char* fmt, const char* detail = "") {
    char msg[256];
    snprintf(msg, sizeof(msg), fmt, detail);
    return set_last_error(code, msg);
}

}  // namespace

extern "C" {

int decdec_tp_layout(uint32_t world, uint32_t max_n, size_t* flags_off, size_t* slots_off, size_t* slot_stride, size_t* bytes) {
    if (world == 0 || world > kTpMaxWorld || max_n == 0) return tp_fail(DECDEC_E_INVALID, "tp: world must be 1..8 and max_n > 0");
    const TpLayout L = tp_layout(world, max_n);
    if (flags_off) *flags_off = L.flags_off;
    if (slots_off) *slots_off = L.slots_off;
    if (slot_stride) *slot_stride = L.slot_stride;
    if (bytes) *bytes = L.bytes;
    return 0;
}

int decdec_tp_create(uint32_t world, uint32_t rank, uint32_t max_n, uintptr_t* comm_out, unsigned char* ipc_handle_out) {
    if (!comm_out) return tp_fail(DECDEC_E_INVALID, "tp: null output handle");
    if (world == 0 || world > kTpMaxWorld || rank >= world) return tp_fail(DECDEC_E_INVALID, "tp: world must be 1..8 and rank < world");
    if (max_n == 0 || max_n > kTpMaxCta * kTpThreads * 4u) return tp_fail(DECDEC_E_UNSUPPORTED, "tp: max_n must be 1..65536");
    TpComm* c = new TpComm();
    memset(c, 0, sizeof(*c));
    c->world = world; c->rank = rank; c->max_n = max_n;
    c->L = tp_layout(world, max_n);
    c->grid = (max_n + kTpThreads * 4u - 1) / (kTpThreads * 4u);       // every launch has this many blocks, so their call counters stay in step
    const char* wp = getenv("DECDEC_TP_WAIT_POLLS");
    c->wait_polls = (wp && *wp) ? (uint32_t)strtoul(wp, nullptr, 10) : (1u << 21);     // about a second
    if (c->wait_polls == 0) c->wait_polls = 1;
    cudaError_t e = cudaGetDevice(&c->device);
    if (e == cudaSuccess) e = cudaMalloc(&c->local, c->L.bytes);
    if (e == cudaSuccess) e = cudaMemset(c->local, 0, c->L.bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e == cudaSuccess && ipc_handle_out) {
        cudaIpcMemHandle_t h;
        e = cudaIpcGetMemHandle(&h, c->local);
        if (e == cudaSuccess) memcpy(ipc_handle_out, &h, sizeof(h));
    }
    if (e != cudaSuccess) {
        if (c->local) cudaFree(c->local);
        delete c;
        cudaGetLastError();
        return tp_fail(DECDEC_E_CUDA, "tp: buffer set-up failed: %s", cudaGetErrorString(e));
    }
    c->peers[rank] = c->local;
    c->connected = world == 1;
    *comm_out = reinterpret_cast<uintptr_t>(c);
    return 0;
}

int decdec_tp_local_ptr(uintptr_t comm, void** ptr_out) {
    TpComm* c = reinterpret_cast<TpComm*>(comm);
    if (!c || !ptr_out) return tp_fail(DECDEC_E_INVALID, "tp: null handle");
    *ptr_out = c->local;
    return 0;
}

int decdec_tp_connect_ipc(uintptr_t comm, const unsigned char* handles) {
    TpComm* c = reinterpret_cast<TpComm*>(comm);
    if (!c || !handles) return tp_fail(DECDEC_E_INVALID, "tp: null handle");
    for (uint32_t s = 0; s < c->world; ++s) {
        if (s == c->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)s * sizeof(h), sizeof(h));
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return tp_fail(DECDEC_E_CUDA, "tp: cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
        }
        c->peers[s] = static_cast<unsigned char*>(p);
        c->opened[s] = true;
    }
    c->connected = true;
    return 0;
}

int decdec_tp_connect_ptrs(uintptr_t comm, const uintptr_t* peer_ptrs) {
    TpComm* c = reinterpret_cast<TpComm*>(comm);
    if (!c || !peer_ptrs) return tp_fail(DECDEC_E_INVALID, "tp: null handle");
    for (uint32_t s = 0; s < c->world; ++s) {
        if (s == c->rank) continue;
        if (!peer_ptrs[s]) return tp_fail(DECDEC_E_INVALID, "tp: null peer pointer");
        c->peers[s] = reinterpret_cast<unsigned char*>(peer_ptrs[s]);
    }
    c->connected = true;
    return 0;
}

int decdec_tp_allreduce(uintptr_t comm, void* y_dev, uint32_t n, int dtype, void* stream) {
    TpComm* c = reinterpret_cast<TpComm*>(comm);
    if (!c || !y_dev) return tp_fail(DECDEC_E_INVALID, "tp: null handle or output");
    if (!c->connected) return tp_fail(DECDEC_E_INVALID, "tp: peers are not connected");
    if (dtype != FP32 && dtype != FP16 && dtype != BF16) return tp_fail(DECDEC_E_INVALID, "Unsupported data type.");
    const uint32_t esz = dtype == FP32 ? 4 : 2, ept = 16 / esz;
    if (n == 0 || n > c->max_n) return tp_fail(DECDEC_E_INVALID, "tp: n exceeds the size the communicator was created for");
    if (n % ept || (reinterpret_cast<uintptr_t>(y_dev) & 15u)) return tp_fail(DECDEC_E_INVALID, "tp: y must be 16-byte aligned and n a multiple of 16 bytes");
    TpArgs a;
    memset(&a, 0, sizeof(a));
    for (uint32_t s = 0; s < c->world; ++s) a.peers[s] = c->peers[s];
    a.world = c->world; a.rank = c->rank; a.n = n;
    a.flags_off = (uint32_t)c->L.flags_off; a.slots_off = (uint32_t)c->L.slots_off; a.slot_stride = c->L.slot_stride;
    a.wait_polls = c->wait_polls;
    const uint32_t grid = c->grid;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    // programmatic dependent launch: the blocks become resident while the GEMV before them drains
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kTpThreads);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    const char* pe = getenv("DECDEC_PDL");
    attr[0].val.programmaticStreamSerializationAllowed = (pe && *pe == '0') ? 0 : 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e;
    switch (dtype) {
        case FP32: e = cudaLaunchKernelEx(&cfg, k_tp_allreduce<FP32>, a, y_dev); break;
        case FP16: e = cudaLaunchKernelEx(&cfg, k_tp_allreduce<FP16>, a, y_dev); break;
        default: e = cudaLaunchKernelEx(&cfg, k_tp_allreduce<BF16>, a, y_dev); break;
    }
    if (e != cudaSuccess) return tp_fail(DECDEC_E_CUDA, "tp: launch failed: %s", cudaGetErrorString(e));
    return 0;
}

int decdec_tp_status(uintptr_t comm, uint32_t* calls_out, uint32_t* error_out) {
    TpComm* c = reinterpret_cast<TpComm*>(comm);
    if (!c) return tp_fail(DECDEC_E_INVALID, "tp: null handle");
    uint32_t h[4] = {0, 0, 0, 0};
    cudaError_t e = cudaMemcpy(h, c->local, sizeof(h), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return tp_fail(DECDEC_E_CUDA, "tp: status read failed: %s", cudaGetErrorString(e));
    if (calls_out) *calls_out = h[0];
    if (error_out) *error_out = h[2];
    return 0;
}

int decdec_tp_destroy(uintptr_t comm) {
    TpComm* c = reinterpret_cast<TpComm*>(comm);
    if (!c) return 0;
    for (uint32_t s = 0; s < c->world; ++s)
        if (c->opened[s]) cudaIpcCloseMemHandle(c->peers[s]);
    if (c->local) cudaFree(c->local);
    delete c;
    return 0;
}

}  // extern "C"
