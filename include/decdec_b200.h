/*
 * decdec_b200 - C ABI of the B200 (sm_100a) implementation of the DecDEC decode hot path.
 *
 * Every entry point is what a foreign-function binding of the reference's `decdec_ext` module would
 * bind for that function: plain pointers, sizes, a dtype tag and a CUDA stream; no torch types.
 * "Reference" below is SNU-ARC/DecDEC; citations are paths inside that repository.
 *
 * Conventions
 *   - all functions return 0 on success, a negative DECDEC_E_* code on failure;
 *     decdec_last_error() gives the message of the last failure on the calling thread;
 *   - `dtype` is DECDEC_FP32 / DECDEC_FP16 / DECDEC_BF16 and names the element type of activations,
 *     outputs, scales, LUTs, alpha and q_bias of that call;
 *   - a linear layer is y[N] = W[N,K] x[K]; K = in_features, N = out_features;
 *   - every compute entry point ACCUMULATES into y (y += ...), like the reference kernels;
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued, never synchronised;
 *   - pointers named *_dev must be device-accessible, *_host must be host memory;
 *   - the library keeps one small accumulator workspace per (device, stream).  The first compute call on a
 *     device allocates (its own and sixteen spare ones, 2 MB each) and therefore must not happen during stream capture.
 *     A stream first seen while it is capturing takes a spare; when the spares are used up it shares the
 *     device's first workspace, and that graph must then not run concurrently with work on the owning stream.
 *     Calls that share a stream are ordered; calls on different streams use different workspaces.
 */
#ifndef DECDEC_B200_H
#define DECDEC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { DECDEC_FP32 = 0, DECDEC_FP16 = 1, DECDEC_BF16 = 2 };

enum {
    DECDEC_OK = 0,
    DECDEC_E_INVALID = -1,      /* bad argument (shape, dtype, alignment, null pointer) */
    DECDEC_E_UNSUPPORTED = -2,  /* valid in the reference but not implemented here */
    DECDEC_E_CUDA = -3,         /* a CUDA runtime call failed */
    DECDEC_E_NOMEM = -4,        /* allocation failed */
    DECDEC_E_DEVICE = -5        /* an earlier launch on the stream gave up on a bounded wait (see decdec_stream_status) */
};

/* Launch geometry of a config; replaces the dict of read_dec_config (dec_config.cu:337-354). */
typedef struct decdec_config_info {
    int32_t num_chunks;            /* ceil(K / 1024) */
    int32_t chunk_size;            /* 1024 */
    int32_t k_chunk;               /* channels selected per chunk */
    int32_t channels_per_tb;       /* packed residual columns (8 outputs each) per DEC thread block */
    int32_t n_tb;                  /* DEC thread blocks actually launched */
    int32_t block_dim_x;           /* 256 */
    int32_t block_dim_y;           /* 1 */
    int32_t shared_memory_size;    /* dynamic shared memory of a DEC-only launch, bytes */
    int32_t reduced_shared_memory; /* always 0: the reduced mode of the reference does not exist here */
} decdec_config_info;

const char* decdec_last_error(void);

/* Version / build probe: returns the compute capability the kernels were compiled for (100). */
int decdec_compiled_arch(void);

/* ---- device-side failures.  NO COUNTERPART IN THE REFERENCE (it ignores launch and device errors,
 * dec_config.cu:204-208).  Every wait inside the kernels of this library is bounded; a thread block that gives up
 * stores a code into the error word of the (device, stream) workspace: 1 = a wait for a shared-memory stage ran
 * out (DECDEC_PIPE_WAIT_NS, default 50 ms), 2 = the launch did not get the shared-memory layout it was sized for.
 * The output of that launch is then incomplete.  The word lives in mapped host memory, so every later compute call
 * on that stream sees it without a copy and fails with DECDEC_E_DEVICE until the stream is reset.
 *   decdec_stream_status  *error_out = the word (0 = fine); does not synchronise.
 *   decdec_stream_reset   waits for the stream, clears the word and the accumulator workspace. */
int decdec_stream_status(void* stream, uint32_t* error_out);
int decdec_stream_reset(void* stream);

/* ---- context (reference: create_dec_context, dec_context.cu:62-103) ------------------------------
 * num_tb: thread blocks given to the compensation role.  selected_rows_dev / selected_acts_dev:
 * caller-owned device buffers of `buffer_size` int32 / dtype elements; after a fused call they hold
 * the selection, before an unfused call the caller writes the rows there.  The context borrows them. */
int decdec_create_context(uint32_t num_tb, int32_t* selected_rows_dev, void* selected_acts_dev,
                          uint32_t buffer_size, int dtype, uintptr_t* out_ctx);
/* The reference has no destructor for contexts (they leak); this one is an addition. */
int decdec_destroy_context(uintptr_t ctx);

/* ---- config (reference: create/update/destroy/read_dec_config, dec_config.cu:247-354) -------------
 * q_residual: int32 [K, N/8] (packed 4-bit residual, cheatsheet.py:99-125).  If q_residual_on_device
 * is 0 the data is copied into pinned, device-mapped host memory owned by the config and fetched
 * zero-copy at run time; otherwise the device pointer is used as is (the reference prints a warning).
 * reordered_scales: dtype [N], layout [nibble][N/8]; copied into device memory owned by the config.
 * thresholds_host: dtype [K] on the host, BORROWED: entries [0] and [k-1] are read at every launch
 * (decdec.cu:66-67), so the caller keeps it alive. */
int decdec_create_config(uintptr_t ctx, uint32_t k_chunk, const int32_t* q_residual, int q_residual_on_device,
                         uint32_t K, uint32_t N, const void* reordered_scales, int scales_on_device,
                         const void* thresholds_host, int dtype, uintptr_t* out_cfg);
int decdec_update_config(uintptr_t cfg, uintptr_t new_ctx, uint32_t k_chunk);
int decdec_destroy_config(uintptr_t cfg);
int decdec_read_config(uintptr_t cfg, decdec_config_info* out);

/* ---- compensation alone (reference: dec / unfused_dec, decdec.cu:139-146, :238-245) ---------------
 * x_dev: dtype [K]; y_dev: dtype [N], accumulated into.  `dec` selects k_chunk channels per 1024
 * (bucket rule of dec.cu:78-182, ascending channel index inside a bucket) and publishes them in the
 * context buffers; `unfused_dec` takes the k rows the caller wrote into selected_rows_dev. */
int decdec_dec(uintptr_t cfg, const void* x_dev, void* y_dev, uint32_t K, uint32_t N, int dtype, void* stream);
int decdec_unfused_dec(uintptr_t cfg, const void* x_dev, void* y_dev, uint32_t K, uint32_t N, int dtype, void* stream);

/* ---- base GEMVs ------------------------------------------------------------------------------------
 * anyprec (reference: anyprec_gemv, decdec.cu:324-333): qweight int32 [planes >= bitwidth, N, K/32],
 *   lut dtype [N, 2^bitwidth]; bitwidth 3..8; fp16/bf16 only.  `planes` is the size of dim 0.
 * lutgemm (reference: lutgemm_gemv, decdec.cu:485-496): qweight int32 [K/32, bitwidth, N],
 *   alpha dtype [K/group, bitwidth, N], q_bias dtype [K/group, N]; bitwidth 1..8; N % 8 == 0.
 * sqllm (reference: sqllm_gemv, decdec.cu:594-603): qweight int32 [K*bitwidth/32, N],
 *   lut dtype [N, 2^bitwidth]; bitwidth 3 or 4. */
int decdec_anyprec_gemv(const void* x_dev, void* y_dev, const int32_t* qweight, uint32_t planes, const void* lut,
                        uint32_t N, uint32_t K, int bitwidth, int dtype, void* stream);
int decdec_lutgemm_gemv(const void* x_dev, void* y_dev, const int32_t* qweight, const void* alpha, const void* q_bias,
                        uint32_t N, uint32_t K, int bitwidth, int group_size, int dtype, void* stream);
int decdec_sqllm_gemv(const void* x_dev, void* y_dev, const int32_t* qweight, const void* lut,
                      uint32_t N, uint32_t K, int bitwidth, int dtype, void* stream);

/* lutgemm GEMV that allocates nothing.  NO COUNTERPART IN THE REFERENCE.
 * Same arguments and result as decdec_lutgemm_gemv.  The accumulator workspace that the other entry
 * points obtain with cudaMalloc is replaced by a fixed array inside the library (held by every GPU
 * that loads the library until the process exits), so the call is usable by hosts that may not call
 * cudaMalloc at that point: plug-ins of an application that owns all device memory, and real-time loops
 * that forbid calls which may synchronise the device.  Limits and duties of the caller:
 *   - out_features <= 32768, otherwise DECDEC_E_UNSUPPORTED;
 *   - the first call on a device resolves the array's address; make it before any stream capture;
 *   - all calls on one GPU share the array: calls that overlap in time on the GPU race. */
int decdec_lutgemm_gemv_noalloc(const void* x_dev, void* y_dev, const int32_t* qweight, const void* alpha,
                                const void* q_bias, uint32_t N, uint32_t K, int bitwidth, int group_size, int dtype,
                                void* stream);

/* Dense weights of a binary-coded layer for the prefill GEMM.  NO COUNTERPART IN THE REFERENCE BINDING: the reference
 * builds this tensor with a chain of torch ops on every prefill call (end-to-end/LUTGEMMLinear.py:41-82).
 * out_dev dtype [K, N] (in_features x out_features, the right operand of `x @ W`), same arithmetic as that
 * expression: the planes' +-alpha are summed, rounded to dtype, and q_bias is added in dtype. */
int decdec_lutgemm_dequant(const int32_t* qweight, const void* alpha, const void* q_bias, void* out_dev,
                           uint32_t N, uint32_t K, int bitwidth, int group_size, int dtype, void* stream);

/* ---- tensor-parallel output exchange.  NO COUNTERPART IN THE REFERENCE (it has no tensor parallelism). -------
 * One-shot push all-reduce of the [n] partial outputs of a row-parallel projection over NVLink peer memory:
 * every rank stores its vector into every peer's buffer as 16-byte lines that carry the call number beside the
 * payload (no fence, no separate flag), waits (bounded) for the peers' lines and sums in rank order, in one
 * kernel per rank.  Replaces ncclAllReduce for these 8-16 KB vectors.
 *
 *   decdec_tp_create       allocates this rank's exchange buffer on the current device; ipc_handle_out (64 bytes,
 *                          may be null) receives its cudaIpcMemHandle_t for the other processes.
 *   decdec_tp_connect_ipc  handles = [world][64] bytes, entry `rank` ignored: opens the peers' buffers.
 *   decdec_tp_connect_ptrs same, for buffers that are already addressable (several GPUs in one process).
 *   decdec_tp_allreduce    y_dev[n] <- sum over ranks, in place, on `stream`.  All ranks must make the same
 *                          sequence of calls with the same n.  Capturable in a CUDA graph.  n <= max_n,
 *                          n*sizeof(dtype) a multiple of 16, y_dev 16-byte aligned.
 *   decdec_tp_status       calls completed and the error word (1 = a wait ran out: a peer's lines did not arrive
 *                          within DECDEC_TP_WAIT_POLLS polls, default 2^21, about a second; that block's part of y was left unsummed).
 *   decdec_tp_layout       byte offsets inside an exchange buffer (call counters [world][64] u32 of which the first
 *                          row is used, slots [2][world][stride]; a slot is a sequence of lines {u32 payload, u32 call,
 *                          u32 payload, u32 call}).
 */
int decdec_tp_layout(uint32_t world, uint32_t max_n, size_t* flags_off, size_t* slots_off, size_t* slot_stride, size_t* bytes);
int decdec_tp_create(uint32_t world, uint32_t rank, uint32_t max_n, uintptr_t* comm_out, unsigned char* ipc_handle_out);
int decdec_tp_local_ptr(uintptr_t comm, void** ptr_out);
int decdec_tp_connect_ipc(uintptr_t comm, const unsigned char* handles);
int decdec_tp_connect_ptrs(uintptr_t comm, const uintptr_t* peer_ptrs);
int decdec_tp_allreduce(uintptr_t comm, void* y_dev, uint32_t n, int dtype, void* stream);
int decdec_tp_status(uintptr_t comm, uint32_t* calls_out, uint32_t* error_out);
int decdec_tp_destroy(uintptr_t comm);

/* anyprec_dequant (reference: decdec.cu:386-393): out_dev dtype [N, K] dense weights. */
int decdec_anyprec_dequant(const int32_t* qweight, const void* lut, void* out_dev,
                           uint32_t N, uint32_t K, int bitwidth, int dtype, void* stream);

/* ---- fused: base GEMV + compensation in ONE launch (reference: dec_anyprec / dec_lutgemm /
 * dec_sqllm, decdec.cu:609-779, which fork the GEMV onto a second stream).  The first thread blocks
 * of the grid run the compensation role, the rest the GEMV; both add into the same fp32
 * accumulator, rounded once into y. */
int decdec_dec_anyprec(uintptr_t cfg, const void* x_dev, void* y_dev, const int32_t* qweight, uint32_t planes,
                       const void* lut, uint32_t N, uint32_t K, int bitwidth, int dtype, void* stream);
int decdec_dec_lutgemm(uintptr_t cfg, const void* x_dev, void* y_dev, const int32_t* qweight, const void* alpha,
                       const void* q_bias, uint32_t N, uint32_t K, int bitwidth, int group_size, int dtype, void* stream);
int decdec_dec_sqllm(uintptr_t cfg, const void* x_dev, void* y_dev, const int32_t* qweight, const void* lut,
                     uint32_t N, uint32_t K, int bitwidth, int dtype, void* stream);

/* ---- GEMV next to an SM-occupying busy kernel (reference: dummy_anyprec / dummy_lutgemm /
 * dummy_sqllm, decdec.cu:874-1013): `dummy_sm` blocks of 1024 threads spin for `dummy_iters`
 * iterations on `stream` while the GEMV runs on a library-owned side stream; joined before return. */
int decdec_dummy_anyprec(const void* x_dev, void* y_dev, const int32_t* qweight, uint32_t planes, const void* lut,
                         uint32_t N, uint32_t K, int bitwidth, int dtype, int dummy_sm, long long dummy_iters, void* stream);
int decdec_dummy_lutgemm(const void* x_dev, void* y_dev, const int32_t* qweight, const void* alpha, const void* q_bias,
                         uint32_t N, uint32_t K, int bitwidth, int group_size, int dtype, int dummy_sm,
                         long long dummy_iters, void* stream);
int decdec_dummy_sqllm(const void* x_dev, void* y_dev, const int32_t* qweight, const void* lut,
                       uint32_t N, uint32_t K, int bitwidth, int dtype, int dummy_sm, long long dummy_iters, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DECDEC_B200_H */
