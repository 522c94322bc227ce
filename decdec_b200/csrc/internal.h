// Internal launch interface between the host-side API (host.cu) and the kernel translation units.
#pragma once
#include "common.cuh"
#include "gemv_bcq.cuh"
#include "gemv_anyprec.cuh"
#include "gemv_sqllm.cuh"
#include "gemv_bcq_pipe.cuh"
#include "gemv_anyprec_pipe.cuh"

namespace dd {

// Each launcher starts ONE grid: blocks [0, d.n_cta) run the compensation role, the rest the GEMV.
cudaError_t launch_dec_only(int dt, const DecParams& d, const FinParams& f, cudaStream_t s);
cudaError_t launch_bcq(int dt, const BcqParams& g, const DecParams& d, const FinParams& f, cudaStream_t s);
bool bcq_pipe_geometry(uint32_t N, uint32_t K, uint32_t bits, uint32_t group, int dt, uint32_t n_kslices, PipeGeom* geo,
                       uint32_t sm_budget);   // SMs the GEMV thread blocks may fill in one wave
cudaError_t launch_bcq_pipe(int dt, const BcqParams& g, const DecParams& d, const FinParams& f, const PipeGeom& geo, cudaStream_t s);
cudaError_t launch_anyprec(int dt, const ApParams& g, const DecParams& d, const FinParams& f, cudaStream_t s);
bool anyprec_pipe_geometry(uint32_t N, uint32_t K, uint32_t bits, ApPipeGeom* geo, uint32_t sm_budget = 148, bool gemv_only = false);
cudaError_t launch_anyprec_pipe(int dt, const ApParams& g, const DecParams& d, const FinParams& f, const ApPipeGeom& geo, cudaStream_t s);
cudaError_t launch_sqllm(int dt, const SqParams& g, const DecParams& d, const FinParams& f, cudaStream_t s);
cudaError_t launch_ap_dequant(int dt, const uint32_t* qweight, const void* lut, void* out, uint32_t N, uint32_t K,
                              uint32_t bits, cudaStream_t s);
cudaError_t launch_bcq_dequant(int dt, const uint32_t* qweight, const void* alpha, const void* q_bias, void* out, uint32_t N,
                               uint32_t K, uint32_t bits, uint32_t group, cudaStream_t s);
cudaError_t launch_burner(int blocks, long long iters, cudaStream_t s);

int set_last_error(int code, const char* msg);
uint32_t device_sms();
size_t dec_only_smem();
size_t anyprec_smem(uint32_t K, bool fast3);
size_t sqllm_smem(uint32_t K);

}  // namespace dd
