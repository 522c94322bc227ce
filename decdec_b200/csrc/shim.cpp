// decdec_ext: the Python module of the reference (decdec_extension/bindings.cpp:17-41), rebuilt as a
// thin torch/pybind11 shim over the C ABI of libdecdec_b200.so.  It checks tensors the way the
// reference's host launchers do (decdec_extension/decdec.cu, dec_config.cu, dec_context.cu), takes
// pointers, sizes and the current CUDA stream from torch, and translates status codes into the
// RuntimeError the reference raises through TORCH_CHECK.  No kernels live here.
#include <torch/extension.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <pybind11/stl.h>

#include <mutex>
#include <unordered_map>

#include "decdec_b200.h"

namespace {

int dt_of(const torch::Tensor& t) {
    switch (t.scalar_type()) {
        case at::kFloat: return DECDEC_FP32;
        case at::kHalf: return DECDEC_FP16;
        case at::kBFloat16: return DECDEC_BF16;
        default: TORCH_CHECK(false, "Unsupported data type."); return -1;
    }
}

void ok(int code) { TORCH_CHECK(code == 0, decdec_last_error()); }

void* cur_stream() { return static_cast<void*>(c10::cuda::getCurrentCUDAStream().stream()); }

// tensors the C side borrows; the reference leaves their lifetime to the caller, keeping a reference
// here costs nothing and removes a class of use-after-free
std::mutex g_mu;
std::unordered_map<uintptr_t, std::vector<torch::Tensor>> g_keep;

void io_checks(const torch::Tensor& input, const torch::Tensor& output) {
    TORCH_CHECK(input.scalar_type() == output.scalar_type(), "Mismatched data types between input and output tensors. input type: ",
                input.scalar_type(), ", output type: ", output.scalar_type());
    TORCH_CHECK(input.is_cuda() && output.is_cuda(), "input and output tensors must be on GPU.");
    TORCH_CHECK(input.dim() == 3, "input tensor must be of shape (batch_size, seq_len, hidden_size).");
    TORCH_CHECK(output.dim() == 3, "output tensor must be of shape (batch_size, seq_len, hidden_size).");
    TORCH_CHECK(input.size(0) == 1, "Batch size must be 1 for input tensor.");
    TORCH_CHECK(output.size(0) == 1, "Batch size must be 1 for output tensor.");
    TORCH_CHECK(input.size(1) == 1, "Sequence length must be 1 for input tensor.");
    TORCH_CHECK(output.size(1) == 1, "Sequence length must be 1 for output tensor.");
    TORCH_CHECK(input.is_contiguous(), "input tensor must be contiguous.");
    TORCH_CHECK(output.is_contiguous(), "output tensor must be contiguous.");
}

// ---- context / config ---------------------------------------------------------------------------------

uintptr_t create_dec_context(uint32_t num_tb, torch::Tensor rows, torch::Tensor acts) {
    TORCH_CHECK(rows.is_cuda(), "selected_rows_buffer must be on GPU.");
    TORCH_CHECK(acts.is_cuda(), "selected_activations_buffer must be on GPU.");
    TORCH_CHECK(rows.numel() == acts.numel(), "selected_rows_buffer and selected_activations_buffer must be of the same size.");
    TORCH_CHECK(rows.scalar_type() == at::kInt, "selected_rows_buffer must be of type int.");
    TORCH_CHECK(rows.is_contiguous(), "selected_rows_buffer must be contiguous.");
    TORCH_CHECK(acts.is_contiguous(), "selected_activations_buffer must be contiguous.");
    c10::cuda::CUDAGuard guard(rows.device());
    uintptr_t h = 0;
    ok(decdec_create_context(num_tb, rows.data_ptr<int32_t>(), acts.data_ptr(), (uint32_t)acts.numel(), dt_of(acts), &h));
    std::lock_guard<std::mutex> lk(g_mu);
    g_keep[h] = {rows, acts};
    return h;
}

uintptr_t create_dec_config(uintptr_t ctx, uint32_t k_chunk, torch::Tensor q_residual, torch::Tensor scales, torch::Tensor thresholds) {
    TORCH_CHECK(thresholds.is_cpu(), "thresholds must be on CPU.");
    TORCH_CHECK(scales.scalar_type() == thresholds.scalar_type(), "reordered_scales and thresholds must have the same data type.");
    TORCH_CHECK(q_residual.scalar_type() == at::kInt, "q_residual must be of type int.");
    TORCH_CHECK(q_residual.is_contiguous(), "q_residual must be contiguous.");
    TORCH_CHECK(scales.is_contiguous(), "reordered_scales must be contiguous.");
    TORCH_CHECK(thresholds.is_contiguous(), "thresholds must be contiguous.");
    TORCH_CHECK(q_residual.dim() == 2 && scales.dim() == 1, "q_residual must be [K, N/8] and reordered_scales [N].");
    const uint32_t K = (uint32_t)q_residual.size(0), N = (uint32_t)scales.size(0);
    TORCH_CHECK((uint64_t)q_residual.size(1) * 8 == N, "q_residual must have out_features / 8 columns.");
    TORCH_CHECK(thresholds.numel() >= K, "thresholds must have in_features entries.");
    if (q_residual.is_cuda()) {
        printf("DecDEC WARNING: q_residual is on GPU. This is NOT the intended setup; zero-copy memory will NOT be used.\n");
    }
    c10::cuda::OptionalCUDAGuard guard;
    if (q_residual.is_cuda()) guard.set_device(q_residual.device());
    else if (scales.is_cuda()) guard.set_device(scales.device());
    else {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = g_keep.find(ctx);
        if (it != g_keep.end()) guard.set_device(it->second[0].device());
    }
    uintptr_t h = 0;
    ok(decdec_create_config(ctx, k_chunk, q_residual.data_ptr<int32_t>(), q_residual.is_cuda() ? 1 : 0, K, N, scales.data_ptr(),
                            scales.is_cuda() ? 1 : 0, thresholds.data_ptr(), dt_of(scales), &h));
    std::lock_guard<std::mutex> lk(g_mu);
    g_keep[h] = {thresholds};
    if (q_residual.is_cuda()) g_keep[h].push_back(q_residual);
    return h;
}

std::unordered_map<std::string, int> read_dec_config(uintptr_t cfg) {
    decdec_config_info i;
    ok(decdec_read_config(cfg, &i));
    return {{"num_chunks", i.num_chunks}, {"chunk_size", i.chunk_size}, {"k_chunk", i.k_chunk},
            {"channels_per_tb", i.channels_per_tb}, {"n_tb", i.n_tb}, {"block_dim_x", i.block_dim_x},
            {"block_dim_y", i.block_dim_y}, {"shared_memory_size", i.shared_memory_size},
            {"reduced_shared_memory", i.reduced_shared_memory}};
}

void update_dec_config(uintptr_t cfg, uintptr_t new_ctx, uint32_t k_chunk) { ok(decdec_update_config(cfg, new_ctx, k_chunk)); }

void destroy_dec_config(uintptr_t cfg) {
    ok(decdec_destroy_config(cfg));
    std::lock_guard<std::mutex> lk(g_mu);
    g_keep.erase(cfg);
}

// ---- compensation alone --------------------------------------------------------------------------------

void dec(uintptr_t cfg, torch::Tensor input, torch::Tensor output) {
    io_checks(input, output);
    c10::cuda::CUDAGuard guard(input.device());
    ok(decdec_dec(cfg, input.data_ptr(), output.data_ptr(), (uint32_t)input.size(2), (uint32_t)output.size(2), dt_of(input), cur_stream()));
}

void unfused_dec(uintptr_t cfg, torch::Tensor input, torch::Tensor output) {
    io_checks(input, output);
    c10::cuda::CUDAGuard guard(input.device());
    ok(decdec_unfused_dec(cfg, input.data_ptr(), output.data_ptr(), (uint32_t)input.size(2), (uint32_t)output.size(2), dt_of(input), cur_stream()));
}

// ---- base GEMVs -----------------------------------------------------------------------------------------

void anyprec_checks(const torch::Tensor& input, const torch::Tensor& output, const torch::Tensor& qweight, const torch::Tensor& lut, int bitwidth) {
    TORCH_CHECK(bitwidth >= 3 && bitwidth <= 8, "Bitwidth must be between 3 and 8.");
    TORCH_CHECK(input.scalar_type() == lut.scalar_type() && input.scalar_type() == output.scalar_type(),
                "Mismatched data types between input, lut, and output tensors.");
    TORCH_CHECK(qweight.scalar_type() == at::kInt, "qweight tensor must be of type int.");
    io_checks(input, output);
    TORCH_CHECK(lut.dim() == 2 && lut.size(1) == (1 << bitwidth) && lut.size(0) == output.size(2),
                "lut tensor must be of shape (output_feat, 2 ** bitwidth). Expected (", output.size(2), ", ", 1 << bitwidth, ").");
    TORCH_CHECK(qweight.dim() == 3 && qweight.size(0) >= bitwidth && qweight.size(2) == input.size(2) / 32 && qweight.size(1) == output.size(2),
                "qweight tensor must be of shape (>=bitwidth, output_feat, input_feat / 32). Expected (>=", bitwidth, ", ", output.size(2), ", ", input.size(2) / 32, ").");
    TORCH_CHECK(qweight.is_contiguous(), "qweight tensor must be contiguous.");
    TORCH_CHECK(lut.is_contiguous(), "lut tensor must be contiguous.");
    TORCH_CHECK(input.scalar_type() != at::kFloat, "Any-Precision GEMV does not support float data type. Please use half or bfloat16.");
}

void anyprec_gemv(torch::Tensor input, torch::Tensor output, torch::Tensor qweight, torch::Tensor lut, int bitwidth) {
    anyprec_checks(input, output, qweight, lut, bitwidth);
    c10::cuda::CUDAGuard guard(input.device());
    ok(decdec_anyprec_gemv(input.data_ptr(), output.data_ptr(), qweight.data_ptr<int32_t>(), (uint32_t)qweight.size(0), lut.data_ptr(),
                           (uint32_t)output.size(2), (uint32_t)input.size(2), bitwidth, dt_of(input), cur_stream()));
}

torch::Tensor anyprec_dequant(torch::Tensor qweight, torch::Tensor lut, int bitwidth) {
    TORCH_CHECK(lut.scalar_type() != at::kFloat, "Any-Precision Dequantization does not support float data type. Please use half or bfloat16.");
    TORCH_CHECK(qweight.dim() == 3 && qweight.scalar_type() == at::kInt && qweight.is_cuda() && lut.is_cuda(), "qweight must be a 3-D int tensor on GPU");
    const int64_t N = qweight.size(1), K = qweight.size(2) * 32;
    c10::cuda::CUDAGuard guard(qweight.device());
    auto weight = torch::empty({N, K}, torch::TensorOptions().dtype(lut.dtype()).device(qweight.device()));
    ok(decdec_anyprec_dequant(qweight.data_ptr<int32_t>(), lut.data_ptr(), weight.data_ptr(), (uint32_t)N, (uint32_t)K, bitwidth, dt_of(lut), cur_stream()));
    return weight;
}

void lutgemm_checks(const torch::Tensor& input, const torch::Tensor& output, const torch::Tensor& q_weight, const torch::Tensor& alpha,
                    const torch::Tensor& q_bias, int bitwidth, int group_size) {
    TORCH_CHECK(bitwidth >= 1 && bitwidth <= 8, "Bitwidth must be between 1 and 8.");
    TORCH_CHECK(input.scalar_type() == alpha.scalar_type() && input.scalar_type() == q_bias.scalar_type() && input.scalar_type() == output.scalar_type(),
                "Mismatched data types between input, alpha, q_bias, and output tensors.");
    io_checks(input, output);
    TORCH_CHECK(q_weight.is_contiguous(), "q_weight tensor must be contiguous.");
    TORCH_CHECK(alpha.is_contiguous(), "alpha tensor must be contiguous.");
    TORCH_CHECK(q_bias.is_contiguous(), "q_bias tensor must be contiguous.");
    TORCH_CHECK(group_size > 0, "group_size must be positive.");
    const int64_t k = input.size(2), m = output.size(2), groups = k / group_size;
    TORCH_CHECK(q_weight.dim() == 3 && q_weight.size(0) == k / 32 && q_weight.size(1) == bitwidth && q_weight.size(2) == m,
                "q_weight tensor must be of shape (input_feat / 32, bitwidth, output_feat). Expected (", k / 32, ", ", bitwidth, ", ", m, ").");
    TORCH_CHECK(alpha.dim() == 3 && alpha.size(0) == groups && alpha.size(1) == bitwidth && alpha.size(2) == m,
                "alpha tensor must be of shape (num_groups, bitwidth, output_feat). Expected (", groups, ", ", bitwidth, ", ", m, ").");
    TORCH_CHECK(q_bias.dim() == 2 && q_bias.size(0) == groups && q_bias.size(1) == m, "q_bias tensor must be of shape (num_groups, output_feat).");
}

void lutgemm_gemv(torch::Tensor input, torch::Tensor output, torch::Tensor q_weight, torch::Tensor alpha, torch::Tensor q_bias, int bitwidth, int group_size) {
    lutgemm_checks(input, output, q_weight, alpha, q_bias, bitwidth, group_size);
    c10::cuda::CUDAGuard guard(input.device());
    ok(decdec_lutgemm_gemv(input.data_ptr(), output.data_ptr(), q_weight.data_ptr<int32_t>(), alpha.data_ptr(), q_bias.data_ptr(),
                           (uint32_t)output.size(2), (uint32_t)input.size(2), bitwidth, group_size, dt_of(input), cur_stream()));
}

void sqllm_checks(const torch::Tensor& input, const torch::Tensor& output, const torch::Tensor& qweight, const torch::Tensor& lut, int bitwidth) {
    TORCH_CHECK(bitwidth == 3 || bitwidth == 4, "Bitwidth must be 3 or 4.");
    TORCH_CHECK(input.scalar_type() == lut.scalar_type() && input.scalar_type() == output.scalar_type(),
                "Mismatched data types between input, lut, and output tensors.");
    TORCH_CHECK(qweight.scalar_type() == at::kInt, "qweight tensor must be of type int.");
    io_checks(input, output);
    TORCH_CHECK(lut.dim() == 2 && lut.size(1) == (1 << bitwidth) && lut.size(0) == output.size(2), "lut tensor must be of shape (output_feat, 2 ** bitwidth).");
    TORCH_CHECK(qweight.dim() == 2 && qweight.size(1) == lut.size(0) && qweight.size(0) == input.size(2) * bitwidth / 32,
                "qweight tensor must be of shape (input_feat * bitwidth / 32, output_feat).");
    TORCH_CHECK(qweight.is_contiguous(), "qweight tensor must be contiguous.");
    TORCH_CHECK(lut.is_contiguous(), "lut tensor must be contiguous.");
}

void sqllm_gemv(torch::Tensor input, torch::Tensor output, torch::Tensor qweight, torch::Tensor lut, int bitwidth) {
    sqllm_checks(input, output, qweight, lut, bitwidth);
    c10::cuda::CUDAGuard guard(input.device());
    ok(decdec_sqllm_gemv(input.data_ptr(), output.data_ptr(), qweight.data_ptr<int32_t>(), lut.data_ptr(), (uint32_t)output.size(2),
                         (uint32_t)input.size(2), bitwidth, dt_of(input), cur_stream()));
}

// ---- fused ------------------------------------------------------------------------------------------------

void dec_anyprec(uintptr_t cfg, torch::Tensor input, torch::Tensor output, torch::Tensor qweight, torch::Tensor lut, int bitwidth) {
    TORCH_CHECK(input.scalar_type() == at::kHalf || input.scalar_type() == at::kBFloat16, "Unsupported data type.");
    anyprec_checks(input, output, qweight, lut, bitwidth);
    c10::cuda::CUDAGuard guard(input.device());
    ok(decdec_dec_anyprec(cfg, input.data_ptr(), output.data_ptr(), qweight.data_ptr<int32_t>(), (uint32_t)qweight.size(0), lut.data_ptr(),
                          (uint32_t)output.size(2), (uint32_t)input.size(2), bitwidth, dt_of(input), cur_stream()));
}

void dec_lutgemm(uintptr_t cfg, torch::Tensor input, torch::Tensor output, torch::Tensor q_weight, torch::Tensor alpha, torch::Tensor q_bias,
                 int bitwidth, int group_size) {
    lutgemm_checks(input, output, q_weight, alpha, q_bias, bitwidth, group_size);
    c10::cuda::CUDAGuard guard(input.device());
    ok(decdec_dec_lutgemm(cfg, input.data_ptr(), output.data_ptr(), q_weight.data_ptr<int32_t>(), alpha.data_ptr(), q_bias.data_ptr(),
                          (uint32_t)output.size(2), (uint32_t)input.size(2), bitwidth, group_size, dt_of(input), cur_stream()));
}

void dec_sqllm(uintptr_t cfg, torch::Tensor input, torch::Tensor output, torch::Tensor q_weight, torch::Tensor lut, int bitwidth) {
    sqllm_checks(input, output, q_weight, lut, bitwidth);
    c10::cuda::CUDAGuard guard(input.device());
    ok(decdec_dec_sqllm(cfg, input.data_ptr(), output.data_ptr(), q_weight.data_ptr<int32_t>(), lut.data_ptr(), (uint32_t)output.size(2),
                        (uint32_t)input.size(2), bitwidth, dt_of(input), cur_stream()));
}

// ---- GEMV beside the busy kernel ----------------------------------------------------------------------------

void dummy_anyprec(torch::Tensor input, torch::Tensor output, torch::Tensor qweight, torch::Tensor lut, int bitwidth, int dummy_sm, long long dummy_iters) {
    TORCH_CHECK(input.scalar_type() == at::kHalf || input.scalar_type() == at::kBFloat16, "dummy_anyprec supports FP16/BF16 only.");
    anyprec_checks(input, output, qweight, lut, bitwidth);
    c10::cuda::CUDAGuard guard(input.device());
    ok(decdec_dummy_anyprec(input.data_ptr(), output.data_ptr(), qweight.data_ptr<int32_t>(), (uint32_t)qweight.size(0), lut.data_ptr(),
                            (uint32_t)output.size(2), (uint32_t)input.size(2), bitwidth, dt_of(input), dummy_sm, dummy_iters, cur_stream()));
}

void dummy_lutgemm(torch::Tensor input, torch::Tensor output, torch::Tensor qweight, torch::Tensor alpha, torch::Tensor qbias, int bitwidth,
                   int group_size, int dummy_sm, long long dummy_iters) {
    lutgemm_checks(input, output, qweight, alpha, qbias, bitwidth, group_size);
    c10::cuda::CUDAGuard guard(input.device());
    ok(decdec_dummy_lutgemm(input.data_ptr(), output.data_ptr(), qweight.data_ptr<int32_t>(), alpha.data_ptr(), qbias.data_ptr(),
                            (uint32_t)output.size(2), (uint32_t)input.size(2), bitwidth, group_size, dt_of(input), dummy_sm, dummy_iters, cur_stream()));
}

void dummy_sqllm(torch::Tensor input, torch::Tensor output, torch::Tensor qweight, torch::Tensor lut, int bitwidth, int dummy_sm, long long dummy_iters) {
    TORCH_CHECK(bitwidth == 3 || bitwidth == 4, "SQLLM bitwidth must be 3 or 4.");
    sqllm_checks(input, output, qweight, lut, bitwidth);
    c10::cuda::CUDAGuard guard(input.device());
    ok(decdec_dummy_sqllm(input.data_ptr(), output.data_ptr(), qweight.data_ptr<int32_t>(), lut.data_ptr(), (uint32_t)output.size(2),
                          (uint32_t)input.size(2), bitwidth, dt_of(input), dummy_sm, dummy_iters, cur_stream()));
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("create_dec_context", &create_dec_context, "Create DECContext (returns pointer)");
    m.def("create_dec_config", &create_dec_config, "Create DECConfig (returns pointer)");
    m.def("read_dec_config", &read_dec_config, "Read info from a DECConfig pointer");
    m.def("update_dec_config", &update_dec_config, "Update a DECConfig pointer");
    m.def("destroy_dec_config", &destroy_dec_config, "Destroy a DECConfig pointer");
    m.def("dec", &dec, "standalone DEC");
    m.def("unfused_dec", &unfused_dec, "DEC without row selection, for testing purposes");
    m.def("anyprec_dequant", &anyprec_dequant, "ANYPREC dequantization");
    m.def("anyprec_gemv", &anyprec_gemv, "ANYPREC GEMV");
    m.def("lutgemm_gemv", &lutgemm_gemv, "LUTGEMM GEMV");
    m.def("sqllm_gemv", &sqllm_gemv, "SQLLM GEMV");
    m.def("dec_anyprec", &dec_anyprec, "ANYPREC with DEC");
    m.def("dec_lutgemm", &dec_lutgemm, "LUTGEMM with DEC");
    m.def("dec_sqllm", &dec_sqllm, "SQLLM with DEC");
    m.def("dummy_anyprec", &dummy_anyprec, "ANYPREC GEMV with dummy SM blocker");
    m.def("dummy_lutgemm", &dummy_lutgemm, "LUTGEMM GEMV with dummy SM blocker");
    m.def("dummy_sqllm", &dummy_sqllm, "SQLLM GEMV with dummy SM blocker");
}
