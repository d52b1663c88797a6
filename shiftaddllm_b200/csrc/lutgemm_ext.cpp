// The compiled `lutgemm` extension module: the five functions the reference's extension exports
// (lut_gemm/lutgemm_cuda.cpp:43-98, registered at :225-230), same names, argument order and
// accumulate-into-`output` contract, bound to the sm_100a library behind the C ABI of
// include/sal_lutgemm.h.  It replaces lut_gemm/lutgemm_cuda.cpp + lut_gemm/setup_lut.py: reference code
// that does `import lutgemm` (lut_gemm/quant.py:5) runs on it unchanged.
//
// Deliberate differences from the reference's module: arguments are checked (dtype, device,
// contiguity, sizes) and a bad call raises instead of reading out of bounds; the kernels go to torch's
// current stream (the reference launches on the legacy default stream, mv_fp16_bias.hpp:591-645); the
// GIL is released around each call; every entry point takes batch inputs (M > 1 rows).
// There is no CPU path: CPU tensors are refused.

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <map>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "sal_lutgemm.h"

namespace {

void require(const torch::Tensor &t, c10::ScalarType dtype, const char *name) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor (there is no CPU path)");
    TORCH_CHECK(t.scalar_type() == dtype, name, " must have dtype ", c10::toString(dtype), ", got ", c10::toString(t.scalar_type()));
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

void check_status(int rc, const char *what) {
    if (rc == SAL_OK) return;
    std::string msg = std::string(what) + " failed: " + sal_status_string(rc) + " (status " + std::to_string(rc) + ")";
    if (rc == SAL_E_LAUNCH) msg += std::string("; CUDA: ") + sal_last_cuda_error();
    TORCH_CHECK(false, msg);
}

// Zero-filled scratch for the split-K reduction, one buffer per (device, stream), grown on demand.
// Calls on one stream are ordered, so one buffer per stream is race-free.  Outgrown buffers are kept:
// a CUDA graph captured earlier may still name them.
struct Scratch {
    std::mutex mutex;
    std::map<std::pair<int, void *>, torch::Tensor> current;
    std::vector<torch::Tensor> outgrown;

    torch::Tensor get(int device, void *stream, size_t need) {
        std::lock_guard<std::mutex> lock(mutex);
        auto key = std::make_pair(device, stream);
        auto it = current.find(key);
        if (it != current.end() && (size_t)it->second.numel() >= need) return it->second;
        if (it != current.end()) outgrown.push_back(it->second);
        torch::Tensor ws = torch::zeros({(int64_t)need}, torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCUDA, device));
        current[key] = ws;
        return ws;
    }
};
Scratch g_scratch;

struct Call {
    const void *bw, *alpha, *x;
    void *y;
    int M, K, N, q;
    torch::Tensor ws;
    void *stream;
};

// Common checks of the reference's argument list; returns the raw pointers, the row count and the scratch.
Call prepare(const torch::Tensor &output, const torch::Tensor &bWeight, const torch::Tensor &alpha, c10::ScalarType alpha_dtype,
             const torch::Tensor &d_input, int mSize, int kSize, int nb, int64_t alpha_numel) {
    require(output, torch::kFloat16, "output");
    require(bWeight, torch::kInt32, "bWeight");
    require(alpha, alpha_dtype, "alpha");
    require(d_input, torch::kFloat16, "d_input");
    const int64_t n = mSize, k = kSize, q = nb;
    TORCH_CHECK(n > 0 && k > 0 && q > 0 && k % 32 == 0, "mSize, kSize, nb must be positive and kSize a multiple of 32");
    TORCH_CHECK(bWeight.numel() == (k / 32) * q * n, "bWeight must hold (kSize/32)*nb*mSize = ", (k / 32) * q * n, " words, has ", bWeight.numel());
    TORCH_CHECK(alpha.numel() == alpha_numel, "alpha must hold ", alpha_numel, " elements, has ", alpha.numel());
    TORCH_CHECK(d_input.numel() % k == 0 && output.numel() % n == 0, "input/output sizes do not match kSize/mSize");
    const int64_t m = d_input.numel() / k;
    TORCH_CHECK(output.numel() / n == m, "output holds ", output.numel() / n, " rows but input holds ", m);
    const auto dev = output.device();
    TORCH_CHECK(bWeight.device() == dev && alpha.device() == dev && d_input.device() == dev, "all tensors must live on the same device");
    Call c;
    c.bw = bWeight.data_ptr();
    c.alpha = alpha.data_ptr();
    c.x = d_input.data_ptr();
    c.y = output.data_ptr();
    c.M = (int)m, c.K = (int)k, c.N = (int)n, c.q = (int)q;
    c10::cuda::CUDAGuard guard(dev);
    c.stream = at::cuda::getCurrentCUDAStream(dev.index()).stream();
    c.ws = g_scratch.get(dev.index(), c.stream, sal_workspace_bytes(c.M, c.N));
    return c;
}

// output += sum_b alpha[g,b,:] * (B_b^T x); alpha fp16 [num_groups, nb, mSize]  (lutgemm_cuda.cpp:43-52)
void lutgemm_compute_shift_scale(torch::Tensor output, torch::Tensor bWeight, torch::Tensor alpha, torch::Tensor d_input, int mSize,
                                 int kSize, int nb, int num_groups) {
    Call c = prepare(output, bWeight, alpha, torch::kFloat16, d_input, mSize, kSize, nb, (int64_t)num_groups * nb * mSize);
    c10::cuda::CUDAGuard guard(output.device());
    check_status(sal_lutgemv_shift_scale(c.bw, c.alpha, nullptr, c.x, c.y, c.M, c.K, c.N, c.q, num_groups, SAL_ACCUMULATE,
                                         c.ws.data_ptr(), (size_t)c.ws.numel(), c.stream),
                 "lutgemm_compute_shift_scale");
}

// alpha, q_bias fp16 [num_groups, mSize]; plane b scaled by alpha / 2**(b+1)  (lutgemm_cuda.cpp:88-98)
void lutgemm_compute(torch::Tensor output, torch::Tensor bWeight, torch::Tensor alpha, torch::Tensor q_bias, torch::Tensor d_input,
                     int mSize, int kSize, int nb, int num_groups) {
    require(q_bias, torch::kFloat16, "q_bias");
    TORCH_CHECK(q_bias.numel() == (int64_t)num_groups * mSize, "q_bias must hold num_groups*mSize elements");
    Call c = prepare(output, bWeight, alpha, torch::kFloat16, d_input, mSize, kSize, nb, (int64_t)num_groups * mSize);
    c10::cuda::CUDAGuard guard(output.device());
    check_status(sal_lutgemv_compute(c.bw, c.alpha, q_bias.data_ptr(), nullptr, c.x, c.y, c.M, c.K, c.N, c.q, num_groups, SAL_ACCUMULATE,
                                     c.ws.data_ptr(), (size_t)c.ws.numel(), c.stream),
                 "lutgemm_compute");
}

// alpha fp16 [kSize/8, nb, num_groups]  (lutgemm_cuda.cpp:54-63)
void lutgemm_compute_block(torch::Tensor output, torch::Tensor bWeight, torch::Tensor alpha, torch::Tensor d_input, int mSize, int kSize,
                           int nb, int num_groups) {
    Call c = prepare(output, bWeight, alpha, torch::kFloat16, d_input, mSize, kSize, nb, (int64_t)(kSize / 8) * nb * num_groups);
    c10::cuda::CUDAGuard guard(output.device());
    check_status(sal_lutgemm_block(c.bw, c.alpha, nullptr, c.x, c.y, c.M, c.K, c.N, c.q, num_groups, SAL_ACCUMULATE, c.ws.data_ptr(),
                                   (size_t)c.ws.numel(), c.stream),
                 "lutgemm_compute_block");
}

// alpha int16 [kSize/8, nb, num_groups], three 3-bit exponents  (lutgemm_cuda.cpp:65-74)
void lutgemm_compute_block_shift(torch::Tensor output, torch::Tensor bWeight, torch::Tensor alpha, torch::Tensor d_input, int mSize,
                                 int kSize, int nb, int num_groups, int num_apot) {
    (void)num_apot;  // fixed at three fields by the encoding, as in the reference kernel (mv_fp16_bias.hpp:294-297)
    Call c = prepare(output, bWeight, alpha, torch::kInt16, d_input, mSize, kSize, nb, (int64_t)(kSize / 8) * nb * num_groups);
    c10::cuda::CUDAGuard guard(output.device());
    check_status(sal_lutgemm_block_shift(c.bw, c.alpha, nullptr, c.x, c.y, c.M, c.K, c.N, c.q, num_groups, SAL_ACCUMULATE,
                                         c.ws.data_ptr(), (size_t)c.ws.numel(), c.stream),
                 "lutgemm_compute_block_shift");
}

// alpha int8 [kSize/8, nb, num_groups, num_apot]; -128 = no term  (lutgemm_cuda.cpp:76-85): the call of LutLinear.forward
void lutgemm_compute_block_shiftInt8(torch::Tensor output, torch::Tensor bWeight, torch::Tensor alpha, torch::Tensor d_input, int mSize,
                                     int kSize, int nb, int num_groups, int num_apot) {
    Call c = prepare(output, bWeight, alpha, torch::kInt8, d_input, mSize, kSize, nb, (int64_t)(kSize / 8) * nb * num_groups * num_apot);
    c10::cuda::CUDAGuard guard(output.device());
    check_status(sal_lutgemm_block_shift_int8(c.bw, c.alpha, nullptr, c.x, c.y, c.M, c.K, c.N, c.q, num_groups, num_apot, SAL_ACCUMULATE,
                                              c.ws.data_ptr(), (size_t)c.ws.numel(), c.stream),
                 "lutgemm_compute_block_shiftInt8");
}

// Extension over the reference's list: output = bias + product in one kernel (no bias.clone()), mode A.
void lutgemv_fused(torch::Tensor output, torch::Tensor bWeight, torch::Tensor alpha, c10::optional<torch::Tensor> bias,
                   torch::Tensor d_input, int mSize, int kSize, int nb, int num_groups, bool pdl) {
    Call c = prepare(output, bWeight, alpha, torch::kFloat16, d_input, mSize, kSize, nb, (int64_t)num_groups * nb * mSize);
    const void *b = nullptr;
    if (bias.has_value()) {
        require(*bias, torch::kFloat16, "bias");
        TORCH_CHECK(bias->numel() == mSize, "bias must hold mSize elements");
        b = bias->data_ptr();
    }
    c10::cuda::CUDAGuard guard(output.device());
    check_status(sal_lutgemv_shift_scale(c.bw, c.alpha, b, c.x, c.y, c.M, c.K, c.N, c.q, num_groups, pdl ? SAL_PDL : 0u, c.ws.data_ptr(),
                                         (size_t)c.ws.numel(), c.stream),
                 "lutgemv_fused");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "BCQ LUT-GEMM for NVIDIA B200 (sm_100a): drop-in for ShiftAddLLM's compiled lutgemm extension";
    namespace py = pybind11;
    using release = py::call_guard<py::gil_scoped_release>;
    m.def("lutgemm_compute", &lutgemm_compute, "lutgemm_compute", release());
    m.def("lutgemm_compute_shift_scale", &lutgemm_compute_shift_scale, "lutgemm_compute_shift_scale", release());
    m.def("lutgemm_compute_block", &lutgemm_compute_block, "lutgemm_compute_block", release());
    m.def("lutgemm_compute_block_shift", &lutgemm_compute_block_shift, "lutgemm_compute_block_shift", release());
    m.def("lutgemm_compute_block_shiftInt8", &lutgemm_compute_block_shiftInt8, "lutgemm_compute_block_shiftInt8", release());
    m.def("lutgemv_fused", &lutgemv_fused, "output = bias + product (mode A), optionally with programmatic dependent launch",
          py::arg("output"), py::arg("bWeight"), py::arg("alpha"), py::arg("bias"), py::arg("d_input"), py::arg("mSize"), py::arg("kSize"),
          py::arg("nb"), py::arg("num_groups"), py::arg("pdl") = false, release());
    m.def("sal_version", []() { return sal_version(); });
}
