// Torch extension `moonpoly` (pybind module) + dispatcher library `moonpoly_ops`, the surface the
// reference exposes from moonpoly/core/moonpoly_gemm.cu:160-558 and :1738-1927 and that its vLLM
// Linear patch calls (integrations/vllm/v0.10.0/moonpoly_linear.patch:487-516).  Op schemas are
// those of moonpoly_gemm.cu:516-524.  Everything here is tensor bookkeeping: checks, output
// allocation, the current stream; the computation is one call into the C ABI.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include <optional>
#include <stdexcept>
#include <string>

#include "../../include/moonpoly_abi.h"

namespace {

void require(bool cond, const std::string& msg) {
  if (!cond) throw std::invalid_argument(msg);
}

void check(int rc) {
  if (rc == MP_OK || rc == MP_ERR_UNALIGNED_K) return;   // misaligned K: the reference computes nothing, silently
  if (rc == MP_ERR_INVALID_ARG || rc == MP_ERR_LAYOUT || rc == MP_ERR_BAD_PID || rc == MP_ERR_WORKSPACE)
    throw std::invalid_argument(mp_last_error_string());
  throw std::runtime_error(mp_last_error_string());
}

int dtype_code(const at::Tensor& t) {
  if (t.scalar_type() == at::kHalf) return MP_FP16;
  if (t.scalar_type() == at::kChar) return MP_INT8;
  if (t.scalar_type() == at::kFloat) return MP_FP32;
  if (t.scalar_type() == at::kBFloat16)
    throw std::invalid_argument(
        "BF16 core GEMM has been removed. Convert tensors to torch.float16 before calling MoonPoly.");
  throw std::invalid_argument("Unsupported torch data type");
}

void* stream_of(const at::Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

int64_t norm_split(int64_t s) { return s <= 0 ? 2 : s; }

// ------------------------------------------------------------------------------------------ linear
at::Tensor linear_cuda(const at::Tensor& x, const at::Tensor& w) {
  require(x.is_cuda() && w.is_cuda(), "Tensors must be on CUDA device");
  require(x.dim() == 2 && w.dim() == 2, "linear: input and weight must be 2D");
  require(x.size(1) == w.size(1), "linear: weight shape mismatch");
  require(x.scalar_type() == w.scalar_type(), "linear: input and weight dtypes differ");
  const int dt = dtype_code(x);
  c10::cuda::CUDAGuard guard(x.device());
  const at::Tensor xc = x.contiguous(), wc = w.contiguous();
  at::Tensor y = at::empty({x.size(0), w.size(0)}, x.options().dtype(dt == MP_INT8 ? at::kInt : x.scalar_type()));
  check(mp_linear(dt, (int)x.size(0), (int)w.size(0), (int)x.size(1), xc.data_ptr(), wc.data_ptr(), y.data_ptr(),
                  stream_of(x)));
  return y;
}

// Extension beyond the reference's op set: Linear with the bias add fused into the epilogue, fp16 or bf16.
at::Tensor linear_bias_cuda(const at::Tensor& x, const at::Tensor& w, const std::optional<at::Tensor>& bias) {
  require(x.is_cuda() && w.is_cuda(), "Tensors must be on CUDA device");
  require(x.dim() == 2 && w.dim() == 2, "linear_bias: input and weight must be 2D");
  require(x.size(1) == w.size(1), "linear_bias: weight shape mismatch");
  require(x.scalar_type() == w.scalar_type(), "linear_bias: input and weight dtypes differ");
  require(x.scalar_type() == at::kHalf || x.scalar_type() == at::kBFloat16, "linear_bias: fp16 or bf16 only");
  c10::cuda::CUDAGuard guard(x.device());
  const at::Tensor xc = x.contiguous(), wc = w.contiguous();
  at::Tensor bc;
  if (bias.has_value() && bias->defined()) {
    require(bias->is_cuda() && bias->scalar_type() == x.scalar_type() && bias->numel() == w.size(0),
            "linear_bias: bias must be a CUDA tensor of N elements in the input dtype");
    bc = bias->contiguous();
  }
  at::Tensor y = at::empty({x.size(0), w.size(0)}, x.options());
  check(mp_linear_bias(x.scalar_type() == at::kHalf ? MP_FP16 : MP_BF16, (int)x.size(0), (int)w.size(0), (int)x.size(1),
                       xc.data_ptr(), wc.data_ptr(), bc.defined() ? bc.data_ptr() : nullptr, y.data_ptr(), stream_of(x)));
  return y;
}

// The measured decode plans live inside the online selector of the library, so the C++-selector
// op is the plain op (non-fp16 / non-2-D / non-contiguous inputs take this route in the reference too).
at::Tensor linear_cpp_selector_cuda(const at::Tensor& x, const at::Tensor& w) { return linear_cuda(x, w); }

void fp16_pair_checks(const char* op, const at::Tensor& a, const at::Tensor& b) {
  require(a.is_cuda() && b.is_cuda(), std::string(op) + ": tensors must be CUDA");
  require(a.scalar_type() == at::kHalf && b.scalar_type() == at::kHalf, std::string(op) + ": tensors must be float16");
  require(a.dim() == 2 && b.dim() == 2, std::string(op) + ": tensors must be 2D");
}

int64_t fp16_workspace_size(const at::Tensor& x, const at::Tensor& w, int64_t pid, int64_t split) {
  fp16_pair_checks("fp16_workspace_size", x, w);
  require(w.size(1) == x.size(1), "fp16_workspace_size: weight shape mismatch");
  size_t bytes = 0;   // Linear (M,N,K) runs as RCC (m,n,k) = (N,M,K)
  check(mp_workspace_size(MP_FP16, (int)pid, (int)w.size(0), (int)x.size(0), (int)x.size(1), (int)norm_split(split), &bytes));
  return (int64_t)bytes;
}

int64_t fp16_rcc_workspace_size(const at::Tensor& a, const at::Tensor& b_col, int64_t pid, int64_t split) {
  fp16_pair_checks("fp16_rcc_workspace_size", a, b_col);
  require(b_col.size(0) == a.size(1), "fp16_rcc_workspace_size: B logical shape must be [k, n]");
  size_t bytes = 0;
  check(mp_workspace_size(MP_FP16, (int)pid, (int)a.size(0), (int)b_col.size(1), (int)a.size(1), (int)norm_split(split), &bytes));
  return (int64_t)bytes;
}

void workspace_checks(const char* op, const at::Tensor& ws, size_t need, void** ptr, size_t* bytes) {
  *ptr = nullptr;
  *bytes = 0;
  if (need == 0) return;
  require(ws.defined(), std::string(op) + ": workspace is required for this pid");
  require(ws.is_cuda() && ws.scalar_type() == at::kByte && ws.is_contiguous(),
          std::string(op) + ": workspace must be contiguous CUDA uint8 tensor");
  require((size_t)ws.numel() >= need, std::string(op) + ": workspace buffer too small");
  *ptr = ws.data_ptr();
  *bytes = (size_t)ws.numel();
}

void linear_fp16_pid_ws_out(const at::Tensor& x, const at::Tensor& w, at::Tensor& out, int64_t pid,
                            const at::Tensor& workspace, int64_t split) {
  const char* op = "linear_fp16_pid_ws_out";
  fp16_pair_checks(op, x, w);
  require(out.is_cuda() && out.scalar_type() == at::kHalf && out.dim() == 2, std::string(op) + ": output must be a 2D CUDA float16 tensor");
  require(x.is_contiguous() && w.is_contiguous() && out.is_contiguous(), std::string(op) + ": input/weight/output must be contiguous");
  const int64_t M = x.size(0), K = x.size(1), N = w.size(0);
  require(w.size(1) == K, std::string(op) + ": weight shape mismatch");
  require(out.size(0) == M && out.size(1) == N, std::string(op) + ": output shape must be [M, N]");
  split = norm_split(split);
  size_t need = 0;
  check(mp_workspace_size(MP_FP16, (int)pid, (int)N, (int)M, (int)K, (int)split, &need));
  void* ws_ptr; size_t ws_bytes;
  workspace_checks(op, workspace, need, &ws_ptr, &ws_bytes);
  c10::cuda::CUDAGuard guard(x.device());
  check(mp_gemm_rcc_pid(MP_FP16, (int)pid, (int)split, (int)N, (int)M, (int)K, w.data_ptr(), x.data_ptr(), out.data_ptr(),
                        1.0f, 0.0f, ws_ptr, ws_bytes, stream_of(x)));
}

at::Tensor linear_fp16_pid_ws(const at::Tensor& x, const at::Tensor& w, int64_t pid, const at::Tensor& workspace,
                              int64_t split) {
  fp16_pair_checks("linear_fp16_pid_ws", x, w);
  at::Tensor out = at::empty({x.size(0), w.size(0)}, x.options());
  linear_fp16_pid_ws_out(x, w, out, pid, workspace, split);
  return out;
}

void fp16_rcc_pid_ws_out(const at::Tensor& a, const at::Tensor& b_col, at::Tensor& c_col, int64_t pid,
                         const at::Tensor& workspace, int64_t split) {
  const char* op = "fp16_rcc_pid_ws_out";
  fp16_pair_checks(op, a, b_col);
  require(c_col.is_cuda() && c_col.scalar_type() == at::kHalf && c_col.dim() == 2, std::string(op) + ": output must be a 2D CUDA float16 tensor");
  require(a.is_contiguous(), std::string(op) + ": A must be contiguous row-major");
  const int64_t m = a.size(0), k = a.size(1), n = b_col.size(1);
  require(b_col.size(0) == k, std::string(op) + ": B logical shape must be [k, n]");
  require(c_col.size(0) == m && c_col.size(1) == n, std::string(op) + ": output logical shape must be [m, n]");
  require(b_col.stride(0) == 1 && b_col.stride(1) == k, std::string(op) + ": B must use packed column-major strides [1, k]");
  require(c_col.stride(0) == 1 && c_col.stride(1) == m, std::string(op) + ": C must use packed column-major strides [1, m]");
  split = norm_split(split);
  size_t need = 0;
  check(mp_workspace_size(MP_FP16, (int)pid, (int)m, (int)n, (int)k, (int)split, &need));
  void* ws_ptr; size_t ws_bytes;
  workspace_checks(op, workspace, need, &ws_ptr, &ws_bytes);
  c10::cuda::CUDAGuard guard(a.device());
  check(mp_gemm_rcc_pid(MP_FP16, (int)pid, (int)split, (int)m, (int)n, (int)k, a.data_ptr(), b_col.data_ptr(),
                        c_col.data_ptr(), 1.0f, 0.0f, ws_ptr, ws_bytes, stream_of(a)));
}

// Forced pid with run-time split-K; the library's own per-stream scratch is used.
at::Tensor linear_cpp_forced_pid(const at::Tensor& x, const at::Tensor& w, int64_t pid, int64_t split) {
  if (!x.is_cuda() || !w.is_cuda() || x.scalar_type() != at::kHalf || w.scalar_type() != at::kHalf || x.dim() != 2 ||
      w.dim() != 2 || !x.is_contiguous() || !w.is_contiguous())
    return linear_cuda(x, w);
  require(x.size(1) == w.size(1), "linear_cpp_forced_pid: weight shape mismatch");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor out = at::empty({x.size(0), w.size(0)}, x.options());
  check(mp_gemm_rcc_pid(MP_FP16, (int)pid, (int)norm_split(split), (int)w.size(0), (int)x.size(0), (int)x.size(1),
                        w.data_ptr(), x.data_ptr(), out.data_ptr(), 1.0f, 0.0f, nullptr, 0, stream_of(x)));
  return out;
}

// ------------------------------------------------------------------------------------------ scaled int8
at::Tensor scaled_int8_mm(const at::Tensor& a, const at::Tensor& b, const at::Tensor& a_scales,
                          const at::Tensor& b_scales, const std::optional<at::Tensor>& bias, at::ScalarType out_dtype) {
  require(a.is_cuda() && b.is_cuda(), "scaled_int8_mm: tensors must be CUDA");
  require(a.scalar_type() == at::kChar && b.scalar_type() == at::kChar, "A must be int8; B must be int8");
  require(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(0), "scaled_int8_mm: A must be [M,K] and B [K,N]");
  require(out_dtype == at::kHalf || out_dtype == at::kBFloat16, "Unsupported output dtype");
  require(a_scales.scalar_type() == at::kFloat && b_scales.scalar_type() == at::kFloat, "scales must be float32");
  const int64_t M = a.size(0), K = a.size(1), N = b.size(1);
  require(a_scales.numel() == 1 || a_scales.numel() == M, "A scales must be a scalar or [M,1]");
  require(b_scales.numel() == 1 || b_scales.numel() == N, "B scales must be a scalar or [1,N]");
  c10::cuda::CUDAGuard guard(a.device());
  const at::Tensor ac = a.contiguous();
  const at::Tensor b_nk = b.t().contiguous();            // no copy when the caller passed weight.t()
  const at::Tensor sa = a_scales.contiguous(), sb = b_scales.contiguous();
  at::Tensor bias_c;
  const void* bias_ptr = nullptr;
  if (bias.has_value() && bias->defined()) {
    require(bias->scalar_type() == out_dtype, "Bias dtype mismatch");
    require(bias->numel() == N, "bias must have N elements");
    bias_c = bias->contiguous();
    bias_ptr = bias_c.data_ptr();
  }
  at::Tensor out = at::empty({M, N}, a.options().dtype(out_dtype));
  check(mp_scaled_mm_i8((int)M, (int)N, (int)K, ac.data_ptr<int8_t>(), (int)K, b_nk.data_ptr<int8_t>(), (int)K,
                        sa.data_ptr<float>(), sa.numel() == 1, sb.data_ptr<float>(), sb.numel() == 1, bias_ptr,
                        out.data_ptr(), (int)N, out_dtype == at::kHalf ? 0 : 1, stream_of(a)));
  return out;
}

std::tuple<int, int, int, int> scaled_mm_config(int id) {
  int v[4];
  check(mp_scaled_mm_config(id, v));
  return {v[0], v[1], v[2], v[3]};
}

// ------------------------------------------------------------------------------------------ Meta kernels
at::Tensor linear_meta(const at::Tensor& x, const at::Tensor& w) {
  return at::empty_symint({x.sym_size(0), w.sym_size(0)}, x.options());
}
at::Tensor linear_bias_meta(const at::Tensor& x, const at::Tensor& w, const std::optional<at::Tensor>&) {
  return at::empty_symint({x.sym_size(0), w.sym_size(0)}, x.options());
}
int64_t ws_size_meta(const at::Tensor&, const at::Tensor&, int64_t, int64_t) { return 0; }
at::Tensor linear_ws_meta(const at::Tensor& x, const at::Tensor& w, int64_t, const at::Tensor&, int64_t) {
  return at::empty_symint({x.sym_size(0), w.sym_size(0)}, x.options());
}
void out_meta(const at::Tensor&, const at::Tensor&, at::Tensor&, int64_t, const at::Tensor&, int64_t) {}

}  // namespace

TORCH_LIBRARY(moonpoly_ops, m) {
  m.def("linear(Tensor input, Tensor weight) -> Tensor");
  m.def("linear_cpp_selector(Tensor input, Tensor weight) -> Tensor");
  m.def("linear_bias(Tensor input, Tensor weight, Tensor? bias=None) -> Tensor");      // not in the reference's op set
  m.def("fp16_workspace_size(Tensor input, Tensor weight, int pid, int split_k_slices=2) -> int");
  m.def("fp16_rcc_workspace_size(Tensor a, Tensor b_col, int pid, int split_k_slices=2) -> int");
  m.def("linear_fp16_pid_ws(Tensor input, Tensor weight, int pid, Tensor workspace, int split_k_slices=2) -> Tensor");
  m.def("linear_fp16_pid_ws_out(Tensor input, Tensor weight, Tensor(a!) output, int pid, Tensor workspace, int split_k_slices=2) -> ()");
  m.def("fp16_rcc_pid_ws_out(Tensor a, Tensor b_col, Tensor(a!) c_col, int pid, Tensor workspace, int split_k_slices=2) -> ()");
}

TORCH_LIBRARY_IMPL(moonpoly_ops, CUDA, m) {
  m.impl("linear", &linear_cuda);
  m.impl("linear_cpp_selector", &linear_cpp_selector_cuda);
  m.impl("linear_bias", &linear_bias_cuda);
  m.impl("fp16_workspace_size", &fp16_workspace_size);
  m.impl("fp16_rcc_workspace_size", &fp16_rcc_workspace_size);
  m.impl("linear_fp16_pid_ws", &linear_fp16_pid_ws);
  m.impl("linear_fp16_pid_ws_out", &linear_fp16_pid_ws_out);
  m.impl("fp16_rcc_pid_ws_out", &fp16_rcc_pid_ws_out);
}

TORCH_LIBRARY_IMPL(moonpoly_ops, Meta, m) {
  m.impl("linear", &linear_meta);
  m.impl("linear_cpp_selector", &linear_meta);
  m.impl("linear_bias", &linear_bias_meta);
  m.impl("fp16_workspace_size", &ws_size_meta);
  m.impl("fp16_rcc_workspace_size", &ws_size_meta);
  m.impl("linear_fp16_pid_ws", &linear_ws_meta);
  m.impl("linear_fp16_pid_ws_out", &out_meta);
  m.impl("fp16_rcc_pid_ws_out", &out_meta);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "MoonPoly GEMM for B200 (sm_100a): torch binding above the C ABI of libmoonpoly_gemm.so";
  m.def("linear", &linear_cuda, py::arg("A"), py::arg("B"));
  m.def("linear_cpp_selector", &linear_cpp_selector_cuda, py::arg("A"), py::arg("B"));
  m.def("linear_bias", &linear_bias_cuda, py::arg("A"), py::arg("B"), py::arg("bias") = py::none());
  m.def("linear_cpp_forced_pid", &linear_cpp_forced_pid, py::arg("A"), py::arg("B"), py::arg("pid"), py::arg("split_k"));
  m.def("fp16_workspace_size", &fp16_workspace_size, py::arg("A"), py::arg("B"), py::arg("pid"), py::arg("split_k_slices") = 2);
  m.def("linear_fp16_pid_ws", &linear_fp16_pid_ws, py::arg("A"), py::arg("B"), py::arg("pid"), py::arg("workspace"),
        py::arg("split_k_slices") = 2);
  m.def("scaled_int8_mm",
        [](const at::Tensor& a, const at::Tensor& b, const at::Tensor& sa, const at::Tensor& sb,
           const std::optional<at::Tensor>& bias, py::object out_dtype) {
          const at::ScalarType dt = out_dtype.is_none() ? at::kHalf : torch::python::detail::py_object_to_dtype(out_dtype);
          return scaled_int8_mm(a, b, sa, sb, bias, dt);
        },
        py::arg("A"), py::arg("B"), py::arg("A_scales"), py::arg("B_scales"), py::arg("bias") = py::none(),
        py::arg("out_dtype") = py::none());
  m.def("predict_int8_scaled_mm_kernel", [](int mm, int n, int k) { return mp_scaled_mm_predict(mm, n, k); },
        py::arg("m"), py::arg("n"), py::arg("k"));
  m.def("get_int8_scaled_mm_kernel_config", &scaled_mm_config, py::arg("kernel_id"));
  m.def("select_plan", [](int dtype, int mm, int n, int k) {
    mp_plan p;
    check(mp_select_plan(dtype, mm, n, k, &p));
    return std::make_tuple(p.pattern, p.pid, p.split_k, p.split_n, p.estimated_ms);
  });
  m.def("launch_count", []() { return mp_launch_count(); });
}
