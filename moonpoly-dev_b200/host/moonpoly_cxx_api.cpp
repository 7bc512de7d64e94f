// C++ API of the reference (namespace moonpoly) as forwards to the C ABI.  Error behaviour follows
// the reference: std::invalid_argument for bad dtype / layout / Pattern-2 arguments
// (core/fp16/fp16_dispatch.cu:25, core/fp16/fp16_rcc.cu:83-90), std::runtime_error for workspace
// and CUDA failures (core/fp16/fp16_rcc.cu:2634-2642), and the " k is not aligned" message with no
// computation for a misaligned K (core/fp16/fp16_rcc.cu:3280-3282).
#include <iostream>
#include <stdexcept>

#include "../../include/moonpoly_abi.h"
#include "moonpoly.cuh"

namespace moonpoly {
namespace {

void check(int rc) {
  switch (rc) {
    case MP_OK:
      return;
    case MP_ERR_UNALIGNED_K:
      std::cout << " k is not aligned, please check!" << std::endl;
      return;
    case MP_ERR_INVALID_ARG:
    case MP_ERR_LAYOUT:
    case MP_ERR_BAD_PID:
      throw std::invalid_argument(mp_last_error_string());
    default:
      throw std::runtime_error(mp_last_error_string());
  }
}

void forced_fp16(int pid, int split, int m, int n, int k, const cutlass::half_t* A, const cutlass::half_t* B,
                 cutlass::half_t* C, float a, float b, void* ws, size_t ws_bytes, cudaStream_t s) {
  check(mp_gemm_rcc_pid(MP_FP16, pid, split, m, n, k, A, B, C, a, b, ws, ws_bytes, s));
}

size_t ws_size(int pid, int m, int n, int k, int split) {
  size_t bytes = 0;
  check(mp_workspace_size(MP_FP16, pid, m, n, k, split, &bytes));
  return bytes;
}

}  // namespace

int num_sms() { return mp_num_sms(); }

void moonpoly_gemm(MoonpolyDataType dtype, int m, int n, int k, void* A, bool ac, void* B, bool bc, void* C, bool cc,
                   float alpha, float beta, cudaStream_t stream) {
  check(mp_gemm(static_cast<int>(dtype), m, n, k, A, ac, B, bc, C, cc, alpha, beta, stream));
}

void moonpolyLinear(MoonpolyDataType dtype, int m, int n, int k, void* A, void* B, void* C, cudaStream_t stream) {
  check(mp_linear(static_cast<int>(dtype), m, n, k, A, B, C, stream));
}

void run_fp16_gemm(int m, int n, int k, const cutlass::half_t* A, bool ac, const cutlass::half_t* B, bool bc,
                   cutlass::half_t* C, bool cc, float alpha, float beta, cudaStream_t stream) {
  check(mp_gemm(MP_FP16, m, n, k, A, ac, B, bc, C, cc, alpha, beta, stream));
}

void run_int8_gemm(int m, int n, int k, const int8_t* A, bool ac, const int8_t* B, bool bc, int32_t* C, bool cc,
                   int ialpha, int ibeta, cudaStream_t stream) {
  check(mp_gemm(MP_INT8, m, n, k, A, ac, B, bc, C, cc, static_cast<float>(ialpha), static_cast<float>(ibeta), stream));
}

void run_fp32_gemm(int m, int n, int k, const float* A, bool ac, const float* B, bool bc, float* C, bool cc,
                   float alpha, float beta, cudaStream_t stream) {
  check(mp_gemm(MP_FP32, m, n, k, A, ac, B, bc, C, cc, alpha, beta, stream));
}

Fp16OnlinePlan select_fp16_online_plan_row_col_col(int m, int n, int k) {
  mp_plan p;
  check(mp_select_plan(MP_FP16, m, n, k, &p));
  return Fp16OnlinePlan{static_cast<Fp16PolyPattern>(p.pattern), p.pid, p.split_k, p.split_n, p.estimated_ms};
}

void run_fp16_online_gemm_row_col_col(int m, int n, int k, const cutlass::half_t* A, const cutlass::half_t* B,
                                      cutlass::half_t* C, float a, float b, cudaStream_t stream) {
  check(mp_gemm_rcc(MP_FP16, m, n, k, A, B, C, a, b, stream));
}

void get_gemm_alignment_fp16_row_col_col(int pid, int* alignment) { check(mp_pid_info(MP_FP16, pid, nullptr, alignment)); }
void get_gemm_shared_mem_fp16_row_col_col(int pid, int* shared_mem) { check(mp_pid_info(MP_FP16, pid, shared_mem, nullptr)); }
void get_gemm_alignment_int8_row_col_col(int pid, int* alignment) { check(mp_pid_info(MP_INT8, pid, nullptr, alignment)); }
void get_gemm_shared_mem_int8_row_col_col(int pid, int* shared_mem) { check(mp_pid_info(MP_INT8, pid, shared_mem, nullptr)); }
void get_gemm_alignment_fp32_row_col_col(int pid, int* alignment) { check(mp_pid_info(MP_FP32, pid, nullptr, alignment)); }
void get_gemm_shared_mem_fp32_row_col_col(int pid, int* shared_mem) { check(mp_pid_info(MP_FP32, pid, shared_mem, nullptr)); }

void run_moonpoly_selected_gemm_fp16_row_col_col(int pid, int m, int n, int k, const cutlass::half_t* A,
                                                 const cutlass::half_t* B, cutlass::half_t* C, float a, float b,
                                                 cudaStream_t stream) {
  forced_fp16(pid, 1, m, n, k, A, B, C, a, b, nullptr, 0, stream);
}

size_t get_gemm_workspace_size_fp16_row_col_col(int pid, int m, int n, int k, int split) {
  return ws_size(pid, m, n, k, split);
}

void run_moonpoly_selected_gemm_fp16_row_col_col_with_workspace(int pid, int m, int n, int k,
                                                                const cutlass::half_t* A, const cutlass::half_t* B,
                                                                cutlass::half_t* C, float a, float b, void* ws,
                                                                size_t ws_bytes, int split, cudaStream_t stream) {
  forced_fp16(pid, split, m, n, k, A, B, C, a, b, ws, ws_bytes, stream);
}

#define MOONPOLY_STREAMK(PID)                                                                                      \
  size_t get_fp16_p##PID##_streamk_workspace_size_row_col_col(int m, int n, int k, int split) {                    \
    return ws_size(PID, m, n, k, split);                                                                           \
  }
MOONPOLY_STREAMK(40)
MOONPOLY_STREAMK(66)
MOONPOLY_STREAMK(42)
MOONPOLY_STREAMK(43)
MOONPOLY_STREAMK(44)
#undef MOONPOLY_STREAMK

void run_fp16_p40_streamk_singleton_row_col_col(int m, int n, int k, const cutlass::half_t* A,
                                                const cutlass::half_t* B, cutlass::half_t* C, float a, float b,
                                                int split, cudaStream_t stream) {
  forced_fp16(40, split, m, n, k, A, B, C, a, b, nullptr, 0, stream);
}
void run_fp16_p40_streamk_row_col_col(int m, int n, int k, const cutlass::half_t* A, const cutlass::half_t* B,
                                      cutlass::half_t* C, float a, float b, void* ws, size_t ws_bytes, int split,
                                      cudaStream_t stream) {
  if (split <= 0) split = 2;
  if (ws_size(40, m, n, k, split) > 0 && ws == nullptr)
    throw std::runtime_error("P40 StreamK workspace is null");
  forced_fp16(40, split, m, n, k, A, B, C, a, b, ws, ws_bytes, stream);
}
void run_fp16_p66_streamk_row_col_col(int m, int n, int k, const cutlass::half_t* A, const cutlass::half_t* B,
                                      cutlass::half_t* C, float a, float b, int split, cudaStream_t stream) {
  forced_fp16(66, split, m, n, k, A, B, C, a, b, nullptr, 0, stream);
}
void run_fp16_p42_streamk_row_col_col(int m, int n, int k, const cutlass::half_t* A, const cutlass::half_t* B,
                                      cutlass::half_t* C, float a, float b, int split, cudaStream_t stream) {
  forced_fp16(42, split, m, n, k, A, B, C, a, b, nullptr, 0, stream);
}
void run_fp16_p43_streamk_row_col_col(int m, int n, int k, const cutlass::half_t* A, const cutlass::half_t* B,
                                      cutlass::half_t* C, float a, float b, int split, cudaStream_t stream) {
  forced_fp16(43, split, m, n, k, A, B, C, a, b, nullptr, 0, stream);
}
void run_fp16_p44_streamk_row_col_col(int m, int n, int k, const cutlass::half_t* A, const cutlass::half_t* B,
                                      cutlass::half_t* C, float a, float b, int split, cudaStream_t stream) {
  forced_fp16(44, split, m, n, k, A, B, C, a, b, nullptr, 0, stream);
}

void run_fp16_pattern2_twin_gemm_row_col_col(int m, int n, int k, int split_n, const cutlass::half_t* A,
                                             const cutlass::half_t* B, cutlass::half_t* C, float a, float b,
                                             cudaStream_t stream) {
  check(mp_twin_gemm_fp16(m, n, k, split_n, A, B, C, a, b, stream));
}

void run_moonpoly_selected_gemm_int8_row_col_col(int pid, int m, int n, int k, const int8_t* A, const int8_t* B,
                                                 int32_t* C, int alpha, int beta, cudaStream_t stream) {
  // the reference returns silently on a misaligned K here (core/int8/i8_rcc.cu:3164-3166)
  const int rc = mp_gemm_rcc_pid(MP_INT8, pid, 1, m, n, k, A, B, C, static_cast<float>(alpha),
                                 static_cast<float>(beta), nullptr, 0, stream);
  if (rc != MP_ERR_UNALIGNED_K) check(rc);
}

void run_moonpoly_selected_gemm_fp32_row_col_col(int pid, int m, int n, int k, const float* A, const float* B,
                                                 float* C, float a, float b, cudaStream_t stream) {
  check(mp_gemm_rcc_pid(MP_FP32, pid, 1, m, n, k, A, B, C, a, b, nullptr, 0, stream));
}

}  // namespace moonpoly
