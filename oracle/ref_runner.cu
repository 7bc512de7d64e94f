// TEST INFRASTRUCTURE -- command-line driver around the REFERENCE'S OWN GEMM entry points
// (moonpoly/include/moonpoly.cuh), linked by oracle/build_ref_kernels.sh with the reference's
// kernels compiled from the reference tree.  It lets the test-suite run the reference, the CPU
// oracle and the product on identical inputs.  The product never links, loads or runs this file.
//
//   mp_ref_runner <manifest>
//
// The manifest is a text file with one case per line:
//   <op> <m> <n> <k> <pid> <split> <alpha> <beta> <input file> <output file>
// ops (RCC convention: A row-major [m,k]; B stored [n,k]; C stored [n,m]):
//   fp16_auto   moonpoly::run_fp16_gemm              (online selector)
//   fp16_pid    moonpoly::run_moonpoly_selected_gemm_fp16_row_col_col_with_workspace(pid, ..., split)
//   fp16_twin   moonpoly::run_fp16_pattern2_twin_gemm_row_col_col, split_n = <split>
//   int8_auto   moonpoly::run_int8_gemm
//   int8_pid    moonpoly::run_moonpoly_selected_gemm_int8_row_col_col
//   fp32_auto   moonpoly::run_fp32_gemm
//   fp32_pid    moonpoly::run_moonpoly_selected_gemm_fp32_row_col_col
//   fp16_plan   prints "plan <pattern> <pid> <split_k> <split_n>" of select_fp16_online_plan_row_col_col
// The input file holds A, then B, then (when beta != 0) the old C, as raw arrays; the output file
// receives C.  One line "ok <index>" is printed per finished case, so a caller sees how far a run
// got when the reference exits on an internal error (its CUTLASS_CHECK calls exit()).
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#include "moonpoly.cuh"

namespace {

void die(const std::string& msg) {
  std::fprintf(stderr, "mp_ref_runner: %s\n", msg.c_str());
  std::exit(2);
}

void cuda_ok(cudaError_t e, const char* what) {
  if (e != cudaSuccess) die(std::string(what) + ": " + cudaGetErrorString(e));
}

std::vector<char> read_file(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) die("cannot open " + path);
  return std::vector<char>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}

}  // namespace

int main(int argc, char** argv) {
  if (argc != 2) die("usage: mp_ref_runner <manifest>");
  std::ifstream mf(argv[1]);
  if (!mf) die(std::string("cannot open manifest ") + argv[1]);
  std::string line;
  int index = 0;
  while (std::getline(mf, line)) {
    if (line.empty() || line[0] == '#') continue;
    std::istringstream ss(line);
    std::string op, in_path, out_path;
    long long m, n, k;
    int pid, split;
    float alpha, beta;
    if (!(ss >> op >> m >> n >> k >> pid >> split >> alpha >> beta >> in_path >> out_path)) die("bad manifest line: " + line);

    if (op == "fp16_plan") {
      const moonpoly::Fp16OnlinePlan p = moonpoly::select_fp16_online_plan_row_col_col((int)m, (int)n, (int)k);
      std::printf("plan %d %d %d %d\n", (int)p.pattern, p.pid, p.split_k, p.split_n);
      std::printf("ok %d\n", index++);
      std::fflush(stdout);
      continue;
    }

    cuda_ok(cudaSetDevice(0), "cudaSetDevice");       // the plan query above needs no device
    const bool is_f16 = op.rfind("fp16", 0) == 0, is_i8 = op.rfind("int8", 0) == 0, is_f32 = op.rfind("fp32", 0) == 0;
    if (!is_f16 && !is_i8 && !is_f32) die("unknown op " + op);
    const size_t ein = is_f16 ? 2 : is_i8 ? 1 : 4, eout = is_f16 ? 2 : 4;
    const size_t a_bytes = (size_t)m * k * ein, b_bytes = (size_t)n * k * ein, c_bytes = (size_t)m * n * eout;
    const bool has_c = beta != 0.0f;
    const std::vector<char> in = read_file(in_path);
    if (in.size() != a_bytes + b_bytes + (has_c ? c_bytes : 0)) die("input file of unexpected size: " + in_path);

    void *dA = nullptr, *dB = nullptr, *dC = nullptr;
    cuda_ok(cudaMalloc(&dA, a_bytes + 16), "cudaMalloc A");
    cuda_ok(cudaMalloc(&dB, b_bytes + 16), "cudaMalloc B");
    cuda_ok(cudaMalloc(&dC, c_bytes + 16), "cudaMalloc C");
    cuda_ok(cudaMemcpy(dA, in.data(), a_bytes, cudaMemcpyHostToDevice), "copy A");
    cuda_ok(cudaMemcpy(dB, in.data() + a_bytes, b_bytes, cudaMemcpyHostToDevice), "copy B");
    if (has_c) cuda_ok(cudaMemcpy(dC, in.data() + a_bytes + b_bytes, c_bytes, cudaMemcpyHostToDevice), "copy C");
    else cuda_ok(cudaMemset(dC, 0xFF, c_bytes), "fill C");     // NaN / -1 pattern: untouched outputs show up

    using half = cutlass::half_t;
    const int im = (int)m, in_ = (int)n, ik = (int)k;
    if (op == "fp16_auto") {
      moonpoly::run_fp16_gemm(im, in_, ik, (const half*)dA, false, (const half*)dB, true, (half*)dC, true, alpha, beta);
    } else if (op == "fp16_pid") {
      moonpoly::run_moonpoly_selected_gemm_fp16_row_col_col_with_workspace(pid, im, in_, ik, (const half*)dA, (const half*)dB,
                                                                          (half*)dC, alpha, beta, nullptr, 0, split);
    } else if (op == "fp16_twin") {
      moonpoly::run_fp16_pattern2_twin_gemm_row_col_col(im, in_, ik, split, (const half*)dA, (const half*)dB, (half*)dC,
                                                        alpha, beta);
    } else if (op == "int8_auto") {
      moonpoly::run_int8_gemm(im, in_, ik, (const int8_t*)dA, false, (const int8_t*)dB, true, (int32_t*)dC, true,
                              (int)alpha, (int)beta);
    } else if (op == "int8_pid") {
      moonpoly::run_moonpoly_selected_gemm_int8_row_col_col(pid, im, in_, ik, (const int8_t*)dA, (const int8_t*)dB,
                                                            (int32_t*)dC, (int)alpha, (int)beta);
    } else if (op == "fp32_auto") {
      moonpoly::run_fp32_gemm(im, in_, ik, (const float*)dA, false, (const float*)dB, true, (float*)dC, true, alpha, beta);
    } else if (op == "fp32_pid") {
      moonpoly::run_moonpoly_selected_gemm_fp32_row_col_col(pid, im, in_, ik, (const float*)dA, (const float*)dB, (float*)dC,
                                                            alpha, beta);
    } else {
      die("unknown op " + op);
    }
    cuda_ok(cudaDeviceSynchronize(), "kernel");
    std::vector<char> out(c_bytes);
    cuda_ok(cudaMemcpy(out.data(), dC, c_bytes, cudaMemcpyDeviceToHost), "copy back");
    std::ofstream of(out_path, std::ios::binary);
    of.write(out.data(), (std::streamsize)out.size());
    if (!of) die("cannot write " + out_path);
    cudaFree(dA); cudaFree(dB); cudaFree(dC);
    std::printf("ok %d\n", index++);
    std::fflush(stdout);
  }
  return 0;
}
