// Host-side cost API of the reference.  The reference declares these `extern` inside its kernel
// files (moonpoly/core/fp16/fp16_rcc.cu:29-36, core/fp32/fp32_rcc.cu:27-30, core/int8/i8_rcc.cu:23-26)
// and defines them in core/fp16/fp16_rcc_cost.cu:143-279, core/fp32/fp32_rcc_cost.cu:92-233 and
// core/int8/i8_rcc_cost.cu:105-246; its profilers link to them.  Same namespaces, names and
// parameter lists here.  Arguments follow the reference's feature convention: `ims` is the extent
// tiled by a pid's pm (RCC n), `ins` the extent tiled by pn (RCC m).  Values are milliseconds
// predicted by this library's tables, which are fitted on B200.
#pragma once

#include "moonpoly.cuh"

namespace moonpoly {
namespace fp16 {
namespace row_col_col {
extern const int num_gemm_primary;
float analytic_gemm_cost_model(int ims, int ins, int iks, int pid);
float fitted_gemm_cost_model(int ims, int ins, int iks, int pid);
float gemm_cost_model(int ims, int ins, int iks, int pid);
float gemm_reduction_cost_model(int ims, int ins, int iks, int pid, int split_k_slices);
float gemm_splitk_cost_model(int ims, int ins, int iks, int pid, int split_k_slices);
int cutlass_gemm_predict(int m, int n, int k);
void dump_cost_model(int ims, int ins, int iks, int pid);
}  // namespace row_col_col
}  // namespace fp16

namespace fp32 {
namespace simt {
namespace row_col_col {
float gemm_cost_model(int ims, int ins, int iks, int pid);
float gemm_splitk_cost_model(int ims, int ins, int iks, int split_k_slices);
int cutlass_gemm_predict(int m, int n, int k);
}  // namespace row_col_col
}  // namespace simt
}  // namespace fp32

namespace int8 {
namespace row_col_col {
float gemm_cost_model(int ims, int ins, int iks, int pid);
float gemm_splitk_cost_model(int ims, int ins, int iks, int split_k_slices);
int cutlass_gemm_predict(int m, int n, int k);
}  // namespace row_col_col
}  // namespace int8
}  // namespace moonpoly
