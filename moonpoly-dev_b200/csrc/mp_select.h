// Host-side pid tables, cost models and online selectors (no CUDA in this file).
//
// The pid numbering, the metadata order [pm, pn, pk] (pm tiles RCC n, pn tiles RCC m), the K
// alignment contract and the grouping into primary / split-K / elite pids follow the reference
// (moonpoly/core/fp16/fp16_rcc_cost.cu:15-36, generated/fp16/rcc/candidates.cu:35-65,
// generated/fp16/rcc/splitk_candidates.inc:2764-2858); the tiles behind each pid are Blackwell
// tiles: one operand on the 128-row UMMA-M side, the other on a 16..256 wide UMMA-N side.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "../../include/moonpoly_abi.h"

namespace mp {

// How a pid maps onto the tcgen05 kernel.
struct TileCfg {
  bool valid;
  // orient 0: RCC m (rows of A) on UMMA-M, RCC n tiled by bn.  orient 1: RCC n (rows of B) on
  // UMMA-M, RCC m tiled by bn.  For FP32 (CUDA-core tiles) ti x tj is the CTA tile over (m, n).
  int orient;
  int bn;
  int align;          // k must be a multiple of this (the reference's per-pid contract)
  bool split_capable; // member of the reference's split-K capable set
  int ti, tj;         // FP32 only
  int xm;             // 2: 256-row tiles (two 128-row halves on the UMMA-M side share each bn-wide tile); else 1
};

TileCfg tile_cfg(int dtype, int pid);
bool pid_exists(int dtype, int pid);
// [pm, pn, pk] as reported by get_gemm_shared_mem_*: pm tiles RCC n, pn tiles RCC m.
void pid_tile_meta(int dtype, int pid, int out[3]);

// Cost of running `pid` with `split_k` slices on RCC (m, n, k), in milliseconds.  Feature
// convention of the reference: feature_m = n, feature_n = m (core/fp16/fp16_rcc.cu:451-458).
float cost_ms(int dtype, int pid, int split_k, int m, int n, int k);

// The split-K hand-off / reduction term of cost_ms alone, and the cheapest primary pid for a shape.
float reduction_cost_ms(int dtype, int pid, int split_k, int m, int n);
int predict_primary_pid(int dtype, int m, int n, int k, float* ms);

// Online selection (memoised per shape and flag state).
mp_plan select_plan(int dtype, int m, int n, int k);

// Pattern-2 helpers (core/fp16/fp16_rcc.cu:63-73).
int choose_pattern2_split_n(int n);

// scaled int8 matmul tile choice: config id 0..5, plus a split-K factor for small problems.
struct ScaledCfg { int id; int orient; int bn; int split_k; bool stream; int xm; };   // stream: use the streaming kernel when the problem fits it; xm 2: 256-row tiles
ScaledCfg scaled_mm_select(int M, int N, int K);
void scaled_mm_config_meta(int id, int out[4]);
constexpr int kScaledConfigCount = 6;

int elite_fp16_pids(int* pids, int capacity);
// pid ranges 90..205, 216..321 and 400..439 (generated/fp16/rcc/candidates.cu:62-65)
bool is_explicit_neighborhood_fp16_pid(int pid);

void reload_env();
int num_sms_for_model();
void set_num_sms_for_model(int sms);

}  // namespace mp
