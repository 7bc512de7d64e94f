// Host-side pid tables, cost models and online selectors.  See mp_select.h.
#include "mp_select.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <mutex>
#include <utility>
#include <vector>

namespace mp {
namespace {

constexpr float kInf = std::numeric_limits<float>::infinity();

// ------------------------------------------------------------------------------------------------
// pid tables
// ------------------------------------------------------------------------------------------------
struct U { int8_t orient; int16_t bn; int8_t align; };

// FP16 primary pids 0..40.  The reference's tile (pm over n, pn over m) decides the class:
// the dimension with the larger tile goes on the 128-row UMMA-M side, the other is tiled by
// bn = its reference tile rounded up to a multiple of 16.
constexpr U kFp16Primary[41] = {
    {0, 16, 8},  {0, 128, 8}, {0, 64, 8},  {0, 64, 8},  {0, 16, 8},  {1, 16, 8},  {0, 16, 8},
    {1, 256, 2}, {1, 16, 8},  {1, 16, 2},  {0, 32, 1},  {0, 64, 2},  {1, 64, 2},  {1, 16, 2},
    {0, 96, 8},  {0, 80, 8},  {1, 32, 8},  {1, 32, 8},  {0, 32, 8},  {0, 16, 8},  {0, 80, 8},
    {0, 16, 4},  {1, 96, 8},  {0, 256, 8}, {1, 16, 4},  {1, 16, 8},  {0, 16, 4},  {0, 64, 4},
    {0, 16, 8},  {0, 16, 1},  {0, 192, 8}, {1, 192, 8}, {0, 32, 2},  {0, 96, 1},  {0, 64, 8},
    {0, 16, 2},  {0, 32, 2},  {1, 32, 8},  {0, 16, 1},  {0, 32, 8},  {1, 32, 8},
};
// split-K capable primary pids (core/fp16/fp16_rcc.cu:3067-3090)
constexpr int kFp16SplitPids[17] = {4, 6, 7, 12, 13, 15, 19, 20, 23, 24, 25, 29, 31, 32, 33, 37, 39};
// elite set (generated/fp16/rcc/candidates.cu:35-60)
constexpr int kEliteExtra[5] = {400, 407, 413, 425, 439};
// "explicit neighbourhood" pids 90..205 and 216..321 (generated/fp16/rcc/candidates.cu:62-65): in the
// reference every one of them is a 16-token-wide tile (pm = 16) over 8..128 weight rows; here they share the
// 128 x 16 tile.  These need K % 4 == 0 only, the others K % 8 == 0 (candidates.cu, explicit_neighborhood_alignment).
constexpr int kFp16ExplicitAlign4[45] = {114, 115, 116, 117, 118, 119, 126, 127, 128, 129, 130, 131, 138, 139, 140,
                                         141, 142, 143, 148, 152, 155, 158, 161, 163, 168, 173, 178, 183, 189, 194,
                                         198, 203, 225, 232, 268, 269, 276, 277, 283, 290, 306, 310, 313, 319, 321};
inline bool fp16_explicit_range(int pid) { return (pid >= 90 && pid <= 205) || (pid >= 216 && pid <= 321); }

// INT8 primary pids 0..45 (moonpoly/core/int8/i8_rcc_cost.cu:16-38 tile classes).
constexpr U kInt8Primary[46] = {
    {0, 64, 4},   {1, 64, 8},   {0, 64, 4},  {0, 64, 1},   {0, 64, 1},   {0, 256, 4},  {0, 128, 8},
    {1, 256, 4},  {0, 64, 4},   {0, 64, 16}, {0, 64, 16},  {1, 64, 8},   {0, 64, 16},  {1, 256, 8},
    {0, 256, 16}, {0, 64, 16},  {1, 64, 16}, {0, 128, 4},  {0, 64, 16},  {1, 256, 16}, {0, 64, 16},
    {0, 256, 8},  {0, 128, 8},  {0, 128, 4}, {1, 64, 4},   {0, 128, 8},  {0, 256, 16}, {0, 128, 16},
    {0, 64, 8},   {0, 128, 16}, {0, 128, 1}, {0, 64, 2},   {0, 64, 8},   {0, 64, 16},  {0, 64, 4},
    {1, 64, 16},  {0, 64, 8},   {1, 64, 8},  {0, 128, 4},  {0, 128, 2},  {0, 64, 8},   {0, 64, 16},
    {0, 128, 16}, {1, 64, 16},  {0, 64, 2},  {1, 64, 16},
};

// FP32 primary pids 0..39: CTA tile (ti over m, tj over n) snapped to the instantiated SIMT tiles.
struct F { int16_t ti, tj; };
constexpr F kFp32Primary[40] = {
    {32, 32},  {32, 32},   {64, 32},   {32, 32},   {32, 32},  {32, 32},   {64, 32},   {32, 64},
    {64, 32},  {128, 32},  {32, 32},   {32, 32},   {32, 64},  {64, 64},   {128, 32},  {32, 128},
    {32, 32},  {32, 32},   {64, 32},   {64, 64},   {32, 64},  {32, 128},  {128, 64},  {64, 128},
    {128, 32}, {64, 128},  {128, 64},  {128, 64},  {64, 128}, {128, 32},  {64, 128},  {128, 128},
    {64, 128}, {128, 128}, {128, 128}, {128, 128}, {128, 128}, {128, 128}, {128, 128}, {128, 128},
};

bool in_list(const int* xs, int count, int v) {
  for (int i = 0; i < count; ++i)
    if (xs[i] == v) return true;
  return false;
}

int fp16_base_pid(int pid) {   // pids 400..439 reuse the primary tiles (splitk_candidates.json)
  if (pid == 407) return 8;
  if (pid == 439) return 7;
  return pid - 400;
}

// ------------------------------------------------------------------------------------------------
// environment flags (names and defaults of the reference, App. D of its sources:
// core/fp16/fp16_rcc.cu:110-144,146-149,289-311,363-373,433-436,466-471,490)
// ------------------------------------------------------------------------------------------------
struct Env {
  int p3_min_k = 2048, p3_min_part_k = 512;
  int p2_min_n = 512;
  float p2_max_tail_ratio = 0.25f, p2_margin = 0.90f, p3_margin = 0.97f;
  float gen_margin = 1.0f;
  // FP32 split-K gates: the reference's defaults are 1024 / 256 (its split pays later); these kernels gain from
  // K = 256 on (510 x 512 x 512: 35 -> 23 us with 4 slices), the cost model decides above the gate
  int fp32_p3_min_k = 256, fp32_p3_min_part_k = 64;
  float fp32_p3_margin = 0.97f;
  int int8_p3_min_k = 2048, int8_p3_min_part_k = 512;
  float int8_p3_margin = 0.97f;
  bool disable_fitted = false;
};
Env g_env;
std::once_flag g_env_once;
std::atomic<unsigned> g_env_epoch{1};

bool flag_value(const char* raw, bool dflt) {
  if (raw == nullptr) return dflt;
  // "0", "false", "FALSE", "off", "OFF" are false; anything else is true.
  if (raw[0] == '0' && raw[1] == '\0') return false;
  if (!std::strcmp(raw, "false") || !std::strcmp(raw, "FALSE") || !std::strcmp(raw, "off") ||
      !std::strcmp(raw, "OFF"))
    return false;
  return true;
}
inline bool env_flag(const char* name, bool dflt) { return flag_value(std::getenv(name), dflt); }
int env_int(const char* name, int dflt) {
  const char* raw = std::getenv(name);
  if (!raw) return dflt;
  char* end = nullptr;
  long v = std::strtol(raw, &end, 10);
  return end == raw ? dflt : (int)v;
}
float env_float(const char* name, float dflt) {
  const char* raw = std::getenv(name);
  if (!raw) return dflt;
  char* end = nullptr;
  float v = std::strtof(raw, &end);
  return (end == raw || !std::isfinite(v)) ? dflt : v;
}

void load_env() {
  Env e;
  e.p3_min_k = env_int("MOONPOLY_PATTERN3_MIN_K", 2048);
  e.p3_min_part_k = env_int("MOONPOLY_PATTERN3_MIN_PART_K", 512);
  e.p2_min_n = env_int("MOONPOLY_PATTERN2_MIN_N", 512);
  e.p2_max_tail_ratio = env_float("MOONPOLY_PATTERN2_MAX_TAIL_RATIO", 0.25f);
  e.p2_margin = env_float("MOONPOLY_PATTERN2_MARGIN", 0.90f);
  e.p3_margin = env_float("MOONPOLY_PATTERN3_MARGIN", 0.97f);
  e.gen_margin = env_float("MOONPOLY_GENERATED_SELECTOR_MARGIN", 1.0f);
  e.fp32_p3_min_k = env_int("MOONPOLY_FP32_PATTERN3_MIN_K", 256);
  e.fp32_p3_min_part_k = env_int("MOONPOLY_FP32_PATTERN3_MIN_PART_K", 64);
  e.fp32_p3_margin = env_float("MOONPOLY_FP32_PATTERN3_MARGIN", 0.97f);
  e.int8_p3_min_k = env_int("MOONPOLY_INT8_PATTERN3_MIN_K", 2048);
  e.int8_p3_min_part_k = env_int("MOONPOLY_INT8_PATTERN3_MIN_PART_K", 512);
  e.int8_p3_margin = env_float("MOONPOLY_INT8_PATTERN3_MARGIN", 0.97f);
  const char* dis = std::getenv("MOONPOLY_DISABLE_FITTED_COST");
  const char* legacy = std::getenv("MOONPOLY_USE_FITTED_COST");
  e.disable_fitted = (dis && dis[0] != '\0' && dis[0] != '0') || (legacy && legacy[0] == '0');
  g_env = e;
}
const Env& env() {
  std::call_once(g_env_once, load_env);
  return g_env;
}

// Flags that callers toggle between calls in one process (the reference's FP32/INT8 tests set
// MOONPOLY_*_FORCE_SPLITK between two calls; its Pattern-2 evaluation clears the enable flags
// mid-run).  Read with a raw getenv on every call and folded into the plan-cache key.
struct LiveFlags {
  bool p2, p3, gen, decode_strict, gen_strict, p2_regular, fp32_p3, int8_p3;
  int fp32_force, int8_force;
  unsigned key() const {
    return (unsigned)p2 | (unsigned)p3 << 1 | (unsigned)gen << 2 | (unsigned)decode_strict << 3 |
           (unsigned)gen_strict << 4 | (unsigned)p2_regular << 5 | (unsigned)fp32_p3 << 6 |
           (unsigned)int8_p3 << 7 | ((unsigned)(fp32_force & 0xff)) << 8 |
           ((unsigned)(int8_force & 0xff)) << 16;
  }
};
LiveFlags read_live_flags(int dtype) {
  LiveFlags f{};
  if (dtype == MP_FP16) {
    f.p2 = env_flag("MOONPOLY_ENABLE_PATTERN2", true);
    f.p3 = env_flag("MOONPOLY_ENABLE_PATTERN3", true);
    f.gen = env_flag("MOONPOLY_ENABLE_GENERATED_SELECTOR", true);
    f.decode_strict = env_flag("MOONPOLY_LLM_DECODE_SELECTOR_STRICT", true);
    f.gen_strict = env_flag("MOONPOLY_GENERATED_SELECTOR_STRICT", false);
    f.p2_regular = env_flag("MOONPOLY_PATTERN2_ALLOW_REGULAR", false);
  } else if (dtype == MP_FP32) {
    f.fp32_p3 = env_flag("MOONPOLY_ENABLE_FP32_PATTERN3", true);
    f.fp32_force = env_int("MOONPOLY_FP32_PATTERN3_FORCE_SPLITK", 0);
    f.gen = env_flag("MOONPOLY_ENABLE_GENERATED_SELECTOR", true);
  } else {
    f.int8_p3 = env_flag("MOONPOLY_ENABLE_INT8_PATTERN3", true);
    f.gen = env_flag("MOONPOLY_ENABLE_GENERATED_SELECTOR", true);
    f.int8_force = env_int("MOONPOLY_INT8_PATTERN3_FORCE_SPLITK", 0);
  }
  return f;
}

// One pass over the environment block per call: a hash of every MOONPOLY_* entry.  As long as the
// hash is unchanged the flag values parsed last time are still right, so the per-call cost is a
// single scan instead of one getenv per flag.
extern "C" char** environ;
uint64_t moonpoly_env_hash() {
  uint64_t h = 1469598103934665603ull;
  for (char** e = environ; e != nullptr && *e != nullptr; ++e) {
    const char* s = *e;
    if (s[0] != 'M' || s[1] != 'O' || s[2] != 'O' || s[3] != 'N' || std::strncmp(s, "MOONPOLY_", 9) != 0) continue;
    for (; *s; ++s) h = (h ^ (unsigned char)*s) * 1099511628211ull;
    h = (h ^ 0xffu) * 1099511628211ull;
  }
  return h;
}
LiveFlags live_flags(int dtype) {
  struct Cached { uint64_t hash; bool valid; LiveFlags f; };
  thread_local Cached cache[3] = {};
  const uint64_t h = moonpoly_env_hash();
  Cached& c = cache[dtype == MP_FP16 ? 0 : dtype == MP_FP32 ? 1 : 2];
  if (!c.valid || c.hash != h) { c.f = read_live_flags(dtype); c.hash = h; c.valid = true; }
  return c.f;
}

// ------------------------------------------------------------------------------------------------
// cost model
// ------------------------------------------------------------------------------------------------
std::atomic<int> g_num_sms{148};

inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// Fitted tables in the reference's artefact layout (per-pid piecewise-linear time per wave in
// k_iter), refit on B200.  Generated by py/moonpoly_b200/refit.py.
#include "generated/mp_fitted_cost.inc"

struct Fit { const int* valid; const int* nseg; const int (*maxk)[3]; const double (*slope)[3];
             const double (*icpt)[3]; int count; const double* red_fixed; const double* red_tile; };

Fit fit_for(int dtype) {
  if (dtype == MP_FP16)
    return {fitted_fp16::kPidValid, fitted_fp16::kSegmentCount, fitted_fp16::kSegmentMaxKiter,
            fitted_fp16::kSegmentSlope, fitted_fp16::kSegmentIntercept, fitted_fp16::kCandidateCount,
            fitted_fp16::kFixedMsPerExtraSlice, fitted_fp16::kTileMsPerExtraSlice};
  if (dtype == MP_INT8)
    return {fitted_int8::kPidValid, fitted_int8::kSegmentCount, fitted_int8::kSegmentMaxKiter,
            fitted_int8::kSegmentSlope, fitted_int8::kSegmentIntercept, fitted_int8::kCandidateCount,
            fitted_int8::kFixedMsPerExtraSlice, fitted_int8::kTileMsPerExtraSlice};
  return {fitted_fp32::kPidValid, fitted_fp32::kSegmentCount, fitted_fp32::kSegmentMaxKiter,
          fitted_fp32::kSegmentSlope, fitted_fp32::kSegmentIntercept, fitted_fp32::kCandidateCount,
          fitted_fp32::kFixedMsPerExtraSlice, fitted_fp32::kTileMsPerExtraSlice};
}

const Fit& fit_of(int dtype) {     // MP_FP16 = 0, MP_INT8 = 1, MP_FP32 = 2
  static const Fit fits[3] = {fit_for(MP_FP16), fit_for(MP_INT8), fit_for(MP_FP32)};
  return fits[dtype == MP_FP16 ? 0 : dtype == MP_INT8 ? 1 : 2];
}

// slot in the fitted tables: primary pids keep their number; 400.. keep theirs (table has 440 slots)
float fitted_unit_ms(int dtype, int pid, int k_iter) {
  const Fit& f = fit_of(dtype);
  if (pid < 0 || pid >= f.count || !f.valid[pid] || f.nseg[pid] <= 0) return kInf;
  int seg = f.nseg[pid] - 1;
  for (int i = 0; i < f.nseg[pid]; ++i)
    if (k_iter <= f.maxk[pid][i]) { seg = i; break; }
  const double u = f.slope[pid][seg] * k_iter + f.icpt[pid][seg];
  return u > 0.0 ? (float)u : kInf;
}

// First-principles time of one work unit (one tile x one K slice) on one SM, in ms:
// per K block the slower of tensor issue and the CTA's share of HBM bandwidth, plus a fixed
// pipeline-fill + epilogue term.
float analytic_unit_ms(int dtype, const TileCfg& c, int k_iter, int units_in_flight) {
  const int sms = g_num_sms.load(std::memory_order_relaxed);
  if (dtype == MP_FP32) {
    const double flops = 2.0 * c.ti * c.tj * 16.0;              // per K step of 16
    const double peak_sm = 60.0e12 / sms;                       // CUDA-core FFMA, sustained
    const double eff = std::min(1.0, (double)(c.ti * c.tj) / (128.0 * 128.0) * 0.6 + 0.4);
    const double bytes = (c.ti + c.tj) * 16.0 * 4.0;
    const double bw = std::min(6.4e12 / std::max(1, std::min(units_in_flight, sms)), 150.0e9);
    const double t = std::max(flops / (peak_sm * eff), bytes / bw);
    return (float)((k_iter * t + 1.5e-6) * 1.0e3);
  }
  const double kb_elems = dtype == MP_INT8 ? 128.0 : 64.0;
  const double peak_sm = (dtype == MP_INT8 ? 3.2e15 : 1.6e15) / sms;
  const double flops = 2.0 * 128.0 * c.bn * kb_elems;
  const double bytes = (128.0 + c.bn) * 128.0;
  const double bw = std::min(6.4e12 / std::max(1, std::min(units_in_flight, sms)), 180.0e9);
  const double t = std::max(flops / peak_sm, bytes / bw);
  const double epi = 0.4e-6 + 128.0 * c.bn * 2.0 / 400.0e9;
  return (float)((k_iter * t + 1.2e-6 + epi) * 1.0e3);
}

constexpr float kLaunchMs = 0.0022f;

float reduction_ms(int dtype, int pid, const TileCfg& c, int tiles, int split_k) {
  if (split_k <= 1) return 0.0f;
  const Fit& f = fit_of(dtype);
  const int extra = split_k - 1;
  if (!g_env.disable_fitted && pid >= 0 && pid < f.count && f.valid[pid] && f.red_fixed[pid] >= 0.0) {
    const double r = f.red_fixed[pid] * extra + f.red_tile[pid] * std::max(1, tiles) * extra;
    return (float)std::max(0.0, r);
  }
  // analytic prior: partials are written once and read once through L2, plus a fixed hand-off
  const int sms = g_num_sms.load(std::memory_order_relaxed);
  const double words = dtype == MP_FP32 ? (double)c.ti * c.tj : 128.0 * c.bn;
  const double bytes = 2.0 * words * 4.0 * split_k * std::max(1, tiles);
  return (float)((0.6e-6 + bytes / (3.0e12 * std::min(1.0, std::max(1, tiles) * 4.0 / sms))) * 1.0e3);
}

}  // namespace

int num_sms_for_model() { return g_num_sms.load(); }
void set_num_sms_for_model(int sms) {
  if (sms > 0) g_num_sms.store(sms);
}

// ------------------------------------------------------------------------------------------------
// pid metadata
// ------------------------------------------------------------------------------------------------
TileCfg tile_cfg(int dtype, int pid) {
  TileCfg c{};
  if (dtype == MP_FP16) {
    int base = -1;
    bool split = false;
    if (pid >= 0 && pid <= 40) {
      base = pid;
      split = in_list(kFp16SplitPids, 17, pid) || pid == 40;
    } else if (pid >= 400 && pid <= 439) {
      base = fp16_base_pid(pid);
      split = true;
    } else if (pid == 66) {
      base = 40; split = true;
    } else if (pid == 42) {
      base = 0; split = true;
    } else if (pid == 43) {
      base = 9; split = true;      // 64x16 class
    } else if (pid == 44) {
      base = 37; split = true;     // 64x32 class
    } else if (pid == 1100) {
      // library-native skinny streaming kernel (min(m,n) <= 8): orient 2, no tile in the UMMA sense
      c.valid = true; c.orient = 2; c.bn = 16; c.align = 8; c.split_capable = false;
      return c;
    } else if (pid == 1101) {
      // library-native streaming warp-MMA kernel (min(m,n) <= 64): orient 3
      c.valid = true; c.orient = 3; c.bn = 64; c.align = 8; c.split_capable = false;
      return c;
    } else if (pid >= 1000 && pid < 1064) {
      // library-native tiles (no counterpart in the reference's pid space): pid = 1000 + 32*orient + bn/16
      const int bn = ((pid - 1000) & 31) * 16;
      if (bn < 16 || bn > 256) return c;
      c.valid = true; c.orient = (pid - 1000) >> 5; c.bn = bn; c.align = 8; c.split_capable = true;
      return c;
    } else if (pid >= 1200 && pid < 1264) {
      // library-native 256-row tiles: pid = 1200 + 32*orient + bn/16
      const int bn = ((pid - 1200) & 31) * 16;
      if (bn < 16 || bn > 256) return c;
      c.valid = true; c.orient = (pid - 1200) >> 5; c.bn = bn; c.align = 8; c.split_capable = true; c.xm = 2;
      return c;
    } else if (fp16_explicit_range(pid)) {
      c.valid = true; c.orient = 0; c.bn = 16; c.align = in_list(kFp16ExplicitAlign4, 45, pid) ? 4 : 8;
      c.split_capable = true;
      return c;
    }
    if (base < 0) return c;
    const U& u = kFp16Primary[base];
    c.valid = true; c.orient = u.orient; c.bn = u.bn; c.align = u.align; c.split_capable = split;
    if (pid == 407) c.align = 8;
    if (pid == 43 || pid == 44) c.align = 8;
    return c;
  }
  if (dtype == MP_INT8) {
    if (pid == 1101) {            // library-native streaming warp-MMA kernel (min(m,n) <= 64)
      c.valid = true; c.orient = 3; c.bn = 64; c.align = 16; c.split_capable = false;
      return c;
    }
    if ((pid >= 1000 && pid < 1064) || (pid >= 1200 && pid < 1264)) {
      // library-native tiles, same numbering as for FP16: 1000 + 32*orient + bn/16 (128-row), 1200 + ... (256-row)
      const int base = pid >= 1200 ? 1200 : 1000;
      const int bn = ((pid - base) & 31) * 16;
      if (bn < 16 || bn > 256) return c;
      c.valid = true; c.orient = (pid - base) >> 5; c.bn = bn; c.align = 16; c.split_capable = true;
      c.xm = base == 1200 ? 2 : 1;
      return c;
    }
    if (pid < 0 || pid > 45) return c;
    const U& u = kInt8Primary[pid];
    c.valid = true; c.orient = u.orient; c.bn = u.bn; c.align = u.align; c.split_capable = true;
    return c;
  }
  if (dtype == MP_FP32) {
    if (pid == 1101) {            // library-native FP32 streaming kernel (min(m,n) <= 64)
      c.valid = true; c.orient = 3; c.ti = 64; c.tj = 64; c.align = 4; c.split_capable = false;
      return c;
    }
    if (pid < 0 || pid > 39) return c;
    c.valid = true; c.ti = kFp32Primary[pid].ti; c.tj = kFp32Primary[pid].tj; c.align = 1;
    c.split_capable = true;
    return c;
  }
  return c;
}

bool pid_exists(int dtype, int pid) { return tile_cfg(dtype, pid).valid; }

void pid_tile_meta(int dtype, int pid, int out[3]) {
  const TileCfg c = tile_cfg(dtype, pid);
  if (!c.valid) { out[0] = out[1] = out[2] = 0; return; }
  if (dtype == MP_FP32) { out[0] = c.tj; out[1] = c.ti; out[2] = 16; return; }
  if (c.orient == 3) { out[0] = 16; out[1] = 64; out[2] = 32; return; }     // streaming kernel: 16 streamed rows per CTA x up to 64 rows
  if (c.orient == 2) { out[0] = 16; out[1] = 8; out[2] = 1024; return; }   // skinny kernel: 16 streamed rows per CTA x up to 8 rows
  const int rows = c.xm == 2 ? 256 : 128;
  out[0] = c.orient == 0 ? c.bn : rows;   // pm: tile over RCC n
  out[1] = c.orient == 0 ? rows : c.bn;   // pn: tile over RCC m
  out[2] = dtype == MP_INT8 ? 128 : 64;
}

namespace {
// pid metadata resolved once (the selector evaluates ~90 pids per unseen shape)
struct PidMeta { TileCfg cfg; int meta[3]; };
struct MetaTables {
  PidMeta fp16[440], int8[46], fp32[40], native[64], native256[64], native_i8[64], native256_i8[64], skinny, streaming, streaming_i8, streaming_f32;
  MetaTables() {
    skinny.cfg = tile_cfg(MP_FP16, 1100); pid_tile_meta(MP_FP16, 1100, skinny.meta);
    streaming.cfg = tile_cfg(MP_FP16, 1101); pid_tile_meta(MP_FP16, 1101, streaming.meta);
    streaming_i8.cfg = tile_cfg(MP_INT8, 1101); pid_tile_meta(MP_INT8, 1101, streaming_i8.meta);
    streaming_f32.cfg = tile_cfg(MP_FP32, 1101); pid_tile_meta(MP_FP32, 1101, streaming_f32.meta);
    for (int p = 0; p < 64; ++p) { native[p].cfg = tile_cfg(MP_FP16, 1000 + p); pid_tile_meta(MP_FP16, 1000 + p, native[p].meta); }
    for (int p = 0; p < 64; ++p) { native256[p].cfg = tile_cfg(MP_FP16, 1200 + p); pid_tile_meta(MP_FP16, 1200 + p, native256[p].meta); }
    for (int p = 0; p < 64; ++p) { native_i8[p].cfg = tile_cfg(MP_INT8, 1000 + p); pid_tile_meta(MP_INT8, 1000 + p, native_i8[p].meta); }
    for (int p = 0; p < 64; ++p) { native256_i8[p].cfg = tile_cfg(MP_INT8, 1200 + p); pid_tile_meta(MP_INT8, 1200 + p, native256_i8[p].meta); }
    for (int p = 0; p < 440; ++p) { fp16[p].cfg = tile_cfg(MP_FP16, p); pid_tile_meta(MP_FP16, p, fp16[p].meta); }
    for (int p = 0; p < 46; ++p) { int8[p].cfg = tile_cfg(MP_INT8, p); pid_tile_meta(MP_INT8, p, int8[p].meta); }
    for (int p = 0; p < 40; ++p) { fp32[p].cfg = tile_cfg(MP_FP32, p); pid_tile_meta(MP_FP32, p, fp32[p].meta); }
  }
};
const PidMeta* pid_meta(int dtype, int pid) {
  static const MetaTables t;
  if (pid < 0) return nullptr;
  if (dtype == MP_FP16) {
    if (pid == 1100) return &t.skinny;
    if (pid == 1101) return &t.streaming;
    if (pid >= 1000 && pid < 1064) return t.native[pid - 1000].cfg.valid ? &t.native[pid - 1000] : nullptr;
    if (pid >= 1200 && pid < 1264) return t.native256[pid - 1200].cfg.valid ? &t.native256[pid - 1200] : nullptr;
    return pid < 440 && t.fp16[pid].cfg.valid ? &t.fp16[pid] : nullptr;
  }
  if (dtype == MP_INT8) {
    if (pid == 1101) return &t.streaming_i8;
    if (pid >= 1000 && pid < 1064) return t.native_i8[pid - 1000].cfg.valid ? &t.native_i8[pid - 1000] : nullptr;
    if (pid >= 1200 && pid < 1264) return t.native256_i8[pid - 1200].cfg.valid ? &t.native256_i8[pid - 1200] : nullptr;
    return pid < 46 ? &t.int8[pid] : nullptr;
  }
  if (dtype == MP_FP32) return pid == 1101 ? &t.streaming_f32 : pid < 40 ? &t.fp32[pid] : nullptr;
  return nullptr;
}
inline int cdiv(int a, int b) { return (a + b - 1) / b; }
}  // namespace

float cost_ms(int dtype, int pid, int split_k, int m, int n, int k) {
  const PidMeta* pm = pid_meta(dtype, pid);
  if (pm == nullptr || m <= 0 || n <= 0 || k <= 0) return kInf;
  const TileCfg& c = pm->cfg;
  const int* meta = pm->meta;
  const unsigned S = (unsigned)std::max(1, split_k);
  // unsigned 32-bit divisions: an unseen shape costs ~90 of these evaluations
  const unsigned lm = std::max(1u, ((unsigned)n + (unsigned)meta[0] - 1u) / (unsigned)meta[0]);   // feature_m = n
  const unsigned ln = std::max(1u, ((unsigned)m + (unsigned)meta[1] - 1u) / (unsigned)meta[1]);   // feature_n = m
  const unsigned kd = (unsigned)meta[2] * S;
  const int k_iter = (int)std::max(1u, ((unsigned)k + kd - 1u) / kd);
  const unsigned long long units = (unsigned long long)lm * ln * S;
  const unsigned sms = (unsigned)g_num_sms.load(std::memory_order_relaxed);
  const int waves = units <= sms ? 1 : units < (1ull << 32) ? (int)(((unsigned)units + sms - 1u) / sms)
                                                            : (int)((units + sms - 1ull) / sms);
  static const bool* disable_fitted = &env().disable_fitted;      // g_env lives for the whole process; reload_env rewrites it in place
  float unit = kInf;
  if (!*disable_fitted) unit = fitted_unit_ms(dtype, pid, k_iter);
  float total;
  if (std::isfinite(unit) && unit > 0.0f) {
    total = waves * unit;
  } else {
    unit = analytic_unit_ms(dtype, c, k_iter, (int)std::min<unsigned long long>(units, sms));
    total = waves * unit + kLaunchMs;
  }
  return total + reduction_ms(dtype, pid, c, (int)(lm * ln), (int)S);
}

// Split-K hand-off and reduction term alone (gemm_reduction_cost_model of the reference).
float reduction_cost_ms(int dtype, int pid, int split_k, int m, int n) {
  const PidMeta* pm = pid_meta(dtype, pid);
  if (pm == nullptr || m <= 0 || n <= 0) return kInf;
  const int lm = std::max(1, cdiv(n, pm->meta[0]));
  const int ln = std::max(1, cdiv(m, pm->meta[1]));
  return reduction_ms(dtype, pid, pm->cfg, lm * ln, std::max(1, split_k));
}

int choose_pattern2_split_n(int n) {
  constexpr int tile_n = 128;
  int split_n = (n * 3 / 4 / tile_n) * tile_n;
  if (split_n <= 0) split_n = tile_n;
  if (split_n >= n) split_n = ((n / tile_n) - 1) * tile_n;
  return split_n;
}

// ------------------------------------------------------------------------------------------------
// online selection
// ------------------------------------------------------------------------------------------------
namespace {

// Measured decode plans for Linear(M,N,K) shapes: same record layout as the reference's
// generated/fp16/rcc/llm_decode_selector.inc (m, n, k, pid, split_k); values measured on B200.
struct DecodeEntry { int m, n, k, pid, split_k; };
// Measured plans for RCC shapes, bucketed over the dynamic dimension: a row applies when
// m_lo <= m <= m_hi, n_lo <= n <= n_hi, k matches and m has the row's alignment class
// (0 any, 1 m % 8 == 0, 2 m % 8 != 0: C columns are then not 16-byte aligned).
struct PlanRow { int m_lo, m_hi, n_lo, n_hi, k, align_class, pid, split_k; float ms; };
#include "generated/mp_decode_selector.inc"
// Measured plans of the INT8 scaled matmul out[M,N] = A[M,K] * B[N,K]^T: a row applies to M in
// [m_lo, m_hi] with the row's exact (N, K).  orient 0 / 1: tile of the tensor-core kernel (tokens /
// channels on the 128-row side, the other side tiled by bn); orient 3: the streaming kernel; orient 4 / 5:
// orient 0 / 1 with 256-row tiles.
struct ScaledPlanRow { int m_lo, m_hi, n, k, orient, bn, split_k; float ms; };
#include "generated/mp_scaled_plans.inc"

// Without a measured row: up to how many narrow-side rows the INT8 streaming kernel beats the
// tiles, by the size of the streamed operand (measured on B200: 4096x4096 ... 28672x4096)
bool int8_prefers_stream(int narrow, long long wide_rows, int k) {
  if (narrow < 1 || k < 16 || k % 16 != 0) return false;
  const long long bytes = wide_rows * (long long)k;
  if (narrow <= 8) return true;
  if (narrow <= 16) return bytes <= (64ll << 20);
  if (narrow <= 32) return bytes <= (32ll << 20);
  return false;
}

inline void consider(mp_plan& best, int pattern, int pid, int split_k, int split_n, float ms, float margin) {
  if (!std::isfinite(ms) || ms <= 0.0f) return;
  if (ms < best.estimated_ms * margin) {
    best.pattern = pattern; best.pid = pid; best.split_k = split_k; best.split_n = split_n;
    best.estimated_ms = ms;
  }
}

bool pattern3_k_gate(int k, int split_k, int min_tile_k, int min_k, int min_part_k) {
  if (split_k <= 1 || k < min_k || k < min_tile_k * split_k) return false;
  return (k + split_k - 1) / split_k >= min_part_k;
}

int best_primary(int dtype, int count, int m, int n, int k, float* ms_out) {
  int best = -1;
  float best_ms = kInf;
  for (int pid = 0; pid < count; ++pid) {
    const TileCfg c = tile_cfg(dtype, pid);
    if (!c.valid || k % c.align != 0) continue;
    const float ms = cost_ms(dtype, pid, 1, m, n, k);
    if (ms < best_ms) { best_ms = ms; best = pid; }
  }
  if (ms_out) *ms_out = best_ms;
  return best;
}

}  // namespace

// Cheapest primary pid under the K-alignment contract (cutlass_gemm_predict of the reference).
int predict_primary_pid(int dtype, int m, int n, int k, float* ms) {
  const int count = dtype == MP_FP16 ? 40 : dtype == MP_INT8 ? 46 : 40;
  const int pid = best_primary(dtype, count, m, n, k, ms);
  return pid < 0 ? 0 : pid;
}

namespace {

mp_plan select_fp16(int m, int n, int k, const LiveFlags& lf) {
  const Env& e = env();
  mp_plan best{MP_PATTERN_SINGLE, 0, 1, 0, kInf};

  // (1) measured plans: Linear (M,N,K) entries match RCC (m = N, n = M)
  bool matched = false;
  if (lf.gen) {
    for (int i = 0; i < kDecodeSelectorCount; ++i) {
      const DecodeEntry& d = kDecodeSelector[i];
      if (d.m == n && d.n == m && d.k == k) {
        const int S = std::max(1, d.split_k);
        if (S > 1 && !pattern3_k_gate(k, S, 64, e.p3_min_k, e.p3_min_part_k)) continue;
        const TileCfg c = tile_cfg(MP_FP16, d.pid);
        if (!c.valid || k % c.align != 0) continue;
        consider(best, (S > 1 || c.split_capable) ? MP_PATTERN_SPLITK : MP_PATTERN_SINGLE, d.pid, S, 0,
                 cost_ms(MP_FP16, d.pid, S, m, n, k), e.gen_margin);
        matched = true;
      }
    }
    // rows are looked up through an index sorted by k (built once): a shape scans only its own K's rows
    static const std::vector<std::pair<int, int>> by_k = [] {
      std::vector<std::pair<int, int>> v;
      for (int i = 0; i < kMeasuredPlanCount; ++i) v.emplace_back(kMeasuredPlans[i].k, i);
      std::stable_sort(v.begin(), v.end(), [](const std::pair<int, int>& a, const std::pair<int, int>& b) { return a.first < b.first; });
      return v;
    }();
    auto it = std::lower_bound(by_k.begin(), by_k.end(), std::make_pair(k, -1));
    for (; it != by_k.end() && it->first == k; ++it) {
      const PlanRow& r = kMeasuredPlans[it->second];
      if (m < r.m_lo || m > r.m_hi || n < r.n_lo || n > r.n_hi) continue;
      if ((r.align_class == 1 && m % 8 != 0) || (r.align_class == 2 && m % 8 == 0)) continue;
      const int S = std::max(1, r.split_k);
      const TileCfg c = tile_cfg(MP_FP16, r.pid);
      if (!c.valid || k % c.align != 0) continue;
      consider(best, S > 1 ? MP_PATTERN_SPLITK : MP_PATTERN_SINGLE, r.pid, S, 0, r.ms, e.gen_margin);
      matched = true;
    }
    if (matched && (lf.decode_strict || lf.gen_strict)) return best;
  }

  // (2) Pattern-1: best single primary pid 0..39
  for (int pid = 0; pid < 40; ++pid) {
    const TileCfg c = tile_cfg(MP_FP16, pid);
    if (k % c.align != 0) continue;
    consider(best, MP_PATTERN_SINGLE, pid, 1, 0, cost_ms(MP_FP16, pid, 1, m, n, k), 1.0f);
  }

  // (3) Pattern-3: split-capable pids x {2,4,8}, must beat the best by the margin
  if (lf.p3) {
    static constexpr int kSplit[3] = {2, 4, 8};
    for (int pid : kFp16SplitPids) {
      const TileCfg c = tile_cfg(MP_FP16, pid);
      if (k % c.align != 0) continue;
      for (int S : kSplit) {
        if (!pattern3_k_gate(k, S, 64, e.p3_min_k, e.p3_min_part_k)) continue;
        consider(best, MP_PATTERN_SPLITK, pid, S, 0, cost_ms(MP_FP16, pid, S, m, n, k), e.p3_margin);
      }
    }
  }

  // (4) Pattern-2: a 128-wide main region plus a narrow tail region in one launch
  if (lf.p2 && k % 8 == 0 && n >= e.p2_min_n) {
    constexpr int tile_n = 128;
    int split_n = 0;
    const int tail = n % tile_n;
    bool ok = false;
    if (tail == 0) {
      if (lf.p2_regular) {
        split_n = choose_pattern2_split_n(n);
        ok = split_n > 0 && split_n < n && split_n % tile_n == 0;
      }
    } else if ((float)tail / tile_n <= e.p2_max_tail_ratio) {
      split_n = (n / tile_n) * tile_n;
      ok = split_n > 0 && split_n < n;
    }
    if (ok) {
      float ms0, ms1;
      best_primary(MP_FP16, 40, m, split_n, k, &ms0);
      best_primary(MP_FP16, 40, m, n - split_n, k, &ms1);
      // both regions share one launch: critical path of the two plus the schedule's tail imbalance
      const float ms = std::max(ms0, ms1) + 0.0008f;
      consider(best, MP_PATTERN_COMBINE, -1, 1, split_n, ms, e.p2_margin);
    }
  }

  // (5) Library-native refinements of a cost-model choice (never of a measured row), with the tile kept:
  //  - an RCC m that is not a multiple of 8 leaves the rows of C[n, m] unaligned; with the rows of A on the TMEM
  //    lanes (orient 0) a warp still writes 64 contiguous bytes per column, the other way round every lane writes
  //    2-byte pieces of 16 different rows (2047 x 2048 x 2048: 55 us against 20 us);
  //  - 256-row tiles (pids 1200+) once a tile at least 192 wide fills half the GPU that way: a third less operand
  //    traffic per FLOP (4096 x 4096 x 4104: 177 -> 135 us, 2297 x 5120 x 5120: 184 -> 96 us with both).
  //  - at most 16 rows on the narrow side: the streaming kernel (pid 1101), which the measured tables pick for every
  //    such bucket of every tuned layer (3 x 5120 x 5120: 10 us; the best tile needs a split-K pass).
  if (lf.gen && !matched && k % 8 == 0 && k >= 16 && std::min(m, n) <= 16 && best.pattern != MP_PATTERN_COMBINE) {
    const double bytes = 2.0 * ((double)m * k + (double)n * k + (double)m * n);
    return mp_plan{MP_PATTERN_SINGLE, 1101, 1, 0, (float)(bytes / 6.0e9 + 2.5e-3)};
  }
  if (lf.gen && !matched && k % 8 == 0 && best.pid >= 0 && best.pid < 440 &&
      (best.pattern == MP_PATTERN_SINGLE || best.pattern == MP_PATTERN_SPLITK)) {
    const TileCfg c = tile_cfg(MP_FP16, best.pid);
    if (c.valid && (c.orient == 0 || c.orient == 1) && c.bn >= 16 && c.bn <= 256 && c.bn % 16 == 0) {
      const int orient = (m % 8 != 0 && m >= 128) ? 0 : c.orient;      // a short m belongs on the bn side whatever its alignment
      const int P = orient == 0 ? m : n, Q = orient == 0 ? n : m;
      const int sms = g_num_sms.load(std::memory_order_relaxed);
      const bool wide = best.pattern == MP_PATTERN_SINGLE && c.bn >= 192 && P >= 512 &&
                        cdiv(P, 256) * cdiv(Q, c.bn) >= sms / 2;
      if (wide || orient != c.orient) {
        best.pid = (wide ? 1200 : 1000) + 32 * orient + c.bn / 16;
        if (wide) best.estimated_ms *= 0.88f;
      }
    }
  }
  return best;
}

mp_plan select_simple(int dtype, int count, int m, int n, int k, bool p3_enabled, int forced, int min_tile_k,
                      int min_k, int min_part_k, float margin, int k_align_for_split) {
  float ms = kInf;
  int pid = best_primary(dtype, count, m, n, k, &ms);
  if (pid < 0) pid = 0;
  mp_plan best{MP_PATTERN_SINGLE, pid, 1, 0, ms};
  if (p3_enabled) {
    // the dedicated split-K tile of the reference (fp32: 128x64x8, int8: 128x128x64) is pid -1
    const int split_pid = dtype == MP_FP32 ? 23 : 6;
    if (forced > 1) {
      best.pattern = MP_PATTERN_SPLITK; best.pid = -1; best.split_k = forced;
      best.estimated_ms = cost_ms(dtype, split_pid, forced, m, n, k);
      return best;
    }
    static constexpr int kSplit[3] = {2, 4, 8};
    for (int S : kSplit) {
      if (k % k_align_for_split != 0) continue;
      if (!pattern3_k_gate(k, S, min_tile_k, min_k, min_part_k)) continue;
      const float c = cost_ms(dtype, split_pid, S, m, n, k);
      if (std::isfinite(c) && c > 0.0f && c < best.estimated_ms * margin) {
        best.pattern = MP_PATTERN_SPLITK; best.pid = -1; best.split_k = S; best.estimated_ms = c;
      }
    }
  }
  return best;
}

// plan cache: 2048 sets of two ways (the most recent plan of a set sits in way 0), one mutex; a lookup is a hash,
// a lock and two compares
struct CacheLine { int dtype, m, n, k; unsigned flags, epoch; mp_plan plan; };
constexpr int kCacheSets = 2048;
CacheLine g_cache[kCacheSets][2];
std::mutex g_cache_mu;

inline unsigned hash_shape(int dtype, int m, int n, int k, unsigned flags) {
  uint64_t h = (uint64_t)(unsigned)m * 0x9E3779B97F4A7C15ull;
  h ^= ((uint64_t)(unsigned)n + 0x7F4A7C15ull) * 0xBF58476D1CE4E5B9ull;
  h ^= ((uint64_t)(unsigned)k + 0x1CE4E5B9ull) * 0x94D049BB133111EBull;
  h ^= (uint64_t)flags * 0x2545F4914F6CDD1Dull + (uint64_t)dtype;
  return (unsigned)(h >> 40) & (kCacheSets - 1);
}
inline bool line_is(const CacheLine& c, int dtype, int m, int n, int k, unsigned flags, unsigned epoch) {
  return c.epoch == epoch && c.dtype == dtype && c.m == m && c.n == n && c.k == k && c.flags == flags;
}

}  // namespace

mp_plan select_plan(int dtype, int m, int n, int k) {
  const LiveFlags lf = live_flags(dtype);
  const unsigned fkey = lf.key();
  const unsigned epoch = g_env_epoch.load(std::memory_order_acquire);
  const unsigned slot = hash_shape(dtype, m, n, k, fkey);
  {
    std::lock_guard<std::mutex> g(g_cache_mu);
    CacheLine* set = g_cache[slot];
    if (line_is(set[0], dtype, m, n, k, fkey, epoch)) return set[0].plan;
    if (line_is(set[1], dtype, m, n, k, fkey, epoch)) {
      std::swap(set[0], set[1]);
      return set[0].plan;
    }
  }
  mp_plan plan;
  const Env& e = env();
  if (dtype == MP_FP16) {
    plan = select_fp16(m, n, k, lf);
  } else if (dtype == MP_FP32) {
    plan = select_simple(MP_FP32, 40, m, n, k, lf.fp32_p3, lf.fp32_force, 8, e.fp32_p3_min_k,
                         e.fp32_p3_min_part_k, e.fp32_p3_margin, 1);
    // few rows on one side: the FP32 streaming kernel (library-native pid 1101) replaces tile + split-K pass
    if (lf.gen && lf.fp32_force <= 1 && std::min(m, n) >= 1 && std::min(m, n) <= 64 && k >= 4 && k % 4 == 0) {
      const double bytes = 4.0 * ((double)m * k + (double)n * k + (double)m * n);
      plan = mp_plan{MP_PATTERN_SINGLE, 1101, 1, 0, (float)(bytes / 6.0e9 + 3.0e-3)};
    }
  } else {
    plan = select_simple(MP_INT8, 46, m, n, k, lf.int8_p3, lf.int8_force, 64, e.int8_p3_min_k,
                         e.int8_p3_min_part_k, e.int8_p3_margin, 16);
    // few rows on the narrow side: the streaming kernel (library-native pid 1101) beats every tile; it is part
    // of this library's generated plans, so the same flag gates it
    if (lf.gen && lf.int8_force <= 1 && int8_prefers_stream(std::min(m, n), std::max(m, n), k)) {
      const double bytes = (double)m * k + (double)n * k + 4.0 * m * n;
      plan = mp_plan{MP_PATTERN_SINGLE, 1101, 1, 0, (float)(bytes / 6.0e9 + 2.5e-3)};
    }
    // the measured scaled-matmul plans describe the same int8 main loop on the same (m, n, k): use them for the
    // plain int32-output GEMM as well (the epilogues differ, the ranking of the tiles hardly does)
    bool int8_row = false;
    if (lf.gen && lf.int8_force <= 1 && k % 16 == 0) {
      for (int i = 0; i < kScaledPlanCount; ++i) {
        const ScaledPlanRow& r = kScaledPlans[i];
        if (r.n != n || r.k != k || m < r.m_lo || m > r.m_hi) continue;
        int8_row = true;
        if (r.orient == 3) {
          if (std::min(m, n) <= 64) plan = mp_plan{MP_PATTERN_SINGLE, 1101, 1, 0, r.ms};
        } else {
          const int S = std::max(1, r.split_k);
          const int pid = (r.orient >= 4 ? 1200 : 1000) + 32 * (r.orient & 1) + r.bn / 16;
          plan = mp_plan{S > 1 ? MP_PATTERN_SPLITK : MP_PATTERN_SINGLE, pid, S, 0, r.ms};
        }
        break;
      }
    }
    // a cost-model choice with a tile at least 192 wide moves to its 256-row version once that fills half the GPU
    // (the same refinement as for FP16: a third less operand traffic per MAC)
    if (lf.gen && !int8_row && lf.int8_force <= 1 && k % 16 == 0 && plan.pattern == MP_PATTERN_SINGLE && plan.pid >= 0 &&
        plan.pid < 46) {
      const TileCfg c = tile_cfg(MP_INT8, plan.pid);
      if (c.valid && (c.orient == 0 || c.orient == 1) && c.bn >= 192 && c.bn <= 256 && c.bn % 16 == 0) {
        const int P = c.orient == 0 ? m : n, Q = c.orient == 0 ? n : m;
        const int sms = g_num_sms.load(std::memory_order_relaxed);
        if (P >= 512 && cdiv(P, 256) * cdiv(Q, c.bn) >= sms / 2) {
          plan.pid = 1200 + 32 * c.orient + c.bn / 16;
          plan.estimated_ms *= 0.88f;
        }
      }
    }
  }
  if (std::getenv("MOONPOLY_DEBUG_ONLINE_SELECTOR")) {
    std::fprintf(stdout, "[moonpoly][%s] online m=%d n=%d k=%d -> Pattern%d pid=%d split_k=%d split_n=%d est_ms=%g\n",
                 dtype == MP_FP16 ? "fp16" : dtype == MP_FP32 ? "fp32" : "int8", m, n, k, plan.pattern,
                 plan.pid, plan.split_k, plan.split_n, plan.estimated_ms);
  }
  {
    std::lock_guard<std::mutex> g(g_cache_mu);
    g_cache[slot][1] = g_cache[slot][0];
    g_cache[slot][0] = CacheLine{dtype, m, n, k, fkey, epoch, plan};
  }
  return plan;
}

void reload_env() {
  std::call_once(g_env_once, [] {});
  load_env();
  g_env_epoch.fetch_add(1, std::memory_order_acq_rel);
}

// ------------------------------------------------------------------------------------------------
// scaled int8 matmul configs: (tile over tokens M, tile over channels N, tile_k, alignment)
// ------------------------------------------------------------------------------------------------
namespace {
struct SC { int orient; int bn; int tile_m, tile_n; };
// orient 0: tokens (A rows) on UMMA-M, channels tiled by bn.  orient 1: channels (B rows) on
// UMMA-M, tokens tiled by bn.
constexpr SC kScaled[kScaledConfigCount] = {
    {0, 128, 128, 128}, {1, 64, 64, 128}, {1, 32, 32, 128}, {1, 16, 16, 128}, {0, 256, 128, 256}, {1, 256, 256, 128},
};
}  // namespace

void scaled_mm_config_meta(int id, int out[4]) {
  out[0] = kScaled[id].tile_m; out[1] = kScaled[id].tile_n; out[2] = 128; out[3] = 16;
}

ScaledCfg scaled_mm_select(int M, int N, int K) {
  ScaledCfg best{0, kScaled[0].orient, kScaled[0].bn, 1, false, 1};
  float best_ms = kInf;
  const int sms = g_num_sms.load(std::memory_order_relaxed);
  static constexpr int kSplit[4] = {1, 2, 4, 8};
  for (int id = 0; id < kScaledConfigCount; ++id) {
    const SC& s = kScaled[id];
    TileCfg c{}; c.valid = true; c.orient = s.orient; c.bn = s.bn;
    const int tiles = ceil_div(M, s.tile_m) * ceil_div(N, s.tile_n);
    for (int S : kSplit) {
      if (S > 1 && (K < 2048 || (K + S - 1) / S < 512)) continue;
      const int k_iter = std::max(1, ceil_div(K, 128LL * S));
      const long long units = (long long)tiles * S;
      const int waves = std::max(1, ceil_div(units, sms));
      float ms = waves * analytic_unit_ms(MP_INT8, c, k_iter, (int)std::min<long long>(units, sms)) +
                 reduction_ms(MP_INT8, -1, c, tiles, S);
      // padded work is wasted tensor time: prefer the tile that fits M
      if (ms < best_ms) { best_ms = ms; best = ScaledCfg{id, s.orient, s.bn, S, false, 1}; }
    }
  }
  best.stream = int8_prefers_stream(std::min(M, N), std::max(M, N), K);
  {
    // 256-row tiles once a tile at least 192 wide fills half the GPU that way (measured rows below may override)
    const int P = best.orient == 0 ? M : N, Q = best.orient == 0 ? N : M;
    if (best.split_k == 1 && best.bn >= 192 && P >= 512 && ceil_div(P, 256) * ceil_div(Q, best.bn) >= sms / 2) best.xm = 2;
  }
  // measured rows win over the model; `id` stays the model's choice among the six public configurations
  if (env_flag("MOONPOLY_ENABLE_GENERATED_SELECTOR", true)) {
    for (int i = 0; i < kScaledPlanCount; ++i) {
      const ScaledPlanRow& r = kScaledPlans[i];
      if (r.n != N || r.k != K || M < r.m_lo || M > r.m_hi) continue;
      best.stream = r.orient == 3;
      if (r.orient != 3) {
        best.orient = r.orient & 1; best.xm = r.orient >= 4 ? 2 : 1; best.bn = r.bn; best.split_k = std::max(1, r.split_k);
      }
      break;
    }
  }
  return best;
}

bool is_explicit_neighborhood_fp16_pid(int pid) { return fp16_explicit_range(pid) || (pid >= 400 && pid <= 439); }

int elite_fp16_pids(int* pids, int capacity) {
  int count = 0;
  for (int pid = 0; pid < 40; ++pid, ++count)
    if (pids && count < capacity) pids[count] = pid;
  for (int pid : kEliteExtra) {
    if (pids && count < capacity) pids[count] = pid;
    ++count;
  }
  return count;
}

}  // namespace mp
