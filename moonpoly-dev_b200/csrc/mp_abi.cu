// C ABI of libmoonpoly_gemm.so: argument checks, plan selection, tensor-map set-up, launches.
// See include/moonpoly_abi.h for the contract of every entry point.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "../../include/moonpoly_abi.h"
#include "mp_gemv.cuh"
#include "mp_stream_mma.cuh"
#include "mp_select.h"
#include "mp_simt_gemm.cuh"
#include "mp_umma_gemm.cuh"

namespace {

using namespace mp;

thread_local char g_err[512] = "";
// Programmatic dependent launch of the tensor-core kernel (prologue overlaps the previous kernel's
// tail).  MOONPOLY_DISABLE_PDL=1 turns it off.
const bool g_use_pdl = [] {
  const char* v = std::getenv("MOONPOLY_DISABLE_PDL");
  return !(v && v[0] && v[0] != '0');
}();
// Stream-K head for tile counts that are not a multiple of the grid (see run_umma).
// MOONPOLY_DISABLE_STREAMK=1 turns it off (read at load and again by mp_reload_env).
bool streamk_from_env() {
  const char* v = std::getenv("MOONPOLY_DISABLE_STREAMK");
  return !(v && v[0] && v[0] != '0');
}
std::atomic<bool> g_use_streamk{streamk_from_env()};
// Split-K inside a thread-block cluster (partials exchanged through distributed shared memory instead of
// the global scratch; see run_umma).  Bit-identical to the scratch path, but measured slower on B200
// (M = 128, N = K = 4096: 15.3 us against 14.1 us; the cluster launch costs more than the exchange saves), so
// it is off unless MOONPOLY_ENABLE_CLUSTER_SPLITK=1 (read at load and again by mp_reload_env).
bool cluster_splitk_from_env() {
  const char* v = std::getenv("MOONPOLY_ENABLE_CLUSTER_SPLITK");
  return v && v[0] && v[0] != '0';
}
std::atomic<bool> g_use_cluster_splitk{cluster_splitk_from_env()};
std::atomic<unsigned long long> g_launches{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define MP_CUDA_TRY(expr)                                                                         \
  do {                                                                                            \
    cudaError_t e__ = (expr);                                                                     \
    if (e__ != cudaSuccess)                                                                       \
      return fail(MP_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__,  \
                  __LINE__);                                                                      \
  } while (0)

// ------------------------------------------------------------------------------------------------
// per-device state
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

struct DeviceState {
  bool ready = false;
  int sms = 0;
  int cc = 0;
  bool attrs[9] = {false, false, false, false, false, false, false, false, false};
  bool tile_f32_attrs[12] = {};
};
constexpr int kMaxDevices = 32;
DeviceState g_dev[kMaxDevices];
EncodeTiledFn g_encode = nullptr;
std::mutex g_mu;

int device_state(DeviceState** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(MP_ERR_CUDA, "no CUDA device: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(MP_ERR_CUDA, "device index %d out of range", dev);
  DeviceState& d = g_dev[dev];
  if (!d.ready) {
    std::lock_guard<std::mutex> g(g_mu);
    if (!d.ready) {
      int major = 0, minor = 0;
      MP_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
      MP_CUDA_TRY(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
      MP_CUDA_TRY(cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev));
      d.cc = major * 10 + minor;
      if (g_encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        MP_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
        if (fn == nullptr || q != cudaDriverEntryPointSuccess)
          return fail(MP_ERR_CUDA, "driver has no cuTensorMapEncodeTiled");
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
      }
      set_num_sms_for_model(d.sms);
      d.ready = true;
    }
  }
  if (d.cc != 100 && d.cc != 103)
    return fail(MP_ERR_UNSUPPORTED, "device compute capability %d.%d is not sm_100: this library has no other path",
                d.cc / 10, d.cc % 10);
  *out = &d;
  return MP_OK;
}

// ------------------------------------------------------------------------------------------------
// scratch pool: one buffer per (device, stream), grown on demand, counters kept zero by the kernels
// ------------------------------------------------------------------------------------------------
struct Scratch {
  int dev; cudaStream_t stream; uint8_t* ptr; size_t bytes; size_t counter_bytes;
};
std::vector<Scratch> g_scratch;

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// The partials start behind the counter area the buffer was created with (`have_counters`), which
// may be larger than what this call asks for: capacity is tested against that real layout.
bool scratch_must_grow(size_t have_bytes, size_t have_counters, size_t want_counters, size_t partial_bytes) {
  return have_counters < want_counters || have_bytes < std::max(have_counters, want_counters) + partial_bytes;
}

bool stream_is_capturing(cudaStream_t stream) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &st) != cudaSuccess) { cudaGetLastError(); return false; }
  return st != cudaStreamCaptureStatusNone;
}

int get_scratch(cudaStream_t stream, size_t counter_bytes, size_t partial_bytes, uint8_t** counters,
                uint8_t** partials) {
  int dev = 0;
  MP_CUDA_TRY(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> g(g_mu);
  Scratch* s = nullptr;
  for (auto& e : g_scratch)
    if (e.dev == dev && e.stream == stream) { s = &e; break; }
  const size_t want_counters = std::max<size_t>(round_up(counter_bytes, 256), 1 << 16);
  if (s == nullptr || scratch_must_grow(s->bytes, s->counter_bytes, want_counters, partial_bytes)) {
    // Grow: a fresh, larger buffer.  The old one is kept (work already queued may still use it).  Allocating would
    // invalidate a stream capture in progress: refuse instead, the caller runs the shape once before capturing.
    if (stream_is_capturing(stream))
      return fail(MP_ERR_WORKSPACE, "the split-K scratch must grow, which cannot happen while the stream is being "
                                    "captured: run this shape once before the capture");
    const size_t cb = std::max(want_counters, s ? s->counter_bytes : 0);
    const size_t total = cb + std::max<size_t>(round_up(partial_bytes, 1 << 20) * 2, 8 << 20);
    uint8_t* p = nullptr;
    MP_CUDA_TRY(cudaMalloc(&p, total));
    MP_CUDA_TRY(cudaMemsetAsync(p, 0, cb, stream));
    if (s == nullptr) {
      g_scratch.push_back(Scratch{dev, stream, p, total, cb});
      s = &g_scratch.back();
    } else {
      s->ptr = p; s->bytes = total; s->counter_bytes = cb;
    }
  }
  *counters = s->ptr;
  *partials = s->ptr + s->counter_bytes;
  return MP_OK;
}

// Second pool, same rules: padded copies of operands whose rows miss the tensor path's 16-byte alignment.
std::vector<Scratch> g_pad_scratch;

int get_pad_scratch(cudaStream_t stream, size_t bytes, uint8_t** out) {
  int dev = 0;
  MP_CUDA_TRY(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> g(g_mu);
  Scratch* s = nullptr;
  for (auto& e : g_pad_scratch)
    if (e.dev == dev && e.stream == stream) { s = &e; break; }
  if (s == nullptr || s->bytes < bytes) {
    // a fresh buffer with head-room; never while the stream is being captured (the call then keeps the plain tiles)
    if (stream_is_capturing(stream)) return MP_ERR_WORKSPACE;
    const size_t total = std::max<size_t>(round_up(bytes + bytes / 2, 1 << 20), 16 << 20);
    uint8_t* p = nullptr;
    if (cudaMalloc(&p, total) != cudaSuccess) {
      cudaGetLastError();           // not an error of the call: the caller falls back to the CUDA-core kernels
      return MP_ERR_WORKSPACE;
    }
    if (s == nullptr) {
      g_pad_scratch.push_back(Scratch{dev, stream, p, total, 0});
      s = &g_pad_scratch.back();
    } else {
      // only work of this stream reads the old copies: once it has drained, the buffer can go (operand copies can
      // be gigabytes, so unlike the split-K scratch the old buffer is not kept)
      if (cudaStreamSynchronize(stream) == cudaSuccess) cudaFree(s->ptr);
      cudaGetLastError();
      s->ptr = p; s->bytes = total;
    }
  }
  *out = s->ptr;
  return MP_OK;
}

// dst[r][0..kp) = src[r][0..k) followed by zeros; kp * sizeof(T) is a multiple of 16 and dst is 16-byte aligned.
// One thread builds one 16-byte word from scalar loads (the source rows have no alignment beyond the element's).
template <typename T>
__global__ void pad_rows_kernel(const T* __restrict__ src, long long ld, T* __restrict__ dst, int rows, int k, int kp) {
  constexpr int kPer = 16 / (int)sizeof(T);
  const int words = kp / kPer;
  const long long total = (long long)rows * words;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / words), c0 = (int)(i - (long long)r * words) * kPer;
    alignas(16) T v[kPer];
#pragma unroll
    for (int e = 0; e < kPer; ++e) v[e] = c0 + e < k ? src[(long long)r * ld + c0 + e] : T(0);
    *reinterpret_cast<uint4*>(dst + (long long)r * kp + c0) = *reinterpret_cast<const uint4*>(v);
  }
}

// ------------------------------------------------------------------------------------------------
// Built-in scratch of mp_gemm_rcc_pid_static_scratch: lives in every GPU that loads the library,
// from load to exit.  The name is a host-side stand-in; kernels get the address that
// cudaGetSymbolAddress returns for the current device.
// ------------------------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = 8u << 20;   // 8 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
std::atomic<void*> g_static_scratch_ptr[kMaxDevices] = {};

// ------------------------------------------------------------------------------------------------
// problem description shared by all dtypes
// ------------------------------------------------------------------------------------------------
struct Problem {
  int dtype;                 // MP_FP16 / MP_INT8 / MP_FP32
  int epi;                   // EPI_* (tensor path) -- SEPI_* share the numbering for 0..2
  int m, n, k;               // rows of A, rows of B (stored [n,k]), reduction length
  const void* A; long long lda;
  const void* B; long long ldb;
  void* C; long long c_stride_m, c_stride_n;
  float alpha = 1.0f, beta = 0.0f;
  int ialpha = 1, ibeta = 0;
  const float* a_scales = nullptr; const float* b_scales = nullptr;
  int a_scalar = 0, b_scalar = 0;
  const void* bias = nullptr;
  int out_bf16 = 0;
  int bf16 = 0;              // dtype MP_FP16 with bf16 operands and output (mp_linear_bias with MP_BF16)
  int bias_on_m = 0;         // 16-bit float GEMM with `bias`: 1 = indexed by the rows of A (the Linear mapping's channels)
  // fused all-gather: further bases that receive the same output (the other GPUs' copies of the buffer)
  void* peers[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  int num_peers = 0;
};

struct Launch {
  int orient = 0, bn = 128, split_k = 1;
  int xm = 1;            // 2: 256 x bn tiles (two 128-row halves of X share every Y tile); one region only
  int kc = 0;                 // K blocks per stage; 0 = choose
  int split_n = 0, bn1 = 0;   // twin: second region [split_n, n) with its own UMMA-N
  void* workspace = nullptr; size_t workspace_bytes = 0;
  // schedule check (no launch, no device needed): receives 8 ints per work unit, see mp_debug_schedule
  int* dry_units = nullptr; int dry_capacity = 0; int* dry_count = nullptr; int* dry_grid = nullptr;
};

int elem_bytes(int dtype) { return dtype == MP_FP16 ? 2 : dtype == MP_INT8 ? 1 : 4; }

// Tensor maps are pure functions of (pointer, extents, pitch, box): a small per-thread cache saves
// the driver call (about a microsecond each) when a caller reuses its buffers, as serving does.
struct TmapKey {
  const void* ptr; long long rows, k, ld; int box_rows, kc, dtype;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && rows == o.rows && k == o.k && ld == o.ld && box_rows == o.box_rows && kc == o.kc &&
           dtype == o.dtype;
  }
};
struct TmapSlot { TmapKey key; bool valid; CUtensorMap map; };
constexpr int kTmapSlots = 256;
thread_local TmapSlot t_tmap_cache[kTmapSlots];

// kc == 0: 2-D map [rows][k] with a (128 bytes x box_rows) box.  kc > 0 (k a multiple of one
// 128-byte K block): 3-D map [k/kb][rows][kb] with a (128 bytes x box_rows x kc) box.
int make_tmap(CUtensorMap* tm, int dtype, const void* ptr, long long rows, long long k, long long ld, int box_rows,
              int kc) {
  const TmapKey key{ptr, rows, k, ld, box_rows, kc, dtype};
  uint64_t h = reinterpret_cast<uintptr_t>(ptr) * 0x9E3779B97F4A7C15ull;
  h ^= (uint64_t)rows * 0xBF58476D1CE4E5B9ull + (uint64_t)k * 0x94D049BB133111EBull + (uint64_t)box_rows * 131 + kc;
  TmapSlot& slot = t_tmap_cache[(h >> 32) & (kTmapSlots - 1)];
  if (slot.valid && slot.key == key) {
    *tm = slot.map;
    return MP_OK;
  }
  const int eb = elem_bytes(dtype);
  const cuuint64_t kb = (cuuint64_t)(128 / eb);
  cuuint64_t gdim[3] = {(cuuint64_t)k, (cuuint64_t)rows, 1};
  cuuint64_t gstride[2] = {(cuuint64_t)(ld * eb), 128};
  cuuint32_t box[3] = {(cuuint32_t)kb, (cuuint32_t)box_rows, (cuuint32_t)kc};
  cuuint32_t estr[3] = {1, 1, 1};
  if (kc > 0) { gdim[0] = kb; gdim[2] = (cuuint64_t)k / kb; }
  const CUtensorMapDataType dt = dtype == MP_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const CUresult r = g_encode(tm, dt, kc > 0 ? 3 : 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MP_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  slot.key = key;
  slot.map = *tm;
  slot.valid = true;
  return MP_OK;
}

bool tma_compatible(const Problem& p) {
  const int eb = elem_bytes(p.dtype);
  if (p.k <= 0) return false;
  if ((reinterpret_cast<uintptr_t>(p.A) & 15) || (reinterpret_cast<uintptr_t>(p.B) & 15)) return false;
  if ((p.lda * eb) % 16 != 0 || (p.ldb * eb) % 16 != 0) return false;
  return true;
}

// Operands whose rows miss the 16-byte alignment (K * element size not a multiple of 16, an odd leading dimension
// or base address) cannot be described to TMA (FP16, INT8) or read with 16-byte loads (the FP32 tile kernels).
// Entries that own their scratch copy such operands once into zero-padded, aligned rows (K rounded up to 128 bytes:
// zeros add nothing to a dot product) and run the fast path on the copies; the plain CUDA-core tiles remain the
// fall-back when the copy cannot be allocated and for entries whose memory the caller manages.
// MOONPOLY_DISABLE_PAD=1 turns the copies off.
bool pad_disabled() {
  const char* v = std::getenv("MOONPOLY_DISABLE_PAD");
  return v && v[0] && v[0] != '0';
}

bool pad_operands(Problem& p, cudaStream_t stream) {
  if (p.k <= 0 || p.m <= 0 || p.n <= 0 || tma_compatible(p) || pad_disabled()) return false;
  const int eb = elem_bytes(p.dtype);
  const int per128 = 128 / eb;
  const long long kp = ((long long)p.k + per128 - 1) / per128 * per128;
  const size_t a_bytes = round_up((size_t)p.m * kp * eb, 256), b_bytes = round_up((size_t)p.n * kp * eb, 256);
  uint8_t* buf = nullptr;
  if (get_pad_scratch(stream, a_bytes + b_bytes, &buf) != MP_OK) return false;
  const auto launch = [&](const void* src, long long ld, void* dst, int rows) {
    const long long words = (long long)rows * (kp * eb / 16);
    const int grid = (int)std::min<long long>((words + 255) / 256, 148 * 16);
    if (eb == 4)
      pad_rows_kernel<uint32_t><<<grid, 256, 0, stream>>>(reinterpret_cast<const uint32_t*>(src), ld,
                                                          reinterpret_cast<uint32_t*>(dst), rows, p.k, (int)kp);
    else if (eb == 2)
      pad_rows_kernel<uint16_t><<<grid, 256, 0, stream>>>(reinterpret_cast<const uint16_t*>(src), ld,
                                                          reinterpret_cast<uint16_t*>(dst), rows, p.k, (int)kp);
    else
      pad_rows_kernel<uint8_t><<<grid, 256, 0, stream>>>(reinterpret_cast<const uint8_t*>(src), ld,
                                                         reinterpret_cast<uint8_t*>(dst), rows, p.k, (int)kp);
    g_launches.fetch_add(1, std::memory_order_relaxed);
  };
  launch(p.A, p.lda, buf, p.m);
  launch(p.B, p.ldb, buf + a_bytes, p.n);
  if (cudaGetLastError() != cudaSuccess) return false;
  p.A = buf; p.lda = kp;
  p.B = buf + a_bytes; p.ldb = kp;
  p.k = (int)kp;
  return true;
}

size_t umma_workspace_bytes(const Problem& p, const Launch& l, size_t* counter_bytes) {
  const int P = l.orient == 0 ? p.m : p.n;
  const int Q = l.orient == 0 ? p.n : p.m;
  const int xm = (l.xm == 2 && l.split_n <= 0) ? 2 : 1;
  const int tiles_p = (P + kUmmaM * xm - 1) / (kUmmaM * xm);
  long long tiles;
  int bn_max = l.bn;
  if (l.split_n > 0) {
    tiles = (long long)tiles_p * ((l.split_n + l.bn - 1) / l.bn + (Q - l.split_n + l.bn1 - 1) / l.bn1);
    bn_max = std::max(l.bn, l.bn1);
  } else {
    tiles = (long long)tiles_p * ((Q + l.bn - 1) / l.bn);
  }
  const size_t cb = round_up((size_t)tiles * 16 * sizeof(unsigned), 256);   // [tile][quadrant][arrived, claimed, left, -]
  if (counter_bytes) *counter_bytes = cb;
  if (l.split_k <= 1) return 0;
  return cb + (size_t)tiles * l.split_k * xm * bn_max * kUmmaM * 4;
}

template <int KIND, int EPI, bool SPLIT, bool CLUSTER = false>
int launch_umma_t(DeviceState& d, int attr_slot, const CUtensorMap& tx, const CUtensorMap& ty0,
                  const CUtensorMap& ty1, const UmmaParams& up, int grid, size_t smem, cudaStream_t stream) {
  auto kern = umma_gemm_kernel<KIND, EPI, SPLIT, CLUSTER>;
  if (!d.attrs[attr_slot]) {
    MP_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget));
    d.attrs[attr_slot] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(SPLIT ? kUmmaThreads : kUmmaThreadsWide);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (g_use_pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (CLUSTER) {       // the K slices of a tile form one cluster: consecutive CTAs, grid is a multiple of it
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = (unsigned)up.cluster_k;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  MP_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tx, ty0, ty1, up));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return MP_OK;
}

// Tensor-core path (FP16 / INT8).
int run_umma(const Problem& p, Launch l, cudaStream_t stream) {
  const bool dry = l.dry_count != nullptr;
  DeviceState* d = nullptr;
  DeviceState model{};                      // schedule checks run without a GPU: the modelled SM count stands in
  if (dry) { model.sms = mp::num_sms_for_model(); d = &model; }
  else if (int rc = device_state(&d)) return rc;

  UmmaParams up{};
  const bool swap = l.orient == 1;
  const void* X = swap ? p.B : p.A;
  const void* Y = swap ? p.A : p.B;
  const long long ldx = swap ? p.ldb : p.lda, ldy = swap ? p.lda : p.ldb;
  up.P = swap ? p.n : p.m;
  up.Q = swap ? p.m : p.n;
  up.K = p.k;
  up.out = p.C;
  up.out_stride_p = swap ? p.c_stride_n : p.c_stride_m;
  up.out_stride_q = swap ? p.c_stride_m : p.c_stride_n;
  const int xm = (l.xm == 2 && l.split_n <= 0) ? 2 : 1;
  up.xm = xm;
  up.tiles_p = (up.P + kUmmaM * xm - 1) / (kUmmaM * xm);
  up.group_p = 8;
  int bn_max = l.bn;
  if (l.split_n > 0) {
    up.num_regions = 2;
    up.reg[0] = Region{0, l.split_n, l.bn, (l.split_n + l.bn - 1) / l.bn, 0};
    up.reg[1] = Region{l.split_n, up.Q, l.bn1, (up.Q - l.split_n + l.bn1 - 1) / l.bn1,
                       up.tiles_p * up.reg[0].tiles_q};
    up.total_tiles = up.tiles_p * (up.reg[0].tiles_q + up.reg[1].tiles_q);
    bn_max = std::max(l.bn, l.bn1);
  } else {
    up.num_regions = 1;
    up.reg[0] = Region{0, up.Q, l.bn, (up.Q + l.bn - 1) / l.bn, 0};
    up.reg[1] = up.reg[0];
    up.total_tiles = up.tiles_p * up.reg[0].tiles_q;
  }
  const int kb_elems = p.dtype == MP_INT8 ? 128 : 64;
  up.kb_total = (p.k + kb_elems - 1) / kb_elems;
  // K blocks per stage: wide boxes move far more bytes per TMA instruction; keep >= 3 stages
  const int kb_bytes = xm * kXTileBytes + bn_max * kRowBytes;
  // the scaled epilogue stages the tile's scales and bias in shared memory (up to 8 warps x 1.5 KB)
  const int epi_reserve = p.epi == EPI_SCALED ? 12288 : 0;
  const int smem_for_stages = kSmemBudget - 1024 - 256 - kClusterBarBytes - epi_reserve;
  int kc = l.kc;
  if (kc <= 0) kc = (smem_for_stages / (4 * kb_bytes) >= 3) ? 4 : (smem_for_stages / (2 * kb_bytes) >= 3) ? 2 : 1;
  while (kc > 1 && smem_for_stages / (kc * kb_bytes) < 2) kc >>= 1;
  // at most 31 slices: the reduction tracks claimed shares in one 32-bit mask (one bit seals it)
  int S = std::max(1, std::min(std::min(l.split_k, 31), up.kb_total));
  up.kb_per_slice = ((up.kb_total + S - 1) / S + kc - 1) / kc * kc;     // slices start on a stage boundary
  S = (up.kb_total + up.kb_per_slice - 1) / up.kb_per_slice;              // every slice non-empty
  up.split_k = S;
  l.split_k = S;
  up.kc = kc;
  up.wide = ((long long)p.k * elem_bytes(p.dtype)) % 128 == 0 ? 1 : 0;
  // L2 prefetch ahead of the dependency wait pays when the launch is a short, memory-bound stream
  // (few K blocks per CTA); cap it at 512 KB per CTA
  up.prefetch_kb = g_use_pdl ? std::min(up.kb_per_slice, (512 * 1024) / kb_bytes) : 0;
  up.stage_bytes = kc * kb_bytes;
  up.stages = std::min(kMaxStages, smem_for_stages / up.stage_bytes);
  up.alpha = p.alpha; up.beta = p.beta; up.ialpha = p.ialpha; up.ibeta = p.ibeta;
  up.ws_tile_words = xm * bn_max * kUmmaM;
  up.ws_half_words = bn_max * kUmmaM;
  up.scale_p = swap ? p.b_scales : p.a_scales;
  up.scale_q = swap ? p.a_scales : p.b_scales;
  up.scale_p_scalar = swap ? p.b_scalar : p.a_scalar;
  up.scale_q_scalar = swap ? p.a_scalar : p.b_scalar;
  up.n_on_p = swap ? 1 : 0;
  up.bias = p.bias;
  up.out_bf16 = p.out_bf16;
  up.ab_bf16 = p.bf16;
  up.bias_on_p = p.epi == EPI_F16 ? (swap ? !p.bias_on_m : p.bias_on_m) : 0;
  up.num_peers = p.num_peers;
  for (int i = 0; i < p.num_peers; ++i) up.peer_out[i] = p.peers[i];

  up.ws_slices = S;
  const long long units = (long long)up.total_tiles * up.split_k;
  const int grid = (int)std::min<long long>(units, d->sms);
  up.helpers_ok = units <= grid ? 1 : 0;

  // Stream-K head.  With T tiles on G persistent CTAs, T mod G tiles are left for a last, partly
  // empty wave.  Instead, those r tiles go first and are cut along K into contiguous runs of
  // sk_ipc K blocks, one run per CTA (a run may end one tile and begin the next); the tiles are
  // completed through the split-K scratch, and the other T - r tiles follow as whole waves.  Runs
  // are never shorter than a quarter of K, so a tile has at most ~5 contributors.
  size_t sk_cb = 0, sk_pb = 0;
  if (g_use_streamk.load(std::memory_order_relaxed) && S == 1 && up.num_regions == 1 && up.total_tiles > grid && grid == d->sms) {
    const int r = up.total_tiles % grid;
    // measured on B200: pays while the remainder is at most half a wave (r/G = 0.30: -17 %, 0.46: -5 %,
    // 0.59 and above: the completion traffic costs more than the idle SMs did)
    if (r > 0 && 2 * r <= grid && up.kb_total >= 8 * kc) {
      long long ipc = ((long long)r * up.kb_total + grid - 1) / grid;
      ipc = std::max<long long>(ipc, (up.kb_total + 3) / 4);
      ipc = (ipc + kc - 1) / kc * kc;
      const int max_slices = (int)((up.kb_total + ipc - 2) / ipc + 1);
      sk_cb = round_up((size_t)r * 16 * sizeof(unsigned), 256);
      sk_pb = (size_t)r * max_slices * xm * bn_max * kUmmaM * 4;
      if (l.workspace == nullptr || l.workspace_bytes >= sk_cb + sk_pb) {
        up.sk_tiles = r;
        up.sk_ipc = (int)ipc;
        up.ws_slices = max_slices;
      }
    }
  }

  if (dry) {
    // walk every CTA's units exactly as the kernel's roles do and hand them to the caller
    int count = 0;
    for (int cta = 0; cta < grid; ++cta) {
      UnitWalk walk(up, cta, grid);
      UnitCoord u;
      while (walk.next(up, u)) {
        if (count < l.dry_capacity) {
          int* o = l.dry_units + 8 * (size_t)count;
          o[0] = cta; o[1] = u.tile; o[2] = u.tp; o[3] = u.tq; o[4] = u.kb0; o[5] = u.kb1; o[6] = u.slice; o[7] = u.nslices;
        }
        ++count;
      }
    }
    *l.dry_count = count;
    if (l.dry_grid) { l.dry_grid[0] = grid; l.dry_grid[1] = up.total_tiles; l.dry_grid[2] = up.kb_total; l.dry_grid[3] = up.ws_slices;
                      l.dry_grid[4] = up.sk_tiles; l.dry_grid[5] = up.xm; l.dry_grid[6] = up.helpers_ok; l.dry_grid[7] = up.split_k; }
    return MP_OK;
  }

  // Split-K inside a cluster: when every work unit has a CTA of its own and there are 2, 4 or 8 slices, the
  // slices of a tile are launched as one cluster and exchange partials through distributed shared memory;
  // no scratch, no counters.  The parked tile (bn x 128 words) reuses the pipeline stages.
  const bool cluster = g_use_cluster_splitk.load(std::memory_order_relaxed) && (S == 2 || S == 4 || S == 8) &&
                       up.sk_tiles == 0 && units == grid && xm == 1 &&
                       (size_t)bn_max * kUmmaM * 4 <= (size_t)up.stages * up.stage_bytes;
  up.cluster_k = cluster ? S : 0;

  if (!cluster && (S > 1 || up.sk_tiles > 0)) {
    size_t cb = sk_cb;
    const size_t need = up.sk_tiles > 0 ? sk_cb + sk_pb : umma_workspace_bytes(p, l, &cb);
    uint8_t *counters = nullptr, *partials = nullptr;
    if (l.workspace != nullptr) {
      if (l.workspace_bytes < need)
        return fail(MP_ERR_WORKSPACE, "workspace of %zu bytes given, %zu needed", l.workspace_bytes, need);
      if (reinterpret_cast<uintptr_t>(l.workspace) & 15)
        return fail(MP_ERR_WORKSPACE, "workspace must be 16-byte aligned");
      counters = reinterpret_cast<uint8_t*>(l.workspace);
      partials = counters + cb;
      MP_CUDA_TRY(cudaMemsetAsync(counters, 0, cb, stream));   // caller memory: contents unknown
    } else {
      if (int rc = get_scratch(stream, cb, need - cb, &counters, &partials)) return rc;
    }
    up.ws_counters = reinterpret_cast<unsigned*>(counters);
    up.ws_partials = reinterpret_cast<uint32_t*>(partials);
  }

  CUtensorMap tx, ty0, ty1;
  const int map_kc = up.wide ? up.kc : 0;
  if (int rc = make_tmap(&tx, p.dtype, X, up.P, p.k, ldx, kUmmaM * xm, map_kc)) return rc;
  if (int rc = make_tmap(&ty0, p.dtype, Y, up.Q, p.k, ldy, up.reg[0].bn, map_kc)) return rc;
  if (up.num_regions == 2) {
    if (int rc = make_tmap(&ty1, p.dtype, Y, up.Q, p.k, ldy, up.reg[1].bn, map_kc)) return rc;
  } else {
    ty1 = ty0;
  }

  const size_t smem = (size_t)up.stages * up.stage_bytes + 8 * (2 * up.stages + 4) + 16 + kClusterBarBytes + 1024 + epi_reserve;
  if (cluster) {
    if (p.dtype == MP_FP16) return launch_umma_t<KIND_F16, EPI_F16, true, true>(*d, 6, tx, ty0, ty1, up, grid, smem, stream);
    if (p.epi == EPI_I32) return launch_umma_t<KIND_I8, EPI_I32, true, true>(*d, 7, tx, ty0, ty1, up, grid, smem, stream);
    return launch_umma_t<KIND_I8, EPI_SCALED, true, true>(*d, 8, tx, ty0, ty1, up, grid, smem, stream);
  }
  // kernels whose every unit is a whole tile run the variant without the reduction (8 epilogue warps)
  if (up.split_k > 1 || up.sk_tiles > 0) {
    if (p.dtype == MP_FP16) return launch_umma_t<KIND_F16, EPI_F16, true>(*d, 0, tx, ty0, ty1, up, grid, smem, stream);
    if (p.epi == EPI_I32) return launch_umma_t<KIND_I8, EPI_I32, true>(*d, 1, tx, ty0, ty1, up, grid, smem, stream);
    return launch_umma_t<KIND_I8, EPI_SCALED, true>(*d, 2, tx, ty0, ty1, up, grid, smem, stream);
  }
  if (p.dtype == MP_FP16) return launch_umma_t<KIND_F16, EPI_F16, false>(*d, 3, tx, ty0, ty1, up, grid, smem, stream);
  if (p.epi == EPI_I32) return launch_umma_t<KIND_I8, EPI_I32, false>(*d, 4, tx, ty0, ty1, up, grid, smem, stream);
  return launch_umma_t<KIND_I8, EPI_SCALED, false>(*d, 5, tx, ty0, ty1, up, grid, smem, stream);
}

// CUDA-core path (FP32 always; FP16 / INT8 when TMA's alignment rules are not met).
template <typename TIn, int EPI, int TI, int TJ>
int launch_simt_t(const SimtParams& sp, cudaStream_t stream) {
  dim3 grid((sp.m + TI - 1) / TI, (sp.n + TJ - 1) / TJ, sp.split_k);
  simt_gemm_kernel<TIn, EPI, TI, TJ><<<grid, 256, 0, stream>>>(sp);
  MP_CUDA_TRY(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (sp.split_k > 1) {
    using TAcc = typename SimtAcc<TIn>::type;
    const size_t total = (size_t)sp.m * sp.n;
    const int blocks = (int)std::min<size_t>((total + 255) / 256, 148 * 8);
    simt_splitk_reduce_kernel<TAcc, EPI><<<blocks, 256, 0, stream>>>(sp);
    MP_CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
  }
  return MP_OK;
}

// FP32: tiles of 64 / 128 on 16-byte aligned rows take the throughput kernel (same sums, same order)
template <int TI, int TJ>
int launch_simt_f32(const SimtParams& sp, cudaStream_t stream) {
  constexpr bool big = (TI == 64 || TI == 128) && (TJ == 64 || TJ == 128);
  if constexpr (big) {
    const bool aligned = sp.lda % 4 == 0 && sp.ldb % 4 == 0 && (reinterpret_cast<uintptr_t>(sp.A) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(sp.B) & 15) == 0;
    if (aligned) {
      dim3 grid((sp.m + TI - 1) / TI, (sp.n + TJ - 1) / TJ, sp.split_k);
      if constexpr (TI == 64 && TJ == 64) sgemm_f32_kernel<16, 16, 4, 4><<<grid, 256, 0, stream>>>(sp);
      else sgemm_f32_kernel<TI / 8, TJ / 8, 8, 8><<<grid, (TI / 8) * (TJ / 8), 0, stream>>>(sp);
      MP_CUDA_TRY(cudaGetLastError());
      g_launches.fetch_add(1, std::memory_order_relaxed);
      if (sp.split_k > 1) {
        const size_t total = (size_t)sp.m * sp.n;
        const int blocks = (int)std::min<size_t>((total + 255) / 256, 148 * 8);
        simt_splitk_reduce_kernel<float, SEPI_F32><<<blocks, 256, 0, stream>>>(sp);
        MP_CUDA_TRY(cudaGetLastError());
        g_launches.fetch_add(1, std::memory_order_relaxed);
      }
      return MP_OK;
    }
  }
  return launch_simt_t<float, SEPI_F32, TI, TJ>(sp, stream);
}

int run_simt(const Problem& p, int ti, int tj, int split_k, void* workspace, size_t workspace_bytes,
             cudaStream_t stream) {
  DeviceState* d = nullptr;
  if (int rc = device_state(&d)) return rc;
  SimtParams sp{};
  sp.m = p.m; sp.n = p.n; sp.k = p.k;
  sp.A = p.A; sp.B = p.B; sp.C = p.C;
  sp.lda = p.lda; sp.ldb = p.ldb;
  sp.c_stride_i = p.c_stride_m; sp.c_stride_j = p.c_stride_n;
  sp.alpha = p.alpha; sp.beta = p.beta; sp.ialpha = p.ialpha; sp.ibeta = p.ibeta;
  sp.a_scales = p.a_scales; sp.b_scales = p.b_scales; sp.a_scalar = p.a_scalar; sp.b_scalar = p.b_scalar;
  sp.bias = p.bias; sp.out_bf16 = p.out_bf16; sp.bias_on_i = p.bias_on_m;
  int S = std::max(1, split_k);
  if (p.k > 0) S = std::min(S, (p.k + 15) / 16); else S = 1;
  sp.k_per_slice = p.k > 0 ? ((p.k + S - 1) / S + 15) / 16 * 16 : 0;
  if (p.k > 0) S = (p.k + sp.k_per_slice - 1) / sp.k_per_slice;
  sp.split_k = S;
  if (S > 1) {
    const size_t need = (size_t)S * p.m * p.n * 4;
    if (workspace != nullptr) {
      if (workspace_bytes < need)
        return fail(MP_ERR_WORKSPACE, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
      sp.partials = workspace;
    } else {
      uint8_t *c = nullptr, *part = nullptr;
      if (int rc = get_scratch(stream, 256, need, &c, &part)) return rc;
      sp.partials = part;
    }
  }
  if (p.dtype == MP_FP32) {
    if (ti == 32 && tj == 32) return launch_simt_f32<32, 32>(sp, stream);
    if (ti == 64 && tj == 32) return launch_simt_f32<64, 32>(sp, stream);
    if (ti == 32 && tj == 64) return launch_simt_f32<32, 64>(sp, stream);
    if (ti == 128 && tj == 32) return launch_simt_f32<128, 32>(sp, stream);
    if (ti == 32 && tj == 128) return launch_simt_f32<32, 128>(sp, stream);
    if (ti == 128 && tj == 64) return launch_simt_f32<128, 64>(sp, stream);
    if (ti == 64 && tj == 128) return launch_simt_f32<64, 128>(sp, stream);
    if (ti == 128 && tj == 128) return launch_simt_f32<128, 128>(sp, stream);
    return launch_simt_f32<64, 64>(sp, stream);
  }
  if (p.dtype == MP_FP16 && p.bf16) return launch_simt_t<__nv_bfloat16, SEPI_F16, 64, 64>(sp, stream);
  if (p.dtype == MP_FP16) return launch_simt_t<__half, SEPI_F16, 64, 64>(sp, stream);
  if (p.epi == EPI_I32) return launch_simt_t<int8_t, SEPI_I32, 64, 64>(sp, stream);
  return launch_simt_t<int8_t, SEPI_SCALED, 64, 64>(sp, stream);
}

// Skinny FP16 path: one side of the problem has at most 8 rows; the other operand is streamed once.
template <int T>
int launch_gemv_t(const GemvParams& gp, cudaStream_t stream) {
  const int rows_per_cta = kGemvWarps * kGemvRowsPerWarp;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((gp.R + rows_per_cta - 1) / rows_per_cta));
  cfg.blockDim = dim3(kGemvWarps * 32);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_use_pdl ? 1 : 0;
  MP_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemv_f16_kernel<T>, gp));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return MP_OK;
}

bool gemv_compatible(const Problem& p) {
  return p.dtype == MP_FP16 && p.epi == EPI_F16 && std::min(p.m, p.n) <= 8 && std::min(p.m, p.n) >= 1 && p.k >= 8 &&
         (p.k * 2) % 16 == 0 &&  // the kernel walks K in whole 16-byte chunks (a padded leading dimension does not help)
         tma_compatible(p);      // same rule: 16-byte aligned rows
}

int run_gemv(const Problem& p, cudaStream_t stream) {
  DeviceState* d = nullptr;
  if (int rc = device_state(&d)) return rc;
  GemvParams gp{};
  const bool narrow_is_a = p.m <= p.n;          // direct mapping: few rows of A against the rows of B
  gp.W = reinterpret_cast<const __half*>(narrow_is_a ? p.B : p.A);
  gp.ldw = narrow_is_a ? p.ldb : p.lda;
  gp.X = reinterpret_cast<const __half*>(narrow_is_a ? p.A : p.B);
  gp.ldx = narrow_is_a ? p.lda : p.ldb;
  gp.R = narrow_is_a ? p.n : p.m;
  gp.T = narrow_is_a ? p.m : p.n;
  gp.K = p.k;
  gp.out = reinterpret_cast<__half*>(p.C);
  gp.stride_r = narrow_is_a ? p.c_stride_n : p.c_stride_m;
  gp.stride_t = narrow_is_a ? p.c_stride_m : p.c_stride_n;
  gp.alpha = p.alpha; gp.beta = p.beta;
  switch (gp.T) {
    case 1: return launch_gemv_t<1>(gp, stream);
    case 2: return launch_gemv_t<2>(gp, stream);
    case 3: return launch_gemv_t<3>(gp, stream);
    case 4: return launch_gemv_t<4>(gp, stream);
    case 5: return launch_gemv_t<5>(gp, stream);
    case 6: return launch_gemv_t<6>(gp, stream);
    case 7: return launch_gemv_t<7>(gp, stream);
    default: return launch_gemv_t<8>(gp, stream);
  }
}

// Streaming warp-MMA path: one side of the problem has at most 64 rows; the other operand is streamed once.
template <int KIND, int EPI, int NT, int UNROLL, int MINB>
int launch_stream_t(const StreamParams& sp, int row_ctas, cudaStream_t stream) {
  // every block of rows is taken by t_split neighbouring token parts, each of them by k_split consecutive CTAs
  // (one cluster) that cut K
  const int ks = std::max(1, sp.k_split);
  const int grid = row_ctas * std::max(1, sp.t_split) * ks;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kStreamWarps * 32);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (g_use_pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (ks > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = (unsigned)ks;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  MP_CUDA_TRY(cudaLaunchKernelEx(&cfg, stream_mma_kernel<KIND, EPI, NT, UNROLL, MINB>, sp));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return MP_OK;
}

template <int KIND, int EPI>
int launch_stream_nt(const StreamParams& sp, int row_ctas, cudaStream_t stream) {
  const int rows = sp.t_split > 1 ? sp.t_per : sp.T;       // rows of X one CTA works against
  if (rows <= 8) return launch_stream_t<KIND, EPI, 1, 8, 2>(sp, row_ctas, stream);
  if (rows <= 16) return launch_stream_t<KIND, EPI, 2, 8, 2>(sp, row_ctas, stream);
  if (rows <= 32) return launch_stream_t<KIND, EPI, 4, 8, 2>(sp, row_ctas, stream);
  return launch_stream_t<KIND, EPI, 8, 4, 2>(sp, row_ctas, stream);
}

// CTAs along the rows of W: a whole multiple of the SM count (at most two per SM) when the rows allow it, else one
// CTA per `rows_per_cta` rows.
int stream_row_ctas(int R, int sms, int rows_per_cta) {
  const int per_sm = std::min(2, R / (8 * sms));
  return per_sm >= 1 ? per_sm * sms : std::max(1, (R + rows_per_cta - 1) / rows_per_cta);
}

// K split of the streaming kernel (see StreamParams::k_split).  0 = the library's rule, 1 = off, 2 / 4 / 8 = forced;
// MOONPOLY_STREAM_KSPLIT overrides the rule the same way.
int stream_ksplit_from_env() {
  const char* v = std::getenv("MOONPOLY_STREAM_KSPLIT");
  return v && v[0] ? std::atoi(v) : 0;
}
std::atomic<int> g_stream_ksplit{stream_ksplit_from_env()};

// Token split of the streaming kernel (see StreamParams::t_split).  0 = the library's rule below, 1 = off,
// 2 / 4 / 8 = forced; MOONPOLY_STREAM_TSPLIT overrides the rule the same way.
int stream_tsplit_from_env() {
  const char* v = std::getenv("MOONPOLY_STREAM_TSPLIT");
  return v && v[0] ? std::atoi(v) : 0;
}
std::atomic<int> g_stream_tsplit{stream_tsplit_from_env()};

// When to split the tokens.  Measured on B200 (Linear mapping, FP16): with N = K = 4096 the repeated reads of W
// cost more than the narrower X saves (M = 16: 12.2 us split in two against 8.3 us; M = 32: 15.2 against 11.1),
// and the same holds for every layer with enough rows to give each SM a CTA.  The split pays only when the rows are
// too few to fill the GPU (N = 1024, K = 8192: M = 16 10.0 -> 8.0 us, M = 32 14.7 -> 10.6 us), where it doubles the
// number of CTAs: two parts when one CTA per 8 rows leaves SMs idle and there are more than 8 rows of X.
int stream_tsplit_rule(int ctas, int T, int sms) {
  return (T > 8 && ctas < sms) ? 2 : 1;
}

// When to split K over a cluster.  A whole-K CTA keeps at most 64 KB of W in flight (8 warps x 32 lanes x 16 loads
// of 16 bytes), and the HBM queue needs about two such CTAs per SM to stay full; a weight with fewer than
// 8 * 2 * SMs rows cannot give that many.  The K parts (a power of two) multiply the CTAs up to two per SM, as long
// as every CTA still streams at least 192 KB of W: below that the cluster's start-up and exchange cost more than
// the extra loads in flight bring.  Measured on B200 (FP16, Linear mapping): (M, N, K) = (1, 1024, 28672) 24.0 us
// whole-K, 18.2 / 16.8 / 29.2 us with 2 / 4 / 8 parts; (8, 1024, 28672) 25.8 -> 18.0 us with 4; (1, 2048, 28672)
// 28.6 -> 25.6 us with 2 (4 parts: 39.2 us, four CTAs per SM no longer run together); (1, 1024, 8192) 6.5 us
// whole-K against 6.8 / 6.9 us with 2 / 4 parts, (8, 2048, 8192) 9.3 against 9.9 us: too short to pay.
int stream_ksplit_rule(int R, int K, int elt, int sms) {
  if (R / (8 * sms) >= 2) return 1;
  const bool one_per_sm = R / (8 * sms) >= 1;
  const int row_ctas = one_per_sm ? sms : (R + kStreamRows - 1) / kStreamRows;
  const double rows_per_cta = one_per_sm ? (double)R / sms : (double)std::min(R, kStreamRows);
  const double bytes_per_cta = rows_per_cta * K * elt;
  int ks = 1;
  while (ks < 8 && row_ctas * ks * 2 <= 2 * sms && bytes_per_cta / (ks * 2) >= 192.0 * 1024.0) ks *= 2;
  return ks;
}

// Launch shape of the streaming kernel: K split first (it cuts both operands per CTA), then the token split for
// what is still short of one wave.  forced_ck < 0 forces -forced_ck K parts, forced_tsplit > 0 the token parts.
struct StreamShape { int row_ctas, k_split, t_split, t_per; };

StreamShape stream_launch_shape(int R, int T, int K, int elt, int sms, int forced_ck, int forced_tsplit) {
  StreamShape sh{};
  int ks = forced_ck < 0 ? -forced_ck : g_stream_ksplit.load(std::memory_order_relaxed);
  if (ks == 0) ks = stream_ksplit_rule(R, K, elt, sms);
  while (ks > 1 && (long long)K * elt < 4096ll * ks) ks >>= 1;      // every warp keeps a full batch of loads
  ks = std::max(1, std::min(ks, 8));
  sh.k_split = ks;
  sh.row_ctas = stream_row_ctas(R, sms, ks > 1 ? kStreamRows : 8);
  // token split: parts of 8 or 16 rows of X per CTA, never an empty part
  int ts = forced_tsplit > 0 ? forced_tsplit : g_stream_tsplit.load(std::memory_order_relaxed);
  if (ts == 0) ts = stream_tsplit_rule(sh.row_ctas * ks, T, sms);
  ts = std::max(1, std::min(ts, (T + 7) / 8));
  sh.t_per = 0;
  if (ts > 1) {
    sh.t_per = ((T + ts - 1) / ts + 7) / 8 * 8;
    ts = (T + sh.t_per - 1) / sh.t_per;
  }
  sh.t_split = ts;
  return sh;
}

bool stream_compatible(const Problem& p) {
  if (!(p.dtype == MP_FP16 && p.epi == EPI_F16) && p.dtype != MP_INT8) return false;
  return std::min(p.m, p.n) <= 64 && std::min(p.m, p.n) >= 1 && p.k >= 16 &&
         ((long long)p.k * elem_bytes(p.dtype)) % 16 == 0 &&   // K is walked in whole 16-byte chunks
         tma_compatible(p);      // same rule: 16-byte aligned rows
}

// forced_ck: 0 = the library decides; < 0 = -forced_ck K parts (-1: whole-K CTAs).
int run_stream(const Problem& p, cudaStream_t stream, int forced_ck = 0, int forced_tsplit = 0) {
  DeviceState* d = nullptr;
  if (int rc = device_state(&d)) return rc;
  StreamParams sp{};
  const bool narrow_is_a = p.m <= p.n;
  sp.W = narrow_is_a ? p.B : p.A;
  sp.ldw = narrow_is_a ? p.ldb : p.lda;
  sp.X = narrow_is_a ? p.A : p.B;
  sp.ldx = narrow_is_a ? p.lda : p.ldb;
  sp.R = narrow_is_a ? p.n : p.m;
  sp.T = narrow_is_a ? p.m : p.n;
  sp.K = p.k;
  sp.out = p.C;
  sp.stride_r = narrow_is_a ? p.c_stride_n : p.c_stride_m;
  sp.stride_t = narrow_is_a ? p.c_stride_m : p.c_stride_n;
  sp.alpha = p.alpha; sp.beta = p.beta; sp.ialpha = p.ialpha; sp.ibeta = p.ibeta;
  // scaled epilogue: tokens are the rows of A, channels the rows of B
  sp.chan_scale = p.b_scales; sp.chan_scalar = p.b_scalar;
  sp.tok_scale = p.a_scales; sp.tok_scalar = p.a_scalar;
  sp.chan_on_r = (p.epi == EPI_F16 && p.bias_on_m) ? (narrow_is_a ? 0 : 1) : (narrow_is_a ? 1 : 0);
  sp.bias = p.bias; sp.out_bf16 = p.out_bf16;
  sp.num_peers = p.num_peers;
  for (int i = 0; i < p.num_peers; ++i) sp.peer_out[i] = p.peers[i];
  const StreamShape shape = stream_launch_shape(sp.R, sp.T, sp.K, elem_bytes(p.dtype), d->sms, forced_ck, forced_tsplit);
  sp.k_split = shape.k_split;
  sp.t_split = shape.t_split;
  sp.t_per = shape.t_per;
  const int row_ctas = shape.row_ctas;
  if (p.dtype == MP_FP16 && p.bf16) return launch_stream_nt<STREAM_BF16, STREAM_EPI_F16>(sp, row_ctas, stream);
  if (p.dtype == MP_FP16) return launch_stream_nt<STREAM_F16, STREAM_EPI_F16>(sp, row_ctas, stream);
  if (p.epi == EPI_I32) return launch_stream_nt<STREAM_I8, STREAM_EPI_I32>(sp, row_ctas, stream);
  return launch_stream_nt<STREAM_I8, STREAM_EPI_SCALED>(sp, row_ctas, stream);
}

// FP32 streaming kernel: one side of the problem has at most 64 rows.
bool skinny_f32_compatible(const Problem& p) {
  const auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  return p.dtype == MP_FP32 && std::min(p.m, p.n) >= 1 && std::min(p.m, p.n) <= 64 && p.k >= 4 && p.k % 4 == 0 &&
         p.lda % 4 == 0 && p.ldb % 4 == 0 && al(p.A) && al(p.B);
}

template <int ROWS, int UNROLL>
int launch_gemv_f32(const SkinnyF32Params& sp, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((sp.R + ROWS - 1) / ROWS));
  cfg.blockDim = dim3(kGemvF32Warps * 32);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_use_pdl ? 1 : 0;
  MP_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemv_f32_kernel<ROWS, UNROLL>, sp));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return MP_OK;
}

template <int RH, int RI, int TJ>
int launch_tile_f32(DeviceState& d, int slot, const SkinnyF32Params& sp, int ks, cudaStream_t stream) {
  auto kern = tile_f32_kernel<RH, RI, TJ>;
  constexpr int smem = tile_f32_smem_bytes<RH, RI, TJ>();
  static_assert(smem <= kSmemBudget, "ring too large");
  if (!d.tile_f32_attrs[slot]) {
    MP_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    d.tile_f32_attrs[slot] = true;
  }
  constexpr int rows = RH * 4 * RI;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((sp.R + rows - 1) / rows), (unsigned)ks, 1);
  cfg.blockDim = dim3(kTileF32Threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (g_use_pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (ks > 1) {                    // the K parts of a row block form one cluster
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = (unsigned)ks;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  MP_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, sp));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return MP_OK;
}

template <int RH, int RI>
int launch_tile_f32_t(DeviceState& d, const SkinnyF32Params& sp, int ks, cudaStream_t stream) {
  constexpr int base = RH == 2 ? 8 : (RI == 4 ? 4 : 0);
  if (sp.T <= 16) return launch_tile_f32<RH, RI, 2>(d, base + 0, sp, ks, stream);
  if (sp.T <= 24) return launch_tile_f32<RH, RI, 3>(d, base + 1, sp, ks, stream);
  if (sp.T <= 40) return launch_tile_f32<RH, RI, 5>(d, base + 2, sp, ks, stream);
  return launch_tile_f32<RH, RI, 8>(d, base + 3, sp, ks, stream);
}

// Shape of the FP32 tile launch: 32 rows per CTA (the squarest tile against up to 64 narrow rows keeps the bytes
// an SM pulls from L2 per FMA lowest) and as many K parts per cluster (a power of two, at most 8, at least one
// 128-float chunk each) as keep the grid within one wave.  Measured on 37 x 1024 x 1024: 32 rows x 4 parts 6.4 us,
// 16 x 2 7.7 us, 8 x 1 9.8 us, one warp per row pair 33 us.  MOONPOLY_F32_TILE="rows,parts" (rows 8, 16 or 32)
// overrides the shape for experiments.
void tile_f32_rule(const SkinnyF32Params& sp, int sms, int* rows, int* ks) {
  static const char* env = std::getenv("MOONPOLY_F32_TILE");
  const int chunks = (sp.K + kTileF32KC - 1) / kTileF32KC;
  int r = 32, k = 1;
  if (env && std::sscanf(env, "%d,%d", &r, &k) >= 1 && (r == 8 || r == 16 || r == 32)) {
    k = std::max(1, std::min(k, 8));
  } else {
    r = 32;
    const int blocks = (sp.R + r - 1) / r;
    k = 1;
    while (k < 8 && blocks * k * 2 <= sms) k *= 2;
  }
  *rows = r;
  *ks = std::max(1, std::min(k, chunks));
}

int run_skinny_f32(const Problem& p, cudaStream_t stream) {
  DeviceState* d = nullptr;
  if (int rc = device_state(&d)) return rc;
  SkinnyF32Params sp{};
  const bool narrow_is_a = p.m <= p.n;
  sp.W = reinterpret_cast<const float*>(narrow_is_a ? p.B : p.A);
  sp.ldw = narrow_is_a ? p.ldb : p.lda;
  sp.X = reinterpret_cast<const float*>(narrow_is_a ? p.A : p.B);
  sp.ldx = narrow_is_a ? p.lda : p.ldb;
  sp.R = narrow_is_a ? p.n : p.m;
  sp.T = narrow_is_a ? p.m : p.n;
  sp.K = p.k;
  sp.out = reinterpret_cast<float*>(p.C);
  sp.stride_r = narrow_is_a ? p.c_stride_n : p.c_stride_m;
  sp.stride_t = narrow_is_a ? p.c_stride_m : p.c_stride_n;
  sp.alpha = p.alpha; sp.beta = p.beta;
  if (sp.T > 8) {
    int rows = 32, ks = 1;
    tile_f32_rule(sp, d->sms, &rows, &ks);
    return rows == 32 ? launch_tile_f32_t<2, 4>(*d, sp, ks, stream)
         : rows == 16 ? launch_tile_f32_t<1, 4>(*d, sp, ks, stream) : launch_tile_f32_t<1, 2>(*d, sp, ks, stream);
  }
  // at most 8 narrow rows: the streaming kernel; four rows per CTA once two rows per CTA are more than 16 CTAs per SM
  if (sp.R >= 32 * d->sms) return launch_gemv_f32<4, 4>(sp, stream);
  return launch_gemv_f32<2, 8>(sp, stream);
}

int check_rcc_args(int dtype, int m, int n, int k, const void* A, const void* B, const void* C) {
  if (dtype != MP_FP16 && dtype != MP_INT8 && dtype != MP_FP32)
    return fail(MP_ERR_INVALID_ARG, "Unsupported data type %d", dtype);
  if (m < 0 || n < 0 || k < 0) return fail(MP_ERR_INVALID_ARG, "negative problem size (%d,%d,%d)", m, n, k);
  if (m > 0 && n > 0 && (C == nullptr || (k > 0 && (A == nullptr || B == nullptr))))
    return fail(MP_ERR_INVALID_ARG, "null operand pointer");
  return MP_OK;
}

Problem rcc_problem(int dtype, int m, int n, int k, const void* A, const void* B, void* C, float alpha, float beta) {
  Problem p{};
  p.dtype = dtype;
  p.epi = dtype == MP_INT8 ? EPI_I32 : EPI_F16;
  p.m = m; p.n = n; p.k = k;
  p.A = A; p.lda = k; p.B = B; p.ldb = k;
  p.C = C; p.c_stride_m = 1; p.c_stride_n = m;
  p.alpha = alpha; p.beta = beta;
  p.ialpha = (int)alpha; p.ibeta = (int)beta;
  return p;
}

// The tensor-core launch a pid stands for on problem `p`.  The streaming pids (orient 2 / 3) name
// kernels of their own; for shapes those do not cover they fall back to a narrow tensor tile whose
// orientation follows the problem.  run_pid and mp_workspace_size both derive the launch here, so
// the reported workspace size always matches what the call will need.
Launch umma_launch_for(const Problem& p, const TileCfg& c, int split_k) {
  Launch l;
  l.split_k = std::max(1, split_k);
  if (c.orient == 2) {
    l.orient = p.m <= p.n ? 1 : 0; l.bn = 16;
  } else if (c.orient == 3) {
    l.orient = p.m <= p.n ? 1 : 0; l.bn = std::min(64, std::max(16, (std::min(p.m, p.n) + 15) / 16 * 16));
  } else {
    l.orient = c.orient; l.bn = c.bn; l.xm = c.xm == 2 ? 2 : 1;
  }
  return l;
}

// Runs one pid (or the dedicated split-K tile when pid < 0) on an RCC problem.
int run_pid(const Problem& p, int pid, int split_k, void* ws, size_t ws_bytes, cudaStream_t stream) {
  if (p.m == 0 || p.n == 0) return MP_OK;
  const int eff_pid = pid >= 0 ? pid : (p.dtype == MP_FP32 ? 23 : 6);
  const TileCfg c = tile_cfg(p.dtype, eff_pid);
  if (!c.valid) return fail(MP_ERR_BAD_PID, "pid %d has no kernel for dtype %d", pid, p.dtype);
  if (p.dtype == MP_FP32) {
    if (c.orient == 3) {          // the FP32 streaming kernel; shapes it does not cover take a 64x64 tile
      if (skinny_f32_compatible(p)) return run_skinny_f32(p, stream);
      return run_simt(p, 64, 64, split_k, ws, ws_bytes, stream);
    }
    return run_simt(p, c.ti, c.tj, split_k, ws, ws_bytes, stream);
  }
  if (!tma_compatible(p)) return run_simt(p, 64, 64, split_k, ws, ws_bytes, stream);
  // the skinny CUDA-core kernel serves plain FP16 only: bf16 operands, a fused bias or extra destinations take the
  // warp-MMA streaming kernel instead
  const bool plain = !p.bf16 && p.bias == nullptr && p.num_peers == 0;
  if (c.orient == 2 && plain && gemv_compatible(p)) return run_gemv(p, stream);        // the skinny streaming kernel
  if ((c.orient == 3 || (c.orient == 2 && !plain)) && stream_compatible(p)) return run_stream(p, stream);    // the streaming warp-MMA kernel
  Launch l = umma_launch_for(p, c, split_k);
  l.workspace = ws; l.workspace_bytes = ws_bytes;
  return run_umma(p, l, stream);
}

int run_twin(const Problem& p, int split_n, cudaStream_t stream) {
  if (p.m == 0 || p.n == 0) return MP_OK;
  if (!tma_compatible(p)) {
    // two plain launches with the reference's pointer offsets (core/fp16/fp16_rcc.cu:101-103)
    Problem p0 = p; p0.n = split_n;
    Problem p1 = p; p1.n = p.n - split_n;
    p1.B = reinterpret_cast<const uint8_t*>(p.B) + (size_t)split_n * p.ldb * 2;
    p1.C = reinterpret_cast<uint8_t*>(p.C) + (size_t)split_n * p.c_stride_n * 2;
    if (int rc = run_simt(p0, 64, 64, 1, nullptr, 0, stream)) return rc;
    return run_simt(p1, 64, 64, 1, nullptr, 0, stream);
  }
  Launch l;
  l.orient = 0;
  l.bn = (split_n % 256 == 0) ? 256 : 128;
  l.split_n = split_n;
  const int tail = p.n - split_n;
  l.bn1 = std::min(64, (tail + 15) / 16 * 16);
  l.split_k = 1;
  return run_umma(p, l, stream);
}

}  // namespace

// ================================================================================================
// exported entry points
// ================================================================================================
extern "C" {

const char* mp_last_error_string(void) { return g_err; }
const char* mp_version(void) { return "moonpoly-b200 0.1 (sm_100a)"; }
unsigned long long mp_launch_count(void) { return g_launches.load(); }

int mp_num_sms(void) {
  DeviceState* d = nullptr;
  if (device_state(&d) != MP_OK) return 0;
  return d->sms;
}

int mp_reload_env(void) {
  mp::reload_env();
  g_use_streamk.store(streamk_from_env(), std::memory_order_relaxed);
  g_use_cluster_splitk.store(cluster_splitk_from_env(), std::memory_order_relaxed);
  g_stream_tsplit.store(stream_tsplit_from_env(), std::memory_order_relaxed);
  g_stream_ksplit.store(stream_ksplit_from_env(), std::memory_order_relaxed);
  return MP_OK;
}

int mp_select_plan(int dtype, int m, int n, int k, mp_plan* plan) {
  if (plan == nullptr) return fail(MP_ERR_INVALID_ARG, "plan is null");
  if (dtype != MP_FP16 && dtype != MP_INT8 && dtype != MP_FP32)
    return fail(MP_ERR_INVALID_ARG, "Unsupported data type %d", dtype);
  if (m <= 0 || n <= 0 || k <= 0) return fail(MP_ERR_INVALID_ARG, "non-positive problem size");
  *plan = mp::select_plan(dtype, m, n, k);
  return MP_OK;
}

int mp_pid_info(int dtype, int pid, int tile[3], int* alignment) {
  const TileCfg c = tile_cfg(dtype, pid);
  if (!c.valid) return fail(MP_ERR_BAD_PID, "pid %d has no kernel for dtype %d", pid, dtype);
  if (tile) pid_tile_meta(dtype, pid, tile);
  if (alignment) *alignment = c.align;
  return MP_OK;
}

int mp_cost_ms(int dtype, int pid, int split_k, int m, int n, int k, float* ms) {
  if (ms == nullptr) return fail(MP_ERR_INVALID_ARG, "ms is null");
  if (!pid_exists(dtype, pid)) return fail(MP_ERR_BAD_PID, "pid %d has no kernel for dtype %d", pid, dtype);
  *ms = mp::cost_ms(dtype, pid, split_k, m, n, k);
  return MP_OK;
}

int mp_cost_reduction_ms(int dtype, int pid, int split_k, int m, int n, float* ms) {
  if (ms == nullptr) return fail(MP_ERR_INVALID_ARG, "ms is null");
  if (!pid_exists(dtype, pid)) return fail(MP_ERR_BAD_PID, "pid %d has no kernel for dtype %d", pid, dtype);
  *ms = mp::reduction_cost_ms(dtype, pid, split_k, m, n);
  return MP_OK;
}

int mp_cost_predict_pid(int dtype, int m, int n, int k, int* pid, float* ms) {
  if (pid == nullptr) return fail(MP_ERR_INVALID_ARG, "pid is null");
  if (dtype != MP_FP16 && dtype != MP_INT8 && dtype != MP_FP32)
    return fail(MP_ERR_INVALID_ARG, "Unsupported data type %d", dtype);
  if (m <= 0 || n <= 0 || k <= 0) return fail(MP_ERR_INVALID_ARG, "non-positive problem size");
  *pid = mp::predict_primary_pid(dtype, m, n, k, ms);
  return MP_OK;
}

int mp_debug_scratch_must_grow(size_t have_bytes, size_t have_counter_bytes, size_t want_counter_bytes,
                               size_t partial_bytes) {
  return scratch_must_grow(have_bytes, have_counter_bytes, want_counter_bytes, partial_bytes) ? 1 : 0;
}

int mp_debug_stream_launch(int dtype, int m, int n, int k, int out[4]) {
  if (out == nullptr || (dtype != MP_FP16 && dtype != MP_INT8) || m < 1 || n < 1 || k < 1)
    return fail(MP_ERR_INVALID_ARG, "mp_debug_stream_launch: FP16 or INT8, positive sizes");
  const int R = std::max(m, n), T = std::min(m, n);
  const StreamShape sh = stream_launch_shape(R, T, k, elem_bytes(dtype), mp::num_sms_for_model(), 0, 0);
  out[0] = sh.row_ctas; out[1] = sh.k_split; out[2] = sh.t_split;
  out[3] = sh.row_ctas * sh.k_split * sh.t_split;
  return MP_OK;
}

int mp_debug_f32_tile_launch(int m, int n, int k, int out[3]) {
  if (out == nullptr || m < 1 || n < 1 || k < 1) return fail(MP_ERR_INVALID_ARG, "mp_debug_f32_tile_launch: positive sizes");
  SkinnyF32Params sp{};
  sp.R = std::max(m, n); sp.T = std::min(m, n); sp.K = k;
  int rows = 32, ks = 1;
  tile_f32_rule(sp, mp::num_sms_for_model(), &rows, &ks);
  out[0] = rows; out[1] = ks; out[2] = (sp.R + rows - 1) / rows * ks;
  return MP_OK;
}

int mp_elite_fp16_pids(int* pids, int capacity) { return mp::elite_fp16_pids(pids, capacity); }
int mp_is_explicit_neighborhood_pid(int pid) { return mp::is_explicit_neighborhood_fp16_pid(pid) ? 1 : 0; }

int mp_debug_schedule(int dtype, int orient, int bn, int kc, int split_k, int m, int n, int k, int* units,
                      int capacity, int* count, int* info) {
  if (dtype != MP_FP16 && dtype != MP_INT8) return fail(MP_ERR_INVALID_ARG, "the tile schedule exists for FP16 and INT8");
  if (count == nullptr || m <= 0 || n <= 0 || k <= 0) return fail(MP_ERR_INVALID_ARG, "bad arguments");
  const int xm = (orient == 4 || orient == 5) ? 2 : 1;
  if (xm == 2) orient -= 4;
  if ((orient != 0 && orient != 1) || bn < 16 || bn > 256 || bn % 16 != 0) return fail(MP_ERR_INVALID_ARG, "bad tile");
  Problem p = rcc_problem(dtype, m, n, k, reinterpret_cast<const void*>(16), reinterpret_cast<const void*>(16),
                          reinterpret_cast<void*>(16), 1.0f, 0.0f);
  Launch l;
  l.orient = orient; l.bn = bn; l.kc = kc; l.split_k = std::max(1, split_k); l.xm = xm;
  l.dry_units = units; l.dry_capacity = units ? capacity : 0; l.dry_count = count; l.dry_grid = info;
  return run_umma(p, l, nullptr);
}

int mp_workspace_size(int dtype, int pid, int m, int n, int k, int split_k, size_t* bytes) {
  if (bytes == nullptr) return fail(MP_ERR_INVALID_ARG, "bytes is null");
  *bytes = 0;
  if (split_k <= 0) split_k = 2;
  const int eff_pid = pid >= 0 ? pid : (dtype == MP_FP32 ? 23 : 6);
  const TileCfg c = tile_cfg(dtype, eff_pid);
  if (!c.valid) return fail(MP_ERR_BAD_PID, "pid %d has no kernel for dtype %d", pid, dtype);
  if (split_k <= 1 || m <= 0 || n <= 0 || k <= 0) return MP_OK;
  // the larger of the two paths a call may take (tensor tiles, or CUDA-core tiles for unaligned K)
  const size_t simt = (size_t)split_k * m * n * 4;
  if (dtype == MP_FP32) { *bytes = simt; return MP_OK; }
  Problem p{};
  p.dtype = dtype; p.m = m; p.n = n; p.k = k;
  const Launch l = umma_launch_for(p, c, split_k);
  *bytes = std::max(simt, umma_workspace_bytes(p, l, nullptr));
  return MP_OK;
}

int mp_gemm_rcc_pid(int dtype, int pid, int split_k, int m, int n, int k, const void* A, const void* B, void* C,
                    float alpha, float beta, void* workspace, size_t workspace_bytes, void* stream) {
  if (int rc = check_rcc_args(dtype, m, n, k, A, B, C)) return rc;
  if (split_k <= 0) split_k = 2;
  const TileCfg c = tile_cfg(dtype, pid);
  if (!c.valid) return fail(MP_ERR_BAD_PID, "pid %d has no kernel for dtype %d", pid, dtype);
  if (k % c.align != 0)
    return fail(MP_ERR_UNALIGNED_K, " k is not aligned, please check! (k=%d, pid %d needs k %% %d == 0)", k, pid, c.align);
  const Problem p = rcc_problem(dtype, m, n, k, A, B, C, alpha, beta);
  return run_pid(p, pid, split_k, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

int mp_gemm_rcc_tile(int dtype, int orient, int bn, int kc, int split_k, int m, int n, int k, const void* A,
                     const void* B, void* C, float alpha, float beta, void* stream) {
  if (int rc = check_rcc_args(dtype, m, n, k, A, B, C)) return rc;
  if (dtype == MP_FP32) return fail(MP_ERR_UNSUPPORTED, "explicit tiles exist for the tensor-core dtypes only");
  if (orient == 2) {            // the skinny streaming kernel (bn, kc, split_k unused)
    const Problem pg = rcc_problem(dtype, m, n, k, A, B, C, alpha, beta);
    if (!gemv_compatible(pg)) return fail(MP_ERR_INVALID_ARG, "the skinny kernel needs FP16, min(m,n) <= 8 and 16-byte aligned rows");
    return run_gemv(pg, reinterpret_cast<cudaStream_t>(stream));
  }
  if (orient == 3) {            // the streaming warp-MMA kernel (bn unused; kc = -K parts, split_k = token parts)
    const Problem pg = rcc_problem(dtype, m, n, k, A, B, C, alpha, beta);
    if (!stream_compatible(pg)) return fail(MP_ERR_INVALID_ARG, "the streaming kernel needs FP16 or INT8, min(m,n) <= 64 and 16-byte aligned rows");
    if (kc != 0 && kc != -1 && kc != -2 && kc != -4 && kc != -8)
      return fail(MP_ERR_INVALID_ARG, "streaming kernel: kc = -1 / -2 / -4 / -8 selects that many K parts, 0 lets the library choose");
    return run_stream(pg, reinterpret_cast<cudaStream_t>(stream), kc, split_k > 1 ? split_k : 0);
  }
  const int xm = (orient == 4 || orient == 5) ? 2 : 1;       // orient 4 / 5: orient 0 / 1 with 256-row tiles
  if (xm == 2) orient -= 4;
  if ((orient != 0 && orient != 1) || bn < 16 || bn > 256 || bn % 16 != 0 || (kc != 0 && kc != 1 && kc != 2 && kc != 4))
    return fail(MP_ERR_INVALID_ARG, "bad tile: orient=%d bn=%d kc=%d", orient, bn, kc);
  if (m == 0 || n == 0) return MP_OK;
  const Problem p = rcc_problem(dtype, m, n, k, A, B, C, alpha, beta);
  if (!tma_compatible(p)) return fail(MP_ERR_UNALIGNED_K, "operands do not meet the 16-byte alignment of the tensor path");
  Launch l;
  l.orient = orient; l.bn = bn; l.kc = kc; l.split_k = std::max(1, split_k); l.xm = xm;
  return run_umma(p, l, reinterpret_cast<cudaStream_t>(stream));
}

int mp_twin_gemm_fp16(int m, int n, int k, int split_n, const void* A, const void* B, void* C, float alpha,
                      float beta, void* stream) {
  if (int rc = check_rcc_args(MP_FP16, m, n, k, A, B, C)) return rc;
  if (split_n <= 0) split_n = mp::choose_pattern2_split_n(n);
  if (split_n <= 0 || split_n >= n || split_n % 128 != 0)
    return fail(MP_ERR_INVALID_ARG,
                "Pattern2 FP16 RCC requires 0 < split_n < n and split_n aligned to the OP0 N tile");
  if (k % 8 != 0) return fail(MP_ERR_INVALID_ARG, "Pattern2 FP16 RCC requires K aligned to 8");
  const Problem p = rcc_problem(MP_FP16, m, n, k, A, B, C, alpha, beta);
  return run_twin(p, split_n, reinterpret_cast<cudaStream_t>(stream));
}

int mp_gemm_rcc(int dtype, int m, int n, int k, const void* A, const void* B, void* C, float alpha, float beta,
                void* stream) {
  if (int rc = check_rcc_args(dtype, m, n, k, A, B, C)) return rc;
  if (m == 0 || n == 0) return MP_OK;
  Problem p = rcc_problem(dtype, m, n, k, A, B, C, alpha, beta);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (k == 0) return run_simt(p, 64, 64, 1, nullptr, 0, s);
  pad_operands(p, s);                              // unaligned rows: the plan is then made for the padded K
  const mp_plan plan = mp::select_plan(dtype, m, n, p.k);
  if (dtype == MP_FP16 && plan.pattern == MP_PATTERN_COMBINE) return run_twin(p, plan.split_n, s);
  return run_pid(p, plan.pid, plan.split_k, nullptr, 0, s);
}

int mp_gemm(int dtype, int m, int n, int k, const void* A, int a_col_major, const void* B, int b_col_major, void* C,
            int c_col_major, float alpha, float beta, void* stream) {
  if (dtype != MP_FP16 && dtype != MP_INT8 && dtype != MP_FP32)
    return fail(MP_ERR_INVALID_ARG, "Unsupported data type");
  if (!(!a_col_major && b_col_major && c_col_major))
    return fail(MP_ERR_LAYOUT, "Unsupported layout: only A row-major, B column-major, C column-major is served");
  return mp_gemm_rcc(dtype, m, n, k, A, B, C, alpha, beta, stream);
}

int mp_linear(int dtype, int M, int N, int K, const void* X, const void* W, void* Y, void* stream) {
  return mp_gemm(dtype, N, M, K, W, 0, X, 1, Y, 1, 1.0f, 0.0f, stream);
}

// ------------------------------------------------------------------------------------------------
// Column-parallel Linear fused with the all-gather of its output, and the cross-GPU flag barrier that follows
// ------------------------------------------------------------------------------------------------
int mp_linear_gather(int dtype, int M, int N_local, int K, const void* X, const void* W_shard, void* const* dst,
                     int n_dst, long long ld_dst, long long col_offset, void* stream) {
  if (dtype != MP_FP16) return fail(MP_ERR_UNSUPPORTED, "the fused all-gather Linear is served for FP16");
  if (dst == nullptr || n_dst < 1 || n_dst > 8) return fail(MP_ERR_INVALID_ARG, "1 to 8 destination buffers are supported, got %d", n_dst);
  if (M < 0 || N_local < 0 || K < 0 || col_offset < 0 || ld_dst < col_offset + N_local)
    return fail(MP_ERR_INVALID_ARG, "bad sizes: M=%d N_local=%d K=%d ld=%lld offset=%lld", M, N_local, K, ld_dst, col_offset);
  for (int i = 0; i < n_dst; ++i)
    if (dst[i] == nullptr) return fail(MP_ERR_INVALID_ARG, "destination %d is null", i);
  if (M == 0 || N_local == 0) return MP_OK;
  if (K == 0 || X == nullptr || W_shard == nullptr) return fail(MP_ERR_INVALID_ARG, "null operand pointer or K == 0");
  // Linear -> RCC: m = N_local (A = W), n = M (B = X); C element (channel j, token t) lives at base + t * ld + offset + j
  Problem p = rcc_problem(dtype, N_local, M, K, W_shard, X, reinterpret_cast<__half*>(dst[0]) + col_offset, 1.0f, 0.0f);
  p.c_stride_m = 1;
  p.c_stride_n = ld_dst;
  p.num_peers = n_dst - 1;
  for (int i = 1; i < n_dst; ++i) p.peers[i - 1] = reinterpret_cast<__half*>(dst[i]) + col_offset;
  if (!tma_compatible(p))
    return fail(MP_ERR_UNALIGNED_K, "the fused all-gather Linear needs 16-byte aligned operand rows (K %% 8 == 0)");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  mp_plan plan = mp::select_plan(dtype, N_local, M, K);
  if (plan.pattern == MP_PATTERN_COMBINE) {       // the twin launch writes through the same epilogue
    return run_twin(p, plan.split_n, s);
  }
  return run_pid(p, plan.pid, plan.split_k, nullptr, 0, s);
}

int mp_linear_bias(int dtype, int M, int N, int K, const void* X, const void* W, const void* bias, void* Y, void* stream) {
  if (dtype != MP_FP16 && dtype != MP_BF16)
    return fail(MP_ERR_INVALID_ARG, "mp_linear_bias serves MP_FP16 and MP_BF16, got dtype %d", dtype);
  if (int rc = check_rcc_args(MP_FP16, N, M, K, W, X, Y)) return rc;
  if (M == 0 || N == 0) return MP_OK;
  // Linear -> RCC: m = N (A = W), n = M (B = X); the bias runs along m
  Problem p = rcc_problem(MP_FP16, N, M, K, W, X, Y, 1.0f, 0.0f);
  p.bias = bias;
  p.bias_on_m = 1;
  if (dtype == MP_BF16) { p.bf16 = 1; p.out_bf16 = 1; }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (K == 0) return run_simt(p, 64, 64, 1, nullptr, 0, s);
  pad_operands(p, s);
  const mp_plan plan = mp::select_plan(MP_FP16, N, M, p.k);
  if (plan.pattern == MP_PATTERN_COMBINE) return run_twin(p, plan.split_n, s);
  return run_pid(p, plan.pid, plan.split_k, nullptr, 0, s);
}

namespace {
// One warp: lane r < world first publishes `value` in rank r's flag array at this rank's slot (release at system
// scope, after a system fence: the slab stores of the kernels before it in the stream are visible first), then
// waits until rank r's value has arrived here.  The wait is bounded; on expiry the status word gets a code.
__global__ void peer_barrier_kernel(unsigned* const* flags, int world, int rank, unsigned value,
                                    unsigned long long timeout_ns, int* status) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();
  unsigned* theirs = flags[r] + rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(value) : "memory");
  const unsigned* mine = flags[rank] + r;
  const unsigned long long t0 = mp::globaltimer_ns();
  for (;;) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if ((int)(v - value) >= 0) break;                       // counters only grow (wrap-around safe)
    if (mp::globaltimer_ns() - t0 > timeout_ns) {
      atomicCAS(status, 0, mp::MP_DEV_TIMEOUT_PEER);
      break;
    }
  }
}
}  // namespace

int mp_peer_barrier(unsigned* const* flags_dev, int world, int rank, unsigned value, unsigned timeout_us, void* stream) {
  if (flags_dev == nullptr || world < 1 || world > 8 || rank < 0 || rank >= world)
    return fail(MP_ERR_INVALID_ARG, "bad peer barrier arguments (world %d, rank %d)", world, rank);
  DeviceState* d = nullptr;
  if (int rc = device_state(&d)) return rc;
  int* status = nullptr;
  MP_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), mp::g_mp_status));
  peer_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      flags_dev, world, rank, value, (unsigned long long)(timeout_us ? timeout_us : 1000000u) * 1000ull, status);
  MP_CUDA_TRY(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return MP_OK;
}

int mp_peer_alloc(size_t bytes, void** ptr, unsigned char handle[64]) {
  if (ptr == nullptr || handle == nullptr || bytes == 0) return fail(MP_ERR_INVALID_ARG, "bad arguments");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* p = nullptr;
  MP_CUDA_TRY(cudaMalloc(&p, bytes));
  MP_CUDA_TRY(cudaMemset(p, 0, bytes));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail(MP_ERR_CUDA, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
  }
  std::memcpy(handle, &h, 64);
  *ptr = p;
  return MP_OK;
}

int mp_peer_open(const unsigned char handle[64], void** ptr) {
  if (ptr == nullptr || handle == nullptr) return fail(MP_ERR_INVALID_ARG, "bad arguments");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, 64);
  MP_CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return MP_OK;
}

int mp_peer_close(void* ptr) {
  if (ptr == nullptr) return MP_OK;
  MP_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return MP_OK;
}

int mp_peer_free(void* ptr) {
  if (ptr == nullptr) return MP_OK;
  MP_CUDA_TRY(cudaFree(ptr));
  return MP_OK;
}

int mp_scaled_mm_predict(int M, int N, int K) { return mp::scaled_mm_select(M, N, K).id; }

int mp_scaled_mm_config(int config_id, int out[4]) {
  if (config_id < 0 || config_id >= mp::kScaledConfigCount || out == nullptr)
    return fail(MP_ERR_INVALID_ARG, "Invalid config id: %d", config_id);
  mp::scaled_mm_config_meta(config_id, out);
  return MP_OK;
}

namespace {
int scaled_problem(Problem* p, int M, int N, int K, const int8_t* A, int lda, const int8_t* B_nk, int ldb,
                   const float* a_scales, int a_scalar, const float* b_scales, int b_scalar, const void* bias,
                   void* out, int ldc, int out_dtype) {
  if (M < 0 || N < 0 || K < 0) return fail(MP_ERR_INVALID_ARG, "negative problem size");
  if (M == 0 || N == 0) return -1;          // nothing to do
  if (!A || !B_nk || !out || !a_scales || !b_scales) return fail(MP_ERR_INVALID_ARG, "null operand pointer");
  if (out_dtype != 0 && out_dtype != 1) return fail(MP_ERR_INVALID_ARG, "Unsupported output dtype %d", out_dtype);
  if (lda < K || ldb < K || ldc < N) return fail(MP_ERR_INVALID_ARG, "leading dimension smaller than the row");
  *p = Problem{};
  p->dtype = MP_INT8; p->epi = EPI_SCALED;
  p->m = M; p->n = N; p->k = K;
  p->A = A; p->lda = lda; p->B = B_nk; p->ldb = ldb;
  p->C = out; p->c_stride_m = ldc; p->c_stride_n = 1;
  p->a_scales = a_scales; p->b_scales = b_scales; p->a_scalar = a_scalar ? 1 : 0; p->b_scalar = b_scalar ? 1 : 0;
  p->bias = bias; p->out_bf16 = out_dtype;
  return MP_OK;
}
}  // namespace

int mp_scaled_mm_i8(int M, int N, int K, const int8_t* A, int lda, const int8_t* B_nk, int ldb, const float* a_scales,
                    int a_scalar, const float* b_scales, int b_scalar, const void* bias, void* out, int ldc,
                    int out_dtype, void* stream) {
  Problem p;
  const int rc = scaled_problem(&p, M, N, K, A, lda, B_nk, ldb, a_scales, a_scalar, b_scales, b_scalar, bias, out, ldc,
                                out_dtype);
  if (rc != MP_OK) return rc < 0 ? MP_OK : rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (K > 0) pad_operands(p, s);
  if (K == 0 || !tma_compatible(p)) return run_simt(p, 64, 64, 1, nullptr, 0, s);
  const mp::ScaledCfg cfg = mp::scaled_mm_select(M, N, p.k);
  if (cfg.stream && stream_compatible(p)) return run_stream(p, s);
  Launch l;
  l.orient = cfg.orient; l.bn = cfg.bn; l.split_k = cfg.split_k; l.xm = cfg.xm;
  return run_umma(p, l, s);
}

int mp_scaled_mm_i8_tile(int orient, int bn, int split_k, int M, int N, int K, const int8_t* A, int lda,
                         const int8_t* B_nk, int ldb, const float* a_scales, int a_scalar, const float* b_scales,
                         int b_scalar, const void* bias, void* out, int ldc, int out_dtype, void* stream) {
  Problem p;
  const int rc = scaled_problem(&p, M, N, K, A, lda, B_nk, ldb, a_scales, a_scalar, b_scales, b_scalar, bias, out, ldc,
                                out_dtype);
  if (rc != MP_OK) return rc < 0 ? MP_OK : rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (K == 0 || !tma_compatible(p)) return fail(MP_ERR_INVALID_ARG, "operands miss the 16-byte alignment the tensor-core kernels need");
  if (orient == 3) {
    if (!stream_compatible(p)) return fail(MP_ERR_INVALID_ARG, "the streaming kernel needs min(M,N) <= 64");
    return run_stream(p, s);
  }
  const int xm = (orient == 4 || orient == 5) ? 2 : 1;       // orient 4 / 5: orient 0 / 1 with 256-row tiles
  if (xm == 2) orient -= 4;
  if ((orient != 0 && orient != 1) || bn < 16 || bn > 256 || bn % 16 != 0)
    return fail(MP_ERR_INVALID_ARG, "bad tile: orient=%d bn=%d", orient, bn);
  Launch l;
  l.orient = orient; l.bn = bn; l.split_k = std::max(1, split_k); l.xm = xm;
  return run_umma(p, l, s);
}

int mp_device_status(void* stream, int* device_code) {
  DeviceState* d = nullptr;
  if (int rc = device_state(&d)) return rc;
  if (stream) MP_CUDA_TRY(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)));
  else MP_CUDA_TRY(cudaDeviceSynchronize());
  int code = 0;
  MP_CUDA_TRY(cudaMemcpyFromSymbol(&code, mp::g_mp_status, sizeof(int)));
  if (device_code) *device_code = code;
  if (code != 0) {
    const int zero = 0;
    MP_CUDA_TRY(cudaMemcpyToSymbol(mp::g_mp_status, &zero, sizeof(int)));
    return fail(MP_ERR_DEVICE, "a kernel recorded device status %d (bounded wait expired)", code);
  }
  return MP_OK;
}

// ------------------------------------------------------------------------------------------------
// Forced-pid GEMM that never allocates: its split-K scratch is a fixed array inside the library.
// ------------------------------------------------------------------------------------------------
int mp_gemm_rcc_pid_static_scratch(int dtype, int pid, int split_k, int m, int n, int k, const void* A,
                                   const void* B, void* C, float alpha, float beta, void* stream) {
  if (int rc = check_rcc_args(dtype, m, n, k, A, B, C)) return rc;
  if (split_k <= 0) split_k = 2;
  const TileCfg c = tile_cfg(dtype, pid);
  if (!c.valid) return fail(MP_ERR_BAD_PID, "pid %d has no kernel for dtype %d", pid, dtype);
  if (k % c.align != 0)
    return fail(MP_ERR_UNALIGNED_K, " k is not aligned, please check! (k=%d, pid %d needs k %% %d == 0)", k, pid, c.align);
  size_t need = 0;
  if (int rc = mp_workspace_size(dtype, pid, m, n, k, split_k, &need)) return rc;
  if (need > kStaticScratchBytes)
    return fail(MP_ERR_WORKSPACE,
                "this problem needs %zu bytes of split-K scratch but the built-in array holds %zu; "
                "lower split_k or use mp_gemm_rcc_pid with a workspace of your own",
                need, (size_t)kStaticScratchBytes);
  int dev = -1;
  MP_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(MP_ERR_CUDA, "device index %d out of range", dev);
  void* scratch = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    // set-up, once per device, with that device current: host code only holds a stand-in for the
    // array's name, so ask the runtime for its address on this device
    std::lock_guard<std::mutex> g(g_mu);
    MP_CUDA_TRY(cudaGetSymbolAddress(&scratch, g_static_scratch));
    g_static_scratch_ptr[dev].store(scratch, std::memory_order_release);
  }
  const Problem p = rcc_problem(dtype, m, n, k, A, B, C, alpha, beta);
  // the scratch keeps whatever the previous call left; run_umma clears the counters it needs at
  // zero (a memset on `stream`, not an allocation) before the launch
  return run_pid(p, pid, split_k, scratch, kStaticScratchBytes, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
