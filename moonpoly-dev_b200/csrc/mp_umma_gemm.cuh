// Persistent tcgen05 GEMM for sm_100a:   D[P x Q] = X[P x K] * Y[Q x K]^T
//
// Both operands are K-contiguous ("K-major"), which is what the row-column-column contract of the
// reference gives (A row-major [m,k]; B column-major [k,n], i.e. stored [n,k];
// moonpoly/core/fp16/fp16_rcc.cu:537-544).  The host decides which operand sits on the 128-wide
// UMMA-M side (X) and which on the 16..256-wide UMMA-N side (Y), and passes the element strides of
// the output so that either assignment writes the caller's column-major C (or row-major `out` of
// the scaled int8 matmul) directly.
//
// One launch covers the whole problem ("polymerisation" in one kernel): a device-side schedule walks
// work units = (output tile, K slice).  Tiles may come from two regions with different UMMA-N
// (the Pattern-2 twin GEMM of moonpoly/core/fp16/fp16_rcc.cu:75-108), and K may be cut into slices
// (Pattern-3 / pids 400+); slices park fp32/int32 partials in a workspace and the last slice to
// arrive sums them in slice order, so the result is bit-identical from run to run and no CTA ever
// waits for another.  When every work unit has a CTA of its own and the slice count is 2, 4 or 8, the
// slices of a tile are instead launched as one thread-block cluster and exchange their partials through
// distributed shared memory (CLUSTER variant below): same sums in the same order, no trip through L2.
//
// Roles per CTA (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
// warps 2..5 = epilogue (TMEM lane quadrant = warp % 4).  Accumulators are double-buffered in TMEM
// so the epilogue of one unit overlaps the main loop of the next.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "mp_ptx.cuh"

namespace mp {

__device__ int g_mp_status = 0;   // 0 = ok; otherwise the first MP_DEV_* code any kernel recorded

constexpr int kUmmaM = 128;            // rows of X per tile
constexpr int kRowBytes = 128;         // one K block = 128 bytes of K per row (64 fp16 / 128 int8)
constexpr int kXTileBytes = kUmmaM * kRowBytes;
constexpr int kMaxBN = 256;
constexpr int kTmemCols = 512;
constexpr int kMaxStages = 12;
constexpr int kUmmaThreads = 192;       // kernels that may split K: producer, MMA issuer, 4 epilogue warps
constexpr int kUmmaThreadsWide = 320;   // single-slice kernels: 8 epilogue warps (two per TMEM lane quadrant)
constexpr int kSmemBudget = 232448;    // 227 KB opt-in limit per CTA
constexpr int kClusterBarBytes = 64;   // cluster variant: ready[4 quadrants] + done barriers behind the TMEM slot

enum { KIND_F16 = 0, KIND_I8 = 1 };
enum { EPI_F16 = 0, EPI_I32 = 1, EPI_SCALED = 2 };

struct Region {
  int q_begin;    // first Q index of the region
  int q_end;      // one past the last Q index
  int bn;         // UMMA-N (multiple of 16, <= 256) used for this region
  int tiles_q;    // ceil((q_end - q_begin) / bn)
  int tile_base;  // index of the region's first tile in the launch-wide tile numbering
};

struct UmmaParams {
  int P, Q, K;
  int tiles_p;
  int num_regions;
  Region reg[2];
  int total_tiles;
  int split_k;        // K slices per tile (>= 1); every slice is non-empty
  int kb_total;       // ceil(K / elements per K block)
  int kb_per_slice;   // a multiple of kc
  int kc;             // K blocks per pipeline stage (1, 2 or 4)
  int wide;           // 1: tensor maps are 3-D [K/kb][rows][kb] and one load brings kc K blocks
  int stages;
  int xm;             // 128-row halves of X per tile: 1, or 2 = 256 x bn tiles (two accumulators share every Y tile)
  int stage_bytes;    // kc * (xm * kXTileBytes + bn_max * kRowBytes)
  int group_p;        // raster: tiles are walked in groups of `group_p` rows of tiles
  int prefetch_kb;    // K blocks of a CTA's first unit to prefetch into L2 before the dependency wait
  void* out;
  long long out_stride_p, out_stride_q;   // element strides of `out` along P and Q
  // fused all-gather of a column-parallel Linear: every finished tile is also stored, with the same strides, at
  // these bases -- the same output buffer in the memory of the other GPUs (peer-mapped pointers, plain stores)
  void* peer_out[7];
  int num_peers;
  float alpha, beta;
  int ialpha, ibeta;
  uint32_t* ws_partials;   // [total_tiles][split_k][bn_max / 4][128 rows] 16-byte words
  unsigned* ws_counters;   // [total_tiles][4 quadrants][arrived, claimed, left, -], zero on entry, left zero on exit
  int ws_tile_words;       // xm * bn_max * 128: one slice of one tile (its xm 128-row halves one after the other)
  int ws_half_words;       // bn_max * 128: one 128-row half
  int ws_slices;           // slices per tile in the scratch numbering (split_k, or sk_max_slices for stream-K tiles)
  int helpers_ok;          // 1: all units run concurrently, early slices may help with the reduction
  int cluster_k;           // > 1: the split_k slices of a tile are the CTAs of one cluster (CLUSTER kernels only)
  // stream-K head: the first sk_tiles tiles (single region, split_k == 1) are cut into contiguous runs of
  // sk_ipc K blocks, one run per CTA, so that the remainder of total_tiles / grid does not cost a whole wave
  int sk_tiles, sk_ipc;
  // scaled int8 matmul epilogue
  const float* scale_p; const float* scale_q;   // scales indexed along P / along Q
  int scale_p_scalar, scale_q_scalar;
  int n_on_p;              // 1: P is the weight/output-channel index (b_scales, bias live on P)
  const void* bias;        // in the output type, indexed by output channel; may be null
  int out_bf16;
  // FP16-kind GEMM (EPI_F16): ab_bf16 = 1 reads both operands as bf16 (output then bf16 too, out_bf16 = 1);
  // with `bias` set, bias_on_p says whether the bias index (the output channel) runs along P or along Q
  int ab_bf16;
  int bias_on_p;
};

struct UnitCoord {
  int region, tile, tp, tq, kb0, kb1, slice, nslices;
};

__host__ __device__ __forceinline__ void tile_coords(const UmmaParams& p, UnitCoord& u) {
  u.region = (p.num_regions == 2 && u.tile >= p.reg[1].tile_base) ? 1 : 0;
  const Region& r = p.reg[u.region];
  const int t = u.tile - r.tile_base;
  const int group_sz = p.group_p * r.tiles_q;
  const int g = t / group_sz;
  const int first_p = g * p.group_p;
  const int rows = p.group_p < p.tiles_p - first_p ? p.group_p : p.tiles_p - first_p;
  const int in_g = t - g * group_sz;
  u.tq = in_g / rows;
  u.tp = first_p + (in_g - u.tq * rows);
}

// The work units of one CTA, in the order every role of the CTA walks them: first its run of the
// stream-K head (if any), which may cover the tail of one tile and the head of the next, then the
// uniform units  w = blockIdx.x, blockIdx.x + grid, ...  where unit w is slice w % split_k of tile
// sk_tiles + w / split_k.
struct UnitWalk {
  int sk_cur, sk_end, w, cta, grid;
  __device__ __forceinline__ explicit UnitWalk(const UmmaParams& p) : UnitWalk(p, (int)blockIdx.x, (int)gridDim.x) {}
  // the same walk for CTA `cta_` of a grid of `grid_` CTAs; host code uses it to check schedules
  __host__ __device__ __forceinline__ UnitWalk(const UmmaParams& p, int cta_, int grid_) : cta(cta_), grid(grid_) {
    const long long total = (long long)p.sk_tiles * p.kb_total;
    const long long b = (long long)cta * p.sk_ipc;
    sk_cur = (int)(b < total ? b : total);
    sk_end = (int)(b + p.sk_ipc < total ? b + p.sk_ipc : total);
    w = cta;
  }
  __host__ __device__ __forceinline__ bool next(const UmmaParams& p, UnitCoord& u) {
    if (sk_cur < sk_end) {
      u.tile = sk_cur / p.kb_total;
      u.kb0 = sk_cur - u.tile * p.kb_total;
      const int len = p.kb_total - u.kb0 < sk_end - sk_cur ? p.kb_total - u.kb0 : sk_end - sk_cur;
      u.kb1 = u.kb0 + len;
      const int first_cta = (u.tile * p.kb_total) / p.sk_ipc;
      const int last_cta = ((u.tile + 1) * p.kb_total - 1) / p.sk_ipc;
      u.slice = cta - first_cta;
      u.nslices = last_cta - first_cta + 1;
      sk_cur += len;
      tile_coords(p, u);
      return true;
    }
    const int uniform_units = (p.total_tiles - p.sk_tiles) * p.split_k;
    if (w >= uniform_units) return false;
    const int t = w / p.split_k;
    u.tile = p.sk_tiles + t;
    u.slice = w - t * p.split_k;
    u.nslices = p.split_k;
    u.kb0 = u.slice * p.kb_per_slice;
    u.kb1 = p.kb_total < u.kb0 + p.kb_per_slice ? p.kb_total : u.kb0 + p.kb_per_slice;
    tile_coords(p, u);
    w += grid;
    return true;
  }
};

// ------------------------------------------------------------------------------------ epilogue math
// What the scaled epilogue needs besides the accumulators, fetched once per tile before the
// accumulator is waited for: with ~200 KB of the SM's L1/shared memory given to the pipeline stages
// little L1 is left, and a scale load issued per 16-column chunk cost an L2 round trip each time.
struct ScaledStage {
  const float* sq;       // shared memory: scale along Q for the tile's columns, index q - q_base
  const uint16_t* bq;    // shared memory: bias along Q (when the channels are on Q), same index
  int q_base;
  float sp;              // scale of this thread's row
  uint16_t bp;           // bias of this thread's row (when the channels are on P)
};

__device__ __forceinline__ uint16_t f32_to_out16(float v, int bf16) {
  if (bf16) return __bfloat16_as_ushort(__float2bfloat16_rn(v));
  return __half_as_ushort(__float2half_rn(v));
}

// Final value for one output element from its 32-bit accumulator word.
template <int EPI>
__device__ __forceinline__ void finish_store(const UmmaParams& p, void* out_base, uint32_t accw, int pi, int qi,
                                             float sp, float sq_or_zero) {
  const long long off = (long long)pi * p.out_stride_p + (long long)qi * p.out_stride_q;
  if constexpr (EPI == EPI_F16) {
    // out = RN16(alpha * acc + beta * old); with a bias: out = RN16(out + bias[channel]), added in the output type
    float v = p.alpha * __uint_as_float(accw);
    uint16_t* o = reinterpret_cast<uint16_t*>(out_base) + off;
    if (p.beta != 0.0f)
      v += p.beta * (p.out_bf16 ? __bfloat162float(__ushort_as_bfloat16(*o)) : __half2float(__ushort_as_half(*o)));
    uint16_t h = f32_to_out16(v, p.out_bf16);
    if (p.bias != nullptr) {
      const uint16_t b = reinterpret_cast<const uint16_t*>(p.bias)[p.bias_on_p ? pi : qi];
      if (p.out_bf16) h = __bfloat16_as_ushort(__float2bfloat16_rn(__bfloat162float(__ushort_as_bfloat16(h)) + __bfloat162float(__ushort_as_bfloat16(b))));
      else h = __half_as_ushort(__float2half_rn(__half2float(__ushort_as_half(h)) + __half2float(__ushort_as_half(b))));
    }
    *o = h;
  } else if constexpr (EPI == EPI_I32) {
    int v = p.ialpha * (int)accw;
    int* o = reinterpret_cast<int*>(out_base) + off;
    if (p.ibeta != 0) v += p.ibeta * (*o);
    *o = v;
  } else {
    // out = RN16( a_scale[token] * RN32( b_scale[channel] * RN32(acc) ) ) (+ bias in the output type)
    const float bs = p.n_on_p ? sp : sq_or_zero;
    const float as = p.n_on_p ? sq_or_zero : sp;
    const float t0 = __fmul_rn(__int2float_rn((int)accw), bs);
    const float t1 = __fmul_rn(as, t0);
    uint16_t h = f32_to_out16(t1, p.out_bf16);
    if (p.bias != nullptr) {
      const int ch = p.n_on_p ? pi : qi;
      const uint16_t b = reinterpret_cast<const uint16_t*>(p.bias)[ch];
      if (p.out_bf16) {
        const float s = __bfloat162float(__ushort_as_bfloat16(h)) + __bfloat162float(__ushort_as_bfloat16(b));
        h = __bfloat16_as_ushort(__float2bfloat16_rn(s));
      } else {
        const float s = __half2float(__ushort_as_half(h)) + __half2float(__ushort_as_half(b));
        h = __half_as_ushort(__float2half_rn(s));
      }
    }
    reinterpret_cast<uint16_t*>(out_base)[off] = h;
  }
}

// Store 16 consecutive Q columns [q0, q0+16) of row `pi` from accumulator words r[0..15].
template <int EPI>
__device__ __forceinline__ void store_chunk16_to(const UmmaParams& p, void* out_base, const uint32_t (&r)[16], int pi, int q0,
                                                 int q_end, const ScaledStage& st) {
  if (pi >= p.P) return;
  const int valid = min(16, q_end - q0);
  if (valid <= 0) return;

  if constexpr (EPI == EPI_F16) {
    // fast path: row of D is contiguous in memory and the 32-byte run is aligned
    if (p.out_stride_q == 1 && valid == 16 && p.beta == 0.0f && p.bias == nullptr && !p.out_bf16) {
      __half* o = reinterpret_cast<__half*>(out_base) + (long long)pi * p.out_stride_p + q0;
      if ((reinterpret_cast<uintptr_t>(o) & 15) == 0) {
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const __half2 h = __floats2half2_rn(p.alpha * __uint_as_float(r[2 * j]),
                                              p.alpha * __uint_as_float(r[2 * j + 1]));
          w[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        reinterpret_cast<uint4*>(o)[0] = make_uint4(w[0], w[1], w[2], w[3]);
        reinterpret_cast<uint4*>(o)[1] = make_uint4(w[4], w[5], w[6], w[7]);
        return;
      }
    }
  }
  if constexpr (EPI == EPI_F16) {
    // rows of D are the contiguous index of the output (the 32 lanes of a warp write 64 adjacent
    // bytes per column): one pointer walks the 16 columns, no per-element index arithmetic
    if (p.out_stride_p == 1 && p.beta == 0.0f && p.bias == nullptr && !p.out_bf16) {
      __half* o = reinterpret_cast<__half*>(out_base) + pi + (long long)q0 * p.out_stride_q;
      const long long step = p.out_stride_q;
      if (valid == 16) {
#pragma unroll
        for (int j = 0; j < 16; ++j) o[(long long)j * step] = __float2half_rn(p.alpha * __uint_as_float(r[j]));
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (j < valid) o[(long long)j * step] = __float2half_rn(p.alpha * __uint_as_float(r[j]));
      }
      return;
    }
  }
  if constexpr (EPI == EPI_I32) {
    if (p.out_stride_p == 1 && p.ibeta == 0) {
      int* o = reinterpret_cast<int*>(out_base) + pi + (long long)q0 * p.out_stride_q;
      const long long step = p.out_stride_q;
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (j < valid) o[(long long)j * step] = p.ialpha * (int)r[j];
      return;
    }
  }
  if constexpr (EPI == EPI_I32) {
    if (p.out_stride_q == 1 && valid == 16 && p.ibeta == 0) {
      int* o = reinterpret_cast<int*>(out_base) + (long long)pi * p.out_stride_p + q0;
      if ((reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          reinterpret_cast<uint4*>(o)[j] =
              make_uint4(p.ialpha * (int)r[4 * j], p.ialpha * (int)r[4 * j + 1],
                         p.ialpha * (int)r[4 * j + 2], p.ialpha * (int)r[4 * j + 3]);
        return;
      }
    }
  }

  if constexpr (EPI == EPI_SCALED) {
    const float sp = st.sp;
    const bool has_bias = p.bias != nullptr;
    const float* sqs = st.sq + (q0 - st.q_base);
    // fast path: this thread's 16 outputs are contiguous and 16-byte aligned; the result leaves as
    // two 16-byte stores
    uint16_t* o = reinterpret_cast<uint16_t*>(out_base) + (long long)pi * p.out_stride_p + q0;
    if (p.out_stride_q == 1 && valid == 16 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
      float sq[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 t = reinterpret_cast<const float4*>(sqs)[j];
        sq[4 * j] = t.x; sq[4 * j + 1] = t.y; sq[4 * j + 2] = t.z; sq[4 * j + 3] = t.w;
      }
      uint16_t bq[16];
      if (has_bias) {
        if (p.n_on_p) {
#pragma unroll
          for (int j = 0; j < 16; ++j) bq[j] = st.bp;
        } else {
          const uint4* b4 = reinterpret_cast<const uint4*>(st.bq + (q0 - st.q_base));
          const uint4 t0 = b4[0], t1 = b4[1];
          const uint32_t w[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
#pragma unroll
          for (int j = 0; j < 8; ++j) { bq[2 * j] = (uint16_t)(w[j] & 0xffffu); bq[2 * j + 1] = (uint16_t)(w[j] >> 16); }
        }
      }
      uint32_t packed[8];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float bs = p.n_on_p ? sp : sq[j];
        const float as = p.n_on_p ? sq[j] : sp;
        const float t1 = __fmul_rn(as, __fmul_rn(__int2float_rn((int)r[j]), bs));
        uint16_t h = f32_to_out16(t1, p.out_bf16);
        if (has_bias) {
          if (p.out_bf16) {
            const float sum = __bfloat162float(__ushort_as_bfloat16(h)) + __bfloat162float(__ushort_as_bfloat16(bq[j]));
            h = __bfloat16_as_ushort(__float2bfloat16_rn(sum));
          } else {
            const float sum = __half2float(__ushort_as_half(h)) + __half2float(__ushort_as_half(bq[j]));
            h = __half_as_ushort(__float2half_rn(sum));
          }
        }
        if (j & 1) packed[j >> 1] |= (uint32_t)h << 16;
        else packed[j >> 1] = h;
      }
      reinterpret_cast<uint4*>(o)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      reinterpret_cast<uint4*>(o)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
      return;
    }
    // every other layout: one pointer walks the 16 columns (when the rows of D are the contiguous
    // index of the output, the 32 lanes of a warp write 64 adjacent bytes per column)
    uint16_t* ow = reinterpret_cast<uint16_t*>(out_base) + (long long)pi * p.out_stride_p + (long long)q0 * p.out_stride_q;
    const long long step = p.out_stride_q;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      if (j < valid) {
        const float bs = p.n_on_p ? sp : sqs[j];
        const float as = p.n_on_p ? sqs[j] : sp;
        const float t1 = __fmul_rn(as, __fmul_rn(__int2float_rn((int)r[j]), bs));
        uint16_t h = f32_to_out16(t1, p.out_bf16);
        if (has_bias) {
          const uint16_t b = p.n_on_p ? st.bp : st.bq[q0 - st.q_base + j];
          if (p.out_bf16) {
            const float sum = __bfloat162float(__ushort_as_bfloat16(h)) + __bfloat162float(__ushort_as_bfloat16(b));
            h = __bfloat16_as_ushort(__float2bfloat16_rn(sum));
          } else {
            const float sum = __half2float(__ushort_as_half(h)) + __half2float(__ushort_as_half(b));
            h = __half_as_ushort(__float2half_rn(sum));
          }
        }
        ow[(long long)j * step] = h;
      }
    }
    return;
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    if (j < valid) finish_store<EPI>(p, out_base, r[j], pi, q0 + j, 0.0f, 0.0f);
  }
}

// The caller's output, then the same tile at every peer base (fused all-gather; num_peers is 0 otherwise).
template <int EPI>
__device__ __forceinline__ void store_chunk16(const UmmaParams& p, const uint32_t (&r)[16], int pi, int q0,
                                              int q_end, const ScaledStage& st) {
  store_chunk16_to<EPI>(p, p.out, r, pi, q0, q_end, st);
  for (int d = 0; d < p.num_peers; ++d) store_chunk16_to<EPI>(p, p.peer_out[d], r, pi, q0, q_end, st);
}

// ------------------------------------------------------------------------------------ the kernel
// SPLIT = true: tiles may be finished through the split-K scratch (uniform slices or a stream-K head); the
// reduction needs ~130 registers of partial sums in flight, which leaves room for 4 epilogue warps only.
// SPLIT = false: every unit is a whole tile; the reduction is compiled out and 8 epilogue warps (two per TMEM
// lane quadrant, taking alternate 32-column groups) halve the time a tile needs to leave TMEM -- that time is
// exposed whenever a CTA has a single tile, and always with 256-row tiles.
// CLUSTER = true (implies SPLIT): launched with cluster dimension split_k and exactly one work unit per CTA; the
// CTAs of a cluster are the K slices of one tile.  Each parks its raw accumulators in its OWN shared memory
// (the pipeline stages are idle by then), tells its peers, and sums its share of the tile's columns by reading
// every slice's partials -- its own included -- through distributed shared memory, in slice order 0..S-1: the
// same additions in the same order as the scratch path, so both give bit-identical results.
template <int KIND, int EPI, bool SPLIT, bool CLUSTER = false>
__global__ void __launch_bounds__(SPLIT ? kUmmaThreads : kUmmaThreadsWide, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmY0,
                 const __grid_constant__ CUtensorMap tmY1, const UmmaParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const int stages = p.stages;
  const uint32_t bar_base = smem_base + (uint32_t)stages * (uint32_t)p.stage_bytes;
  // barrier slots (8 bytes each): full[stages] | empty[stages] | tfull[2] | tempty[2] | tmem slot
  auto full_bar = [&](int s) { return bar_base + 8u * (uint32_t)s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (uint32_t)(stages + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (uint32_t)(2 * stages + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (uint32_t)(2 * stages + 2 + b); };
  volatile uint32_t* tmem_slot =
      reinterpret_cast<volatile uint32_t*>(smem + (size_t)stages * p.stage_bytes + 8 * (2 * stages + 4));
  // cluster variant: ready[q] (count = slices) says "quadrant q of every slice is parked", done (count = 4 x
  // slices) says "every warp of the cluster has finished reading": no CTA's shared memory may go away before
  const uint32_t cbar_base = bar_base + 8u * (uint32_t)(2 * stages + 4) + 16u;
  auto ready_bar = [&](int q) { return cbar_base + 8u * (uint32_t)q; };
  const uint32_t done_bar = cbar_base + 32u;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  int* status = &g_mp_status;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), SPLIT ? 4 : 8);
    }
    if constexpr (CLUSTER) {
      for (int q = 0; q < 4; ++q) mbar_init(ready_bar(q), (uint32_t)p.cluster_k);
      mbar_init(done_bar, 4u * (uint32_t)p.cluster_k);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmY0);
    if (p.num_regions == 2) tma_prefetch_desc(&tmY1);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // peers arrive on this CTA's cluster barriers: nobody may do so before they are initialised
  if constexpr (CLUSTER) cluster_sync_all();

  // Programmatic dependent launch: everything above touched only this CTA's shared memory, TMEM
  // and kernel parameters, so it may overlap the tail of the previous kernel in the stream.  Let
  // the next kernel start its own prologue now.  Each role then waits (griddep_wait) before its
  // first access to global memory that the previous kernel may still produce or use: the
  // operands, C, the split-K scratch.  The MMA issuer touches only shared memory and TMEM.
  griddep_launch_dependents();

  constexpr int kElemsPerKb = (KIND == KIND_I8) ? 128 : 64;
  // slices whose partials are in flight together in the split-K reduction; the scaled epilogue needs the
  // registers for itself
  constexpr int kSliceBatch = (EPI == EPI_SCALED) ? 2 : 4;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (one lane)
    if (lane == 0) {
      // While the previous kernel drains, pull the first unit's operands towards L2 (a hint only;
      // whatever the previous kernel still writes reaches L2 as well, so this cannot go stale).
      UnitCoord u;
      if (UnitWalk(p).next(p, u)) {
        const Region& r = p.reg[u.region];
        const CUtensorMap* tmY = u.region ? &tmY1 : &tmY0;
        const int prow = u.tp * kUmmaM * p.xm, qrow = r.q_begin + u.tq * r.bn;
        const int kb_lim = min(u.kb1, u.kb0 + p.prefetch_kb);
        for (int kb = u.kb0; kb < kb_lim; kb += p.kc) {
          if (p.wide) {
            tma_prefetch_3d(&tmX, 0, prow, kb);
            tma_prefetch_3d(tmY, 0, qrow, kb);
          } else {
            for (int c = 0; c < p.kc; ++c) {
              tma_prefetch_2d(&tmX, (kb + c) * kElemsPerKb, prow);
              tma_prefetch_2d(tmY, (kb + c) * kElemsPerKb, qrow);
            }
          }
        }
      }
      griddep_wait();
      uint32_t it = 0;
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      UnitWalk walk(p);
      while (ok && walk.next(p, u)) {
        const Region& r = p.reg[u.region];
        const CUtensorMap* tmY = u.region ? &tmY1 : &tmY0;
        const uint32_t x_bytes = (uint32_t)(p.xm * kXTileBytes);      // X rows of one K block
        const uint32_t tx = (uint32_t)p.kc * (x_bytes + (uint32_t)(r.bn * kRowBytes));
        const uint32_t y_off = (uint32_t)p.kc * x_bytes;
        const int prow = u.tp * kUmmaM * p.xm;
        const int qrow = r.q_begin + u.tq * r.bn;
        for (int kb = u.kb0; kb < u.kb1; kb += p.kc, ++it) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u, status, MP_DEV_TIMEOUT_PRODUCER)) { ok = false; break; }
          const uint32_t a_dst = smem_base + (uint32_t)s * (uint32_t)p.stage_bytes;
          mbar_arrive_expect_tx(full_bar(s), tx);
          if (p.wide) {
            tma_load_3d(a_dst, &tmX, full_bar(s), 0, prow, kb);
            tma_load_3d(a_dst + y_off, tmY, full_bar(s), 0, qrow, kb);
          } else {
            // 2-D maps (K not a multiple of one K block): one box per K block; boxes past the
            // end of K are filled with zeros by the TMA unit and still count their bytes
            for (int c = 0; c < p.kc; ++c) {
              tma_load_2d(a_dst + (uint32_t)c * x_bytes, &tmX, full_bar(s), (kb + c) * kElemsPerKb, prow);
              tma_load_2d(a_dst + y_off + (uint32_t)(c * r.bn * kRowBytes), tmY, full_bar(s),
                          (kb + c) * kElemsPerKb, qrow);
            }
          }
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
      }
      if (!ok) {
        // Give copies that were already issued a bounded chance to land before the CTA retires.
        const uint32_t lo = it > (uint32_t)stages ? it - (uint32_t)stages : 0u;
        for (uint32_t i = lo; i < it; ++i) {
          // no status word: the error already recorded must not cut this drain short
          mbar_wait(full_bar((int)(i % (uint32_t)stages)), (i / (uint32_t)stages) & 1u, nullptr,
                    MP_DEV_TIMEOUT_DRAIN);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (one lane)
    if (lane == 0) {
      // The issuing thread is on the critical path of narrow tiles (a 128 x 64 x 16 MMA lasts ~32
      // cycles), so the loop carries its state instead of recomputing it: stage index and phase
      // are counters, and the operand descriptors of a stage are the descriptor of shared-memory
      // offset 0 plus byte offsets >> 4 added to its address field.
      uint32_t ui = 0;
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      const uint64_t desc0 = umma_smem_desc_sw128(smem_base);
      const uint32_t x16 = (uint32_t)(p.xm * kXTileBytes) >> 4;        // X rows of one K block, in 16-byte units
      const uint32_t stage16 = (uint32_t)p.stage_bytes >> 4;
      UnitWalk walk(p);
      UnitCoord u;
      for (; ok && walk.next(p, u); ++ui) {
        const Region& r = p.reg[u.region];
        // 256-row tiles keep two accumulators (all 512 TMEM columns): one buffer, no overlap with the drain
        const uint32_t buf = p.xm == 2 ? 0u : (ui & 1u);
        const uint32_t use = p.xm == 2 ? ui : (ui >> 1);
        if (!mbar_wait(tempty_bar((int)buf), (use & 1u) ^ 1u, status, MP_DEV_TIMEOUT_MMA_TMEM)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * (uint32_t)kMaxBN;
        const uint32_t idesc = (KIND == KIND_I8) ? umma_idesc(2u, 1u, kUmmaM, (uint32_t)r.bn)
                                                 : umma_idesc(1u, p.ab_bf16 ? 1u : 0u, kUmmaM, (uint32_t)r.bn);
        const uint32_t y16 = (uint32_t)(r.bn * kRowBytes) >> 4;        // Y rows of one K block
        uint32_t first = 0u;                                            // 0 until the accumulators hold a product
        for (int kb = u.kb0; kb < u.kb1; kb += p.kc) {
          if (!mbar_wait(full_bar(s), ph, status, MP_DEV_TIMEOUT_MMA_FULL)) { ok = false; break; }
          tc_fence_after();
          uint64_t ad = desc0 + (uint64_t)((uint32_t)s * stage16);
          uint64_t bd = ad + (uint64_t)((uint32_t)p.kc * x16);
          const int nc = min(p.kc, u.kb1 - kb);     // K blocks of this stage that lie inside the slice
          for (int c = 0; c < nc; ++c, ad += x16, bd += y16) {
            // 4 x 32 bytes of K per 128-byte row; with 256-row tiles both halves of X use the same Y tile
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint32_t acc = kk > 0 ? 1u : first;
              if constexpr (KIND == KIND_I8) umma_i8(d_tmem, ad + 2u * kk, bd + 2u * kk, idesc, acc);
              else umma_f16(d_tmem, ad + 2u * kk, bd + 2u * kk, idesc, acc);
            }
            if (p.xm == 2) {
              const uint64_t ad1 = ad + (uint64_t)(kXTileBytes >> 4);
#pragma unroll
              for (int kk = 0; kk < 4; ++kk) {
                const uint32_t acc = kk > 0 ? 1u : first;
                if constexpr (KIND == KIND_I8) umma_i8(d_tmem + (uint32_t)kMaxBN, ad1 + 2u * kk, bd + 2u * kk, idesc, acc);
                else umma_f16(d_tmem + (uint32_t)kMaxBN, ad1 + 2u * kk, bd + 2u * kk, idesc, acc);
              }
            }
            first = 1u;
          }
          tc_commit(empty_bar(s));      // stage reusable once these MMAs have read it
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
        if (ok) tc_commit(tfull_bar((int)buf));   // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int quad = warp & 3;
    const int half = SPLIT ? 0 : ((warp - 2) >> 2);       // which alternate 32-column groups this warp drains
    constexpr int kColStep = SPLIT ? 32 : 64;
    uint32_t ui = 0;
    bool ok = true;
    griddep_wait();
    UnitWalk walk(p);
    UnitCoord u;
    for (; ok && walk.next(p, u); ++ui) {
      const Region& r = p.reg[u.region];
      const uint32_t buf = p.xm == 2 ? 0u : (ui & 1u);
      const uint32_t use = p.xm == 2 ? ui : (ui >> 1);
      // scaled epilogue: fetch the tile's scales and bias while the accumulator is still being produced
      ScaledStage st{};
      float sp_h[2] = {0.0f, 0.0f};
      uint16_t bp_h[2] = {0, 0};
      if constexpr (EPI == EPI_SCALED) {
        uint8_t* mine = smem + (size_t)stages * p.stage_bytes + 8 * (2 * stages + 4) + 16 + kClusterBarBytes +
                        (size_t)(warp - 2) * 1536;
        float* sq_s = reinterpret_cast<float*>(mine);
        uint16_t* bq_s = reinterpret_cast<uint16_t*>(mine + 1024);
        const int qb = r.q_begin + u.tq * r.bn;
        const bool bias_on_q = p.bias != nullptr && !p.n_on_p;
        __syncwarp();                      // this warp has finished reading the previous tile's values
        for (int j = lane; j < r.bn; j += 32) {
          const int q = qb + j;
          sq_s[j] = q < r.q_end ? p.scale_q[p.scale_q_scalar ? 0 : q] : 0.0f;
          if (bias_on_q) bq_s[j] = q < r.q_end ? reinterpret_cast<const uint16_t*>(p.bias)[q] : (uint16_t)0;
        }
        for (int h = 0; h < p.xm; ++h) {
          const int row = (u.tp * p.xm + h) * kUmmaM + quad * 32 + lane;
          if (row < p.P) {
            sp_h[h] = p.scale_p[p.scale_p_scalar ? 0 : row];
            if (p.bias != nullptr && p.n_on_p) bp_h[h] = reinterpret_cast<const uint16_t*>(p.bias)[row];
          }
        }
        __syncwarp();
        st.sq = sq_s; st.bq = bq_s; st.q_base = qb; st.sp = sp_h[0]; st.bp = bp_h[0];
      }
      if (!mbar_wait(tfull_bar((int)buf), use & 1u, status, MP_DEV_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      uint32_t t_addr = tmem_base + buf * (uint32_t)kMaxBN + ((uint32_t)(quad * 32) << 16);
      const int row_in_tile = quad * 32 + lane;
      int pi = u.tp * kUmmaM * p.xm + row_in_tile;
      const int q_tile0 = r.q_begin + u.tq * r.bn;
      const int q_end = min(r.q_end, q_tile0 + r.bn);

      const int S = u.nslices;               // slices that make up this unit's tile
      if (!SPLIT || S == 1) {
        // two 16-column TMEM loads are in flight before the wait: the round trip, not the data,
        // is what a load costs.  256-row tiles drain their second accumulator (the tile's rows
        // 128..255, TMEM columns 256..511) the same way.
        for (int h = 0; h < p.xm; ++h, t_addr += (uint32_t)kMaxBN, pi += kUmmaM) {
        if constexpr (EPI == EPI_SCALED) { st.sp = sp_h[h]; st.bp = bp_h[h]; }
        {
          for (int c0 = 32 * half; c0 < r.bn; c0 += kColStep) {
            uint32_t v[2][16];
            const bool two = c0 + 16 < r.bn;
            tmem_ld_x16(t_addr + (uint32_t)c0, v[0]);
            if (two) tmem_ld_x16(t_addr + (uint32_t)c0 + 16u, v[1]);
            tmem_ld_wait();
            store_chunk16<EPI>(p, v[0], pi, q_tile0 + c0, q_end, st);
            if (two) store_chunk16<EPI>(p, v[1], pi, q_tile0 + c0 + 16, q_end, st);
          }
        }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar((int)buf));
      } else if constexpr (CLUSTER) {
        // ---- split-K inside a cluster: park the raw accumulators in this CTA's own shared memory as
        // [column / 4][row] 16-byte words (32 lanes = 512 contiguous bytes per access, conflict-free).  The
        // pipeline stages are idle: this CTA's only unit has been consumed by the MMAs that tfull reported.
        const uint32_t xbuf = smem_base + (uint32_t)row_in_tile * 16u;
        for (int c0 = 0; c0 < r.bn; c0 += 32) {
          uint32_t v[2][16];
          const bool two = c0 + 16 < r.bn;
          tmem_ld_x16(t_addr + (uint32_t)c0, v[0]);
          if (two) tmem_ld_x16(t_addr + (uint32_t)c0 + 16u, v[1]);
          tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < 2; ++h)
            if (h == 0 || two) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                st_smem_v4(xbuf + (uint32_t)(((c0 + 16 * h) >> 2) + j) * (uint32_t)(kUmmaM * 16),
                           make_uint4(v[h][4 * j], v[h][4 * j + 1], v[h][4 * j + 2], v[h][4 * j + 3]));
            }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(tempty_bar((int)buf));
          // tell every slice of the tile (this one included) that quadrant `quad` of slice u.slice is parked
          for (int s = 0; s < S; ++s) mbar_arrive_cluster(mapa_shared(ready_bar(quad), (uint32_t)s));
        }
        const bool got = mbar_wait_cluster(ready_bar(quad), 0u, status, MP_DEV_TIMEOUT_CLUSTER);
        if (got) {
          // this CTA finishes share `slice` of the 16-column chunks; every column is summed in slice order 0..S-1
          const int chunks = r.bn >> 4;
          const int c_begin = ((int)u.slice * chunks / S) << 4;
          const int c_end = (((int)u.slice + 1) * chunks / S) << 4;
          for (int c0 = c_begin; c0 < c_end; c0 += 16) {
            uint32_t v[16];
            const uint32_t off = xbuf + (uint32_t)(c0 >> 2) * (uint32_t)(kUmmaM * 16);
            for (int s0 = 0; s0 < S; s0 += kSliceBatch) {
              uint4 x[kSliceBatch][4];
#pragma unroll
              for (int ds = 0; ds < kSliceBatch; ++ds)
                if (s0 + ds < S) {
                  const uint32_t remote = mapa_shared(off, (uint32_t)(s0 + ds));
#pragma unroll
                  for (int j = 0; j < 4; ++j) x[ds][j] = ld_dsmem_v4(remote + (uint32_t)j * (uint32_t)(kUmmaM * 16));
                }
#pragma unroll
              for (int ds = 0; ds < kSliceBatch; ++ds)
                if (s0 + ds < S) {
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const uint32_t w[4] = {x[ds][j].x, x[ds][j].y, x[ds][j].z, x[ds][j].w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                      uint32_t& acc = v[4 * j + e];
                      if (s0 + ds == 0) acc = w[e];
                      else if constexpr (KIND == KIND_I8) acc = (uint32_t)((int)acc + (int)w[e]);
                      else acc = __float_as_uint(__fadd_rn(__uint_as_float(acc), __uint_as_float(w[e])));
                    }
                  }
                }
            }
            store_chunk16<EPI>(p, v, pi, q_tile0 + c0, q_end, st);
          }
        }
        __syncwarp();
        // the peers' shared memory is no longer needed by this warp (also reported after a failed wait, so that a
        // healthy peer can leave)
        if (lane == 0)
          for (int s = 0; s < S; ++s) mbar_arrive_cluster(mapa_shared(done_bar, (uint32_t)s));
        if (!got) { ok = false; break; }
      } else if constexpr (SPLIT) {
        // park this slice's raw accumulators as [tile][slice][half][column / 4][row] 16-byte words: the 32
        // lanes of a warp (32 consecutive rows) then touch 512 contiguous bytes per access, both here
        // and in the reduction below (row-major scratch would scatter each access over 32 lines)
        for (int h = 0; h < p.xm; ++h) {
          uint4* part = reinterpret_cast<uint4*>(p.ws_partials + ((size_t)u.tile * p.ws_slices + u.slice) * (size_t)p.ws_tile_words +
                                                 (size_t)h * p.ws_half_words) + row_in_tile;
          const uint32_t t_half = t_addr + (uint32_t)h * (uint32_t)kMaxBN;
          for (int c0 = 0; c0 < r.bn; c0 += 32) {
            uint32_t v[2][16];
            const bool two = c0 + 16 < r.bn;                       // two TMEM loads in flight per wait
            tmem_ld_x16(t_half + (uint32_t)c0, v[0]);
            if (two) tmem_ld_x16(t_half + (uint32_t)c0 + 16u, v[1]);
            tmem_ld_wait();
#pragma unroll
            for (int hh = 0; hh < 2; ++hh)
              if (hh == 0 || two) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  __stcg(part + (size_t)(((c0 + 16 * hh) >> 2) + j) * kUmmaM,
                         make_uint4(v[hh][4 * j], v[hh][4 * j + 1], v[hh][4 * j + 2], v[hh][4 * j + 3]));
              }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar((int)buf));   // TMEM buffer is free again
        __threadfence();
        __syncwarp();
        // Reduction of this quadrant of the tile.  Share i is the run of 16-column chunks
        // [i*chunks/S, (i+1)*chunks/S).  The warp that arrives last (ticket S-1) knows all S slices are
        // parked: it sums its own share at once, then seals the claim mask and takes every share
        // nobody has registered for.  A warp that arrived earlier may help with the share of its
        // ticket: it registers (a fire-and-forget atomic OR), waits a short, bounded time for the
        // last arrival and then sums the share; if the wait runs out it withdraws the registration --
        // unless the mask is already sealed, which tells it that everything has arrived and that the
        // share has been left to it.  Nothing therefore ever depends on a warp that is waiting (no
        // deadlock when kernels of several streams compete for the SMs), and helping is only tried
        // when all work units run concurrently (one unit per CTA).  Every column is summed in slice
        // order s = 0..S-1 whoever sums it: results are bit-identical from run to run.
        constexpr unsigned kSealed = 0x80000000u;
        unsigned* ctr = p.ws_counters + ((size_t)u.tile * 4 + quad) * 4;   // arrived, claim mask, left, unused
        unsigned ticket = 0;
        if (lane == 0) ticket = atomicAdd(ctr, 1u);
        ticket = __shfl_sync(0xffffffffu, ticket, 0);
        const int chunks = r.bn >> 4;
        const int total_chunks = chunks * p.xm;           // the tile's 128-row halves one after the other
        const bool last = ticket == (unsigned)(S - 1);
        const unsigned all_shares = (1u << S) - 1u;      // S <= 31
        unsigned mine = 0;                      // shares this warp sums
        if (last) {
          mine = 1u << ticket;
        } else if (p.helpers_ok && ((int)ticket + 1) * total_chunks / S > (int)ticket * total_chunks / S) {
          unsigned got = 0;
          if (lane == 0) {
            atomicOr(ctr + 1, 1u << ticket);
            if (counter_wait_ge_for(ctr, (unsigned)S, kHelpWaitNs)) got = 1u << ticket;
            else if (atomicAnd(ctr + 1, ~(1u << ticket)) & kSealed) got = 1u << ticket;
          }
          mine = __shfl_sync(0xffffffffu, got, 0);
        }
        for (int round = 0; round < 2; ++round) {
          if (round == 1) {
            if (!last) break;
            unsigned rest = 0;
            if (lane == 0) rest = all_shares & ~atomicOr(ctr + 1, all_shares | kSealed) & ~(1u << ticket);
            mine = __shfl_sync(0xffffffffu, rest, 0);
          }
          if (mine != 0) __threadfence();
          while (mine != 0) {
            const int share = __ffs((int)mine) - 1;
            mine &= mine - 1;
            const int sb = share * total_chunks / S, se = (share + 1) * total_chunks / S;
            for (int h = 0; h < p.xm; ++h) {
            const int lo = max(sb, h * chunks) - h * chunks, hi = min(se, (h + 1) * chunks) - h * chunks;
            if (lo >= hi) continue;
            const int c_begin = lo << 4, c_end = hi << 4;
            const int pi_h = pi + h * kUmmaM;
            if constexpr (EPI == EPI_SCALED) { st.sp = sp_h[h]; st.bp = bp_h[h]; }
          const uint4* base = reinterpret_cast<const uint4*>(p.ws_partials + (size_t)u.tile * p.ws_slices * (size_t)p.ws_tile_words +
                                                             (size_t)h * p.ws_half_words) + row_in_tile;
          const size_t slice_words16 = (size_t)p.ws_tile_words >> 2;
          // 32 columns per pass (the last pass may be half wide); the loads of up to kSliceBatch slices
          // are all in flight before the first is consumed
          for (int c0 = c_begin; c0 < c_end; c0 += 32) {
            const int nq = (c_end - c0 >= 32) ? 8 : 4;      // 16-byte words in this pass
            uint32_t v[32];
            for (int s0 = 0; s0 < S; s0 += kSliceBatch) {
              uint4 x[kSliceBatch][8];
#pragma unroll
              for (int ds = 0; ds < kSliceBatch; ++ds)
                if (s0 + ds < S) {
                  const uint4* ps = base + (size_t)(s0 + ds) * slice_words16 + (size_t)(c0 >> 2) * kUmmaM;
#pragma unroll
                  for (int j = 0; j < 8; ++j)
                    if (j < nq) x[ds][j] = __ldcg(ps + (size_t)j * kUmmaM);
                }
#pragma unroll
              for (int ds = 0; ds < kSliceBatch; ++ds)
                if (s0 + ds < S) {
#pragma unroll
                  for (int j = 0; j < 8; ++j)
                    if (j < nq) {
                      const uint32_t w[4] = {x[ds][j].x, x[ds][j].y, x[ds][j].z, x[ds][j].w};
#pragma unroll
                      for (int e = 0; e < 4; ++e) {
                        uint32_t& acc = v[4 * j + e];
                        if (s0 + ds == 0) acc = w[e];
                        else if constexpr (KIND == KIND_I8) acc = (uint32_t)((int)acc + (int)w[e]);
                        else acc = __float_as_uint(__fadd_rn(__uint_as_float(acc), __uint_as_float(w[e])));
                      }
                    }
                }
            }
            store_chunk16<EPI>(p, *reinterpret_cast<const uint32_t(*)[16]>(&v[0]), pi_h, q_tile0 + c0, q_end, st);
            if (nq == 8)
              store_chunk16<EPI>(p, *reinterpret_cast<const uint32_t(*)[16]>(&v[16]), pi_h, q_tile0 + c0 + 16, q_end, st);
          }
            }
          }
        }
        __syncwarp();
        if (lane == 0) {
          // the last warp to leave restores the counters (nobody polls or claims any more)
          if (atomicAdd(ctr + 2, 1u) == (unsigned)(S - 1)) { ctr[0] = 0u; ctr[1] = 0u; ctr[2] = 0u; }
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  if constexpr (CLUSTER) {
    // this CTA's shared memory must outlive every peer's reads of it
    if (threadIdx.x == 0 && p.cluster_k > 1) mbar_wait_cluster(done_bar, 0u, status, MP_DEV_TIMEOUT_CLUSTER);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace mp
