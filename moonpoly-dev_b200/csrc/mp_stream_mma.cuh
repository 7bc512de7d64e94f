// Streaming GEMM for a narrow side of at most 64 rows (FP16, INT8): the wide operand W[R,K] goes
// from HBM straight into registers, already in the fragment layout of the warp-level tensor
// instruction (m16n8k16 for FP16, m16n8k32 for INT8), and is multiplied against the few rows of
// X[T,K] that sit in L1/L2.  There is no shared-memory pipeline, no TMEM and no split-K hand-off
// through global memory, so the kernel has none of the latency chains (barrier round trips,
// accumulator drain, partial-sum exchange) that bound the tcgen05 kernel when the whole problem is
// a ~5 us HBM stream.
//
//   acc[r][t] = sum_k W[r,k] * X[t,k]          (fp32 for FP16 inputs, exact int32 for INT8)
//   FP16:        out = alpha * acc + beta * out                       (fp16)
//   INT8 plain:  out = ialpha * acc + ibeta * out                     (int32)
//   INT8 scaled: out = RN16(a_s[token] * RN32(b_s[channel] * RN32(acc))) (+ bias in the output type)
//
// Work split: one CTA of 8 warps owns up to 16 rows of W at a time; warp w takes the w-th eighth
// of K for those rows, and the 8 partial 16 x T blocks are added in a fixed order through shared
// memory (deterministic).  A dot product does not care in which order k is visited as long as both
// operands agree, so a lane loads 16 contiguous bytes of its row and spreads them over the k-slots
// of two consecutive MMAs; the X fragment is loaded with the same rule.  Every load of W is a full
// 16-byte vector and the four lanes of a row cover 64 contiguous bytes.  Two optional splits multiply
// the CTAs when the rows of W cannot fill the GPU: the rows of X over neighbouring CTAs (t_split) and K
// over the CTAs of a cluster (k_split); see StreamParams.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace mp {

enum { STREAM_F16 = 0, STREAM_I8 = 1, STREAM_BF16 = 2 };
enum { STREAM_EPI_F16 = 0, STREAM_EPI_I32 = 1, STREAM_EPI_SCALED = 2 };

struct StreamParams {
  const void* W; long long ldw;       // wide operand, R rows (ld in elements)
  const void* X; long long ldx;       // narrow operand, T rows
  void* out; long long stride_r, stride_t;
  int R, T, K;                         // K * element size % 16 == 0, rows 16-byte aligned
  float alpha, beta;
  int ialpha, ibeta;
  // scaled epilogue: channel = W row when chan_on_r, else X row; the other index is the token
  const float* chan_scale; const float* tok_scale;
  int chan_scalar, tok_scalar, chan_on_r, out_bf16;
  const void* bias;                    // in the output type, indexed by channel; may be null
  // Token split: t_split > 1 gives every block of W rows to t_split neighbouring CTAs, each against its own
  // t_per rows of X (a multiple of 8).  W is then read t_split times, but the repeats hit L2 (neighbouring CTAs
  // run together), HBM still sees it once, and every CTA keeps a narrow X that stays in L1.
  int t_split, t_per;
  // K split: k_split > 1 gives every (row block, token part) to k_split consecutive CTAs -- one thread-block cluster
  // -- each streaming its own contiguous range of K; the partial 16 x T blocks meet through distributed shared
  // memory in rank order (deterministic).  For weights with so few rows that whole-K CTAs cannot keep enough loads
  // in flight to fill the HBM queue (R ~ 1024..2048: the projections of a model sharded over 4-8 GPUs).
  int k_split;
  // fused all-gather of a column-parallel Linear: the same output buffer in the memory of the other GPUs
  // (peer-mapped pointers, same strides); every result is stored there too with plain stores
  void* peer_out[7];
  int num_peers;
};

constexpr int kStreamWarps = 8;        // K is split eight ways inside a CTA
constexpr int kStreamRows = 16;        // W rows per tile (the M of the warp-level MMA)

__device__ __forceinline__ void mma_m16n8k16_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_m16n8k16_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                  uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_m16n8k32_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int EPI>
__device__ __forceinline__ void stream_finish_to(const StreamParams& p, void* out_base, uint32_t accw, int r, int t) {
  const long long off = (long long)r * p.stride_r + (long long)t * p.stride_t;
  if constexpr (EPI == STREAM_EPI_F16) {
    // 16-bit float output (fp16, or bf16 when out_bf16): RN16(alpha * acc + beta * old), then + bias in that type
    uint16_t* o = reinterpret_cast<uint16_t*>(out_base) + off;
    float v = p.alpha * __uint_as_float(accw);
    if (p.beta != 0.0f)
      v += p.beta * (p.out_bf16 ? __bfloat162float(__ushort_as_bfloat16(*o)) : __half2float(__ushort_as_half(*o)));
    uint16_t h = p.out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
    if (p.bias != nullptr) {
      const uint16_t b = reinterpret_cast<const uint16_t*>(p.bias)[p.chan_on_r ? r : t];
      if (p.out_bf16) h = __bfloat16_as_ushort(__float2bfloat16_rn(__bfloat162float(__ushort_as_bfloat16(h)) + __bfloat162float(__ushort_as_bfloat16(b))));
      else h = __half_as_ushort(__float2half_rn(__half2float(__ushort_as_half(h)) + __half2float(__ushort_as_half(b))));
    }
    *o = h;
  } else if constexpr (EPI == STREAM_EPI_I32) {
    int* o = reinterpret_cast<int*>(out_base) + off;
    int v = p.ialpha * (int)accw;
    if (p.ibeta != 0) v += p.ibeta * (*o);
    *o = v;
  } else {
    const int ch = p.chan_on_r ? r : t, tok = p.chan_on_r ? t : r;
    const float bs = p.chan_scale[p.chan_scalar ? 0 : ch];
    const float as = p.tok_scale[p.tok_scalar ? 0 : tok];
    const float t0 = __fmul_rn(__int2float_rn((int)accw), bs);
    const float t1 = __fmul_rn(as, t0);
    uint16_t h = p.out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(t1)) : __half_as_ushort(__float2half_rn(t1));
    if (p.bias != nullptr) {
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

template <int EPI>
__device__ __forceinline__ void stream_finish(const StreamParams& p, uint32_t accw, int r, int t) {
  stream_finish_to<EPI>(p, p.out, accw, r, t);
  for (int d = 0; d < p.num_peers; ++d) stream_finish_to<EPI>(p, p.peer_out[d], accw, r, t);
}

__device__ __forceinline__ uint32_t stream_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void stream_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t stream_ld_dsmem(uint32_t local_addr, uint32_t rank) {
  uint32_t remote, v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
  return v;
}

// NT = number of 8-row groups of X covered (T <= 8 * NT); UNROLL = K blocks (64 bytes of each row)
// in flight per warp; MINB = CTAs that must fit on an SM.  The grid is a whole multiple of the SM
// count whenever there are enough rows, and CTA i takes the contiguous rows [i*R/G, (i+1)*R/G):
// every SM then streams the same number of bytes (+- one row), which a fixed 16-row tiling cannot
// give.
template <int KIND, int EPI, int NT, int UNROLL, int MINB>
__global__ void __launch_bounds__(kStreamWarps * 32, MINB)
stream_mma_kernel(const StreamParams p) {
  __shared__ uint32_t red[kStreamWarps][kStreamRows][NT * 8 + 1];
  constexpr int kElt = KIND == STREAM_I8 ? 1 : 2;          // bytes per element
  constexpr int kChunkElems = 16 / kElt;                   // elements per 16-byte chunk
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  __shared__ uint32_t part[kStreamRows][NT * 8];
  const int t_split = p.t_split > 1 ? p.t_split : 1;
  const int ks = p.k_split > 1 ? p.k_split : 1;
  const int kq = (int)blockIdx.x % ks;                                 // rank in the cluster = K range
  const int bid = (int)blockIdx.x / ks, nbid = (int)gridDim.x / ks;
  const int rb = bid / t_split, nrb = nbid / t_split;
  const int t0 = (bid - rb * t_split) * p.t_per;                      // first row of X of this CTA
  const int Tl = t_split > 1 ? min(p.t_per, p.T - t0) : p.T;          // rows of X of this CTA
  const int r_begin = (int)((long long)rb * p.R / nrb);
  const int r_end = (int)((long long)(rb + 1) * p.R / nrb);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const char* Wb = reinterpret_cast<const char*>(p.W);
  const char* Xb = reinterpret_cast<const char*>(p.X) + (long long)t0 * p.ldx * (KIND == STREAM_I8 ? 1 : 2);

  // Before the previous kernel of the stream is complete nothing may be read for real, but pulling
  // this CTA's rows of W towards L2 is harmless and joins back-to-back launches into one stream.
  {
    const int row_bytes = p.K * kElt;
    const int lines_per_row = (row_bytes + 127) >> 7;
    for (int i = threadIdx.x; i < (r_end - r_begin) * lines_per_row; i += kStreamWarps * 32) {
      const int r = i / lines_per_row, l = i - r * lines_per_row;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(Wb + (long long)(r_begin + r) * p.ldw * kElt + (size_t)l * 128));
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");

  const int chunks = p.K / kChunkElems;                 // 16-byte chunks per row
  const int blocks = (chunks + 3) >> 2;                 // K blocks of 4 chunks
  const int cta_blk0 = (int)((long long)blocks * kq / ks), cta_blk1 = (int)((long long)blocks * (kq + 1) / ks);
  const int per_warp = (cta_blk1 - cta_blk0 + kStreamWarps - 1) / kStreamWarps;
  const int blk_begin = cta_blk0 + warp * per_warp;
  const int blk_end = min(cta_blk1, blk_begin + per_warp);

  const uint4* xr[NT];
  bool x_ok[NT];
#pragma unroll
  for (int nb = 0; nb < NT; ++nb) {
    x_ok[nb] = nb * 8 + g < Tl;
    xr[nb] = reinterpret_cast<const uint4*>(Xb + (long long)(nb * 8 + g) * p.ldx * kElt);
  }
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  const bool rows_contig = p.stride_r == 1;

  for (int row0 = r_begin; row0 < r_end; row0 += kStreamRows) {
    const bool row_lo_ok = row0 + g < r_end, row_hi_ok = row0 + g + 8 < r_end;
    const uint4* w_lo = reinterpret_cast<const uint4*>(Wb + (long long)(row0 + g) * p.ldw * kElt);
    const uint4* w_hi = reinterpret_cast<const uint4*>(Wb + (long long)(row0 + g + 8) * p.ldw * kElt);

    float accf[NT][4];
    int acci[NT][4];
#pragma unroll
    for (int nb = 0; nb < NT; ++nb)
#pragma unroll
      for (int i = 0; i < 4; ++i) { accf[nb][i] = 0.0f; acci[nb][i] = 0; }

    for (int b0 = blk_begin; b0 < blk_end; b0 += UNROLL) {
      uint4 lo[UNROLL], hi[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int c = (b0 + u) * 4 + t4;
        const bool ok = b0 + u < blk_end && c < chunks;
        lo[u] = ok && row_lo_ok ? __ldcs(w_lo + c) : zero4;   // streamed once: keep X in L1 instead
        hi[u] = ok && row_hi_ok ? __ldcs(w_hi + c) : zero4;
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int c = (b0 + u) * 4 + t4;
        const bool ok = b0 + u < blk_end && c < chunks;
#pragma unroll
        for (int nb = 0; nb < NT; ++nb) {
          const uint4 xv = ok && x_ok[nb] ? __ldg(xr[nb] + c) : zero4;
          if constexpr (KIND == STREAM_I8) {
            mma_m16n8k32_s8(acci[nb], lo[u].x, hi[u].x, lo[u].y, hi[u].y, xv.x, xv.y);
            mma_m16n8k32_s8(acci[nb], lo[u].z, hi[u].z, lo[u].w, hi[u].w, xv.z, xv.w);
          } else if constexpr (KIND == STREAM_BF16) {
            mma_m16n8k16_bf16(accf[nb], lo[u].x, hi[u].x, lo[u].y, hi[u].y, xv.x, xv.y);
            mma_m16n8k16_bf16(accf[nb], lo[u].z, hi[u].z, lo[u].w, hi[u].w, xv.z, xv.w);
          } else {
            mma_m16n8k16_f16(accf[nb], lo[u].x, hi[u].x, lo[u].y, hi[u].y, xv.x, xv.y);
            mma_m16n8k16_f16(accf[nb], lo[u].z, hi[u].z, lo[u].w, hi[u].w, xv.z, xv.w);
          }
        }
      }
    }

    // accumulator fragment: [0],[1] = (row g, cols 2*t4, 2*t4+1); [2],[3] = (row g+8, same cols)
    if (row0 != r_begin) __syncthreads();               // the previous tile's sums have been read
#pragma unroll
    for (int nb = 0; nb < NT; ++nb) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) w[i] = KIND == STREAM_I8 ? (uint32_t)acci[nb][i] : __float_as_uint(accf[nb][i]);
      red[warp][g][nb * 8 + 2 * t4] = w[0];
      red[warp][g][nb * 8 + 2 * t4 + 1] = w[1];
      red[warp][g + 8][nb * 8 + 2 * t4] = w[2];
      red[warp][g + 8][nb * 8 + 2 * t4 + 1] = w[3];
    }
    __syncthreads();

    // the faster-moving index of the output walks whichever of (row, narrow row) is contiguous
    for (int i = threadIdx.x; i < kStreamRows * Tl; i += kStreamWarps * 32) {
      int r, t;
      if (rows_contig) { r = i & (kStreamRows - 1); t = i >> 4; }
      else { t = i % Tl; r = i / Tl; }
      if (row0 + r >= r_end) continue;
      uint32_t accw;
      if constexpr (KIND == STREAM_I8) {
        int v = 0;
#pragma unroll
        for (int w = 0; w < kStreamWarps; ++w) v += (int)red[w][r][t];
        accw = (uint32_t)v;
      } else {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < kStreamWarps; ++w) v += __uint_as_float(red[w][r][t]);
        accw = __float_as_uint(v);
      }
      if (ks == 1) stream_finish<EPI>(p, accw, row0 + r, t0 + t);
      else part[r][t] = accw;
    }
    if (ks > 1) {
      // every K range's 16 x Tl block is in its CTA's shared memory; rank kq finishes its share of the outputs,
      // adding the ranks' partial sums in rank order
      stream_cluster_sync();
      const int n_out = kStreamRows * Tl;
      const int i_begin = n_out * kq / ks, i_end = n_out * (kq + 1) / ks;
      for (int i = i_begin + threadIdx.x; i < i_end; i += kStreamWarps * 32) {
        int r, t;
        if (rows_contig) { r = i & (kStreamRows - 1); t = i >> 4; }
        else { t = i % Tl; r = i / Tl; }
        if (row0 + r >= r_end) continue;
        const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(&part[r][t]));
        uint32_t accw;
        if constexpr (KIND == STREAM_I8) {
          int v = 0;
          for (int q = 0; q < ks; ++q) v += (int)stream_ld_dsmem(addr, (uint32_t)q);
          accw = (uint32_t)v;
        } else {
          float v = 0.0f;
          for (int q = 0; q < ks; ++q) v += __uint_as_float(stream_ld_dsmem(addr, (uint32_t)q));
          accw = __float_as_uint(v);
        }
        stream_finish<EPI>(p, accw, row0 + r, t0 + t);
      }
      stream_cluster_sync();          // the peers have read this CTA's block: it may be overwritten or go away
    }
  }
}


}  // namespace mp
