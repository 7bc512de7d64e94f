// Skinny FP16 GEMM for 1..8 rows on one side ("GEMV-like"): the wide operand W[R,K] is streamed
// from HBM exactly once with 16-byte vector loads, one warp per pair of W rows, while the few rows
// of the narrow operand X[T,K] (T <= 8) come from L1/L2.  Products are accumulated in fp32 and the
// lanes of a warp are combined with shuffles, so there is no shared-memory pipeline, no TMEM and
// no split-K hand-off: for these shapes the kernel is a pure HBM stream and the latency chains of
// the tensor-core kernel (barriers, accumulator drain, partial-sum exchange) are what it avoids.
//
//   out[r * stride_r + t * stride_t] = alpha * sum_k W[r,k] * X[t,k] + beta * out[...]
//
// Serves both mappings of the row-column-column contract: the direct one (few rows of A against
// the rows of B: W = B, X = A) and the Linear one (weight rows in A, few token rows in B).
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace mp {

struct GemvParams {
  const __half* W; long long ldw;     // wide operand, R rows
  const __half* X; long long ldx;     // narrow operand, T rows (T <= 8)
  __half* out; long long stride_r, stride_t;
  int R, T, K;                         // K % 8 == 0, rows 16-byte aligned
  float alpha, beta;
};

constexpr int kGemvWarps = 4;          // warps per CTA
constexpr int kGemvRowsPerWarp = 2;    // W rows a warp works on at a time
constexpr int kGemvUnroll = 8;         // 16-byte chunks of each row in flight per lane

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

template <int T>
__global__ void __launch_bounds__(kGemvWarps * 32)
gemv_f16_kernel(const GemvParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = (blockIdx.x * kGemvWarps + warp) * kGemvRowsPerWarp;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (row0 >= p.R) return;
  const int nrows = min(kGemvRowsPerWarp, p.R - row0);
  const uint4* w0 = reinterpret_cast<const uint4*>(p.W + (long long)row0 * p.ldw);
  const uint4* w1 = reinterpret_cast<const uint4*>(p.W + (long long)(row0 + (nrows > 1 ? 1 : 0)) * p.ldw);
  // These CTAs are small enough to become resident while the previous kernel of the stream still
  // runs.  Until that kernel is complete nothing may be read for real (it may be producing W or X),
  // but pulling this warp's rows of W towards L2 is harmless -- L2 is the point of coherence -- and
  // turns back-to-back launches into one continuous HBM stream.
  {
    const char* b0 = reinterpret_cast<const char*>(w0);
    const char* b1 = reinterpret_cast<const char*>(w1);
    const int row_bytes = p.K * 2;
    for (int off = lane * 128; off < row_bytes; off += 32 * 128) {
      asm volatile("prefetch.global.L2 [%0];" ::"l"(b0 + off));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(b1 + off));
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int chunks = p.K >> 3;                      // 16-byte chunks per row

  // acc[t] = (partial sum for row0, partial sum for row0 + 1): both rows share every X value, so one
  // packed fp32 FMA (two independent IEEE fp32 FMAs in one instruction) advances both
  float2 acc[T];
#pragma unroll
  for (int t = 0; t < T; ++t) acc[t] = make_float2(0.0f, 0.0f);

  // lane l takes chunks l, l+32, l+64, ...: a warp reads 512 contiguous bytes of a row per step
  for (int c0 = lane; c0 < chunks; c0 += 32 * kGemvUnroll) {
    uint4 a[kGemvUnroll], b[kGemvUnroll];
#pragma unroll
    for (int u = 0; u < kGemvUnroll; ++u) {
      const int c = c0 + 32 * u;
      if (c < chunks) {
        // streamed once: do not let W displace X in L1
        a[u] = __ldcs(w0 + c);
        b[u] = __ldcs(w1 + c);
      }
    }
#pragma unroll
    for (int u = 0; u < kGemvUnroll; ++u) {
      const int c = c0 + 32 * u;
      if (c < chunks) {
        float fa[8], fb[8];
        unpack8(a[u], fa);
        unpack8(b[u], fb);
#pragma unroll
        for (int t = 0; t < T; ++t) {
          const uint4 xv = __ldg(reinterpret_cast<const uint4*>(p.X + (long long)t * p.ldx) + c);
          float fx[8];
          unpack8(xv, fx);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            acc[t] = __ffma2_rn(make_float2(fa[i], fb[i]), make_float2(fx[i], fx[i]), acc[t]);
        }
      }
    }
  }

#pragma unroll
  for (int t = 0; t < T; ++t) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      acc[t].x += __shfl_xor_sync(0xffffffffu, acc[t].x, off);
      acc[t].y += __shfl_xor_sync(0xffffffffu, acc[t].y, off);
    }
  }

  // lane (r * T + t) writes output (r, t)
  if (lane < nrows * T) {
    const int r = lane / T, t = lane - r * T;
    float v = 0.0f;
#pragma unroll
    for (int tt = 0; tt < T; ++tt)
      if (tt == t) v = r == 0 ? acc[tt].x : acc[tt].y;
    __half* o = p.out + (long long)(row0 + r) * p.stride_r + (long long)t * p.stride_t;
    v *= p.alpha;
    if (p.beta != 0.0f) v += p.beta * __half2float(*o);
    *o = __float2half_rn(v);
  }
}

}  // namespace mp
