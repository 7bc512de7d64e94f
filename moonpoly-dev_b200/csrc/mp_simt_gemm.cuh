// CUDA-core GEMM tiles:  C[i + j*ldc] = alpha * sum_k A[i*lda + k] * B[j*ldb + k] + beta * C
//
// Used for (a) the FP32 path -- the reference's FP32 kernels are SIMT FFMA, not TF32
// (moonpoly/core/fp32/fp32_rcc.cu:193-2208, OpClassSimt), so exact fp32 multiply-add semantics are
// kept and no tensor core is involved -- and (b) FP16 / INT8 problems whose K or base pointers do
// not meet the 16-byte alignment TMA needs (the reference keeps pids with alignment 1/2/4 for those,
// moonpoly/core/fp16/fp16_rcc_cost.cu:32-36).
//
// A tile of TI x TJ outputs per 256-thread CTA, K walked in steps of 16 through shared memory,
// every thread owning a (TI/16) x (TJ/16) register block.  Optional parallel split-K writes raw
// partials to a workspace (grid.z = slices) and a second kernel sums them in slice order
// (the GemmSplitKParallel + ReduceSplitK arrangement of moonpoly/core/fp32/fp32_rcc.cu:136-187).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace mp {

enum { SEPI_F16 = 0, SEPI_I32 = 1, SEPI_SCALED = 2, SEPI_F32 = 3 };

struct SimtParams {
  int m, n, k;
  const void* A; const void* B; void* C;
  long long lda, ldb;                  // row pitch (elements) of A[m,k] and B[n,k]
  long long c_stride_i, c_stride_j;    // element strides of C along i (rows of A) and j (rows of B)
  float alpha, beta;
  int ialpha, ibeta;
  int split_k, k_per_slice;
  void* partials;                      // [split_k][n][m] accumulators when split_k > 1
  // scaled int8 epilogue: i = token index (a_scales), j = output channel (b_scales, bias)
  const float* a_scales; const float* b_scales;
  int a_scalar, b_scalar;
  const void* bias;
  int out_bf16;
  int bias_on_i;                       // 16-bit float GEMM with a bias: 1 = the bias index is i, 0 = j
};

template <typename T> struct SimtAcc { using type = float; };
template <> struct SimtAcc<int8_t> { using type = int; };

template <typename TIn> __device__ __forceinline__ typename SimtAcc<TIn>::type simt_cvt(TIn v);
template <> __device__ __forceinline__ float simt_cvt<float>(float v) { return v; }
template <> __device__ __forceinline__ float simt_cvt<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float simt_cvt<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ int simt_cvt<int8_t>(int8_t v) { return (int)v; }

template <int EPI, typename TAcc>
__device__ __forceinline__ void simt_finish(const SimtParams& p, TAcc acc, int i, int j) {
  const long long off = (long long)i * p.c_stride_i + (long long)j * p.c_stride_j;
  if constexpr (EPI == SEPI_F32) {
    float v = p.alpha * acc;
    float* o = reinterpret_cast<float*>(p.C) + off;
    if (p.beta != 0.0f) v += p.beta * (*o);
    *o = v;
  } else if constexpr (EPI == SEPI_F16) {
    float v = p.alpha * acc;
    uint16_t* o = reinterpret_cast<uint16_t*>(p.C) + off;
    if (p.beta != 0.0f)
      v += p.beta * (p.out_bf16 ? __bfloat162float(__ushort_as_bfloat16(*o)) : __half2float(__ushort_as_half(*o)));
    uint16_t h = p.out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
    if (p.bias != nullptr) {
      const uint16_t b = reinterpret_cast<const uint16_t*>(p.bias)[p.bias_on_i ? i : j];
      if (p.out_bf16) h = __bfloat16_as_ushort(__float2bfloat16_rn(__bfloat162float(__ushort_as_bfloat16(h)) + __bfloat162float(__ushort_as_bfloat16(b))));
      else h = __half_as_ushort(__float2half_rn(__half2float(__ushort_as_half(h)) + __half2float(__ushort_as_half(b))));
    }
    *o = h;
  } else if constexpr (EPI == SEPI_I32) {
    int v = p.ialpha * acc;
    int* o = reinterpret_cast<int*>(p.C) + off;
    if (p.ibeta != 0) v += p.ibeta * (*o);
    *o = v;
  } else {
    const float bs = p.b_scales[p.b_scalar ? 0 : j];
    const float as = p.a_scales[p.a_scalar ? 0 : i];
    const float t1 = __fmul_rn(as, __fmul_rn(__int2float_rn((int)acc), bs));
    uint16_t h;
    if (p.out_bf16) {
      h = __bfloat16_as_ushort(__float2bfloat16_rn(t1));
      if (p.bias) {
        const float s = __bfloat162float(__ushort_as_bfloat16(h)) +
                        __bfloat162float(__ushort_as_bfloat16(reinterpret_cast<const uint16_t*>(p.bias)[j]));
        h = __bfloat16_as_ushort(__float2bfloat16_rn(s));
      }
    } else {
      h = __half_as_ushort(__float2half_rn(t1));
      if (p.bias) {
        const float s = __half2float(__ushort_as_half(h)) +
                        __half2float(__ushort_as_half(reinterpret_cast<const uint16_t*>(p.bias)[j]));
        h = __half_as_ushort(__float2half_rn(s));
      }
    }
    reinterpret_cast<uint16_t*>(p.C)[off] = h;
  }
}

template <typename TIn, int EPI, int TI, int TJ>
__global__ void __launch_bounds__(256)
simt_gemm_kernel(const SimtParams p) {
  using TAcc = typename SimtAcc<TIn>::type;
  constexpr int TK = 16;
  constexpr int RI = TI / 16, RJ = TJ / 16;
  __shared__ TAcc As[TK][TI + 1];
  __shared__ TAcc Bs[TK][TJ + 1];

  const TIn* A = reinterpret_cast<const TIn*>(p.A);
  const TIn* B = reinterpret_cast<const TIn*>(p.B);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int i0 = blockIdx.x * TI, j0 = blockIdx.y * TJ;
  const int k_begin = blockIdx.z * p.k_per_slice;
  const int k_end = min(p.k, k_begin + p.k_per_slice);

  TAcc acc[RI][RJ];
#pragma unroll
  for (int a = 0; a < RI; ++a)
#pragma unroll
    for (int b = 0; b < RJ; ++b) acc[a][b] = TAcc(0);

  for (int k0 = k_begin; k0 < k_end; k0 += TK) {
    for (int e = threadIdx.x; e < TI * TK; e += 256) {
      const int r = e / TK, kk = e % TK;
      const int gi = i0 + r, gk = k0 + kk;
      As[kk][r] = (gi < p.m && gk < k_end) ? simt_cvt<TIn>(A[(long long)gi * p.lda + gk]) : TAcc(0);
    }
    for (int e = threadIdx.x; e < TJ * TK; e += 256) {
      const int r = e / TK, kk = e % TK;
      const int gj = j0 + r, gk = k0 + kk;
      Bs[kk][r] = (gj < p.n && gk < k_end) ? simt_cvt<TIn>(B[(long long)gj * p.ldb + gk]) : TAcc(0);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      TAcc av[RI], bv[RJ];
#pragma unroll
      for (int a = 0; a < RI; ++a) av[a] = As[kk][tx + 16 * a];
#pragma unroll
      for (int b = 0; b < RJ; ++b) bv[b] = Bs[kk][ty + 16 * b];
#pragma unroll
      for (int a = 0; a < RI; ++a)
#pragma unroll
        for (int b = 0; b < RJ; ++b) {
          if constexpr (sizeof(TIn) == 1) acc[a][b] += av[a] * bv[b];
          else acc[a][b] = fmaf(av[a], bv[b], acc[a][b]);
        }
    }
    __syncthreads();
  }

#pragma unroll
  for (int b = 0; b < RJ; ++b)
#pragma unroll
    for (int a = 0; a < RI; ++a) {
      const int i = i0 + tx + 16 * a, j = j0 + ty + 16 * b;
      if (i < p.m && j < p.n) {
        if (p.split_k > 1) {
          reinterpret_cast<TAcc*>(p.partials)[((size_t)blockIdx.z * p.n + j) * (size_t)p.m + i] = acc[a][b];
        } else {
          simt_finish<EPI, TAcc>(p, acc[a][b], i, j);
        }
      }
    }
}

// Sums split-K partials in slice order s = 0..S-1 and applies the epilogue.
template <typename TAcc, int EPI>
__global__ void __launch_bounds__(256)
simt_splitk_reduce_kernel(const SimtParams p) {
  const size_t total = (size_t)p.m * p.n;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (size_t)gridDim.x * blockDim.x) {
    const int j = (int)(e / p.m), i = (int)(e % p.m);
    const TAcc* src = reinterpret_cast<const TAcc*>(p.partials) + e;
    TAcc acc = src[0];
    for (int s = 1; s < p.split_k; ++s) acc += src[(size_t)s * total];
    simt_finish<EPI, TAcc>(p, acc, i, j);
  }
}

}  // namespace mp

// ------------------------------------------------------------------------------------------------
// FP32 streaming kernel for a narrow side of at most 64 rows: one warp per ROWS rows of the wide
// operand W[R,K]; the lanes read the rows once with 16-byte loads and keep one accumulator per
// (row, narrow row), the rows of X[T,K] come from L1/L2 (each X vector serves ROWS rows), and the
// 32 partial sums of each output meet in a shuffle tree.  A small FP32 problem (37 x 1024 x 1024)
// is one short wave of such warps instead of a few 64x64 tiles with a split-K pass behind them.
//   out[r * stride_r + t * stride_t] = alpha * sum_k W[r,k] * X[t,k] + beta * out[...]
// ------------------------------------------------------------------------------------------------
namespace mp {

struct SkinnyF32Params {
  const float* W; long long ldw;
  const float* X; long long ldx;
  float* out; long long stride_r, stride_t;
  int R, T, K;                          // K % 4 == 0, rows 16-byte aligned
  float alpha, beta;
};

constexpr int kSkinnyF32Warps = 4;

template <int TMAX, int ROWS>
__global__ void __launch_bounds__(kSkinnyF32Warps * 32)
skinny_f32_kernel(const SkinnyF32Params p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r0 = (blockIdx.x * kSkinnyF32Warps + warp) * ROWS;
  if (r0 >= p.R) return;
  const float4* w[ROWS];
  bool ok[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    ok[i] = r0 + i < p.R;
    w[i] = reinterpret_cast<const float4*>(p.W + (long long)(ok[i] ? r0 + i : r0) * p.ldw);
  }
  const int chunks = p.K >> 2;
  float acc[ROWS][TMAX];
#pragma unroll
  for (int i = 0; i < ROWS; ++i)
#pragma unroll
    for (int t = 0; t < TMAX; ++t) acc[i][t] = 0.0f;
  for (int c = lane; c < chunks; c += 32) {
    float4 a[ROWS];
#pragma unroll
    for (int i = 0; i < ROWS; ++i) a[i] = __ldcs(w[i] + c);
#pragma unroll
    for (int t = 0; t < TMAX; ++t) {
      if (t < p.T) {
        const float4 x = __ldg(reinterpret_cast<const float4*>(p.X + (long long)t * p.ldx) + c);
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
          acc[i][t] = fmaf(a[i].x, x.x, acc[i][t]);
          acc[i][t] = fmaf(a[i].y, x.y, acc[i][t]);
          acc[i][t] = fmaf(a[i].z, x.z, acc[i][t]);
          acc[i][t] = fmaf(a[i].w, x.w, acc[i][t]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
#pragma unroll
    for (int t = 0; t < TMAX; ++t) {
      if (t < p.T) {
        float v = acc[i][t];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (ok[i] && lane == (t & 31)) {
          float* o = p.out + (long long)(r0 + i) * p.stride_r + (long long)t * p.stride_t;
          float res = p.alpha * v;
          if (p.beta != 0.0f) res += p.beta * (*o);
          *o = res;
        }
      }
    }
  }
}

// The same computation with the narrow operand staged in shared memory: when X[T,K] fits (T * K * 4 bytes <= 200 KB,
// e.g. 37 x 1024), one CTA of 16 warps per SM copies it in once and its warps then take ROWS rows of W at a time,
// reading W straight from global memory and X from shared memory.  The plain kernel above pulls X through L1 once
// per warp; its rows lie 4 KB apart, the loads of one K chunk fall into few cache sets and most of them miss, so the
// 37 x 1024 x 1024 problem moved ~150 MB from L2 (27 us).  Staged, X crosses L2 once per SM.
constexpr int kSkinnySmemWarps = 16;

template <int TMAX, int ROWS>
__global__ void __launch_bounds__(kSkinnySmemWarps * 32, 1)
skinny_f32_smem_kernel(const SkinnyF32Params p) {
  extern __shared__ __align__(16) float xs_f32[];          // [T][K]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunks = p.K >> 2;
  // rows of this CTA: a contiguous, balanced range
  const int r_begin = (int)((long long)blockIdx.x * p.R / gridDim.x);
  const int r_end = (int)((long long)(blockIdx.x + 1) * p.R / gridDim.x);
  {
    float4* dst = reinterpret_cast<float4*>(xs_f32);
    for (int i = threadIdx.x; i < p.T * chunks; i += kSkinnySmemWarps * 32) {
      const int t = i / chunks, c = i - t * chunks;
      dst[i] = __ldg(reinterpret_cast<const float4*>(p.X + (long long)t * p.ldx) + c);
    }
  }
  __syncthreads();
  const float4* xs4 = reinterpret_cast<const float4*>(xs_f32);
  for (int r0 = r_begin + warp * ROWS; r0 < r_end; r0 += kSkinnySmemWarps * ROWS) {
    const float4* w[ROWS];
    bool ok[ROWS];
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
      ok[i] = r0 + i < r_end;
      w[i] = reinterpret_cast<const float4*>(p.W + (long long)(ok[i] ? r0 + i : r0) * p.ldw);
    }
    float acc[ROWS][TMAX];
#pragma unroll
    for (int i = 0; i < ROWS; ++i)
#pragma unroll
      for (int t = 0; t < TMAX; ++t) acc[i][t] = 0.0f;
    for (int c = lane; c < chunks; c += 32) {
      float4 a[ROWS];
#pragma unroll
      for (int i = 0; i < ROWS; ++i) a[i] = __ldcs(w[i] + c);
#pragma unroll
      for (int t = 0; t < TMAX; ++t) {
        if (t < p.T) {
          const float4 x = xs4[t * chunks + c];
#pragma unroll
          for (int i = 0; i < ROWS; ++i) {
            acc[i][t] = fmaf(a[i].x, x.x, acc[i][t]);
            acc[i][t] = fmaf(a[i].y, x.y, acc[i][t]);
            acc[i][t] = fmaf(a[i].z, x.z, acc[i][t]);
            acc[i][t] = fmaf(a[i].w, x.w, acc[i][t]);
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
#pragma unroll
      for (int t = 0; t < TMAX; ++t) {
        if (t < p.T) {
          float v = acc[i][t];
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
          if (ok[i] && lane == (t & 31)) {
            float* o = p.out + (long long)(r0 + i) * p.stride_r + (long long)t * p.stride_t;
            float res = p.alpha * v;
            if (p.beta != 0.0f) res += p.beta * (*o);
            *o = res;
          }
        }
      }
    }
  }
}

}  // namespace mp
