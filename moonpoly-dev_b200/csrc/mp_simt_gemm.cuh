// CUDA-core GEMM tiles:  C[i + j*ldc] = alpha * sum_k A[i*lda + k] * B[j*ldb + k] + beta * C
//
// Used for (a) the FP32 path -- the reference's FP32 kernels are SIMT FFMA, not TF32
// (moonpoly/core/fp32/fp32_rcc.cu:193-2208, OpClassSimt), so exact fp32 multiply-add semantics are
// kept and no tensor core is involved -- and (b) FP16 / INT8 problems whose K or base pointers do
// not meet the 16-byte alignment TMA needs, when no padded copy of the operands can be made (the
// reference keeps pids with alignment 1/2/4 for those, moonpoly/core/fp16/fp16_rcc_cost.cu:32-36).
//
// Kernels in this file:
//   simt_gemm_kernel    the plain tile: TI x TJ outputs per 256-thread CTA, K walked in steps of 16 through
//                       shared memory, every thread owning a (TI/16) x (TJ/16) register block; any type, any
//                       alignment
//   sgemm_f32_kernel    FP32 tiles of 64 / 128 on 16-byte aligned rows, built for throughput
//   gemv_f32_kernel     FP32, at most 8 rows on the narrow side: a streaming kernel
//   tile_f32_kernel     FP32, 9..64 rows on the narrow side: square-ish tiles, K split over a cluster
// Optional parallel split-K of the tile kernels writes raw partials to a workspace (grid.z = slices) and
// simt_splitk_reduce_kernel sums them in slice order (the GemmSplitKParallel + ReduceSplitK arrangement of
// moonpoly/core/fp32/fp32_rcc.cu:136-187).
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

// FP32 tile kernel for operands whose rows are 16-byte aligned (lda, ldb multiples of 4, aligned bases): the same
// computation as simt_gemm_kernel<float, SEPI_F32, RI*TX, RJ*TY> with every sum formed in the same order (ascending
// k, one fused multiply-add per term), built for throughput.  Global loads are 16 bytes along K, stored transposed
// into shared memory ([k][row], conflict-free), the next K step of 16 is fetched into registers while the current
// one is multiplied (two shared-memory buffers, one barrier per step), a thread owns 4 x 4 or 8 x 8 outputs as groups
// of four neighbouring rows x groups of four neighbouring columns so that both operands arrive as 16-byte
// shared-memory reads,
// and the products go through packed FP32 FMAs (two neighbouring rows per instruction).
template <int TX, int TY, int RI, int RJ>
__global__ void __launch_bounds__(TX * TY)
sgemm_f32_kernel(const SimtParams p) {
  // TX x TY threads with RI x RJ outputs each.  Measured per K step of 16 on one CTA per SM: a 64 x 64 tile as 256
  // threads of 4 x 4 outputs 1.0 us (bound by its shared-memory reads: two 16-byte reads per 8 packed FMAs), as 64
  // threads of 8 x 8 1.3 us (two warps cannot hide the global loads); 128 x 64 as 128 threads of 8 x 8 is 9 % faster
  // than as 256 threads of 8 x 4.  The launch picks 256 x (4 x 4), 128 x (8 x 8) and 256 x (8 x 8).
  constexpr int TK = 16, NT = TX * TY, TI = RI * TX, TJ = RJ * TY, HI = 4 * TX, HJ = 4 * TY;
  constexpr int NA = TI * 4 / NT, NB = TJ * 4 / NT;             // 16-byte global loads per thread and K step
  static_assert((TX == 8 || TX == 16) && (TY == 8 || TY == 16) && (RI == 4 || RI == 8) && (RJ == 4 || RJ == 8) &&
                NA >= 1 && NB >= 1, "tiles of 64 or 128");
  __shared__ __align__(16) float As[2][TK][TI];
  __shared__ __align__(16) float Bs[2][TK][TJ];
  const float* A = reinterpret_cast<const float*>(p.A);
  const float* B = reinterpret_cast<const float*>(p.B);
  const int t = threadIdx.x, tx = t % TX, ty = t / TX;
  const int i0 = blockIdx.x * TI, j0 = blockIdx.y * TJ;
  const int k_begin = blockIdx.z * p.k_per_slice;
  const int k_end = min(p.k, k_begin + p.k_per_slice);

  float4 ra[NA], rb[NB];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int u = 0; u < NA; ++u) {
      const int f = t + NT * u, row = f % TI, kq = f / TI;
      const int gi = i0 + row, gk = k0 + kq * 4;
      float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (gi < p.m) {
        const float* src = A + (long long)gi * p.lda + gk;
        if (gk + 3 < k_end) v = __ldg(reinterpret_cast<const float4*>(src));
        else {
          if (gk < k_end) v.x = __ldg(src);
          if (gk + 1 < k_end) v.y = __ldg(src + 1);
          if (gk + 2 < k_end) v.z = __ldg(src + 2);
        }
      }
      ra[u] = v;
    }
#pragma unroll
    for (int u = 0; u < NB; ++u) {
      const int f = t + NT * u, row = f % TJ, kq = f / TJ;
      const int gj = j0 + row, gk = k0 + kq * 4;
      float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (gj < p.n) {
        const float* src = B + (long long)gj * p.ldb + gk;
        if (gk + 3 < k_end) v = __ldg(reinterpret_cast<const float4*>(src));
        else {
          if (gk < k_end) v.x = __ldg(src);
          if (gk + 1 < k_end) v.y = __ldg(src + 1);
          if (gk + 2 < k_end) v.z = __ldg(src + 2);
        }
      }
      rb[u] = v;
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int u = 0; u < NA; ++u) {
      const int f = t + NT * u, row = f % TI, kq = f / TI;
      As[buf][kq * 4 + 0][row] = ra[u].x; As[buf][kq * 4 + 1][row] = ra[u].y;
      As[buf][kq * 4 + 2][row] = ra[u].z; As[buf][kq * 4 + 3][row] = ra[u].w;
    }
#pragma unroll
    for (int u = 0; u < NB; ++u) {
      const int f = t + NT * u, row = f % TJ, kq = f / TJ;
      Bs[buf][kq * 4 + 0][row] = rb[u].x; Bs[buf][kq * 4 + 1][row] = rb[u].y;
      Bs[buf][kq * 4 + 2][row] = rb[u].z; Bs[buf][kq * 4 + 3][row] = rb[u].w;
    }
  };

  float2 acc[RI / 2][RJ];
#pragma unroll
  for (int a = 0; a < RI / 2; ++a)
#pragma unroll
    for (int b = 0; b < RJ; ++b) acc[a][b] = make_float2(0.0f, 0.0f);

  int cur = 0;
  if (k_begin < k_end) {
    fetch(k_begin);
    stash(0);
  }
  __syncthreads();
  for (int k0 = k_begin; k0 < k_end; k0 += TK) {
    const bool more = k0 + TK < k_end;
    if (more) fetch(k0 + TK);
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float2 a2[RI / 2];
      float bv[RJ];
#pragma unroll
      for (int h = 0; h < RI / 4; ++h) {
        const float4 v = *reinterpret_cast<const float4*>(&As[cur][kk][HI * h + 4 * tx]);
        a2[2 * h] = make_float2(v.x, v.y);
        a2[2 * h + 1] = make_float2(v.z, v.w);
      }
#pragma unroll
      for (int h = 0; h < RJ / 4; ++h) {
        const float4 v = *reinterpret_cast<const float4*>(&Bs[cur][kk][HJ * h + 4 * ty]);
        bv[4 * h] = v.x; bv[4 * h + 1] = v.y; bv[4 * h + 2] = v.z; bv[4 * h + 3] = v.w;
      }
#pragma unroll
      for (int b = 0; b < RJ; ++b) {
        const float2 bb = make_float2(bv[b], bv[b]);
#pragma unroll
        for (int a = 0; a < RI / 2; ++a) acc[a][b] = __ffma2_rn(a2[a], bb, acc[a][b]);
      }
    }
    if (more) stash(cur ^ 1);
    __syncthreads();
    cur ^= 1;
  }

  // thread's rows: i0 + HI*h + 4*tx + e; columns: j0 + HJ*h + 4*ty + e
  const bool vec_out = p.split_k > 1 ? (p.m % 4 == 0)
                                     : (p.c_stride_i == 1 && p.c_stride_j % 4 == 0 &&
                                        (reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
#pragma unroll
  for (int b = 0; b < RJ; ++b) {
    const int j = j0 + HJ * (b / 4) + 4 * ty + (b & 3);
    if (j >= p.n) continue;
#pragma unroll
    for (int h = 0; h < RI / 4; ++h) {
      const int i = i0 + HI * h + 4 * tx;
      if (i >= p.m) continue;
      const float v[4] = {acc[2 * h][b].x, acc[2 * h][b].y, acc[2 * h + 1][b].x, acc[2 * h + 1][b].y};
      if (p.split_k > 1) {
        float* dst = reinterpret_cast<float*>(p.partials) + ((size_t)blockIdx.z * p.n + j) * (size_t)p.m + i;
        if (vec_out && i + 3 < p.m) *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        else
          for (int e = 0; e < 4 && i + e < p.m; ++e) dst[e] = v[e];
      } else if (vec_out && i + 3 < p.m) {
        float* dst = reinterpret_cast<float*>(p.C) + (long long)i + (long long)j * p.c_stride_j;
        float4 o = make_float4(p.alpha * v[0], p.alpha * v[1], p.alpha * v[2], p.alpha * v[3]);
        if (p.beta != 0.0f) {
          const float4 old = *reinterpret_cast<const float4*>(dst);
          o.x += p.beta * old.x; o.y += p.beta * old.y; o.z += p.beta * old.z; o.w += p.beta * old.w;
        }
        *reinterpret_cast<float4*>(dst) = o;
      } else {
        for (int e = 0; e < 4 && i + e < p.m; ++e) simt_finish<SEPI_F32, float>(p, v[e], i + e, j);
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
// FP32 streaming kernel for a narrow side of at most 8 rows of X[T,K] against the rows of the wide operand W[R,K].
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

constexpr int kGemvF32Warps = 8;

// A CTA of 8 warps owns ROWS rows of W; warp w owns the w-th eighth of K and keeps ROWS * UNROLL 16-byte loads of W
// in flight per lane (the same arrangement that lets the FP16 streaming kernel fill the HBM queue), X comes from
// L1/L2 (every X vector serves ROWS rows), the lanes' partial sums meet in a shuffle tree and the eight warps' in
// shared memory, in warp order.  T <= 8.
template <int ROWS, int UNROLL>
__global__ void __launch_bounds__(kGemvF32Warps * 32)
gemv_f32_kernel(const SkinnyF32Params p) {
  __shared__ float red[kGemvF32Warps][ROWS][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r0 = blockIdx.x * ROWS;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const float4* w[ROWS];
  bool ok[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    ok[i] = r0 + i < p.R;
    w[i] = reinterpret_cast<const float4*>(p.W + (long long)(ok[i] ? r0 + i : r0) * p.ldw);
  }
  const int chunks = p.K >> 2;
  const int per_warp = (chunks + kGemvF32Warps - 1) / kGemvF32Warps;
  const int c_begin = warp * per_warp, c_end = min(chunks, c_begin + per_warp);
  float acc[ROWS][8];
#pragma unroll
  for (int i = 0; i < ROWS; ++i)
#pragma unroll
    for (int t = 0; t < 8; ++t) acc[i][t] = 0.0f;
  asm volatile("griddepcontrol.wait;" ::: "memory");          // the previous kernel of the stream may produce W or X
  const float4 zero4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (int c0 = c_begin + lane; c0 < c_end; c0 += 32 * UNROLL) {
    float4 a[ROWS][UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int i = 0; i < ROWS; ++i) a[i][u] = (c0 + 32 * u < c_end && ok[i]) ? __ldcs(w[i] + c0 + 32 * u) : zero4;
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int c = c0 + 32 * u;
      if (c < c_end) {
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          if (t < p.T) {
            const float4 x = __ldg(reinterpret_cast<const float4*>(p.X + (long long)t * p.ldx) + c);
#pragma unroll
            for (int i = 0; i < ROWS; ++i) {
              acc[i][t] = fmaf(a[i][u].x, x.x, acc[i][t]);
              acc[i][t] = fmaf(a[i][u].y, x.y, acc[i][t]);
              acc[i][t] = fmaf(a[i][u].z, x.z, acc[i][t]);
              acc[i][t] = fmaf(a[i][u].w, x.w, acc[i][t]);
            }
          }
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < ROWS; ++i)
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      if (t < p.T) {
        float v = acc[i][t];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0) red[warp][i][t] = v;
      }
    }
  __syncthreads();
  if (threadIdx.x < ROWS * 8) {
    const int i = threadIdx.x >> 3, t = threadIdx.x & 7;
    if (t < p.T && r0 + i < p.R) {
      float v = red[0][i][t];
#pragma unroll
      for (int q = 1; q < kGemvF32Warps; ++q) v += red[q][i][t];
      float* o = p.out + (long long)(r0 + i) * p.stride_r + (long long)t * p.stride_t;
      float res = p.alpha * v;
      if (p.beta != 0.0f) res += p.beta * (*o);
      *o = res;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// FP32 tile kernel for a narrow side of 9..64 rows and a wide side too short to fill the GPU with one warp per row
// pair (37 x 1024 x 1024).  What bounds such a problem is the rate at which one SM pulls operands out of L2 (about
// 100 GB/s), so a CTA takes a tile that is as square as the shape allows -- RH*4*RI rows of W against all T rows of
// X -- over one K part, and the K parts of a row block are the CTAs of one cluster (cluster dims (1, gridDim.y, 1)).
// Operands arrive in K chunks of 128 floats through a four-slot cp.async ring (coalesced 16-byte copies, zero-filled
// past the edges), so a CTA with at most four chunks has all of its input in flight at once.  Inside a chunk the
// eight warps form RH row halves x 8/RH K lanes; the lanes of a warp form a 4 x 8 grid over (rows, narrow rows) with
// an RI x TJ register tile each, accumulated with packed FP32 FMAs (even and odd k in the two halves of a pair), so
// one 16-byte shared-memory read feeds 2*TJ (W) or 2*RI (X) packed FMAs.  The pitch of 132 floats puts the eight X
// rows of a quarter-warp on different banks; the W address is the same across a quarter-warp (broadcast).  The
// K lanes' partial sums meet in shared memory in lane order; with gridDim.y > 1 every CTA leaves its sums in its own
// shared memory and each rank adds its share of the outputs over the ranks, in rank order, through distributed
// shared memory -- the result does not depend on timing.
// ------------------------------------------------------------------------------------------------
constexpr int kTileF32Threads = 256;
constexpr int kTileF32KC = 128;
constexpr int kTileF32Pitch = kTileF32KC + 4;
constexpr int kTileF32Stages = 4;

__device__ __forceinline__ void f32t_cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;          // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void f32t_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void f32t_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ float f32t_ld_cluster(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}
__device__ __forceinline__ void f32t_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int RH, int RI, int TJ>
constexpr int tile_f32_smem_bytes() { return kTileF32Stages * (RH * 4 * RI + 8 * TJ) * kTileF32Pitch * 4; }

template <int RH, int RI, int TJ>
__global__ void __launch_bounds__(kTileF32Threads)
tile_f32_kernel(const SkinnyF32Params p) {
  extern __shared__ __align__(16) float tf_smem[];
  constexpr int KC = kTileF32KC, PITCH = kTileF32Pitch, NS = kTileF32Stages;
  constexpr int KW = 8 / RH;                                  // K lanes (warps) per row half
  constexpr int ROWS = RH * 4 * RI, TT = 8 * TJ, LINES = ROWS + TT, STAGE = LINES * PITCH, OUTS = ROWS * TT;
  static_assert((KW + 1) * OUTS <= NS * STAGE, "the reduction area reuses the staging ring");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rg = lane >> 3, tg = lane & 7;
  const int half = warp / KW, kw = warp % KW;
  const int r_base = blockIdx.x * ROWS;
  const int ks = (int)gridDim.y, rank = (int)blockIdx.y;
  const int chunks_total = (p.K + KC - 1) / KC;
  const int c_begin = (int)((long long)rank * chunks_total / ks);
  const int n_chunks = (int)((long long)(rank + 1) * chunks_total / ks) - c_begin;

  // one warp copies one 512-byte line piece per instruction
  auto stage = [&](int ci, int slot) {
    const int k = (c_begin + ci) * KC + lane * 4;
    const bool k_ok = k < p.K;
    float* base = tf_smem + slot * STAGE + lane * 4;
    for (int line = warp; line < LINES; line += kTileF32Threads / 32) {
      const float* src;
      bool valid;
      if (line < ROWS) {
        const int r = r_base + line;
        valid = k_ok && r < p.R;
        src = p.W + (valid ? (long long)r * p.ldw + k : 0);
      } else {
        const int t = line - ROWS;
        valid = k_ok && t < p.T;
        src = p.X + (valid ? (long long)t * p.ldx + k : 0);
      }
      f32t_cp_async16(static_cast<uint32_t>(__cvta_generic_to_shared(base + line * PITCH)), src, valid);
    }
  };

  float2 acc[RI][TJ];
#pragma unroll
  for (int i = 0; i < RI; ++i)
#pragma unroll
    for (int j = 0; j < TJ; ++j) acc[i][j] = make_float2(0.0f, 0.0f);

  asm volatile("griddepcontrol.wait;" ::: "memory");          // the previous kernel of the stream may produce W or X
#pragma unroll
  for (int s = 0; s < NS - 1; ++s) {
    if (s < n_chunks) stage(s, s);
    f32t_cp_async_commit();
  }
  for (int c = 0; c < n_chunks; ++c) {
    f32t_cp_async_wait<NS - 2>();          // chunk c has landed (this thread's copies) ...
    __syncthreads();                       // ... everyone's; and everyone is done with the slot refilled below
    if (c + NS - 1 < n_chunks) stage(c + NS - 1, (c + NS - 1) % NS);
    f32t_cp_async_commit();
    const float* wb = tf_smem + (c % NS) * STAGE + (half * 4 * RI + rg) * PITCH;
    const float* xb = tf_smem + (c % NS) * STAGE + (ROWS + tg) * PITCH;
#pragma unroll 2
    for (int s = 0; s < KC / 4 / KW; ++s) {
      const int f4 = (kw + KW * s) * 4;
      float4 a[RI], x[TJ];
#pragma unroll
      for (int i = 0; i < RI; ++i) a[i] = *reinterpret_cast<const float4*>(wb + 4 * i * PITCH + f4);
#pragma unroll
      for (int j = 0; j < TJ; ++j) x[j] = *reinterpret_cast<const float4*>(xb + 8 * j * PITCH + f4);
#pragma unroll
      for (int i = 0; i < RI; ++i)
#pragma unroll
        for (int j = 0; j < TJ; ++j) {
          acc[i][j] = __ffma2_rn(make_float2(a[i].x, a[i].y), make_float2(x[j].x, x[j].y), acc[i][j]);
          acc[i][j] = __ffma2_rn(make_float2(a[i].z, a[i].w), make_float2(x[j].z, x[j].w), acc[i][j]);
        }
    }
  }
  f32t_cp_async_wait<0>();
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __syncthreads();                         // the ring is free: it becomes the reduction area

  // partial sums of the K lanes -> red[kw][row * TT + t]; summed in lane order into part[]
  float* red = tf_smem;
  float* part = tf_smem + KW * OUTS;
#pragma unroll
  for (int i = 0; i < RI; ++i)
#pragma unroll
    for (int j = 0; j < TJ; ++j)
      red[kw * OUTS + (half * 4 * RI + rg + 4 * i) * TT + tg + 8 * j] = acc[i][j].x + acc[i][j].y;
  __syncthreads();
  for (int o = threadIdx.x; o < OUTS; o += kTileF32Threads) {
    float v = red[o];
#pragma unroll
    for (int w = 1; w < KW; ++w) v += red[w * OUTS + o];
    part[o] = v;
  }
  if (ks > 1) f32t_cluster_sync();        // every rank's part[] is complete and visible in the cluster
  else __syncthreads();
  {
    // rank q finishes outputs [q * OUTS / ks, (q + 1) * OUTS / ks)
    const int o_begin = rank * OUTS / ks, o_end = (rank + 1) * OUTS / ks;
    const uint32_t part_addr = static_cast<uint32_t>(__cvta_generic_to_shared(part));
    for (int o = o_begin + threadIdx.x; o < o_end; o += kTileF32Threads) {
      const int row = r_base + o / TT, t = o % TT;
      float v = 0.0f;
      if (ks > 1) {
        for (int q = 0; q < ks; ++q) v += f32t_ld_cluster(part_addr + 4u * o, (uint32_t)q);
      } else {
        v = part[o];
      }
      if (row < p.R && t < p.T) {
        float* dst = p.out + (long long)row * p.stride_r + (long long)t * p.stride_t;
        float res = p.alpha * v;
        if (p.beta != 0.0f) res += p.beta * (*dst);
        *dst = res;
      }
    }
  }
  if (ks > 1) f32t_cluster_sync();        // a CTA's shared memory stays alive until its peers have read it
}

}  // namespace mp
