/*
 * C ABI of libmoonpoly_gemm.so -- the B200 (sm_100a) implementation of MoonPoly's
 * row-column-column GEMM path.  Plain C: PODs, raw device pointers, sizes, an opaque stream
 * handle (a cudaStream_t passed as void*; NULL = the legacy default stream).  No C++ or torch
 * types cross this boundary.  Every function returns an mp_status (0 = success) and never
 * throws, prints or exits; mp_last_error_string() describes the calling thread's last failure.
 *
 * "RCC" everywhere: A row-major [m,k] (lda = k), B column-major [k,n] (stored [n,k], ldb = k),
 * C column-major [m,n] (ldc = m).  All data pointers are DEVICE pointers owned by the caller;
 * calls are asynchronous on `stream`.  The library has no CPU fallback: without a CUDA device of
 * compute capability 10.0 every compute entry point fails with MP_ERR_CUDA / MP_ERR_UNSUPPORTED.
 *
 * Each entry point names the reference interface (file:line in skwmw01/MoonPoly-dev) it stands for.
 */
#ifndef MOONPOLY_ABI_H_
#define MOONPOLY_ABI_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum mp_status {
  MP_OK = 0,
  MP_ERR_INVALID_ARG = 1,   /* null pointer, negative size, bad enum value, bad split_n ...      */
  MP_ERR_LAYOUT = 2,        /* layout other than (A row, B col, C col)                            */
  MP_ERR_UNALIGNED_K = 3,   /* k % alignment(pid) != 0; nothing was computed                      */
  MP_ERR_BAD_PID = 4,       /* pid has no kernel                                                  */
  MP_ERR_WORKSPACE = 5,     /* caller workspace null or too small                                 */
  MP_ERR_CUDA = 6,          /* a CUDA runtime/driver call failed                                  */
  MP_ERR_DEVICE = 7,        /* a kernel recorded an error (bounded wait expired ...)              */
  MP_ERR_UNSUPPORTED = 8    /* device is not sm_100 / dtype not served                            */
} mp_status;

/* Values of moonpoly::MoonpolyDataType (moonpoly/include/moonpoly.cuh:20-24).  MP_BF16 has no counterpart there
 * (the reference removed its BF16 core GEMM, moonpoly/core/moonpoly_gemm.cu:74-77); mp_linear_bias accepts it. */
enum { MP_FP16 = 0, MP_INT8 = 1, MP_FP32 = 2, MP_BF16 = 3 };

/* Values of moonpoly::Fp16PolyPattern (moonpoly/include/moonpoly.cuh:33-37). */
enum { MP_PATTERN_SINGLE = 1, MP_PATTERN_COMBINE = 2, MP_PATTERN_SPLITK = 3 };

/* Same fields and order as moonpoly::Fp16OnlinePlan (moonpoly/include/moonpoly.cuh:39-45). */
typedef struct mp_plan {
  int pattern;
  int pid;
  int split_k;
  int split_n;
  float estimated_ms;
} mp_plan;

/* moonpoly::moonpoly_gemm (moonpoly/core/moonpoly_gemm.cu:7-39): dtype switch + layout check
 * (core/fp16/fp16_dispatch.cu:11-27 and siblings).  For MP_INT8 alpha/beta are truncated to int
 * and C is int32.  Layout other than (0,1,1) -> MP_ERR_LAYOUT; unknown dtype -> MP_ERR_INVALID_ARG. */
int mp_gemm(int dtype, int m, int n, int k, const void* A, int a_col_major, const void* B,
            int b_col_major, void* C, int c_col_major, float alpha, float beta, void* stream);

/* moonpoly::moonpolyLinear (moonpoly/core/moonpoly_gemm.cu:41-44): Y[M,N] = X[M,K] * W[N,K]^T,
 * all row-major; remapped to RCC (m = N, n = M, A = W, B = X), alpha = 1, beta = 0. */
int mp_linear(int dtype, int M, int N, int K, const void* X, const void* W, void* Y, void* stream);

/* Linear with the bias add fused into the GEMM's epilogue, FP16 or BF16 (no counterpart in the reference, whose
 * callers add the bias with a second kernel: integrations/vllm/v0.10.0/moonpoly_linear.patch:700-712, and whose
 * core GEMM refuses BF16).  Y[M,N] = X[M,K] * W[N,K]^T (+ bias[N]), all row-major, operands and output of `dtype`
 * (MP_FP16 or MP_BF16), fp32 accumulation.  The result is rounded to the output type first and the bias is then
 * added in the output type -- bit-identical to the two-step `linear` followed by `+ bias`.  bias may be NULL. */
int mp_linear_bias(int dtype, int M, int N, int K, const void* X, const void* W, const void* bias, void* Y, void* stream);

/* run_moonpoly_gemm_{fp16,fp32,int8}_row_col_col (core/fp16/fp16_rcc.cu:3263-3269,
 * core/fp32/fp32_rcc.cu:2272-2282, core/int8/i8_rcc.cu:3143-3157): online selector, then the
 * chosen pattern/pid in one launch. */
int mp_gemm_rcc(int dtype, int m, int n, int k, const void* A, const void* B, void* C, float alpha,
                float beta, void* stream);

/* run_moonpoly_selected_gemm_*_row_col_col[_with_workspace] (core/fp16/fp16_rcc.cu:3271-3295,
 * 3454-3514; core/fp32/fp32_rcc.cu:2284-2299; core/int8/i8_rcc.cu:3159-3169): forced pid with a
 * run-time split-K factor (split_k <= 0 means 2, as everywhere in the reference).  `workspace` may
 * be NULL: the library then uses its own per-stream scratch.  A non-NULL workspace must hold
 * mp_workspace_size() bytes; it needs no initialisation by the caller.
 * k % alignment(pid) != 0 -> MP_ERR_UNALIGNED_K and C is untouched (the reference prints a
 * message and returns without computing). */
int mp_gemm_rcc_pid(int dtype, int pid, int split_k, int m, int n, int k, const void* A,
                    const void* B, void* C, float alpha, float beta, void* workspace,
                    size_t workspace_bytes, void* stream);

/* No counterpart in the reference.  Same contract as mp_gemm_rcc_pid, for callers that must not
 * allocate device memory while they run: an inference server that commits the whole GPU to its
 * weights and KV cache at start-up and treats any later allocation as a bug (it could fail, or
 * stall every stream while the driver maps memory), or a plug-in that lives inside another
 * runtime's memory budget and is not allowed to call cudaMalloc at all.  mp_gemm_rcc_pid with a
 * NULL workspace grows a per-stream scratch on demand; this entry point instead keeps the split-K
 * scratch in an 8 MiB array that is part of the library image on every GPU that loads it.
 *   - It calls no cudaMalloc / cudaFree and nothing else that allocates.
 *   - Problems whose scratch need (mp_workspace_size) exceeds 8 MiB are refused with
 *     MP_ERR_WORKSPACE and a message naming both sizes; nothing is computed.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress);
 *     make that first call before any stream capture begins.
 *   - All calls on a device share the one array, which still holds the previous call's data; the
 *     words that must start at zero are cleared on `stream` before each launch.  Two calls that
 *     overlap on the GPU (different streams) race on it: keep them on one stream or order them. */
int mp_gemm_rcc_pid_static_scratch(int dtype, int pid, int split_k, int m, int n, int k,
                                   const void* A, const void* B, void* C, float alpha, float beta,
                                   void* stream);

/* Tuning entry (no counterpart in the reference, whose tiles are fixed at compile time by its
 * CUTLASS template instantiations): run the FP16 / INT8 tensor-core kernel on an RCC problem with
 * an explicit tile instead of a pid.  orient 0 puts the rows of A on the 128-row UMMA-M side and
 * tiles n by bn; orient 1 puts the rows of B there and tiles m by bn.  bn: multiple of 16 in
 * [16,256].  kc: K blocks (of 128 bytes) per pipeline stage, 1, 2 or 4; 0 lets the library choose.
 * orient 2 and 3 select the streaming kernels instead (2: FP16 CUDA-core, narrow side <= 8 rows;
 * 3: FP16 / INT8 warp-MMA, narrow side <= 64 rows); bn is ignored there, for orient 3 kc = -1, -2,
 * -4, -8 forces that many K parts per cluster and split_k > 1 that many token parts (0 / 1: the
 * library's rules), and MP_ERR_INVALID_ARG is returned when the problem does not fit the kernel.
 * orient 4 and 5 are orient 0 and 1 with 256-row tiles (two 128-row halves share every bn-wide
 * tile of the other operand).
 * The refit tool (per-tile k_iter sweeps) and the tests use it. */
int mp_gemm_rcc_tile(int dtype, int orient, int bn, int kc, int split_k, int m, int n, int k,
                     const void* A, const void* B, void* C, float alpha, float beta, void* stream);

/* Test aid (no counterpart in the reference; needs no GPU): the device-side work schedule of the
 * tensor-core kernel for an RCC problem and an explicit tile, as the kernel's roles walk it.  Every
 * work unit yields 8 ints in `units` (room for `capacity` units): CTA, tile, tile row, tile column,
 * first K block, one past the last K block, slice index, slices of the tile.  `count` receives the
 * number of units; `info` (8 ints, may be NULL): grid, tiles, K blocks, scratch slices per tile,
 * tiles in the stream-K head, 128-row halves per tile, helpers allowed, split_k.  The SM count is
 * the one the cost model uses (148 unless a device has been queried). */
int mp_debug_schedule(int dtype, int orient, int bn, int kc, int split_k, int m, int n, int k,
                      int* units, int capacity, int* count, int* info);

/* Test aid (no counterpart in the reference; needs no GPU): the growth rule of the library's own
 * per-stream split-K scratch.  The buffer holds a counter area (`have_counter_bytes`, fixed when the
 * buffer was created) followed by the partial sums; returns 1 when a call that wants
 * `want_counter_bytes` of counters and `partial_bytes` of partials does not fit `have_bytes`. */
int mp_debug_scratch_must_grow(size_t have_bytes, size_t have_counter_bytes, size_t want_counter_bytes,
                               size_t partial_bytes);

/* Test aids (no counterpart in the reference; need no GPU): the launch shape the library's rules give the
 * streaming warp-MMA kernel for an FP16 / INT8 problem with min(m, n) <= 64 -- out = {CTAs along the rows of the
 * wide operand, K parts per cluster, token parts, grid size} -- and the FP32 tile kernel for a problem with
 * 9 <= min(m, n) <= 64 -- out = {rows per CTA, K parts per cluster, grid size}. */
int mp_debug_stream_launch(int dtype, int m, int n, int k, int out[4]);
int mp_debug_f32_tile_launch(int m, int n, int k, int out[3]);

/* get_gemm_workspace_size_fp16_row_col_col (core/fp16/fp16_rcc.cu:3306-3316), extended to every
 * pid and dtype: bytes of scratch mp_gemm_rcc_pid needs for this problem (0 when split_k == 1). */
int mp_workspace_size(int dtype, int pid, int m, int n, int k, int split_k, size_t* bytes);

/* select_fp16_online_plan_row_col_col (core/fp16/fp16_rcc.cu:3220-3222 -> 423-505),
 * select_fp32_online_plan (core/fp32/fp32_rcc.cu:2225-2267),
 * select_int8_online_plan (core/int8/i8_rcc.cu:3095-3138).  Host only; no device needed. */
int mp_select_plan(int dtype, int m, int n, int k, mp_plan* plan);

/* get_gemm_shared_mem_* / get_gemm_alignment_* (core/fp16/fp16_rcc.cu:3534-3553,
 * core/fp32/fp32_rcc.cu:2302-2311, core/int8/i8_rcc.cu:3171-3181): tile = [pm, pn, pk] where pm
 * tiles RCC n and pn tiles RCC m; alignment = required divisor of k. */
int mp_pid_info(int dtype, int pid, int tile[3], int* alignment);

/* gemm_cost_model / gemm_splitk_cost_model (core/fp16/fp16_rcc_cost.cu:161-237 and the fp32/int8
 * siblings): predicted milliseconds of pid with split_k slices on RCC (m,n,k). */
int mp_cost_ms(int dtype, int pid, int split_k, int m, int n, int k, float* ms);

/* gemm_reduction_cost_model (core/fp16/fp16_rcc_cost.cu:190-210): the split-K hand-off and
 * reduction term of mp_cost_ms alone, for RCC (m, n) and `split_k` slices (0 when split_k <= 1). */
int mp_cost_reduction_ms(int dtype, int pid, int split_k, int m, int n, float* ms);

/* cutlass_gemm_predict (core/fp16/fp16_rcc_cost.cu:256-279, core/fp32/fp32_rcc_cost.cu,
 * core/int8/i8_rcc_cost.cu:232-246): the cheapest primary pid for RCC (m, n, k) among the pids whose
 * K-alignment contract the shape meets; `ms` (may be NULL) receives its predicted milliseconds. */
int mp_cost_predict_pid(int dtype, int m, int n, int k, int* pid, float* ms);

/* run_fp16_pattern2_twin_gemm_row_col_col (core/fp16/fp16_rcc.cu:3297-3304 -> 75-108): columns
 * [0,split_n) and [split_n,n) of C are produced by two tile shapes inside ONE launch.
 * split_n <= 0 picks 3/4 of n rounded down to 128.  Requires 0 < split_n < n, split_n % 128 == 0,
 * k % 8 == 0, else MP_ERR_INVALID_ARG (the reference throws std::invalid_argument). */
int mp_twin_gemm_fp16(int m, int n, int k, int split_n, const void* A, const void* B, void* C,
                      float alpha, float beta, void* stream);

/* Column-parallel Linear fused with the all-gather of its output (no counterpart in the reference, which runs on
 * one GPU; the vLLM integration it patches gathers with a separate NCCL call).  Rank r of g owns W_shard
 * [N_local, K], the rows [col_offset, col_offset + N_local) of the full weight, and computes its slab
 * Y[:, col_offset : col_offset + N_local] of the full row-major output Y[M, ld_dst].  The epilogue stores every
 * finished tile into ALL n_dst copies of Y: dst[0..n_dst) are the bases of the full output buffer on this GPU and,
 * peer-mapped, on the other GPUs of the box (plain stores over NVLink; no TMA, no multicast, no library call).
 * FP16 only, alpha = 1, beta = 0, K % 8 == 0.  A consumer must not read a peer's slab before mp_peer_barrier. */
int mp_linear_gather(int dtype, int M, int N_local, int K, const void* X, const void* W_shard, void* const* dst,
                     int n_dst, long long ld_dst, long long col_offset, void* stream);

/* Cross-GPU flag barrier for mp_linear_gather, one tiny kernel on `stream`.  flags_dev is a DEVICE array of
 * `world` pointers, [r] = rank r's flag array of `world` unsigned words (peer-mapped for r != rank, zero at start).
 * Publishes `value` into slot `rank` of every rank's array (after a system-scope fence, so the slab stores of the
 * kernels before it in the stream are visible first) and waits until every rank's `value` has arrived here.
 * Values must grow from call to call.  The wait is bounded by timeout_us (0 = one second); when it runs out the
 * kernel records a code in the device status word (mp_device_status returns MP_ERR_DEVICE) and returns. */
int mp_peer_barrier(unsigned* const* flags_dev, int world, int rank, unsigned value, unsigned timeout_us,
                    void* stream);

/* Helpers for the two calls above (plain CUDA IPC): a zero-filled device buffer plus the 64-byte handle another
 * process of the same box opens to get a peer-mapped pointer (peer access is enabled on first use). */
int mp_peer_alloc(size_t bytes, void** ptr, unsigned char handle[64]);
int mp_peer_open(const unsigned char handle[64], void** ptr);
int mp_peer_close(void* ptr);
int mp_peer_free(void* ptr);

/* scaled_mm_mikpoly -> cutlass_scaled_mm_mikpoly_unified
 * (core/int8/scaled_mm/scaled_mm_bindings.cpp:20-92, scaled_mm_mikpoly_unified.cu:362-403):
 * out[M,N] (row-major, ldc) = a_scales[m] * (b_scales[n] * int32(A[M,K] * B_nk[N,K]^T)) (+ bias[n]),
 * rounded as the reference's epilogue does (scaled_mm_epilogues_mikpoly.hpp:40-119).
 * a_scales has M entries or one (a_scalar != 0); b_scales N entries or one.  bias is NULL or N
 * values of the output type.  out_dtype: 0 = fp16, 1 = bf16. */
int mp_scaled_mm_i8(int M, int N, int K, const int8_t* A, int lda, const int8_t* B_nk, int ldb,
                    const float* a_scales, int a_scalar, const float* b_scales, int b_scalar,
                    const void* bias, void* out, int ldc, int out_dtype, void* stream);

/* Tuning entry for the scaled matmul (no counterpart in the reference, whose six configurations are
 * fixed CUTLASS instantiations): same arguments as mp_scaled_mm_i8 behind an explicit kernel choice.
 * orient 0 puts the tokens (rows of A) on the 128-row UMMA-M side and tiles the channels by bn,
 * orient 1 puts the channels (rows of B_nk) there and tiles the tokens by bn, orient 3 selects the
 * streaming kernel (narrow side <= 64 rows; bn and split_k ignored), orient 4 / 5 are orient 0 / 1
 * with 256-row tiles.  The refit tool uses it to
 * measure the scaled-matmul plan table. */
int mp_scaled_mm_i8_tile(int orient, int bn, int split_k, int M, int N, int K, const int8_t* A, int lda,
                         const int8_t* B_nk, int ldb, const float* a_scales, int a_scalar,
                         const float* b_scales, int b_scalar, const void* bias, void* out, int ldc,
                         int out_dtype, void* stream);

/* predict_best_sm80_evt_config / get_sm80_evt_config
 * (core/int8/scaled_mm/scaled_mm_mikpoly_unified.cu:405-414): tile id the scaled matmul would
 * pick for (M,N,K), and a tile's (tile_m, tile_n, tile_k, alignment). */
int mp_scaled_mm_predict(int M, int N, int K);
int mp_scaled_mm_config(int config_id, int out[4]);

/* is_paper_elite_fp16_pid / paper_elite_fp16_kernel_count / paper_elite_fp16_pids
 * (generated/fp16/rcc/candidates.cu:35-60). `pids` may be NULL; returns the count. */
int mp_elite_fp16_pids(int* pids, int capacity);

/* is_explicit_neighborhood_pid (generated/fp16/rcc/candidates.cu:62-65): 1 for the FP16 pid ranges
 * 90..205, 216..321 and 400..439, else 0.  Every pid of these ranges has a kernel here. */
int mp_is_explicit_neighborhood_pid(int pid);

/* The reference reads its MOONPOLY_* environment flags on every call (core/fp16/fp16_rcc.cu:110-144).
 * This library caches numeric flags at first use; mp_reload_env() re-reads all of them and drops
 * memoised plans.  The force-split and enable flags that the reference's tests toggle between
 * calls are re-read on every call regardless. */
int mp_reload_env(void);

/* Waits for `stream` (NULL: the whole device) and reports the device-side status word: 0, or the
 * first error a kernel recorded since the last call (then cleared).  Returns MP_ERR_DEVICE when
 * the word was non-zero. */
int mp_device_status(void* stream, int* device_code);

/* Number of SMs of the current device (the reference's constant num_SM = 108,
 * moonpoly/include/moonpoly.cuh:26, becomes a query); <= 0 when no device is present. */
int mp_num_sms(void);

/* Number of kernels this library has launched from the calling process so far. */
unsigned long long mp_launch_count(void);

const char* mp_last_error_string(void);
const char* mp_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MOONPOLY_ABI_H_ */
