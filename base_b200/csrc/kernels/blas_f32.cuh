// f32 GEMV / GEMM kernels behind the cl_cublas_* entry points.
//
// The reference calls cuBLAS for these (base/src/ffi/cuda.rs:1586-1603,
// 1668-1683, 1776-1797) and notes that cuBLAS commits to no summation order
// (lean/lib/AlgorithmLib/ML/Compose.lean:261-285).  These kernels commit to
// one: per lane a sequential fma walk over columns lane*4 + 128*i, then the
// xor butterfly 16,8,4,2,1 — the shape of the reference's own `vec4`
// schedule (lean/lib/AlgorithmLib/ML/Sched.lean:7-64, fold in
// ML/Schema.lean:10-24), with fma instead of mul+add.
#pragma once
#include "common.cuh"

struct SgemvArgs {
  int rows;      // outputs for the transposed (row-major W[rows][cols]) form
  int cols;
  float alpha;
  float beta;
};

// y[r] = alpha * sum_c W[r][c] * x[c] + beta * y[r];  W row-major [rows][cols].
// One warp per 4 rows; 8 warps per CTA.
constexpr int kSgemvWarps = 8;
constexpr int kSgemvRowsPerWarp = 4;

extern "C" __global__ void __launch_bounds__(kSgemvWarps * 32)
sgemv_t_f32(const float *__restrict__ W, const float *__restrict__ x, float *__restrict__ y, SgemvArgs a) {
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int r0 = (blockIdx.x * kSgemvWarps + warp) * kSgemvRowsPerWarp;
  if (r0 >= a.rows) return;
  float acc[kSgemvRowsPerWarp];
#pragma unroll
  for (int i = 0; i < kSgemvRowsPerWarp; ++i) acc[i] = 0.f;
  const bool vec = (a.cols & 3) == 0;
  if (vec) {
    const int n4 = a.cols >> 2;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    for (int c = lane; c < n4; c += 32) {
      const float4 xv = x4[c];
#pragma unroll
      for (int i = 0; i < kSgemvRowsPerWarp; ++i) {
        const int r = min(r0 + i, a.rows - 1);
        const float4 w = __ldcs(reinterpret_cast<const float4 *>(W + size_t(r) * a.cols) + c);
        acc[i] = fmaf(w.x, xv.x, acc[i]);
        acc[i] = fmaf(w.y, xv.y, acc[i]);
        acc[i] = fmaf(w.z, xv.z, acc[i]);
        acc[i] = fmaf(w.w, xv.w, acc[i]);
      }
    }
  } else {
    for (int c = lane; c < a.cols; c += 32) {
      const float xv = x[c];
#pragma unroll
      for (int i = 0; i < kSgemvRowsPerWarp; ++i) {
        const int r = min(r0 + i, a.rows - 1);
        acc[i] = fmaf(W[size_t(r) * a.cols + c], xv, acc[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kSgemvRowsPerWarp; ++i) acc[i] = warp_sum(acc[i]);
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < kSgemvRowsPerWarp; ++i) {
      const int r = r0 + i;
      if (r < a.rows) {
        float v = a.alpha * acc[i];
        if (a.beta != 0.f) v = fmaf(a.beta, y[r], v);
        y[r] = v;
      }
    }
  }
}

// y[c] = alpha * sum_r W[r][c] * x[r] + beta * y[c]  (cuBLAS "N" on the
// column-major view).  One thread per output column, coalesced over c.
extern "C" __global__ void __launch_bounds__(256)
sgemv_n_f32(const float *__restrict__ W, const float *__restrict__ x, float *__restrict__ y, SgemvArgs a) {
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= a.cols) return;
  float acc = 0.f;
  for (int r = 0; r < a.rows; ++r) acc = fmaf(W[size_t(r) * a.cols + c], x[r], acc);
  float v = a.alpha * acc;
  if (a.beta != 0.f) v = fmaf(a.beta, y[c], v);
  y[c] = v;
}

// Column-major C[m x n] = alpha * op(A) * op(B) + beta * C, strided batches.
// One thread per output element; used for small attention-sized products.
struct SgemmArgs {
  int transa, transb, m, n, k;
  float alpha, beta;
  long long stride_a, stride_b, stride_c;
  int lda, ldb, ldc;
};

extern "C" __global__ void __launch_bounds__(256)
sgemm_naive_f32(const float *__restrict__ A, const float *__restrict__ B, float *__restrict__ C, SgemmArgs g) {
  pdl_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  const int batch = blockIdx.y;
  if (idx >= g.m * g.n) return;
  const int i = idx % g.m, j = idx / g.m;
  const float *a = A + size_t(batch) * g.stride_a;
  const float *b = B + size_t(batch) * g.stride_b;
  float *c = C + size_t(batch) * g.stride_c;
  float acc = 0.f;
  for (int p = 0; p < g.k; ++p) {
    const float av = g.transa ? a[size_t(i) * g.lda + p] : a[size_t(p) * g.lda + i];
    const float bv = g.transb ? b[size_t(p) * g.ldb + j] : b[size_t(j) * g.ldb + p];
    acc = fmaf(av, bv, acc);
  }
  float v = g.alpha * acc;
  if (g.beta != 0.f) v = fmaf(g.beta, c[size_t(j) * g.ldc + i], v);
  c[size_t(j) * g.ldc + i] = v;
}

// ---- GEMV in the reference's committed fold order ---------------------------------------------------
// y[r] = W[r] . x with ONE warp per output row and the reference's own arithmetic, so that the result is
// bit-identical to the reference's CPU image of its kernels (applications/warp-check/src/lib.rs:28-116,
// lean/lib/AlgorithmLib/ML/Sched.lean:7-64, ML/Schema.lean:10-44): per lane a sequential walk
// acc = acc + (a * b) with separate multiply and add, then the xor butterfly 16, 8, 4, 2, 1
// (lane = lane + other), result read at lane 0.  walk 0 = vec4 (four contiguous elements per lane per
// trip, the warp strides by 128; needs cols % 128 == 0), 1 = strided (one element per lane per trip, stride
// 32; cols % 32 == 0), 2 = blocked (lane l walks the run l * cols / 32 ...).  For checks and for callers that
// need the reference's bits; the fused kernels above are the fast path.
struct WarpFoldArgs { int rows, cols, walk; };

extern "C" __global__ void __launch_bounds__(256)
gemv_warp_fold_f32(const float *__restrict__ W, const float *__restrict__ x, float *__restrict__ y, WarpFoldArgs a) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  const float *w = W + size_t(row) * a.cols;
  float acc = 0.f;
  if (a.walk == 0) {
    for (int t = 0; t < a.cols / 128; ++t) {
      const int o = t * 128 + lane * 4;
#pragma unroll
      for (int q = 0; q < 4; ++q) acc = __fadd_rn(acc, __fmul_rn(w[o + q], x[o + q]));
    }
  } else if (a.walk == 1) {
    for (int t = 0; t < a.cols / 32; ++t) acc = __fadd_rn(acc, __fmul_rn(w[t * 32 + lane], x[t * 32 + lane]));
  } else {
    const int run = a.cols / 32;
    for (int t = 0; t < run; ++t) acc = __fadd_rn(acc, __fmul_rn(w[lane * run + t], x[lane * run + t]));
  }
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, m));
  if (lane == 0) y[row] = acc;
}
