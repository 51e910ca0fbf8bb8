// MXFP4 mixture-of-experts FFN for decode-sized token counts.
//
// Stages (reference definitions: router Compose.lean:1834-1836, expert
// Compose.lean:1798-1801, combine Compose.lean:1803-1810 under
// lean/lib/AlgorithmLib/ML/; NumPy image applications/ten-qwen/moe.py:26-37):
//   router logits -> top-k (descending logit, ties to the lower expert id)
//   -> softmax over the k selected logits -> per expert
//   down(swiglu(gate_up(x))) -> sum over the k slots in slot order.
// The gpt-oss specifics (router bias, interleaved gate/up rows, clamp,
// alpha, +1 on the linear branch, expert biases) are not in the reference;
// they are fixed by the oracle (oracle/moe_oracle.py) and mirrored here.
//
// Weight layout in HBM ("checkpoint layout", what `load` uploads):
//   codes  [E][R][K/2] u8, two codes per byte, low nibble first
//   scales [E][R][K/32] u8 (UE8M0)
//   bias   [E][R] f32
// with (R, K) = (2I, H) for gate_up (row 2i = gate_i, row 2i+1 = up_i) and
// (H, I) for down.
//
// GEMV mapping: one thread per 32-element block column (16 bytes of codes +
// 1 scale byte per row), so a warp reads 512 contiguous bytes of a row; the
// thread keeps its 32 activations in registers across the CTA's rows, and
// rows are reduced over the warp with the 16-value transposed shuffle tree.
#pragma once
#include "common.cuh"

struct MoeDims {
  int H;        // hidden size
  int I;        // expert intermediate size
  int E;        // experts
  int top_k;
  int T;        // tokens in this call
  float alpha;
  float limit;
};

// ---- router -------------------------------------------------------------------
// logits[t][e] = Wr[e] . x[t] + br[e].  One CTA per expert, all tokens (up to
// 8 per pass) so a router row is read once.
extern "C" __global__ void __launch_bounds__(128)
moe_router_logits(const float *__restrict__ Wr, const float *__restrict__ br,
                  const float *__restrict__ x, float *__restrict__ logits, MoeDims d) {
  pdl_wait();
  const int e = blockIdx.x;
  const int tid = threadIdx.x;
  __shared__ float red[4][8];
  const float4 *w4 = reinterpret_cast<const float4 *>(Wr + size_t(e) * d.H);
  const int n4 = d.H >> 2;
  for (int t0 = 0; t0 < d.T; t0 += 8) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int c = tid; c < n4; c += 128) {
      float4 w = __ldg(w4 + c);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (t0 + i < d.T) {
          float4 xv = __ldg(reinterpret_cast<const float4 *>(x + size_t(t0 + i) * d.H) + c);
          acc[i] = fmaf(w.x, xv.x, acc[i]);
          acc[i] = fmaf(w.y, xv.y, acc[i]);
          acc[i] = fmaf(w.z, xv.z, acc[i]);
          acc[i] = fmaf(w.w, xv.w, acc[i]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = warp_sum(acc[i]);
    if ((tid & 31) == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) red[tid >> 5][i] = acc[i];
    }
    __syncthreads();
    if (tid < 8 && t0 + tid < d.T) {
      float s = ((red[0][tid] + red[1][tid]) + red[2][tid]) + red[3][tid];
      logits[size_t(t0 + tid) * d.E + e] = s + br[e];
    }
    __syncthreads();
  }
}

// ---- top-k + softmax over the selected logits -----------------------------------
// One warp per token.  E <= 128 (4 logits per lane).  Selection is by
// (logit descending, expert id ascending); NaN logits sort last.
// idx_copy (optional): a second place for the indices (shared memory of a fused caller).
B200_DEVICE void topk_softmax_token(const float *__restrict__ logits, int *__restrict__ topk_idx,
                                    float *__restrict__ topk_w, const MoeDims &d, int t, int lane, int *idx_copy = nullptr) {
  float v[4];
  bool taken[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int e = lane + 32 * i;
    float l = (e < d.E) ? logits[size_t(t) * d.E + e] : -INFINITY;
    v[i] = (l == l) ? l : -INFINITY;
    taken[i] = e >= d.E;
  }
  float sel_v[8];
  int sel_e[8];
  for (int j = 0; j < d.top_k && j < 8; ++j) {
    float bv = -INFINITY;
    int be = 0x7fffffff;   // "none": loses every tie
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int e = lane + 32 * i;
      if (!taken[i] && (be == 0x7fffffff || v[i] > bv || (v[i] == bv && e < be))) { bv = v[i]; be = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (oe != 0x7fffffff && (be == 0x7fffffff || ov > bv || (ov == bv && oe < be))) { bv = ov; be = oe; }
    }
    sel_v[j] = bv;
    sel_e[j] = (be == 0x7fffffff) ? 0 : be;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (lane + 32 * i == be) taken[i] = true;
  }
  if (lane == 0) {
    float m = sel_v[0];
    float ex[8], s = 0.f;
    for (int j = 0; j < d.top_k && j < 8; ++j) { ex[j] = __expf(sel_v[j] - m); s += ex[j]; }
    for (int j = 0; j < d.top_k && j < 8; ++j) {
      topk_idx[size_t(t) * d.top_k + j] = sel_e[j];
      if (idx_copy) idx_copy[t * d.top_k + j] = sel_e[j];
      topk_w[size_t(t) * d.top_k + j] = ex[j] / s;
    }
  }
}

extern "C" __global__ void __launch_bounds__(32)
moe_topk_softmax(const float *__restrict__ logits, int *__restrict__ topk_idx,
                 float *__restrict__ topk_w, MoeDims d) {
  pdl_wait();
  topk_softmax_token(logits, topk_idx, topk_w, d, blockIdx.x, threadIdx.x);
}

// ---- shared GEMV core: 16 rows x (K/32 block columns), one token ----------------
// Thread `col` owns block column `col` (< K/32).  Returns, in v[0] of each
// lane, the warp's partial of row row_of_lane16(lane); the caller sums the
// warps of the CTA through shared memory in warp order.
template <int ROWS>
B200_DEVICE void load_rows(const uint8_t *__restrict__ codes, const uint8_t *__restrict__ scales,
                           int K, int col, bool valid, uint4 (&w)[ROWS], uint32_t (&s)[ROWS]) {
  const int kb = K >> 5;
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    if (valid) {
      w[r] = __ldg(reinterpret_cast<const uint4 *>(codes + size_t(r) * (K >> 1)) + col);
      s[r] = __ldg(scales + size_t(r) * kb + col);
    } else {
      w[r] = make_uint4(0, 0, 0, 0);
      s[r] = 127;
    }
  }
}

B200_DEVICE float block_dot32(const uint4 &w, const float (&x)[32]) {
  float v[8];
  float a0 = 0.f, a1 = 0.f;
  e2m1x8_to_f32(w.x, v);
#pragma unroll
  for (int i = 0; i < 8; i += 2) { a0 = fmaf(v[i], x[i], a0); a1 = fmaf(v[i + 1], x[i + 1], a1); }
  e2m1x8_to_f32(w.y, v);
#pragma unroll
  for (int i = 0; i < 8; i += 2) { a0 = fmaf(v[i], x[8 + i], a0); a1 = fmaf(v[i + 1], x[9 + i], a1); }
  e2m1x8_to_f32(w.z, v);
#pragma unroll
  for (int i = 0; i < 8; i += 2) { a0 = fmaf(v[i], x[16 + i], a0); a1 = fmaf(v[i + 1], x[17 + i], a1); }
  e2m1x8_to_f32(w.w, v);
#pragma unroll
  for (int i = 0; i < 8; i += 2) { a0 = fmaf(v[i], x[24 + i], a0); a1 = fmaf(v[i + 1], x[25 + i], a1); }
  return a0 + a1;
}

B200_DEVICE void load_x32(const float *__restrict__ x, int col, bool valid, float (&xr)[32]) {
  if (valid) {
    const float4 *p = reinterpret_cast<const float4 *>(x) + col * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float4 f = p[i];
      xr[4 * i] = f.x; xr[4 * i + 1] = f.y; xr[4 * i + 2] = f.z; xr[4 * i + 3] = f.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) xr[i] = 0.f;
  }
}

constexpr int kGemvThreads = 96;   // 3 warps: up to 96 block columns (K <= 3072)
constexpr int kGemvRows = 16;

// ---- gate_up + clamped SwiGLU ------------------------------------------------------
// grid (2I/16, T*top_k).  CTA (rt, a): assignment a = t*top_k + j uses expert
// topk_idx[a]; computes rows [16 rt, 16 rt + 16) of gate_up, i.e. 8
// activations act[a][8 rt .. 8 rt + 8).
extern "C" __global__ void __launch_bounds__(kGemvThreads)
moe_gate_up_swiglu(const uint8_t *__restrict__ codes, const uint8_t *__restrict__ scales,
                   const float *__restrict__ bias, const float *__restrict__ x,
                   const int *__restrict__ topk_idx, float *__restrict__ act, MoeDims d) {
  const int a = blockIdx.y;
  const int t = a / d.top_k;
  const int row0 = blockIdx.x * kGemvRows;
  const int R = 2 * d.I, K = d.H;
  const int col = threadIdx.x, lane = col & 31, warp = col >> 5;
  const bool valid = col < (K >> 5);
  __shared__ float part[3][kGemvRows];

  pdl_wait();   // topk_idx and x come from the preceding kernels
  const int e = topk_idx[a];
  const uint8_t *cw = codes + (size_t(e) * R + row0) * (K >> 1);
  const uint8_t *sw = scales + (size_t(e) * R + row0) * (K >> 5);
  uint4 w[kGemvRows];
  uint32_t s[kGemvRows];
  load_rows<kGemvRows>(cw, sw, K, col, valid, w, s);
  float xr[32];
  load_x32(x + size_t(t) * K, col, valid, xr);
  pdl_launch_dependents();

  float v[kGemvRows];
#pragma unroll
  for (int r = 0; r < kGemvRows; ++r) v[r] = ue8m0_to_f32(s[r]) * block_dot32(w[r], xr);
  warp_reduce16(v, lane);
  if ((lane & 1) == 0) part[warp][row_of_lane16(lane)] = v[0];
  __syncthreads();
  if (col < kGemvRows / 2) {
    const int rg = 2 * col, ru = 2 * col + 1;
    float g = ((part[0][rg] + part[1][rg]) + part[2][rg]) + bias[size_t(e) * R + row0 + rg];
    float u = ((part[0][ru] + part[1][ru]) + part[2][ru]) + bias[size_t(e) * R + row0 + ru];
    act[size_t(a) * d.I + (row0 >> 1) + col] = swiglu_clamped(g, u, d.alpha, d.limit);
  }
}

// ---- down + weighted combine ----------------------------------------------------------
// grid (H/16, T).  CTA (rt, t) walks the token's top_k slots in slot order:
// y[t][r] = sum_j w[t][j] * (Wd[e_j][r] . act[t*top_k + j] + bd[e_j][r]),
// added to `residual` when that pointer is non-null.  No atomics: the sum
// order is fixed.
extern "C" __global__ void __launch_bounds__(kGemvThreads)
moe_down_combine(const uint8_t *__restrict__ codes, const uint8_t *__restrict__ scales,
                 const float *__restrict__ bias, const float *__restrict__ act,
                 const int *__restrict__ topk_idx, const float *__restrict__ topk_w,
                 const float *__restrict__ residual, float *__restrict__ y, MoeDims d) {
  const int t = blockIdx.y;
  const int row0 = blockIdx.x * kGemvRows;
  const int R = d.H, K = d.I;
  const int col = threadIdx.x, lane = col & 31, warp = col >> 5;
  const bool valid = col < (K >> 5);
  __shared__ float part[3][kGemvRows];
  float out = 0.f;

  // topk_idx was written two kernels back, which has completed before this
  // grid can start (its predecessor signals only after its own wait), so
  // the first slot's weights are fetched before waiting for `act`.
  for (int j = 0; j < d.top_k; ++j) {
    const int a = t * d.top_k + j;
    const int e = topk_idx[a];
    const uint8_t *cw = codes + (size_t(e) * R + row0) * (K >> 1);
    const uint8_t *sw = scales + (size_t(e) * R + row0) * (K >> 5);
    uint4 w[kGemvRows];
    uint32_t s[kGemvRows];
    load_rows<kGemvRows>(cw, sw, K, col, valid, w, s);
    if (j == 0) pdl_wait();
    float xr[32];
    load_x32(act + size_t(a) * K, col, valid, xr);
    float v[kGemvRows];
#pragma unroll
    for (int r = 0; r < kGemvRows; ++r) v[r] = ue8m0_to_f32(s[r]) * block_dot32(w[r], xr);
    warp_reduce16(v, lane);
    if ((lane & 1) == 0) part[warp][row_of_lane16(lane)] = v[0];
    __syncthreads();
    if (col < kGemvRows) {
      float o = ((part[0][col] + part[1][col]) + part[2][col]) + bias[size_t(e) * R + row0 + col];
      out = fmaf(topk_w[a], o, out);
    }
    __syncthreads();
  }
  pdl_launch_dependents();
  if (col < kGemvRows) {
    const size_t o = size_t(t) * R + row0 + col;
    y[o] = residual ? residual[o] + out : out;
  }
}

// ---- dequantised-value dump (bit-exact check of the element path) -------------------
// out[r][k] = scale(r, k/32) * e2m1(code(r, k)) for rows [row0, row0+nrows)
// of one expert matrix, using the same conversion the GEMV uses.
struct DequantArgs { int K; int R; int expert; int row0; int nrows; };

extern "C" __global__ void __launch_bounds__(128)
mxfp4_dequant_rows(const uint8_t *__restrict__ codes, const uint8_t *__restrict__ scales,
                   float *__restrict__ out, DequantArgs a) {
  const int r = blockIdx.x;
  if (r >= a.nrows) return;
  const size_t row = size_t(a.expert) * a.R + a.row0 + r;
  const uint32_t *cw = reinterpret_cast<const uint32_t *>(codes + row * (a.K >> 1));
  const uint8_t *sw = scales + row * (a.K >> 5);
  for (int wi = threadIdx.x; wi < (a.K >> 3); wi += blockDim.x) {
    float v[8];
    e2m1x8_to_f32(cw[wi], v);
    const float sc = ue8m0_to_f32(sw[wi >> 2]);
#pragma unroll
    for (int i = 0; i < 8; ++i) out[size_t(r) * a.K + wi * 8 + i] = sc * v[i];
  }
}
