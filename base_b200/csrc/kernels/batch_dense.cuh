// Dense layers of a decode step for a BATCH of sequences (up to a few hundred tokens): a skinny GEMM
// out[t][r] = sum_k W[r][k] x[t][k] (+ bias, + residual) whose cost is reading W once.  It runs on the
// tcgen05 tensor cores with the weights as they are stored (bf16) and f32-exact activations:
//   * B operand = 8-row groups of W (K-major core matrices, streamed from HBM by bulk copies);
//   * A operand = the tokens: row t = bf16(x[t]), row 32 + t = bf16(x[t] - row t), so that hi + lo carries x to
//     2^-17 relative; M = 64, at most 32 tokens per pass (more tokens = more passes over the same weights);
//   * D (tensor memory, f32) [64 x N]; the epilogue adds the hi and lo rows.
// Same math as the one-token kernels (dense_decode.cuh: W x + bias (+ residual), reference call sites
// lean/lib/AlgorithmLib/Cuda.lean:278-288); only the summation order differs.
//
// Layouts (made once: dense_tc_retile for weights, rows_to_a for activations):
//   W tiled: [K chunk of 64][row group of 8][column group of 8 (16 B)][8 rows][16 B]  -> the row groups a CTA owns
//            are one contiguous piece per chunk (one bulk copy into a ring slot);
//   A tiled: [pass][K chunk of 64][column group][2 * bd_rh(B) rows][16 B]                -> 8 KB per pass and chunk at 32 tokens, less below.
// Every wait is bounded; on timeout a code is stored in *status and the kernel ends.
#pragma once
#include "tc_gemm.cuh"
#include "dense_decode.cuh"
#include "mega_decode.cuh"

constexpr int kBdTokens = 32;          // tokens per pass
constexpr int kBdRows = 64;            // A rows per pass (hi + lo)
constexpr int kBdMaxGroups = 16;       // row groups per unit: N <= 128
constexpr int kBdSlots = 16;          // at most; the ring holds as many slots as fit (a slot = the A piece + this CTA's B piece of one K chunk)
constexpr int kBdRingBytes = 8 * (8192 + kBdMaxGroups * 1024);      // 192 KB
constexpr int kBdThreads = 192;        // warps 0..3: epilogue, warp 4: producer, warp 5: issuer
constexpr uint32_t kBdSpin = 1u << 22;

// ---- weights: row-major bf16 [rows][K] -> tiled ------------------------------------------------
struct DenseRetileArgs { int rows, K; };      // rows % 8 == 0, K % 64 == 0

extern "C" __global__ void __launch_bounds__(256)
dense_tc_retile(const uint4 *__restrict__ src, uint4 *__restrict__ dst, DenseRetileArgs a) {
  const size_t n = size_t(a.rows) * (a.K >> 3);              // 16-byte vectors
  const int cgs = a.K >> 3, RG = a.rows >> 3;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
    const int row = int(i / cgs), cgk = int(i % cgs);
    const int c = cgk >> 3, cg = cgk & 7, g = row >> 3;
    dst[((size_t(c) * RG + g) * 8 + cg) * 8 + (row & 7)] = src[i];
  }
}

// ---- activations: f32 rows -> tiled hi/lo bf16 A operand, with the fused prologues of a layer -------------
// mode 0: x = in[t]                                         (attention output -> o-proj)
// mode 1: h = in[t] + sum_g parts[g][t] (g ascending; the experts' partial sums of every rank), hout[t] = h,
//         x = h * inv * w, inv = 1 / sqrt(mean(h^2) + eps)  (combine + residual + RMSNorm -> qkv / lm_head)
// mode 2: as mode 1 without parts and without the A operand: xn[t] = x only (RMSNorm -> router, experts)
// mode 3: as mode 1 with the experts' combine done here (one GPU, every expert local): parts = the experts' outputs
//         o[t * n_parts + j], xn = the routing weights w[t][j] (read only), n_parts = top_k;
//         h = in[t] + sum_j w[t][j] * o[t * top_k + j], the sum folded in slot order from zero as moe_combine_range does
// One CTA of 256 threads per token; K % 64 == 0, K <= 4096.
struct RowsToAArgs { int K, B, mode, n_parts; long long part_stride; float eps; };

B200_DEVICE uint16_t bd_bf16(float f) { return f32_to_bf16_rne(f); }
// hi rows per pass: 32, or with fewer than 32 tokens their count rounded up to 8 (the A tile of a K chunk is then
// [column group][2 * bd_rh rows][16 B]: fewer bytes for every CTA to copy; the instruction still reads 64 rows, what
// lies behind the tile's rows gives accumulator rows nobody reads)
B200_DEVICE int bd_rh(int B) { return B >= 32 ? 32 : ((B + 7) & ~7); }

B200_DEVICE void rows_to_a_body(const float *__restrict__ in, const float *__restrict__ parts, const float *__restrict__ w,
                                float *__restrict__ hout, float *__restrict__ xn, uint16_t *__restrict__ a_tiled,
                                const RowsToAArgs &a) {
  __shared__ float red[8];
  const int t = blockIdx.x, tid = threadIdx.x, K = a.K;
  const int nchunks = K >> 6;
  float v[16];
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int i4 = tid + 256 * u;            // float4 index
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i4 * 4 < K) {
      x = __ldcg(reinterpret_cast<const float4 *>(in + size_t(t) * K) + i4);
      if (a.mode == 1)
        for (int g = 0; g < a.n_parts; ++g) {
          const float4 p = __ldcg(reinterpret_cast<const float4 *>(parts + size_t(g) * a.part_stride + size_t(t) * K) + i4);
          x.x += p.x; x.y += p.y; x.z += p.z; x.w += p.w;
        }
      if (a.mode == 3) {                                      // the combine of moe_combine_range, then the residual
        float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < a.n_parts; ++j) {
          const float wj = __ldcg(xn + t * a.n_parts + j);
          const float4 p = __ldcg(reinterpret_cast<const float4 *>(parts + size_t(t * a.n_parts + j) * K) + i4);
          y.x = fmaf(wj, p.x, y.x); y.y = fmaf(wj, p.y, y.y); y.z = fmaf(wj, p.z, y.z); y.w = fmaf(wj, p.w, y.w);
        }
        x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
      }
      if (a.mode != 0 && a.mode != 2 && hout) reinterpret_cast<float4 *>(hout + size_t(t) * K)[i4] = x;
    }
    v[4 * u] = x.x; v[4 * u + 1] = x.y; v[4 * u + 2] = x.z; v[4 * u + 3] = x.w;
    ss = fmaf(x.x, x.x, ss); ss = fmaf(x.y, x.y, ss); ss = fmaf(x.z, x.z, ss); ss = fmaf(x.w, x.w, ss);
  }
  if (a.mode != 0) {
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float inv = 1.0f / sqrtf(tot / float(K) + a.eps);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i4 = tid + 256 * u;
      if (i4 * 4 < K) {
        const float4 g = __ldg(reinterpret_cast<const float4 *>(w) + i4);
        v[4 * u] = v[4 * u] * inv * g.x; v[4 * u + 1] = v[4 * u + 1] * inv * g.y;
        v[4 * u + 2] = v[4 * u + 2] * inv * g.z; v[4 * u + 3] = v[4 * u + 3] * inv * g.w;
        if (xn && a.mode != 3) reinterpret_cast<float4 *>(xn + size_t(t) * K)[i4] = make_float4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]);
      }
    }
  }
  if (a.mode == 2 || !a_tiled) return;
  const int pass = t / kBdTokens, r = t % kBdTokens;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int i4 = tid + 256 * u, k = i4 * 4;
    if (k < K) {
      const int c = k >> 6, cg = (k & 63) >> 3, e = k & 7;      // e = 0 or 4
      uint16_t hi[4], lo[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        hi[j] = bd_bf16(v[4 * u + j]);
        lo[j] = bd_bf16(v[4 * u + j] - bf16_lo(uint32_t(hi[j])));
      }
      const int Rh = bd_rh(a.B);
      uint8_t *base = reinterpret_cast<uint8_t *>(a_tiled) + ((size_t(pass) * nchunks + c) * 8 + cg) * (2 * Rh * 16) + e * 2;
      *reinterpret_cast<uint2 *>(base + r * 16) = make_uint2(uint32_t(hi[0]) | (uint32_t(hi[1]) << 16), uint32_t(hi[2]) | (uint32_t(hi[3]) << 16));
      *reinterpret_cast<uint2 *>(base + (Rh + r) * 16) = make_uint2(uint32_t(lo[0]) | (uint32_t(lo[1]) << 16), uint32_t(lo[2]) | (uint32_t(lo[3]) << 16));
    }
  }
}

extern "C" __global__ void __launch_bounds__(256)
rows_to_a(const float *__restrict__ in, const float *__restrict__ parts, const float *__restrict__ w,
          float *__restrict__ hout, float *__restrict__ xn, uint16_t *__restrict__ a_tiled, RowsToAArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  rows_to_a_body(in, parts, w, hout, xn, a_tiled, a);
}

// ---- the GEMM -----------------------------------------------------------------------------------------
// grid = any number of CTAs (148: one per SM); a CTA owns the row groups [RG * b / grid, RG * (b + 1) / grid), cut
// into units of at most kBdMaxGroups.  Jobs = (unit, pass), passes innermost so that a unit's weights are streamed
// again while they are still in L2.  Warp 4 produces (ring of kBdSlots slots: the A piece and the unit's B piece
// of one K chunk), warp 5 issues four K = 16 instructions per chunk and lets tcgen05.commit free the slot,
// warps 0..3 read the accumulator (two of them, so the next job's instructions overlap this read-back), add the
// hi and lo rows through shared memory and finish (bias, residual).
struct DenseTcArgs {
  int rows, K, B;
  int kind;          // 0: out = W x + bias (bias may be null); 1: ... + res[t][row]
  int m64_rows16;    // where accumulator row r of an M = 64 instruction lives: 1: lane 32 (r / 16) + r % 16; 0: lane r
  int out_stride;    // floats between consecutive tokens of out / res
};

struct BdBars {
  uint64_t full[kBdSlots], empty[kBdSlots], done[2], dfree[2];
  uint32_t tmem_base;
  int abort;
};

B200_DEVICE bool bd_wait(uint64_t *bar, uint32_t parity, BdBars *b, int *status, int code) {
  const uint32_t lim = *reinterpret_cast<volatile int *>(&b->abort) ? 4096u : kBdSpin;
  for (uint32_t i = 0; i < lim; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  *reinterpret_cast<volatile int *>(&b->abort) = 1;
  atomicCAS(status, 0, code);
  return false;
}

// Four K = 16 instructions over one K chunk of 64 (the operands advance by two column groups each: a_step 16-byte units
// of A = 2 x (tile rows) x 16 B, 2 x 128 B of B), issued by an elected lane of the converged warp.
// The four go to accumulators d_tmem + i * d_step (d_step = 0: one accumulator): with several accumulators the
// instructions of a chunk do not wait for one another's results, the epilogue adds them up.
B200_DEVICE void bd_mma4_warp(uint32_t d_tmem, uint32_t d_step, uint64_t adesc, uint64_t bdesc, uint32_t idesc, bool accumulate_first,
                              uint64_t a_step) {
  asm volatile(
      "{\n.reg .pred p, p1, e;\n.reg .b64 a1, a2, a3, b1, b2, b3;\n.reg .b32 d1, d2, d3;\n"
      "elect.sync _|e, 0xffffffff;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "setp.eq.b32 p1, %5, 0;\nor.pred p1, p1, p;\n"          // later instructions accumulate unless they own a fresh accumulator
      "add.u32 d1, %0, %5;\nadd.u32 d2, d1, %5;\nadd.u32 d3, d2, %5;\n"
      "add.u64 a1, %1, %6;\nadd.u64 a2, a1, %6;\nadd.u64 a3, a2, %6;\n"
      "add.u64 b1, %2, 16;\nadd.u64 b2, %2, 32;\nadd.u64 b3, %2, 48;\n"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "@e tcgen05.mma.cta_group::1.kind::f16 [d1], a1, b1, %3, p1;\n"
      "@e tcgen05.mma.cta_group::1.kind::f16 [d2], a2, b2, %3, p1;\n"
      "@e tcgen05.mma.cta_group::1.kind::f16 [d3], a3, b3, %3, p1;\n}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(uint32_t(accumulate_first)), "r"(d_step), "l"(a_step)
      : "memory");
}

constexpr int kBdStageStride = kBdMaxGroups * 8 + 1;      // floats per staged accumulator row (padded)
B200_DEVICE int bd_smem_bytes() { return kBdRingBytes + kBdRows * kBdStageStride * 4 + int(sizeof(BdBars)) + 64; }

extern "C" __global__ void __launch_bounds__(kBdThreads, 1)
dense_tc_gemm(const uint8_t *__restrict__ Wt, const uint8_t *__restrict__ At, const float *__restrict__ bias,
              const float *__restrict__ res, float *__restrict__ out, int *__restrict__ status, DenseTcArgs a) {
  uint8_t *ring = dyn_smem;
  float *stage = reinterpret_cast<float *>(dyn_smem + kBdRingBytes);
  BdBars *bars = reinterpret_cast<BdBars *>(dyn_smem + kBdRingBytes + kBdRows * kBdStageStride * 4);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int RG = a.rows >> 3, nchunks = a.K >> 6, passes = (a.B + kBdTokens - 1) / kBdTokens;
  const int g_lo = int((long long)RG * blockIdx.x / gridDim.x), g_hi = int((long long)RG * (blockIdx.x + 1) / gridDim.x);
  const int units = (g_hi - g_lo + kBdMaxGroups - 1) / kBdMaxGroups, jobs = units * passes;
  // the ring is 192 KB (all the shared memory the staging rows and barriers leave): lm_head runs four slots of two
  // 24 KB chunks, qkv / o-proj four or five slots of three chunks
  const int Rh = bd_rh(a.B);
  const uint32_t a_bytes = 256u * uint32_t(Rh);                // the A tile of one pass and K chunk
  // A ring slot holds kc >= 2 consecutive K chunks (the last slot what is left): the hand-over of a slot between
  // producer, tensor core and back (two mbarrier waits, a commit) costs about 0.25 us whatever the slot holds, and
  // with one chunk per slot that, not bytes or instructions, was the kernel's time (measured by leaving the A copies
  // and the instructions out: 17 of 20 us stayed).
  // kc = 2 chunks per slot, or 3 / 4 where three such slots still fit the ring (measured at 32 tokens: qkv 15.1 us with
  // kc = 2 and five slots, 12.9 with kc = 3 and three slots, 13.9 with kc = 4 and two).
  const uint32_t b_max = uint32_t(max(1, min(kBdMaxGroups, g_hi - g_lo))) * 1024u;
  int kc = 2;
  while (kc < 4 && uint32_t(kc + 1) * (a_bytes + b_max) * 3u <= uint32_t(kBdRingBytes)) ++kc;
  const uint32_t slot_bytes = uint32_t(kc) * (a_bytes + b_max);
  const uint32_t n_slots = min(uint32_t(kBdSlots), uint32_t(kBdRingBytes) / slot_bytes);
  const int npairs = (nchunks + kc - 1) / kc;

  if (tid == 0) {
    for (int i = 0; i < kBdSlots; ++i) { mbar_init(&bars->full[i], 1); mbar_init(&bars->empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars->done[i], 1); mbar_init(&bars->dfree[i], 4); }
    bars->abort = 0;
  }
  fence_barrier_init();
  if (warp == 0) tc_alloc(&bars->tmem_base, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  pdl_wait();                         // the activations (and the residual) come from the kernels before
  pdl_launch_dependents();

  if (warp == 4) {
    // ---- producer
    if (lane == 0) {
      uint32_t q = 0;
      for (int j = 0; j < jobs; ++j) {
        const int u = j / passes, pass = j % passes;
        const int g0 = g_lo + u * kBdMaxGroups, ng = min(kBdMaxGroups, g_hi - g0);
        const uint32_t b_bytes = uint32_t(ng) * 1024u;
        const uint8_t *asrc = At + size_t(pass) * nchunks * a_bytes, *bsrc = Wt + size_t(g0) * 1024;
        for (int p = 0; p < npairs; ++p, ++q) {
          const uint32_t s = q % n_slots;
          if (q >= n_slots && !bd_wait(&bars->empty[s], ((q / n_slots) - 1) & 1, bars, status, 61)) { j = jobs; break; }
          uint8_t *dst = ring + size_t(s) * slot_bytes;
          const int c0 = kc * p;
          const uint32_t nck = uint32_t(min(kc, nchunks - c0));
          mbar_expect_tx(&bars->full[s], nck * (a_bytes + b_bytes));
          bulk_g2s(dst, asrc + size_t(c0) * a_bytes, nck * a_bytes, &bars->full[s]);        // consecutive chunks of A are contiguous
          for (uint32_t kk = 0; kk < nck; ++kk)
            bulk_g2s(dst + uint32_t(kc) * a_bytes + kk * b_bytes, bsrc + size_t(c0 + int(kk)) * RG * 1024, b_bytes, &bars->full[s]);
        }
      }
    }
  } else if (warp == 5) {
    // ---- issuer: the whole warp runs the loop, an elected lane issues (operands stay in uniform registers)
    uint32_t q = 0;
    for (int j = 0; j < jobs; ++j) {
      const int u = j / passes;
      const int g0 = g_lo + u * kBdMaxGroups, ng = min(kBdMaxGroups, g_hi - g0), N = ng * 8;
      const uint32_t acc = tmem + uint32_t(j & 1) * 256u;
      const uint32_t d_step = N <= 64 ? 64u : 0u;            // four accumulators of 64 columns, or one of up to 128
      if (j >= 2 && !bd_wait(&bars->dfree[j & 1], ((j >> 1) - 1) & 1, bars, status, 62)) break;
      tc_fence_after_sync();
      const uint32_t idesc = tc_idesc_bf16(kBdRows, N);
      bool ok = true;
      const uint32_t b_bytes = uint32_t(ng) * 1024u;
      for (int p = 0; p < npairs; ++p, ++q) {
        const uint32_t s = q % n_slots;
        ok = bd_wait(&bars->full[s], (q / n_slots) & 1, bars, status, 63);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(ring + size_t(s) * slot_bytes), sb = sa + uint32_t(kc) * a_bytes;
        const int nck = min(kc, nchunks - kc * p);
        for (int kk = 0; kk < nck; ++kk) {
          const uint64_t da = tc_smem_desc(sa + uint32_t(kk) * a_bytes, 2 * Rh * 16, 128);
          const uint64_t db = tc_smem_desc(sb + uint32_t(kk) * b_bytes, 128, 1024);
          bd_mma4_warp(acc, d_step, da, db, idesc, p > 0 || kk > 0, uint64_t(4 * Rh));
        }
        tc_commit_warp(&bars->empty[s], true);
        tc_commit_warp(&bars->done[j & 1], p == npairs - 1);
        __syncwarp();
      }
      if (!ok) break;
    }
  } else {
    // ---- epilogue warps 0..3
    for (int j = 0; j < jobs; ++j) {
      const int u = j / passes, pass = j % passes;
      const int g0 = g_lo + u * kBdMaxGroups, ng = min(kBdMaxGroups, g_hi - g0), N = ng * 8;
      const uint32_t acc = tmem + uint32_t(j & 1) * 256u;
      const int n_acc = N <= 64 ? 4 : 1;
      if (!bd_wait(&bars->done[j & 1], (j >> 1) & 1, bars, status, 64)) break;
      tc_fence_after_sync();
      const int row = a.m64_rows16 ? (lane < 16 ? warp * 16 + lane : -1) : (warp < 2 ? warp * 32 + lane : -1);
      for (int c0 = 0; c0 < N; c0 += 16) {
        float v[16];
        tc_ld16(acc + (uint32_t(warp * 32) << 16) + uint32_t(c0), v);
        for (int i = 1; i < n_acc; ++i) {
          float w[16];
          tc_ld16(acc + (uint32_t(warp * 32) << 16) + uint32_t(i * 64 + c0), w);
#pragma unroll
          for (int q2 = 0; q2 < 16; ++q2) v[q2] += w[q2];
        }
        if (row >= 0) {
#pragma unroll
          for (int i = 0; i < 16; ++i) stage[row * kBdStageStride + c0 + i] = v[i];
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->dfree[j & 1]);
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const int ntok = min(kBdTokens, a.B - pass * kBdTokens);
      for (int idx = tid; idx < ntok * N; idx += 128) {
        const int t = idx / N, n = idx % N, r = g0 * 8 + n;
        float val = stage[t * kBdStageStride + n] + stage[(Rh + t) * kBdStageStride + n];
        if (bias) val += __ldg(bias + r);
        const size_t o = size_t(pass * kBdTokens + t) * a.out_stride + r;
        if (a.kind == 1) val += __ldcg(res + o);
        out[o] = val;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tc_dealloc(tmem, 512);
  }
}
