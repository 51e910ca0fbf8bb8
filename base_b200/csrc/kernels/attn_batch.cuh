// Decode attention for a batch of sequences: same definition as attn_decode.cuh (RoPE, KV append, GQA, sinks,
// sliding window, bf16 cache; reference citations there), organised for many sequences at once.  A CTA owns one
// (sequence, kv head) and a contiguous range of the 128-position slices of its context; it streams the slices
// through a two-stage shared-memory pipeline (cp.async) and keeps a running softmax (maximum, denominator,
// weighted V sum) in registers, warp = q head, so that nothing is merged between slices.  With S > 1 CTAs per
// (sequence, kv head) — few sequences, long context — each writes one partial result and the last one to finish
// merges them in order (as attn_decode does per slice).
#pragma once
#include "attn_decode.cuh"

struct AttnBatchArgs {
  int NQ, NKV, B, cache_len, window, max_pos, qkv_stride;
  float scale;
  int max_splits;        // stride of the partial buffers
  int S;                 // CTAs per (sequence, kv head) = gridDim.x
};

constexpr int kAbThreads = 256;

struct alignas(16) AttnBatchSmem {
  uint16_t k[2][kAttnSplit][72];
  uint16_t v[2][kAttnSplit][72];
  float q[kAttnMaxGroup][64];
  float s[kAttnMaxGroup][kAttnSplit];
  int is_last;
};

B200_DEVICE void ab_prefetch(AttnBatchSmem &sm, int stage, int j0, int nj, size_t head_base, int cache_len,
                             const uint16_t *kcache, const uint16_t *vcache, int tid) {
  for (int idx = tid; idx < nj * 8; idx += kAbThreads) {
    const int row = idx >> 3, ch = idx & 7;
    const size_t src = (head_base + size_t((j0 + row) % cache_len)) * 64 + ch * 8;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(&sm.k[stage][row][ch * 8])), "l"(kcache + src) : "memory");
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(&sm.v[stage][row][ch * 8])), "l"(vcache + src) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

// ---- tensor-core pieces (mma.sync m16n8k16, bf16 inputs, f32 accumulate) --------------------------------------
// A rows 0..7 = the group's q heads (or their probabilities) rounded to bf16, rows 8..15 = what the rounding left
// (x - bf16(x)), so that hi + lo carries the f32 value to 2^-17; the two halves of an accumulator column are added
// afterwards.  K and V are bf16 in the cache, so the products are exact.
B200_DEVICE uint32_t ab_pack_hi(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&h);
}
B200_DEVICE uint32_t ab_pack_lo(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  const float2 f = __bfloat1622float2(h);
  const __nv_bfloat162 l = __floats2bfloat162_rn(a - f.x, b - f.y);
  return *reinterpret_cast<const uint32_t *>(&l);
}
B200_DEVICE void ab_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
B200_DEVICE void ab_ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// grid = (S, NKV, B), 256 threads, dynamic shared memory sizeof(AttnBatchSmem).
// part_o [B][NQ][max_splits][64], part_ml [B][NQ][max_splits][2], counters [B][NKV] (zero on entry, zero on exit).
// Warp w owns positions [16 w, 16 w + 16) of every slice, for all q heads of the group: Q K^T is two n-tiles x four
// k-steps, P V one k-step x eight n-tiles; its running maximum, denominator and output stay in registers over the
// slices and the eight warps are merged once at the end, in warp order.
// The o-proj's A operand (rows_to_a, mode 0, of batch_dense.cuh) written by the attention itself: elements k, k + 1 of
// sequence b as the hi / lo bf16 rows r and Rh + r of the tile [pass][K chunk = q head][column group][2 Rh rows][16 B].
B200_DEVICE void attn_store_a(uint16_t *a_tiled, int b, int B, int NQ, int qh, int lane, float x0, float x1) {
  const int pass = b >> 5, r = b & 31, cg = lane >> 2, e = (2 * lane) & 7;
  const uint16_t h0 = f32_to_bf16_rne(x0), h1 = f32_to_bf16_rne(x1);
  const uint16_t l0 = f32_to_bf16_rne(x0 - bf16_lo(uint32_t(h0))), l1 = f32_to_bf16_rne(x1 - bf16_lo(uint32_t(h1)));
  const int Rh = B >= 32 ? 32 : ((B + 7) & ~7);                   // bd_rh of batch_dense.cuh
  uint8_t *base = reinterpret_cast<uint8_t *>(a_tiled) + ((size_t(pass) * NQ + qh) * 8 + cg) * (2 * Rh * 16) + e * 2;
  *reinterpret_cast<uint32_t *>(base + r * 16) = uint32_t(h0) | (uint32_t(h1) << 16);
  *reinterpret_cast<uint32_t *>(base + (Rh + r) * 16) = uint32_t(l0) | (uint32_t(l1) << 16);
}

extern "C" __global__ void __launch_bounds__(kAbThreads, 2)
attn_decode_batch(const float *__restrict__ qkv, const float *__restrict__ rope, const int *__restrict__ meta,
                  uint16_t *kcache, uint16_t *vcache, const float *__restrict__ sinks, float *__restrict__ part_o,
                  float *__restrict__ part_ml, int *__restrict__ counters, float *__restrict__ attn_out,
                  uint16_t *__restrict__ a_tiled, AttnBatchArgs a) {
  AttnBatchSmem &sm = *reinterpret_cast<AttnBatchSmem *>(dyn_smem);
  constexpr int HD = 64, HALF = 32;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int sx = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = a.NQ / a.NKV, QD = a.NQ * HD;
  const int pos = meta[2 * b + 1];          // written before this step's graph is launched (or by the last step's argmax)
  const int lo_vis = a.window > 0 ? max(0, pos + 1 - a.window) : 0;
  const int nsplit = (pos + 1 - lo_vis + kAttnSplit - 1) / kAttnSplit;
  const int S = min(a.S, nsplit);
  if (sx >= S) return;
  const int s_lo = int((long long)nsplit * sx / S), s_hi = int((long long)nsplit * (sx + 1) / S);
  const size_t head_base = (size_t(b) * a.NKV + kvh) * a.cache_len;
  // the cache rows depend only on the position: request the first slice before waiting for q, k and v
  {
    const int j0 = lo_vis + s_lo * kAttnSplit;
    ab_prefetch(sm, 0, j0, min(kAttnSplit, pos + 1 - j0), head_base, a.cache_len, kcache, vcache, tid);
  }
  pdl_wait();
  pdl_launch_dependents();
  const float *tok = qkv + size_t(b) * a.qkv_stride;
  const int rp = min(pos, a.max_pos - 1);
  const float *sinp = rope + size_t(rp) * HALF, *cosp = rope + size_t(a.max_pos) * HALF + size_t(rp) * HALF;
  {
    const int gq = tid >> 5, d = tid & 31;          // 8 warps = up to 8 q heads of the group
    float rlo = 0.f, rhi = 0.f;
    if (gq < G) {
      const float *q = tok + size_t(kvh * G + gq) * HD;
      const float lo = __ldcg(q + d), hi = __ldcg(q + d + HALF), s = __ldg(sinp + d), cs = __ldg(cosp + d);
      rlo = __fmul_rn(__fsub_rn(__fmul_rn(lo, cs), __fmul_rn(hi, s)), a.scale);
      rhi = __fmul_rn(__fadd_rn(__fmul_rn(lo, s), __fmul_rn(hi, cs)), a.scale);
    }
    sm.q[gq][d] = rlo;
    sm.q[gq][d + HALF] = rhi;
  }
  __syncthreads();
  // ---- this thread's q fragments: head g, dims 16 ks + 2 c (+1) and + 8
  uint32_t qa[4][4];
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    const float2 x0 = *reinterpret_cast<const float2 *>(&sm.q[g][16 * ks + 2 * c]);
    const float2 x1 = *reinterpret_cast<const float2 *>(&sm.q[g][16 * ks + 8 + 2 * c]);
    qa[ks][0] = ab_pack_hi(x0.x, x0.y);
    qa[ks][1] = ab_pack_lo(x0.x, x0.y);
    qa[ks][2] = ab_pack_hi(x1.x, x1.y);
    qa[ks][3] = ab_pack_lo(x1.x, x1.y);
  }
  float M = -INFINITY, L = 0.f;              // head g, this warp's positions; L is this thread's share
  float o[8][4];                             // n-tile (8 dims) x {row g: cols 2c, 2c+1; row g + 8: the same}
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const int p0 = 16 * warp;
#pragma unroll 1
  for (int sl = s_lo; sl < s_hi; ++sl) {
    const int st = (sl - s_lo) & 1;
    const int j0 = lo_vis + sl * kAttnSplit, nj = min(kAttnSplit, pos + 1 - j0);
    if (sl + 1 < s_hi) {
      const int j1 = j0 + kAttnSplit;
      ab_prefetch(sm, st ^ 1, j1, min(kAttnSplit, pos + 1 - j1), head_base, a.cache_len, kcache, vcache, tid);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();                                   // this slice's rows have landed for every thread
    if (sl == nsplit - 1) {
      // the slice that ends at `pos` appends the new row (cache and shared memory) and clears the V rows past it
      const size_t slot = (head_base + size_t(pos % a.cache_len)) * HD;
      const int row = pos - j0;
      if (tid < HALF) {
        const float *k = tok + QD + size_t(kvh) * HD;
        const float lo = __ldcg(k + tid), hi = __ldcg(k + tid + HALF), s = __ldg(sinp + tid), cs = __ldg(cosp + tid);
        const uint16_t blo = f32_to_bf16_rne(__fsub_rn(__fmul_rn(lo, cs), __fmul_rn(hi, s)));
        const uint16_t bhi = f32_to_bf16_rne(__fadd_rn(__fmul_rn(lo, s), __fmul_rn(hi, cs)));
        kcache[slot + tid] = blo;
        kcache[slot + tid + HALF] = bhi;
        sm.k[st][row][tid] = blo;
        sm.k[st][row][tid + HALF] = bhi;
      } else if (tid >= 64 && tid < 128) {
        const int d = tid - 64;
        const uint16_t bv = f32_to_bf16_rne(__ldcg(tok + QD + size_t(a.NKV) * HD + size_t(kvh) * HD + d));
        vcache[slot + d] = bv;
        sm.v[st][row][d] = bv;
      }
      for (int i = tid; i < (kAttnSplit - nj) * 8; i += kAbThreads)      // a zero probability times stale bits must stay zero
        *reinterpret_cast<uint4 *>(&sm.v[st][nj + (i >> 3)][(i & 7) * 8]) = make_uint4(0, 0, 0, 0);
      __syncthreads();
    }
    if (p0 < nj) {
      // ---- scores of positions p0 + {0..7} (tile 0) and p0 + {8..15} (tile 1) for head g
      float sc[2][4];
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        sc[t][0] = sc[t][1] = sc[t][2] = sc[t][3] = 0.f;
        const uint16_t *krow = &sm.k[st][p0 + 8 * t + g][0];
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint32_t b0 = *reinterpret_cast<const uint32_t *>(krow + 16 * ks + 2 * c);
          const uint32_t b1 = *reinterpret_cast<const uint32_t *>(krow + 16 * ks + 8 + 2 * c);
          ab_mma(sc[t], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
        }
      }
      // this thread: head g, positions p0 + 8 t + 2 c (+1); the lo rows (g + 8) are added to the hi rows
      float s4[4];
      float m = -INFINITY;
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int p = p0 + 8 * t + 2 * c + e;
          s4[2 * t + e] = p < nj ? sc[t][e] + sc[t][2 + e] : -INFINITY;
          m = fmaxf(m, s4[2 * t + e]);
        }
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      const float Mn = fmaxf(M, m);
      const float f = (M == -INFINITY) ? 0.f : __expf(M - Mn);
      float pr[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pr[i] = s4[i] == -INFINITY ? 0.f : __expf(s4[i] - Mn);
      L = fmaf(L, f, (pr[0] + pr[1]) + (pr[2] + pr[3]));
      M = Mn;
      // probabilities as the A operand: k = position within the 16: tile 0 -> k 2c, 2c+1; tile 1 -> k 8 + 2c, ...
      const uint32_t pa0 = ab_pack_hi(pr[0], pr[1]), pa1 = ab_pack_lo(pr[0], pr[1]);
      const uint32_t pa2 = ab_pack_hi(pr[2], pr[3]), pa3 = ab_pack_lo(pr[2], pr[3]);
      // V of these 16 positions, transposed by ldmatrix: lane l addresses row p0 + 8 ((l >> 3) & 1) + (l & 7),
      // dims 16 n2 + 8 (l >> 4): registers {0, 1} = n-tile 2 n2, {2, 3} = n-tile 2 n2 + 1
      const uint32_t vbase = smem_u32(&sm.v[st][p0 + 8 * ((lane >> 3) & 1) + (lane & 7)][8 * (lane >> 4)]);
#pragma unroll
      for (int n2 = 0; n2 < 4; ++n2) {
        uint32_t vb[4];
        ab_ldmatrix_x4_trans(vb, vbase + n2 * 32);
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          float (&acc)[4] = o[2 * n2 + h2];
          acc[0] *= f; acc[1] *= f; acc[2] *= f; acc[3] *= f;
          ab_mma(acc, pa0, pa1, pa2, pa3, vb[2 * h2], vb[2 * h2 + 1]);
        }
      }
    }
    __syncthreads();                                   // this stage is free for the slice after next
  }
  // ---- merge the eight warps (disjoint positions), in warp order; the staging area is the idle K stage
  L += __shfl_xor_sync(0xffffffffu, L, 1);
  L += __shfl_xor_sync(0xffffffffu, L, 2);
  float *wo = reinterpret_cast<float *>(&sm.k[0][0][0]);       // [8 warps][8 heads][64]  (16 KB of the 18 KB stage)
  float *wm = reinterpret_cast<float *>(&sm.s[0][0]);          // [8 warps][8 heads] maxima, then denominators
  float *wl = wm + 64;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    *reinterpret_cast<float2 *>(wo + (warp * 8 + g) * 64 + 8 * i + 2 * c) = make_float2(o[i][0] + o[i][2], o[i][1] + o[i][3]);
  }
  if (c == 0) { wm[warp * 8 + g] = M; wl[warp * 8 + g] = L; }
  __syncthreads();
  float o0 = 0.f, o1 = 0.f;
  M = -INFINITY; L = 0.f;
  {
    // thread = (head `warp`, dims 2 lane, 2 lane + 1), as the code below expects
#pragma unroll
    for (int w = 0; w < 8; ++w) M = fmaxf(M, wm[w * 8 + warp]);
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const float mw = wm[w * 8 + warp];
      const float fw = mw == -INFINITY ? 0.f : __expf(mw - M);
      const float2 ov = *reinterpret_cast<const float2 *>(wo + (w * 8 + warp) * 64 + 2 * lane);
      L = fmaf(wl[w * 8 + warp], fw, L);
      o0 = fmaf(ov.x, fw, o0);
      o1 = fmaf(ov.y, fw, o1);
    }
  }
  const int qh = kvh * G + warp;
  if (S == 1) {
    if (warp < G) {
      const float sk = __ldg(sinks + qh);
      const float Mf = fmaxf(M, sk), f = __expf(M - Mf);
      const float Lf = fmaf(L, f, __expf(sk - Mf));
      *reinterpret_cast<float2 *>(attn_out + size_t(b) * QD + size_t(qh) * HD + 2 * lane) = make_float2(o0 * f / Lf, o1 * f / Lf);
      if (a_tiled) attn_store_a(a_tiled, b, a.B, a.NQ, qh, lane, o0 * f / Lf, o1 * f / Lf);
    }
    return;
  }
  if (warp < G) {
    *reinterpret_cast<float2 *>(part_o + ((size_t(b) * a.NQ + qh) * a.max_splits + sx) * HD + 2 * lane) = make_float2(o0, o1);
    if (lane == 0) *reinterpret_cast<float2 *>(part_ml + ((size_t(b) * a.NQ + qh) * a.max_splits + sx) * 2) = make_float2(M, L);
  }
  // ---- the last CTA of this (sequence, kv head) to finish merges the S partial results, in order
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int done = atomicAdd(&counters[b * a.NKV + kvh], 1);
    sm.is_last = (done == S - 1);
    if (sm.is_last) counters[b * a.NKV + kvh] = 0;
  }
  __syncthreads();
  if (!sm.is_last) return;
  __threadfence();
  if (warp < G) {
    const float2 *pm = reinterpret_cast<const float2 *>(part_ml + (size_t(b) * a.NQ + qh) * a.max_splits * 2);
    const float *po = part_o + (size_t(b) * a.NQ + qh) * a.max_splits * HD + 2 * lane;
    float Mm = __ldg(sinks + qh), Lm = 0.f, m0 = 0.f, m1 = 0.f;
#pragma unroll 1
    for (int s = 0; s < S; ++s) {
      const float2 ml = __ldcg(pm + s);
      const float2 pv = __ldcg(reinterpret_cast<const float2 *>(po + size_t(s) * HD));
      const float Mn = fmaxf(Mm, ml.x), f = __expf(Mm - Mn), w = __expf(ml.x - Mn);
      Lm = fmaf(ml.y, w, Lm * f);
      m0 = fmaf(pv.x, w, m0 * f);
      m1 = fmaf(pv.y, w, m1 * f);
      Mm = Mn;
    }
    Lm += __expf(__ldg(sinks + qh) - Mm);
    *reinterpret_cast<float2 *>(attn_out + size_t(b) * QD + size_t(qh) * HD + 2 * lane) = make_float2(m0 / Lm, m1 / Lm);
    if (a_tiled) attn_store_a(a_tiled, b, a.B, a.NQ, qh, lane, m0 / Lm, m1 / Lm);
  }
}
