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

// grid = (S, NKV, B), 256 threads, dynamic shared memory sizeof(AttnBatchSmem).
// part_o [B][NQ][max_splits][64], part_ml [B][NQ][max_splits][2], counters [B][NKV] (zero on entry, zero on exit).
extern "C" __global__ void __launch_bounds__(kAbThreads, 2)
attn_decode_batch(const float *__restrict__ qkv, const float *__restrict__ rope, const int *__restrict__ meta,
                  uint16_t *kcache, uint16_t *vcache, const float *__restrict__ sinks, float *__restrict__ part_o,
                  float *__restrict__ part_ml, int *__restrict__ counters, float *__restrict__ attn_out, AttnBatchArgs a) {
  AttnBatchSmem &sm = *reinterpret_cast<AttnBatchSmem *>(dyn_smem);
  constexpr int HD = 64, HALF = 32;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
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
  float M = -INFINITY, L = 0.f, o0 = 0.f, o1 = 0.f;      // warp = q head, lane = two dimensions
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
    __syncthreads();                                   // this slice's rows have landed for every thread; q is staged
    if (sl == nsplit - 1) {
      // the slice that ends at `pos` appends the new row (cache and shared memory)
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
      __syncthreads();
    }
    // ---- scores: thread = (position, half of the q heads)
    {
      const int p = tid >> 1, h0 = (tid & 1) * 4;
      if (p < nj) {
        float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
        for (int ch = 0; ch < 8; ++ch) {
          const uint4 kw = *reinterpret_cast<const uint4 *>(&sm.k[st][p][ch * 8]);
          const float kf[8] = {bf16_lo(kw.x), bf16_hi(kw.x), bf16_lo(kw.y), bf16_hi(kw.y),
                               bf16_lo(kw.z), bf16_hi(kw.z), bf16_lo(kw.w), bf16_hi(kw.w)};
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            const float4 q0 = *reinterpret_cast<const float4 *>(&sm.q[h0 + h][ch * 8]);
            const float4 q1 = *reinterpret_cast<const float4 *>(&sm.q[h0 + h][ch * 8 + 4]);
            float t = s[h];
            t = fmaf(q0.x, kf[0], t); t = fmaf(q0.y, kf[1], t); t = fmaf(q0.z, kf[2], t); t = fmaf(q0.w, kf[3], t);
            t = fmaf(q1.x, kf[4], t); t = fmaf(q1.y, kf[5], t); t = fmaf(q1.z, kf[6], t); t = fmaf(q1.w, kf[7], t);
            s[h] = t;
          }
        }
#pragma unroll
        for (int h = 0; h < 4; ++h) sm.s[h0 + h][p] = s[h];
      }
    }
    __syncthreads();
    // ---- running softmax and P V: warp = q head
    {
      float v[kAttnSplit / 32], m = -INFINITY;
#pragma unroll
      for (int i = 0; i < kAttnSplit / 32; ++i) {
        const int p = lane + 32 * i;
        v[i] = p < nj ? sm.s[warp][p] : -INFINITY;
        m = fmaxf(m, v[i]);
      }
      m = warp_max(m);
      const float Mn = fmaxf(M, m);
      const float f = (M == -INFINITY) ? 0.f : __expf(M - Mn);
      float l = 0.f;
#pragma unroll
      for (int i = 0; i < kAttnSplit / 32; ++i) {
        const int p = lane + 32 * i;
        const float e = p < nj ? __expf(v[i] - Mn) : 0.f;
        sm.s[warp][p] = e;
        l += e;
      }
      l = warp_sum(l);
      L = fmaf(L, f, l);
      M = Mn;
      __syncwarp();
      float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll 4
      for (int p = 0; p + 1 < nj; p += 2) {
        const float pa = sm.s[warp][p], pb = sm.s[warp][p + 1];
        const uint32_t va = *reinterpret_cast<const uint32_t *>(&sm.v[st][p][2 * lane]);
        const uint32_t vb = *reinterpret_cast<const uint32_t *>(&sm.v[st][p + 1][2 * lane]);
        a0 = fmaf(pa, bf16_lo(va), a0); a1 = fmaf(pa, bf16_hi(va), a1);
        b0 = fmaf(pb, bf16_lo(vb), b0); b1 = fmaf(pb, bf16_hi(vb), b1);
      }
      if (nj & 1) {
        const float pa = sm.s[warp][nj - 1];
        const uint32_t va = *reinterpret_cast<const uint32_t *>(&sm.v[st][nj - 1][2 * lane]);
        a0 = fmaf(pa, bf16_lo(va), a0); a1 = fmaf(pa, bf16_hi(va), a1);
      }
      o0 = fmaf(o0, f, a0 + b0);
      o1 = fmaf(o1, f, a1 + b1);
    }
    __syncthreads();                                   // scores and this stage are free for the next slice
  }
  const int qh = kvh * G + warp;
  if (S == 1) {
    if (warp < G) {
      const float sk = __ldg(sinks + qh);
      const float Mf = fmaxf(M, sk), f = __expf(M - Mf);
      const float Lf = fmaf(L, f, __expf(sk - Mf));
      *reinterpret_cast<float2 *>(attn_out + size_t(b) * QD + size_t(qh) * HD + 2 * lane) = make_float2(o0 * f / Lf, o1 * f / Lf);
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
  }
}
