// Streaming MXFP4 expert GEMV/GEMM for decode-sized token counts.
//
// Same math and the same tiled weight layout as moe_tiled.cuh; what changes
// is how the bytes reach the SM.  Every warp is an independent streaming
// engine: it owns whole 16-row tiles (no split of K, so no cross-warp
// reduction and no CTA-wide barrier in the hot loop) and pulls them through a
// private ring of shared-memory sub-stages with bulk asynchronous copies
// (cp.async.bulk, completion on an mbarrier).  A sub-stage is kSubChunks
// 64-element chunks of one tile: kSubChunks * 512 B of codes followed by
// kSubChunks * 32 B of UE8M0 scale words.  The activations are split into f16
// hi/lo columns ONCE by the producing kernel (xh), and a CTA stages the
// columns of its expert slot with bulk copies too, so there is no per-tile
// prologue at all.
//
// grid = (G, slots).  CTA (b, slot) serves expert active[slot]; its warps take
// tiles gw, gw + G*W, ... with gw = b*W + warp.  Any number of warps per CTA
// (blockDim.x / 32) as long as the dynamic shared memory is sized for it.
//
// Every wait on an mbarrier is bounded: after kSpinLimit failed polls the
// warp records an error code in *status and leaves the kernel.
#pragma once
#include "moe_tiled.cuh"
#include "dense_decode.cuh"

constexpr int kSubChunks = 9;
constexpr int kMaxRingStages = 8;
constexpr int kSubBytes = kSubChunks * (512 + 32);   // 4896
constexpr uint32_t kSpinLimit = 4u << 20;

B200_DEVICE uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

B200_DEVICE void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
B200_DEVICE void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
B200_DEVICE bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok)
               : "r"(smem_u32(bar)), "r"(parity)
               : "memory");
  return ok != 0;
}
// Bounded wait; false on timeout.
B200_DEVICE bool mbar_wait(uint64_t *bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// Plain bulk copy global -> this CTA's shared memory (one destination CTA).
B200_DEVICE void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
B200_DEVICE void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

B200_DEVICE void mma_f16_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                              uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

B200_DEVICE void block_mma2(uint32_t w_lo, uint32_t w_hi, const uint4 &xb, float s_lo, float s_hi,
                            float (&acc)[4]) {
  uint32_t l0, l1, l2, l3, h0, h1, h2, h3;
  cvt_e2m1x8(w_lo, l0, l1, l2, l3);
  cvt_e2m1x8(w_hi, h0, h1, h2, h3);
  float d[4];
  mma_f16_zero(d, l0, h0, l1, h1, xb.x, xb.y);
  mma_f16(d, l2, h2, l3, h3, xb.z, xb.w);
  acc[0] = fmaf(s_lo, d[0], acc[0]);
  acc[1] = fmaf(s_lo, d[1], acc[1]);
  acc[2] = fmaf(s_hi, d[2], acc[2]);
  acc[3] = fmaf(s_hi, d[3], acc[3]);
}

struct StreamArgs {
  MoeDims d;
  int exact;      // 1: two f16 columns (hi, lo) per assignment; 0: one
  int xcols;      // activation columns the shared-memory layout reserves (2..8, even)
  int stages;     // sub-stages in each warp's ring (1..kMaxRingStages)
};

// Shared memory: [x columns: xcols * xs_stride(K) halves][rings: W * stages * kSubBytes][barriers]
B200_DEVICE int stream_x_bytes(int K, int xcols) { return xcols * xs_stride(K) * 2; }

// gate_up reads its activations as f32 rows x32[token][K] and splits them into
// f16 hi/lo columns itself; it writes the SwiGLU outputs both as f32 and as
// act_h[a][2][I] f16 ([.][0] = f16(v), [.][1] = f16(v - hi)), which is what
// down stages with bulk copies.
template <bool GATE_UP>
B200_DEVICE void stream_kernel(const uint4 *__restrict__ tcodes, const uint32_t *__restrict__ tscales,
                               const float *__restrict__ bias, const float *__restrict__ x32,
                               const __half *__restrict__ xh, const int *__restrict__ route,
                               float *__restrict__ out,
                               __half *__restrict__ out_h, int *__restrict__ status, const StreamArgs &sa) {
  const MoeDims d = sa.d;
  const int K = GATE_UP ? d.H : d.I;
  const int R = GATE_UP ? 2 * d.I : d.H;
  const int E = d.E;
  const int chunks = K / kChunkK, tiles = R / kTileRows;
  const int subs = (chunks + kSubChunks - 1) / kSubChunks;
  const int slot = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, W = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int kRingStages = sa.stages;

  __half *xs = reinterpret_cast<__half *>(dyn_smem);
  uint8_t *ring = dyn_smem + stream_x_bytes(K, sa.xcols) + size_t(warp) * kRingStages * kSubBytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(dyn_smem + stream_x_bytes(K, sa.xcols) + size_t(W) * kRingStages * kSubBytes);
  uint64_t *xbar = bars;
  uint64_t *full = bars + 1 + warp * kRingStages;

  if (tid == 0) mbar_init(xbar, 1);
  if (lane == 0) {
    for (int s = 0; s < kRingStages; ++s) mbar_init(full + s, 1);
  }
  fence_barrier_init();
  __syncthreads();

  // gate_up: the routing table comes from the kernel just before, so wait now.
  // down: the table is two kernels back and complete before this grid can
  // start (its predecessor releases its dependents only after its own wait),
  // so the weights are requested first and the wait comes before `act_h`.
  if (GATE_UP) {
    pdl_wait();
    pdl_launch_dependents();
  }
  const int *count = route + 1, *offset = route + 1 + E, *active = offset + E + 1, *perm = active + E;
  if (slot >= route[0]) {
    if (!GATE_UP) { pdl_wait(); pdl_launch_dependents(); }
    return;
  }
  const int e = active[slot];
  const int n_assign = count[e], base = offset[e];
  const uint8_t *tc = reinterpret_cast<const uint8_t *>(tcodes) + size_t(e) * tiles * chunks * 512;
  const uint8_t *ts = reinterpret_cast<const uint8_t *>(tscales) + size_t(e) * tiles * chunks * 32;
  const int gw = blockIdx.x * W + warp, GW = gridDim.x * W;
  const int my_tiles = (gw < tiles) ? (tiles - gw + GW - 1) / GW : 0;
  const int total_sub = my_tiles * subs;
  const int per_pass = sa.exact ? sa.xcols / 2 : sa.xcols;
  uint32_t qbase = 0;   // sub-stages issued by this warp in earlier passes
  const __half *xcol = xs + size_t(g) * xs_stride(K) + 8 * t;

  auto issue = [&](int q) {
    const int tile = gw + (q / subs) * GW, sub = q % subs;
    const int c0 = sub * kSubChunks, n = min(kSubChunks, chunks - c0);
    const int s = (qbase + q) % kRingStages;
    uint8_t *dst = ring + s * kSubBytes;
    mbar_expect_tx(full + s, n * 544);
    bulk_g2s(dst, tc + (size_t(tile) * chunks + c0) * 512, n * 512, full + s);
    bulk_g2s(dst + kSubChunks * 512, ts + (size_t(tile) * chunks + c0) * 32, n * 32, full + s);
  };

  int pass = 0;
  for (int p0 = 0; p0 < n_assign; p0 += per_pass, ++pass) {
    const int np = min(per_pass, n_assign - p0);
    const int ncols = sa.exact ? 2 * np : np;
    if (pass > 0) __syncthreads();     // every warp is done with the previous columns
    // Weights first: they do not depend on the activations.
    if (lane == 0) {
      for (int q = 0; q < min(kRingStages, total_sub); ++q) issue(q);
    }
    if (GATE_UP) {
      // x arrives as f32 rows; split into f16 hi/lo columns here (once per CTA).
      for (int c = 0; c < np; ++c) {
        const int a = perm[base + p0 + c];
        const float *xt = x32 + size_t(a / d.top_k) * K;
        if (sa.exact) {
          stage_x_split(xt, K, xs + size_t(2 * c) * xs_stride(K), xs + size_t(2 * c + 1) * xs_stride(K), tid,
                        blockDim.x);
        } else {
          for (int i = tid; i < K; i += blockDim.x) xs[size_t(c) * xs_stride(K) + i] = __float2half_rn(xt[i]);
        }
      }
      __syncthreads();
    } else {
      if (pass == 0) {
        pdl_wait();
        pdl_launch_dependents();
      }
      if (tid == 0) {
        mbar_expect_tx(xbar, ncols * K * 2);
        for (int c = 0; c < ncols; ++c) {
          const int a = perm[base + p0 + (sa.exact ? (c >> 1) : c)];
          const __half *src = xh + (size_t(a) * 2 + (sa.exact ? (c & 1) : 0)) * K;
          bulk_g2s(xs + size_t(c) * xs_stride(K), src, K * 2, xbar);
        }
      }
      if (!mbar_wait(xbar, pass & 1)) {
        if (lane == 0) atomicExch(status, 1);
        return;
      }
    }
    const bool has_col = g < ncols;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int q = 0; q < total_sub; ++q) {
      const int s = (qbase + q) % kRingStages;
      const uint32_t parity = ((qbase + q) / kRingStages) & 1;
      if (!mbar_wait(full + s, parity)) {
        if (lane == 0) atomicExch(status, 2);
        return;
      }
      const int tile = gw + (q / subs) * GW, sub = q % subs;
      const int c0 = sub * kSubChunks, n = min(kSubChunks, chunks - c0);
      const uint8_t *buf = ring + s * kSubBytes;
      const uint4 *wv = reinterpret_cast<const uint4 *>(buf) + lane;
      const uint32_t *sv = reinterpret_cast<const uint32_t *>(buf + kSubChunks * 512) + g;
#pragma unroll 3
      for (int i = 0; i < n; ++i) {
        const uint4 w = wv[i * 32];
        const uint32_t sw = sv[i * 8];
        uint4 xa = make_uint4(0, 0, 0, 0), xb = make_uint4(0, 0, 0, 0);
        if (has_col) {
          xa = *reinterpret_cast<const uint4 *>(xcol + (c0 + i) * kChunkK);
          xb = *reinterpret_cast<const uint4 *>(xcol + (c0 + i) * kChunkK + 32);
        }
        block_mma2(w.x, w.y, xa, scale_fast<0>(sw), scale_fast<1>(sw), acc);
        block_mma2(w.z, w.w, xb, scale_fast<2>(sw), scale_fast<3>(sw), acc);
      }
      __syncwarp();
      if (lane == 0 && q + kRingStages < total_sub) issue(q + kRingStages);
      if (sub == subs - 1) {
        // ---- epilogue for `tile`: lane holds rows g, g+8 x columns 2t, 2t+1
        const int r0 = tile * kTileRows;
        const float b_lo = bias[size_t(e) * R + r0 + g], b_hi = bias[size_t(e) * R + r0 + g + 8];
        float v[2][2];   // [row half][assignment within lane]
        int na;          // assignments this lane holds
        int a_idx[2];
        if (sa.exact) {
          v[0][0] = acc[0] + acc[1] + b_lo;
          v[1][0] = acc[2] + acc[3] + b_hi;
          v[0][1] = v[1][1] = 0.f;
          na = 1;
          a_idx[0] = t; a_idx[1] = -1;
        } else {
          v[0][0] = acc[0] + b_lo; v[0][1] = acc[1] + b_lo;
          v[1][0] = acc[2] + b_hi; v[1][1] = acc[3] + b_hi;
          na = 2;
          a_idx[0] = 2 * t; a_idx[1] = 2 * t + 1;
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          if (j < na) {
            const bool valid = a_idx[j] < np;
            const int a = valid ? perm[base + p0 + a_idx[j]] : 0;
            if (GATE_UP) {
              // gate rows are even, up rows odd: the partner sits 4 lanes up
              const float u_lo = __shfl_down_sync(0xffffffffu, v[0][j], 4);
              const float u_hi = __shfl_down_sync(0xffffffffu, v[1][j], 4);
              if (valid && (g & 1) == 0) {
                const float y_lo = swiglu_clamped(v[0][j], u_lo, d.alpha, d.limit);
                const float y_hi = swiglu_clamped(v[1][j], u_hi, d.alpha, d.limit);
                const int i_lo = (r0 + g) >> 1, i_hi = (r0 + g + 8) >> 1;
                out[size_t(a) * d.I + i_lo] = y_lo;
                out[size_t(a) * d.I + i_hi] = y_hi;
                const __half h_lo = __float2half_rn(y_lo), h_hi = __float2half_rn(y_hi);
                __half *oh = out_h + size_t(a) * 2 * d.I;
                oh[i_lo] = h_lo;
                oh[i_hi] = h_hi;
                oh[d.I + i_lo] = __float2half_rn(y_lo - __half2float(h_lo));
                oh[d.I + i_hi] = __float2half_rn(y_hi - __half2float(h_hi));
              }
            } else if (valid) {
              out[size_t(a) * R + r0 + g] = v[0][j];
              out[size_t(a) * R + r0 + g + 8] = v[1][j];
            }
          }
        }
        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
      }
    }
    qbase += total_sub;
  }
}

extern "C" __global__ void __launch_bounds__(512)
moe_gate_up_stream(const uint4 *__restrict__ tcodes, const uint32_t *__restrict__ tscales,
                   const float *__restrict__ bias, const float *__restrict__ x,
                   const int *__restrict__ route, float *__restrict__ act, __half *__restrict__ act_h,
                   int *__restrict__ status, StreamArgs sa) {
  stream_kernel<true>(tcodes, tscales, bias, x, nullptr, route, act, act_h, status, sa);
}

extern "C" __global__ void __launch_bounds__(512)
moe_down_stream(const uint4 *__restrict__ tcodes, const uint32_t *__restrict__ tscales,
                const float *__restrict__ bias, const __half *__restrict__ act_h,
                const int *__restrict__ route, float *__restrict__ o, int *__restrict__ status,
                StreamArgs sa) {
  stream_kernel<false>(tcodes, tscales, bias, nullptr, act_h, route, o, nullptr, status, sa);
}

// ---- router + top-k + routing tables in one launch -------------------------------------------
// grid = E CTAs of 128 threads.  CTA e: (optional RMSNorm of every token,
// recomputed per CTA), logits[t][e] = Wr[e] . x[t] + br[e]; CTA 0 also writes
// the normalised rows to xn.  The CTA that finishes last (atomic ticket) runs
// the integer part for all tokens: top-k by (logit desc, expert id asc),
// softmax over the k selected logits, then the routing tables of
// moe_route_tables.  Every logit is produced by exactly one CTA in a fixed
// order, so the result does not depend on which CTA is last.
struct RouteArgs {
  MoeDims d;
  int norm;        // 1: x = rmsnorm(in) * g, eps below
  float eps;
};

extern "C" __global__ void __launch_bounds__(128)
moe_route_fused(const float *__restrict__ in, const float *__restrict__ g, const float *__restrict__ Wr,
                const float *__restrict__ br, float *__restrict__ xn, float *__restrict__ logits,
                int *__restrict__ topk_idx, float *__restrict__ topk_w, int *__restrict__ route,
                int *__restrict__ ticket, RouteArgs ra) {
  const MoeDims d = ra.d;
  const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int H = d.H, E = d.E, k = d.top_k, A = d.T * d.top_k;
  __shared__ float red[33];
  __shared__ int s_last;
  __shared__ int s_count[128];
  __shared__ int s_offset[129];
  // The router row and the norm weights do not depend on the previous kernel:
  // fetch them before the dependency wait.  H <= 3072 (6 float4 per thread).
  constexpr int kV = 6;
  const int n4 = H >> 2;
  const float4 *w4 = reinterpret_cast<const float4 *>(Wr + size_t(e) * H);
  float4 wv[kV], gv[kV];
#pragma unroll
  for (int u = 0; u < kV; ++u) {
    const int c = tid + u * 128;
    wv[u] = c < n4 ? __ldg(w4 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    gv[u] = (ra.norm && c < n4) ? __ldg(reinterpret_cast<const float4 *>(g) + c) : make_float4(1.f, 1.f, 1.f, 1.f);
  }
  const float bias_e = br[e];
  pdl_wait();
  pdl_launch_dependents();
  for (int t = 0; t < d.T; ++t) {
    const float4 *x4 = reinterpret_cast<const float4 *>(in + size_t(t) * H);
    float4 xv[kV];
#pragma unroll
    for (int u = 0; u < kV; ++u) {
      const int c = tid + u * 128;
      xv[u] = c < n4 ? x4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float inv = 1.f;
    if (ra.norm) {
      float ss = 0.f;
#pragma unroll
      for (int u = 0; u < kV; ++u) {
        ss = fmaf(xv[u].x, xv[u].x, ss); ss = fmaf(xv[u].y, xv[u].y, ss);
        ss = fmaf(xv[u].z, xv[u].z, ss); ss = fmaf(xv[u].w, xv[u].w, ss);
      }
      inv = 1.0f / sqrtf(block_sum(ss, red) / float(H) + ra.eps);
    }
    float acc = 0.f;
#pragma unroll
    for (int u = 0; u < kV; ++u) {
      const int c = tid + u * 128;
      float4 v = xv[u];
      if (ra.norm) {
        v.x = v.x * inv * gv[u].x; v.y = v.y * inv * gv[u].y; v.z = v.z * inv * gv[u].z; v.w = v.w * inv * gv[u].w;
      }
      if (e == 0 && xn && c < n4) reinterpret_cast<float4 *>(xn + size_t(t) * H)[c] = v;
      acc = fmaf(wv[u].x, v.x, acc); acc = fmaf(wv[u].y, v.y, acc);
      acc = fmaf(wv[u].z, v.z, acc); acc = fmaf(wv[u].w, v.w, acc);
    }
    const float tot = block_sum(acc, red);
    if (tid == 0) logits[size_t(t) * E + e] = tot + bias_e;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int done = atomicAdd(ticket, 1);
    s_last = (done == E - 1);
    if (s_last) *ticket = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // ---- top-k, one warp per token
  for (int t = warp; t < d.T; t += 4) {
    float v[4];
    bool taken[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int ee = lane + 32 * i;
      const float l = (ee < E) ? __ldcg(logits + size_t(t) * E + ee) : -INFINITY;
      v[i] = (l == l) ? l : -INFINITY;
      taken[i] = ee >= E;
    }
    float sel_v[8];
    int sel_e[8];
    for (int j = 0; j < k && j < 8; ++j) {
      float bv = -INFINITY;
      int be = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int ee = lane + 32 * i;
        if (!taken[i] && (be == 0x7fffffff || v[i] > bv || (v[i] == bv && ee < be))) { bv = v[i]; be = ee; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oe = __shfl_xor_sync(0xffffffffu, be, o);
        if (oe != 0x7fffffff && (be == 0x7fffffff || ov > bv || (ov == bv && oe < be))) { bv = ov; be = oe; }
      }
      sel_v[j] = bv;
      sel_e[j] = (be == 0x7fffffff) ? 0 : be;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (lane + 32 * i == be) taken[i] = true;
    }
    if (lane == 0) {
      float ex[8], sum = 0.f;
      for (int j = 0; j < k && j < 8; ++j) { ex[j] = __expf(sel_v[j] - sel_v[0]); sum += ex[j]; }
      for (int j = 0; j < k && j < 8; ++j) {
        topk_idx[size_t(t) * k + j] = sel_e[j];
        topk_w[size_t(t) * k + j] = ex[j] / sum;
      }
    }
  }
  __syncthreads();
  // ---- routing tables (same layout and order as moe_route_tables)
  int *n_active = route, *count = route + 1, *offset = route + 1 + E, *active = offset + E + 1,
      *perm = active + E;
  if (tid < E) {
    int c = 0;
    for (int a = 0; a < A; ++a) c += (topk_idx[a] == tid);
    s_count[tid] = c;
  }
  __syncthreads();
  if (tid == 0) {
    int run = 0, na = 0;
    for (int ee = 0; ee < E; ++ee) {
      s_offset[ee] = run;
      run += s_count[ee];
      if (s_count[ee] > 0) active[na++] = ee;
    }
    s_offset[E] = run;
    *n_active = na;
    for (int i = na; i < E; ++i) active[i] = -1;
  }
  __syncthreads();
  if (tid < E) count[tid] = s_count[tid];
  if (tid <= E) offset[tid] = s_offset[tid];
  for (int a = tid; a < A; a += 128) {
    const int ee = topk_idx[a];
    int rank = 0;
    for (int b = 0; b < a; ++b) rank += (topk_idx[b] == ee);
    perm[s_offset[ee] + rank] = a;
  }
}
