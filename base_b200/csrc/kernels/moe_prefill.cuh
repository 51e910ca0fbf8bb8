// MXFP4 expert FFN for many tokens (prefill): a grouped GEMM on the 5th-gen
// tensor cores.
//
// Reference definition: per (token, expert) assignment the same expert FFN as in
// decode (lean/lib/AlgorithmLib/ML/Compose.lean:1798-1810, QuantMX.lean:131-186);
// with hundreds of tokens per expert the work is a contraction, the only dense
// one on this path, so it runs on tcgen05 instead of streaming GEMVs.
//
// One CTA computes D[up to 256 tokens x kPfN weight rows] for one (expert, token
// tile, weight tile) as two 128-row MMAs per K step that share the dequantised
// weight chunk: tokens are the M dimension (accumulator row = TMEM lane =
// token), so a thread's 16 consecutive accumulator columns are 16 consecutive
// weight rows: the gate/up pairs of the SwiGLU sit in one thread and the
// outputs of a token are written contiguously.
//   warps 0..11 per 64-column K step: gather the tokens' activation rows (bf16)
//               into the A stage with cp.async, load this tile's MXFP4 codes and
//               UE8M0 scale words (tiled layout of moe_tiled.cuh), dequantise
//               them exactly to bf16 (code x 2^(s-127) has two significant bits)
//               into the B stage, both in the K-major core-matrix layout of
//               tc_gemm.cuh; afterwards the epilogue (bias, clamped SwiGLU or
//               plain, stores).
//   warp 12     lane 0 waits for a full stage, issues four
//               tcgen05.mma.kind::f16 (K = 16 each) per token half and commits to the stage's
//               "empty" mbarrier; the accumulator lives in tensor memory.
// kPfStages stages of 56 KB; every wait is bounded (status word, then the CTA
// frees its tensor memory and leaves).
#pragma once
#include "tc_gemm.cuh"

constexpr int kPfM = 128;          // tokens per MMA (accumulator rows = TMEM lanes)
constexpr int kPfTok = 256;        // tokens per CTA tile: two MMAs share every dequantised weight chunk
constexpr int kPfN = 192;          // weight rows per CTA tile (12 tiles of 16 rows); divides 5760 and 2880
constexpr int kPfStages = 4;
constexpr int kPfWorkers = 384;    // 12 warps: one 16-byte code vector per thread and K step
constexpr int kPfThreads = kPfWorkers + 32;
constexpr int kPfLboA = kPfM * 16 + 16;            // column-group stride of the A tile: padded by 16 B so that the eight
                                                   // column groups of a token row (one gathered 128-byte line) fall into different banks
constexpr int kPfHalfA = 8 * kPfLboA;              // 16512 B: 128 tokens x 64 columns bf16
constexpr int kPfStageA = 2 * kPfHalfA;            // two token halves
constexpr int kPfLboB = kPfN * 16 + 32;            // B tile: padded by 32 B (a quarter-warp stores rows g, g+1 x four column groups)
constexpr int kPfStageB = 8 * kPfLboB;             // 24832 B
constexpr int kPfStageBytes = kPfStageA + kPfStageB;
constexpr int kPfAVec = (kPfTok * 8 + kPfWorkers - 1) / kPfWorkers;   // activation vectors per thread and K step (6)

struct PrefillArgs {
  int E;            // experts (the routing tables' layout depends on it)
  int K;            // reduction length (multiple of 64)
  int R;            // weight rows per expert (multiple of kPfN)
  int gate_up;      // 1: rows interleave gate/up, out = bf16 act [A][R/2]; 0: out = f32 [A][R]
  int top_k;
  float alpha, limit;
};

// route: the routing tables of moe_route_tables ([n_active][count E][offset E+1][active E][perm A]).
// tiles: [0] = number of token tiles, then per tile {expert, first slot in perm, tokens (1..kPfTok)}.
// xin: bf16 rows [.][K]; the row of assignment a is a / top_k (gate_up: the token's x) or a (down: act[a]).
template <bool GATE_UP>
B200_DEVICE void prefill_body(const uint4 *__restrict__ tcodes, const uint32_t *__restrict__ tscales,
                              const float *__restrict__ bias, const uint16_t *__restrict__ xin,
                              const int *__restrict__ route, const int *__restrict__ tiles, void *__restrict__ out,
                              int *__restrict__ status, const PrefillArgs &a) {
  const int *perm = route + 1 + a.E + (a.E + 1) + a.E;
  __shared__ uint64_t full[kPfStages], empty[kPfStages], done_bar;
  __shared__ uint32_t tmem_base;
  __shared__ int s_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wt = blockIdx.x, tt = blockIdx.y;
  if (tt >= tiles[0]) return;
  const int e = tiles[1 + 3 * tt], first = tiles[2 + 3 * tt], ntok = tiles[3 + 3 * tt];
  const int halves = ntok > kPfM ? 2 : 1;
  const int K = a.K, R = a.R, chunks = K / kChunkK, tiles16 = R / kTileRows;
  constexpr int kMmaWarp = kPfWorkers / 32;
  uint8_t *stage0 = dyn_smem;

  if (tid == 0) {
    for (int s = 0; s < kPfStages; ++s) { mbar_init(&full[s], kPfWorkers / 32); mbar_init(&empty[s], 1); }
    mbar_init(&done_bar, 1);
    s_abort = 0;
  }
  fence_barrier_init();
  if (warp == kMmaWarp) tc_alloc(&tmem_base, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_base;

  if (warp == kMmaWarp) {
    // ---- MMA issuer: accumulator of token half h in TMEM columns [256 h, 256 h + kPfN)
    if (lane == 0) {
      const uint32_t idesc = tc_idesc_bf16(kPfM, kPfN);
      for (int c = 0; c < chunks; ++c) {
        const int s = c % kPfStages;
        if (!tc_wait(&full[s], (c / kPfStages) & 1)) { atomicExch(status, 41); s_abort = 1; break; }
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(stage0 + s * kPfStageBytes), sb = sa + kPfStageA;
        for (int h = 0; h < halves; ++h) {
#pragma unroll
          for (int k16 = 0; k16 < 4; ++k16) {
            const uint64_t da = tc_smem_desc(sa + h * kPfHalfA + k16 * 2 * kPfLboA, kPfLboA, 128);
            const uint64_t db = tc_smem_desc(sb + k16 * 2 * kPfLboB, kPfLboB, 128);
            tc_mma_bf16(tmem + 256 * h, da, db, idesc, c > 0 || k16 > 0);
          }
        }
        tc_commit(&empty[s]);
      }
      tc_commit(&done_bar);
    }
  } else {
    // ---- workers: stage the operands
    // activations: 16-byte vectors v = tid + 384 j: token row (v >> 3) of the tile, column group (v & 7)
    const uint16_t *arow[kPfAVec];
    uint32_t adst[kPfAVec], asz[kPfAVec];
#pragma unroll
    for (int j = 0; j < kPfAVec; ++j) {
      const int v = tid + kPfWorkers * j, row = v >> 3, cg = v & 7;
      const bool in_tile = v < kPfTok * 8 && row < halves * kPfM;
      const int asg = (in_tile && row < ntok) ? perm[first + row] : 0;
      arow[j] = xin + size_t(GATE_UP ? asg / a.top_k : asg) * K + cg * 8;
      adst[j] = in_tile ? uint32_t((row >> 7) * kPfHalfA + cg * kPfLboA + (row & 127) * 16) : 0xffffffffu;
      asz[j] = (in_tile && row < ntok) ? 16u : 0u;      // rows past the tile's tokens are zero-filled
    }
    // weights: vector tid: 16-row tile (tid >> 5) of this CTA's 12, lane vector (tid & 31)
    const int t16 = tid >> 5, lv = tid & 31, g = lv >> 2, t = lv & 3;
    const size_t tile0 = (size_t(e) * tiles16 + size_t(wt) * (kPfN / kTileRows) + t16) * chunks;
    const uint4 *wsrc = tcodes + tile0 * 32 + lv;
    const uint32_t *ssrc = tscales + tile0 * 8 + g;
    // activations of step c -> stage c % kPfStages (cp.async, one group per step)
    auto gather = [&](int c) {
      const uint32_t sA = smem_u32(stage0 + (c % kPfStages) * kPfStageBytes);
#pragma unroll
      for (int j = 0; j < kPfAVec; ++j) {
        if (adst[j] != 0xffffffffu)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sA + adst[j]), "l"(arow[j] + c * kChunkK), "r"(asz[j])
                       : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // The weight stream is what has to be kept in flight (424 MB per layer): every thread holds
    // the codes and scales of the next kPfAhead steps in registers (kPfAhead x 20 B x 384 threads
    // = 30 KB per SM on the way at any time).
    constexpr int kPfAhead = 4;
    uint4 wq[kPfAhead];
    uint32_t sq[kPfAhead];
#pragma unroll
    for (int u = 0; u < kPfAhead; ++u) {
      wq[u] = make_uint4(0, 0, 0, 0);
      sq[u] = 0;
      if (u < chunks) {
        wq[u] = __ldcs(wsrc + size_t(u) * 32);
        sq[u] = __ldg(ssrc + size_t(u) * 8);
      }
    }
    bool alive = true;
    gather(0);
    if (chunks > 1) gather(1);
#pragma unroll 1
    for (int c0 = 0; c0 < chunks && alive; c0 += kPfAhead) {
#pragma unroll
      for (int u = 0; u < kPfAhead; ++u) {
        const int c = c0 + u;
        if (c < chunks && alive) {
          const int s = c % kPfStages;
          uint8_t *sB = stage0 + s * kPfStageBytes + kPfStageA;
          // dequantise this step's codes into the B stage, then refill the register slot
          const uint32_t words[4] = {wq[u].x, wq[u].y, wq[u].z, wq[u].w};
          const uint32_t sw = sq[u];
          if (c + kPfAhead < chunks) {
            wq[u] = __ldcs(wsrc + size_t(c + kPfAhead) * 32);
            sq[u] = __ldg(ssrc + size_t(c + kPfAhead) * 8);
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            // word q: row g + 8 (q & 1), 32-element block (q >> 1), elements 8t .. 8t+7; scale byte q
            const float sc = ue8m0_to_f32((sw >> (8 * q)) & 0xffu);
            float f[8];
            e2m1x8_to_f32(words[q], f);
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const __nv_bfloat162 b2 = __floats2bfloat162_rn(f[2 * i] * sc, f[2 * i + 1] * sc);
              o[i] = *reinterpret_cast<const uint32_t *>(&b2);
            }
            const int row = t16 * 16 + g + 8 * (q & 1), cg = 4 * (q >> 1) + t;
            *reinterpret_cast<uint4 *>(sB + cg * kPfLboB + row * 16) = make_uint4(o[0], o[1], o[2], o[3]);
          }
          // the next-but-one step's activations go out before this stage is handed over
          if (c + 2 < chunks) {
            const int s2 = (c + 2) % kPfStages;
            if (c + 2 >= kPfStages && !tc_wait(&empty[s2], ((c + 2) / kPfStages - 1) & 1)) {
              atomicExch(status, 42);
              alive = false;
            }
            if (alive) gather(c + 2);
          }
          // this step's activations have landed once at most the two younger groups are still in flight
          if (c + 2 < chunks) asm volatile("cp.async.wait_group 2;" ::: "memory");
          else if (c + 1 < chunks) asm volatile("cp.async.wait_group 1;" ::: "memory");
          else asm volatile("cp.async.wait_group 0;" ::: "memory");
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&full[s]);        // one arrival per warp: 12 instead of 384 updates of the barrier
        }
      }
    }
  }

  // ---- epilogue: thread = token (TMEM lane quarter warp % 4), a third of the columns per warp
  const bool ok = __syncthreads_and(warp == kMmaWarp ? 1 : tc_wait(&done_bar, 0)) && !s_abort;
  tc_fence_after_sync();
  if (ok && warp < kMmaWarp) {
    const int quarter = warp & 3, third = warp >> 2;
    const float *bp = bias + size_t(e) * R + size_t(wt) * kPfN;
    for (int h = 0; h < halves; ++h) {
      const int row = h * kPfM + quarter * 32 + lane;
      const bool valid = row < ntok;
      const int asg = valid ? perm[first + row] : 0;
#pragma unroll 1
      for (int c0 = third * 64; c0 < third * 64 + 64; c0 += 16) {
        float v[16];
        tc_ld16(tmem + 256 * h + (uint32_t(quarter * 32) << 16) + uint32_t(c0), v);
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] += __ldg(bp + c0 + j);
        if (!valid) continue;
        if (GATE_UP) {
          uint32_t o[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float y0 = swiglu_clamped(v[4 * i], v[4 * i + 1], a.alpha, a.limit);
            const float y1 = swiglu_clamped(v[4 * i + 2], v[4 * i + 3], a.alpha, a.limit);
            const __nv_bfloat162 b2 = __floats2bfloat162_rn(y0, y1);
            o[i] = *reinterpret_cast<const uint32_t *>(&b2);
          }
          uint16_t *dst = reinterpret_cast<uint16_t *>(out) + size_t(asg) * (R >> 1) + ((wt * kPfN + c0) >> 1);
          *reinterpret_cast<uint4 *>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
        } else {
          float *dst = reinterpret_cast<float *>(out) + size_t(asg) * R + wt * kPfN + c0;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            reinterpret_cast<float4 *>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        }
      }
    }
  } else if (!ok && tid == 0) {
    atomicCAS(status, 0, 43);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) tc_dealloc(tmem, 512);
}

extern "C" __global__ void __launch_bounds__(kPfThreads)
moe_prefill_gate_up(const uint4 *__restrict__ tcodes, const uint32_t *__restrict__ tscales,
                    const float *__restrict__ bias, const uint16_t *__restrict__ x_bf16, const int *__restrict__ route,
                    const int *__restrict__ tiles, uint16_t *__restrict__ act_bf16, int *__restrict__ status,
                    PrefillArgs a) {
  prefill_body<true>(tcodes, tscales, bias, x_bf16, route, tiles, act_bf16, status, a);
}

extern "C" __global__ void __launch_bounds__(kPfThreads)
moe_prefill_down(const uint4 *__restrict__ tcodes, const uint32_t *__restrict__ tscales,
                 const float *__restrict__ bias, const uint16_t *__restrict__ act_bf16, const int *__restrict__ route,
                 const int *__restrict__ tiles, float *__restrict__ o, int *__restrict__ status, PrefillArgs a) {
  prefill_body<false>(tcodes, tscales, bias, act_bf16, route, tiles, o, status, a);
}

// ---- routing for many tokens -----------------------------------------------------------------
// Router logits: logits[t][e] = Wr[e] . x[t] + br[e] (f32, same fold as moe_router_logits per
// row: lane-strided float4 walk, xor butterfly).  grid = ceil(T / 4) CTAs of 256 threads: a CTA
// stages four tokens in shared memory, warp w computes experts w, w + 8, ... (with grid.y > 1 the experts are
// divided among grid.y CTAs: many-token callers use grid.y = 1, the batched decode step grid.y = E / 8)
struct RouterManyArgs { int T, H, E; };

// NT tokens per CTA, EW experts per warp at a time.  Every (token, expert) pair walks the token's row in shared memory and
// the expert's row in L2: EW experts share one read of the token's row, NT tokens one read of the expert's row.  The
// per-lane sums and the fold of a pair are the same for any NT and EW, so the logits do not depend on them.
template <int NT, int EW>
B200_DEVICE void router_many_tokens(const float *__restrict__ Wr, const float *__restrict__ br, const float *__restrict__ x,
                                    float *__restrict__ logits, const RouterManyArgs &a) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t0 = blockIdx.x * NT, nt = min(NT, a.T - t0), n4 = a.H >> 2;
  float4 *xs = reinterpret_cast<float4 *>(dyn_smem);            // [NT][H]
  // x may have been written by another GPU while this kernel waited: read it through L2, not the read-only path
  for (int i = tid; i < nt * n4; i += 256) xs[i] = __ldcg(reinterpret_cast<const float4 *>(x + size_t(t0) * a.H) + i);
  __syncthreads();
  const int stride = 8 * gridDim.y;                             // grid.y CTAs share the experts
  for (int e0 = warp + 8 * blockIdx.y; e0 < a.E; e0 += stride * EW) {
    const float4 *w4[EW];
#pragma unroll
    for (int j = 0; j < EW; ++j) w4[j] = reinterpret_cast<const float4 *>(Wr + size_t(min(e0 + j * stride, a.E - 1)) * a.H);
    float acc[EW][NT];
#pragma unroll
    for (int j = 0; j < EW; ++j)
#pragma unroll
      for (int i = 0; i < NT; ++i) acc[j][i] = 0.f;
    for (int c = lane; c < n4; c += 32) {
      float4 w[EW];
#pragma unroll
      for (int j = 0; j < EW; ++j) w[j] = __ldg(w4[j] + c);
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        if (i < nt) {
          const float4 xv = xs[i * n4 + c];
#pragma unroll
          for (int j = 0; j < EW; ++j) {
            acc[j][i] = fmaf(w[j].x, xv.x, acc[j][i]); acc[j][i] = fmaf(w[j].y, xv.y, acc[j][i]);
            acc[j][i] = fmaf(w[j].z, xv.z, acc[j][i]); acc[j][i] = fmaf(w[j].w, xv.w, acc[j][i]);
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < EW; ++j) {
      const int e = e0 + j * stride;
      float mine = 0.f;
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const float v = warp_sum(acc[j][i]);
        if (lane == i) mine = v;
      }
      if (lane < nt && e < a.E) logits[size_t(t0 + lane) * a.E + e] = mine + br[e];
    }
  }
}

// The launch picks the form: grid.x = ceil(T / 8) (and 8 * H * 4 bytes of dynamic shared memory) means 8 tokens per CTA,
// else 4 (4 * H * 4 bytes); a warp with several experts to do (E / (8 x grid.y)) takes 4 (2 with 8 tokens) at a time.
B200_DEVICE void router_many_body(const float *__restrict__ Wr, const float *__restrict__ br, const float *__restrict__ x,
                                  float *__restrict__ logits, const RouterManyArgs &a) {
  const int per_warp = a.E / (8 * int(gridDim.y));
  if (a.T > 4 * int(gridDim.x)) {
    if (per_warp >= 2) router_many_tokens<8, 2>(Wr, br, x, logits, a);
    else router_many_tokens<8, 1>(Wr, br, x, logits, a);
  } else if (per_warp >= 4) {
    router_many_tokens<4, 4>(Wr, br, x, logits, a);
  } else {
    router_many_tokens<4, 1>(Wr, br, x, logits, a);
  }
}

extern "C" __global__ void __launch_bounds__(256)
moe_router_many(const float *__restrict__ Wr, const float *__restrict__ br, const float *__restrict__ x,
                float *__restrict__ logits, RouterManyArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  router_many_body(Wr, br, x, logits, a);
}

// Routing tables and the token-tile list for A = T * top_k assignments, one CTA of 1024 threads.
// Same tables as moe_route_tables (perm: assignments grouped by expert ascending, stable in the
// assignment index); tiles: [0] = n, then {expert, first slot, count <= kPfTok} per tile, experts
// ascending, an expert's tiles in slot order.  E <= 128.
struct TablesManyArgs { int A, E, lo, n; };   // token tiles only for experts [lo, lo + n) (expert-parallel ranks), numbered from lo

// topk_idx may have been written by this CTA just before (moe_topk_tables_many): it is read through L2
B200_DEVICE void route_tables_many_body(const int *topk_idx, int *__restrict__ route, int *__restrict__ tiles,
                                        const TablesManyArgs &a) {
  const int A = a.A, E = a.E, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int *n_active = route, *count = route + 1, *offset = route + 1 + E, *active = offset + E + 1, *perm = active + E;
  __shared__ int s_count[128], s_offset[129], s_run[128];
  __shared__ int s_warp[32][128];          // per chunk: assignments of expert e in warp w
  if (tid < 128) { s_count[tid] = 0; s_run[tid] = 0; }
  __syncthreads();
  for (int i = tid; i < A; i += 1024) atomicAdd(&s_count[__ldcg(topk_idx + i)], 1);      // integer counts: order-free
  __syncthreads();
  if (tid == 0) {
    int run = 0, na = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      s_offset[e] = run;
      if (s_count[e] > 0) active[na++] = e;
      for (int f = 0; f < s_count[e] && e >= a.lo && e < a.lo + a.n; f += kPfTok) {
        tiles[1 + 3 * nt] = e - a.lo;
        tiles[2 + 3 * nt] = run + f;
        tiles[3 + 3 * nt] = min(kPfTok, s_count[e] - f);
        ++nt;
      }
      run += s_count[e];
    }
    s_offset[E] = run;
    *n_active = na;
    for (int i = na; i < E; ++i) active[i] = -1;
    tiles[0] = nt;
  }
  __syncthreads();
  if (tid < E) count[tid] = s_count[tid];
  if (tid <= E) offset[tid] = s_offset[tid];
  // stable ranks, 1024 assignments at a time: rank inside the warp by matching lanes, then the
  // warps before this one in the chunk, then the chunks before (s_run)
  for (int base = 0; base < A; base += 1024) {
    const int i = base + tid;
    const int e = i < A ? __ldcg(topk_idx + i) : -1;
    for (int j = tid; j < 32 * 128; j += 1024) (&s_warp[0][0])[j] = 0;
    __syncthreads();
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int in_warp = __popc(same & ((1u << lane) - 1u));
    if (e >= 0 && in_warp == 0) s_warp[warp][e] = __popc(same);
    __syncthreads();
    if (e >= 0) {
      int before = 0;
      for (int w = 0; w < warp; ++w) before += s_warp[w][e];
      perm[s_offset[e] + s_run[e] + before + in_warp] = i;
    }
    __syncthreads();
    if (tid < E) {
      int tot = 0;
      for (int w = 0; w < 32; ++w) tot += s_warp[w][tid];
      s_run[tid] += tot;
    }
    __syncthreads();
  }
}

extern "C" __global__ void __launch_bounds__(1024)
moe_route_tables_many(const int *__restrict__ topk_idx, int *__restrict__ route, int *__restrict__ tiles,
                      TablesManyArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  route_tables_many_body(topk_idx, route, tiles, a);
}

// Top-k + softmax (one warp per token, as moe_topk_softmax) and the routing tables (count / offset / active / perm, as
// moe_route_tables_many, without the token-tile list) in ONE CTA of 1024 threads, for the batched decode step:
// A = T * top_k <= kTtMaxA assignments.  The indices stay in shared memory; counts by shared-memory atomics (integers:
// order-free), warp 0 scans them, then a warp per expert walks the assignments 32 at a time with ballots and writes the
// permutation (stable in the assignment index by construction, no per-warp histograms).
constexpr int kTtMaxA = 4096;
struct TopkTablesArgs { MoeDims d; TablesManyArgs t; int do_topk; };   // do_topk = 0: topk_idx was written by moe_topk_softmax (many tokens: a warp each, in parallel)

extern "C" __global__ void __launch_bounds__(1024)
moe_topk_tables_many(const float *__restrict__ logits, int *__restrict__ topk_idx, float *__restrict__ topk_w,
                     int *__restrict__ route, TopkTablesArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ int s_idx[kTtMaxA];
  __shared__ int s_count[128], s_offset[129];
  const int A = a.t.A, E = a.t.E, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int T = A / a.d.top_k;
  int *n_active = route, *count = route + 1, *offset = route + 1 + E, *active = offset + E + 1, *perm = active + E;
  if (a.do_topk) {
    for (int t = warp; t < T; t += 32) topk_softmax_token(logits, topk_idx, topk_w, a.d, t, lane, s_idx);
  } else {
    for (int i = tid; i < A; i += 1024) s_idx[i] = __ldcg(topk_idx + i);
  }
  if (tid < 128) s_count[tid] = 0;
  __syncthreads();
  for (int i = tid; i < A; i += 1024) atomicAdd(&s_count[s_idx[i]], 1);          // integer counts: order-free
  __syncthreads();
  if (warp == 0) {
    int run = 0, na = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane, c = e < E ? s_count[e] : 0;
      int inc = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
      }
      if (e < E) { s_offset[e] = run + inc - c; offset[e] = run + inc - c; count[e] = c; }
      const unsigned act = __ballot_sync(0xffffffffu, c > 0);
      if (c > 0) active[na + __popc(act & ((1u << lane) - 1u))] = e;
      na += __popc(act);
      run += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) { s_offset[E] = run; offset[E] = run; *n_active = na; }
    for (int i = na + lane; i < E; i += 32) active[i] = -1;
  }
  __syncthreads();
  // warp w writes the permutation of experts w, w + 32, w + 64, w + 96 in one walk over the assignments
  int at[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) at[j] = warp + 32 * j < E ? s_offset[warp + 32 * j] : 0;
  const unsigned below = (1u << lane) - 1u;
  for (int base = 0; base < A; base += 32) {
    const int e = base + lane < A ? s_idx[base + lane] : -1;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool mine = e == warp + 32 * j;
      const unsigned m = __ballot_sync(0xffffffffu, mine);
      if (mine) perm[at[j] + __popc(m & below)] = base + lane;
      at[j] += __popc(m);
    }
  }
}

// f32 rows -> bf16 (round to nearest even), 8 elements per thread.
struct CvtArgs { long long n8; };

extern "C" __global__ void __launch_bounds__(256)
f32_to_bf16_vec(const float4 *__restrict__ src, uint4 *__restrict__ dst, CvtArgs a) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= a.n8) return;
  const float4 v0 = src[2 * i], v1 = src[2 * i + 1];
  const __nv_bfloat162 b0 = __floats2bfloat162_rn(v0.x, v0.y), b1 = __floats2bfloat162_rn(v0.z, v0.w);
  const __nv_bfloat162 b2 = __floats2bfloat162_rn(v1.x, v1.y), b3 = __floats2bfloat162_rn(v1.z, v1.w);
  dst[i] = make_uint4(*reinterpret_cast<const uint32_t *>(&b0), *reinterpret_cast<const uint32_t *>(&b1),
                      *reinterpret_cast<const uint32_t *>(&b2), *reinterpret_cast<const uint32_t *>(&b3));
}

// Combine restricted to the experts [lo, lo + n) a rank owns: y[t] = sum over the token's slots j whose
// expert is local of w[t][j] * o[t*k + j], slot order (the other ranks add theirs; the sum over ranks is
// the layer's output, lean/lib/AlgorithmLib/ML/Compose.lean:1803-1828).
struct CombineRangeArgs { int H, top_k, lo, n; };

extern "C" __global__ void __launch_bounds__(256)
moe_combine_range(const float *__restrict__ o, const float *__restrict__ topk_w, const int *__restrict__ topk_idx,
                  float *__restrict__ y, CombineRangeArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= a.H) return;
  float v = 0.f;
  for (int j = 0; j < a.top_k; ++j) {
    const int e = topk_idx[t * a.top_k + j];
    if (e >= a.lo && e < a.lo + a.n) v = fmaf(topk_w[t * a.top_k + j], o[size_t(t * a.top_k + j) * a.H + i], v);
  }
  y[size_t(t) * a.H + i] = v;
}
