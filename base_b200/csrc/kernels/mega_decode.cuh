// One persistent kernel for a whole gpt-oss decode step (batch 1).
//
// The step is ~150 dependent GEMV-sized operations of 0.2-35 MB each.  As
// separate launches every one of them pays a drain, a launch and a refill of
// the memory pipeline; measured in place they cost 8-24 us each where the
// bytes alone need 3-7 us.  Here the step is ONE cooperative launch of one
// CTA per SM:
//   * warp 15 is the producer.  It walks the step's weight stream in order
//     (qkv, o-proj, experts' gate_up and down of every layer, lm_head) and
//     keeps a ring of kMegaSlots x 24 KB shared-memory slots filled with
//     cp.async.bulk copies, completion on one mbarrier per slot.  It runs
//     ahead of the consumers across phase boundaries, so HBM keeps streaming
//     while the CTAs meet at a grid barrier; only the experts' gate_up has to
//     wait for data (the router's choice).
//   * warps 0..14 are consumers.  Every CTA owns a contiguous range of output
//     rows (dense) or 16-row tiles (MXFP4) of each operation; its 15 warps
//     split K, so the activations a lane needs sit in registers for the whole
//     phase, and partial sums meet in shared memory every 64 rows.
//   * phases are separated by a grid barrier (one atomic per CTA on a counter
//     that the host zeroes before the launch, then a bounded spin).
// Math, layouts and reference citations are those of the per-operation
// kernels (dense_decode.cuh, attn_decode.cuh, moe_tiled.cuh, moe_stream.cuh);
// only the summation order over K differs (15 slices instead of one walk).
// The code is kept small on purpose (single copy of every consumer loop, rolled
// attention): a first version of 288 KB missed the instruction cache on every
// phase and was 1.6 x slower than this one.
//
// Every wait is bounded.  A wait that runs out stores a code in *status,
// marks the CTA as aborted (later waits give up quickly) and the kernel runs
// to its end without touching out-of-range memory; the host reports the code.
#pragma once
#include "attn_decode.cuh"
#include "moe_mx.cuh"
#include "moe_stream.cuh"

// 15 consumer warps + the producer = 16 warps: 128 registers per thread, and
// K = 2880 splits evenly (45 chunks of 64 = 15 x 3; 360 16-byte vectors = 15 x 24).
constexpr int kMegaConsumers = 15;
constexpr int kMegaThreads = (kMegaConsumers + 1) * 32;      // 512
constexpr int kMegaConsThreads = kMegaConsumers * 32;        // 480
constexpr int kMegaSlots = 7;
constexpr int kMegaSlotBytes = 25088;     // 4 dense rows of K <= 3072 (3 of K = 4096), a 16-row MXFP4 tile, or half a 32-row mx tile
static_assert(kMegaSlotBytes == kMxSlotBytes, "the block-scaled expert path shares the ring");
constexpr uint32_t kMegaSpin = 1u << 20;
constexpr int kMegaMaxTopK = 8;
// Attention inside the step kernel: warps 0..7 work on one (slice, kv head) unit.
constexpr int kMegaAttnWarps = 8;

// Device pointers of one layer / of the step, filled by the host (all 8 bytes wide).
struct MegaLayer {
  const float *ln1; const uint16_t *wqkv; const float *bqkv; const float *sinks;
  const uint16_t *wo; const float *bo; const float *ln2; const float *wr; const float *br;
  const uint8_t *gu_codes; const uint8_t *gu_scales; const float *gu_bias;
  const uint8_t *dn_codes; const uint8_t *dn_scales; const float *dn_bias;
  void *kcache; void *vcache;
  long long cache_len; long long window;
};
static_assert(sizeof(MegaLayer) == 19 * 8, "host mirror assumes 19 x 8 bytes");

struct MegaGlobals {
  const uint16_t *embed; const uint16_t *lm_head; const float *lnf; const float *rope;
  int *meta; float *hA; float *hB; float *qkv; float *attn; float *part_o; float *part_ml; int *counters;
  float *xn; float *rlogits; int *topk_idx; float *topk_w; int *route; float *act; float *o; float *logits;
  int *next_tok; float *am_v; int *am_i; unsigned *sync; int *status;
  const MegaLayer *layers;
  unsigned long long *trace;    // optional: [gridDim.x][kMegaTraceLen] phase time stamps (ns), else null
  float *rpart;                 // [gridDim.x][E rounded up to 32]: per-CTA partial router sums
};
static_assert(sizeof(MegaGlobals) == 28 * 8, "host mirror assumes 28 x 8 bytes");
constexpr int kMegaTraceLen = 512;

struct MegaArgs {
  int layers, H, I, E, top_k, NQ, NKV, V, max_seq;
  float eps, alpha, limit, attn_scale;
  int max_splits;
  int mx;          // 1: expert weights are in the wide block-scaled layout (moe_mx.cuh) and run on the tensor cores
  int kc_gu, kc_dn;   // its chunk sizes (K blocks per ring slot) for gate_up and down
  // Failure-path test hooks (0 in production): the producers leave out ring fill number test_skip_fill - 1, so
  // that the consumers' wait for it runs out; spin = iteration limit of every wait (0: kMegaSpin).
  int test_skip_fill;
  unsigned spin;
};

// One attention unit: kAttnSplit cache rows of a kv head (bf16, padded to 144
// bytes so that 16-byte reads of consecutive rows do not collide), the group's
// rotated q, scores / probabilities.
struct alignas(16) MegaAttnSmem {
  uint16_t k[kAttnSplit][72];
  uint16_t v[kAttnSplit][72];
  float q[kAttnMaxGroup][64];
  float s[kAttnMaxGroup][kAttnSplit];
  int is_last;
};

// Block-scaled expert phases: the staged f32 vector (same place as `xs`), the A operands (8 digit
// rows per K block) of at most two expert slots with the rows the tensor core reads beyond them,
// and the digits' scale bytes [term][96].
struct alignas(16) MegaMxSmem {
  float xs[4096];
  uint8_t a[2][(kMxMaxK / 32) * 128 + 2048];
  uint8_t sf[2][768];
};

struct alignas(16) MegaSmem {
  uint64_t full[kMegaSlots];
  uint64_t empty[kMegaSlots];
  uint64_t route_bar;
  float red[32];
  float part[2][kMegaConsumers][64];
  int r_active[kMegaMaxTopK];     // expert of slot s (ascending expert id)
  int r_assign[kMegaMaxTopK];     // top-k rank of slot s
  float r_gate[kMegaMaxTopK];     // gate of top-k rank j
  int r_sel[kMegaMaxTopK];        // expert of top-k rank j
  int abort;
  uint32_t spin;                  // iteration limit of every wait
  float racc[128];                // router partial sums of this CTA's o-proj rows, per expert
  float rrow[64];                 // h1 values of the super group being finished
  float am_v[2];
  int am_i[2];
  uint64_t done[3];               // block-scaled path: completed by tcgen05.commit when a phase's instructions are done
  uint64_t sready[kMegaSlots];    // block-scaled path: the slot's scale words are in tensor memory (warp 4 -> warp 0)
  uint32_t tmem_base;
  union alignas(16) {
    MegaAttnSmem attn;
    float xs[4096];
    MegaMxSmem mx;
  } u;
};

static_assert(sizeof(MegaSmem) <= 56832, "the host sizes the dynamic shared memory as 7 x 25088 + 56832 (all there is)");

B200_DEVICE int mega_smem_bytes() { return kMegaSlots * kMegaSlotBytes + int(sizeof(MegaSmem)); }

B200_DEVICE void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
B200_DEVICE unsigned ld_acquire_u32(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
B200_DEVICE void cons_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kMegaConsThreads) : "memory"); }

// Bounded mbarrier wait that gives up quickly once the CTA is aborted.
B200_DEVICE bool mega_wait(uint64_t *bar, uint32_t parity, MegaSmem *sm, int *status, int code) {
  if (mbar_try_wait(bar, parity)) return true;       // the common case: the data is already there
  const uint32_t lim = *reinterpret_cast<volatile int *>(&sm->abort) ? 4096u : sm->spin;
  for (uint32_t i = 0; i < lim; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *reinterpret_cast<volatile int *>(status) != 0) break;   // another CTA gave up
  }
  *reinterpret_cast<volatile int *>(&sm->abort) = 1;
  atomicCAS(status, 0, code);
  return false;
}

struct MegaCtx {
  MegaSmem *sm;
  uint8_t *ring;
  const MegaGlobals *g;
  unsigned nbar;       // grid barriers passed
  uint32_t seq;        // ring slots consumed (consumers) or filled (producer)
  int pbuf;            // partial-sum buffer in use
  int tid, lane, warp;
  int nstamp;
  uint32_t ndone;      // block-scaled path: phases finished (parity of the `done` barrier)
  uint32_t nmx;        // block-scaled path: chunks handed from warp 4 to warp 0 so far (index and parity of `sready`)
  uint32_t skip_fill;  // producer, test hook: 1 + the ring fill to leave out (0: none)
};

// Phase time stamp of this CTA (thread 0), when the host asked for a trace.
B200_DEVICE void mega_stamp(MegaCtx &c) {
  if (c.tid == 0 && c.g->trace && c.nstamp < kMegaTraceLen) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    c.g->trace[size_t(blockIdx.x) * kMegaTraceLen + c.nstamp] = t;
  }
  c.nstamp++;
}

// Grid barrier for the consumer warps (the producer only reads immutable weights).
B200_DEVICE void grid_barrier(MegaCtx &c) {
  c.nbar++;
  mega_stamp(c);
  cons_sync();
  if (c.tid == 0) {
    // release-add / acquire-poll: the CTA barriers on both sides extend the ordering to the other threads
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(c.g->sync) : "memory");
    const unsigned target = c.nbar * gridDim.x;
    uint32_t it = 0;
    while (ld_acquire_u32(c.g->sync) < target) {
      ++it;
      if ((it & 63u) == 0 && *reinterpret_cast<volatile int *>(c.g->status) != 0) break;
      if (it > c.sm->spin) { atomicCAS(c.g->status, 0, 10); break; }
    }
  }
  cons_sync();
  mega_stamp(c);
}

// Rows [r0, r1) of an operation with `rows` outputs that this CTA owns.
B200_DEVICE void cta_range(int n, int *lo, int *hi) {
  *lo = int((long long)n * blockIdx.x / gridDim.x);
  *hi = int((long long)n * (blockIdx.x + 1) / gridDim.x);
}

// ---- producer ---------------------------------------------------------------------
// One ring slot: up to two bulk copies (b1 may be 0) landing back to back.
B200_DEVICE void mega_fill(MegaCtx &c, const void *src0, uint32_t b0, const void *src1, uint32_t b1, const void *src2,
                           uint32_t b2) {
  const uint32_t slot = c.seq % kMegaSlots;
  if (c.seq >= kMegaSlots) mega_wait(&c.sm->empty[slot], ((c.seq / kMegaSlots) - 1) & 1, c.sm, c.g->status, 11);
  uint8_t *dst = c.ring + size_t(slot) * kMegaSlotBytes;
  if (c.skip_fill && c.seq + 1 == c.skip_fill) { c.seq++; return; }      // test hook: this slot never fills
  mbar_expect_tx(&c.sm->full[slot], b0 + b1 + b2);
  bulk_g2s(dst, src0, b0, &c.sm->full[slot]);
  if (b1) bulk_g2s(dst + b0, src1, b1, &c.sm->full[slot]);
  if (b2) bulk_g2s(dst + b0 + b1, src2, b2, &c.sm->full[slot]);
  c.seq++;
}

// Block-scaled expert phases: which 8-row groups of which expert slot this CTA owns.  The CTAs are
// divided evenly among the slots (148 = 4 x 37), so a CTA's rows belong to one expert.
B200_DEVICE void mxw_range(int n_slots, int groups, int *slot, int *g0, int *g1) {
  const int cps = max(int(gridDim.x) / n_slots, 1), local = int(blockIdx.x) % cps;
  *slot = int(blockIdx.x) / cps;
  *g0 = *g1 = 0;
  if (*slot < n_slots) {
    *g0 = int((long long)groups * local / cps);
    *g1 = int((long long)groups * (local + 1) / cps);
  }
}

// Rows per ring slot of a dense bf16 matrix with K inputs.
B200_DEVICE int dense_rps(int K) { return K <= 3072 ? 4 : 3; }

// The step's weight stream in consumption order, one fill site for all of it
// (op 0: qkv or, after the last layer, lm_head; 1: o-proj; 2: experts' gate_up; 3: experts' down).
B200_DEVICE void mega_producer(MegaCtx &c, const MegaArgs &a) {
  const MegaGlobals &g = *c.g;
  const int QD = a.NQ * 64, QKV = QD + 2 * a.NKV * 64;
#pragma unroll 1
  for (int l = 0; l <= a.layers; ++l) {
    const bool last = l == a.layers;
    const MegaLayer &ly = g.layers[last ? 0 : l];
#pragma unroll 1
    for (int op = 0; op < (last ? 1 : 4); ++op) {
      const bool dense = op < 2;
      const uint8_t *w0, *w1 = nullptr;
      int n, K, step;
      if (op == 0) { w0 = reinterpret_cast<const uint8_t *>(last ? g.lm_head : ly.wqkv); n = last ? a.V : QKV; K = a.H; }
      else if (op == 1) { w0 = reinterpret_cast<const uint8_t *>(ly.wo); n = a.H; K = QD; }
      else if (op == 2) { w0 = ly.gu_codes; w1 = ly.gu_scales; n = 2 * a.I / (a.mx ? kMxTileRows : kTileRows); K = a.H; }
      else { w0 = ly.dn_codes; w1 = ly.dn_scales; n = a.H / (a.mx ? kMxTileRows : kTileRows); K = a.I; }
      if (op == 2) mega_wait(&c.sm->route_bar, l & 1, c.sm, g.status, 12);     // the router's choice for this layer
      step = dense ? dense_rps(K) : 1;
      const int chunks = K / kChunkK, tiles = n;
      int lo, hi;
      cta_range(dense ? n : a.top_k * tiles, &lo, &hi);
      // block-scaled path: one ring slot per chunk of 8 K blocks of this CTA's rows
      const int kblocks = K >> 5, R = n * (a.mx ? kMxTileRows : kTileRows);
      const bool mx = a.mx && !dense;
      int mslot = 0, g0 = 0, g1 = 0;
      const int mkc = op == 2 ? a.kc_gu : a.kc_dn;
      if (mx) {
        mxw_range(a.top_k, R >> 3, &mslot, &g0, &g1);
        lo = 0;
        hi = g1 > g0 ? (kblocks + mkc - 1) / mkc : 0;
      }
#pragma unroll 1
      for (int i = lo; i < hi; i += step) {
        const uint8_t *s0, *s1 = nullptr, *s2 = nullptr;
        uint32_t b0, b1 = 0, b2 = 0;
        if (dense) {
          s0 = w0 + size_t(i) * K * 2;
          b0 = uint32_t(min(step, hi - i)) * K * 2;
        } else if (mx) {
          // chunk i of this CTA's 8-row groups: one contiguous piece (codes and scale words per group)
          const size_t e = size_t(c.sm->r_active[mslot]);
          const int kcc = min(mkc, kblocks - i * mkc);
          s0 = w0 + e * mxw_matrix_bytes(kblocks, mkc, R) + mxw_chunk_base(i, mkc, R) + size_t(g0) * mxw_group_bytes(kcc);
          b0 = uint32_t((g1 - g0) * mxw_group_bytes(kcc));
        } else {
          const size_t t = size_t(c.sm->r_active[i / tiles]) * tiles + i % tiles;
          s0 = w0 + t * chunks * 512;
          b0 = uint32_t(chunks) * 512;
          s1 = w1 + t * chunks * 32;
          b1 = uint32_t(chunks) * 32;
        }
        mega_fill(c, s0, b0, s1, b1, s2, b2);
      }
    }
  }
}

// ---- consumer: activations --------------------------------------------------------
// The phase's input vector is staged in shared memory (xs, f32) by all
// consumer threads; each thread owns float4 number tid and tid + 512.
struct XVec { float4 v[2]; };

B200_DEVICE float4 f4_zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }

// RMSNorm of the staged vector (Qwen2Proven.lean:304-333 form: x * inv * w) into xs.
B200_DEVICE void mega_norm_to_xs(MegaCtx &c, XVec &x, const float *__restrict__ w, int K, float eps,
                                 float *__restrict__ copy_out) {
  const int n4 = K >> 2;
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    ss = fmaf(x.v[u].x, x.v[u].x, ss); ss = fmaf(x.v[u].y, x.v[u].y, ss);
    ss = fmaf(x.v[u].z, x.v[u].z, ss); ss = fmaf(x.v[u].w, x.v[u].w, ss);
  }
  ss = warp_sum(ss);
  cons_sync();                                   // xs and red are free again
  if (c.lane == 0) c.sm->red[c.warp] = ss;
  cons_sync();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kMegaConsumers; ++i) tot += c.sm->red[i];
  const float inv = 1.0f / sqrtf(tot / float(K) + eps);
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int i = c.tid + u * kMegaConsThreads;
    if (i < n4) {
      const float4 gg = __ldg(reinterpret_cast<const float4 *>(w) + i);
      float4 o = x.v[u];
      o.x = o.x * inv * gg.x; o.y = o.y * inv * gg.y; o.z = o.z * inv * gg.z; o.w = o.w * inv * gg.w;
      reinterpret_cast<float4 *>(c.sm->u.xs)[i] = o;
      if (copy_out) reinterpret_cast<float4 *>(copy_out)[i] = o;
    }
  }
  cons_sync();
}

// h = in + sum_j gate_j * o_j (j in top-k order), as the combine prologue of gemv_fused.
B200_DEVICE void mega_load_combined(MegaCtx &c, XVec &x, const float *in, const float *o, int K, int top_k,
                                    float *hout) {
  const int n4 = K >> 2;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int i = c.tid + u * kMegaConsThreads;
    x.v[u] = i < n4 ? __ldcg(reinterpret_cast<const float4 *>(in) + i) : f4_zero();
  }
  // four experts' outputs at a time, so that their loads travel together with `in`
  for (int j0 = 0; j0 < top_k; j0 += 4) {
    float4 t[4][2];
#pragma unroll
    for (int jj = 0; jj < 4; ++jj)
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int i = c.tid + u * kMegaConsThreads;
        t[jj][u] = (j0 + jj < top_k && i < n4) ? __ldcg(reinterpret_cast<const float4 *>(o + size_t(j0 + jj) * K) + i)
                                               : f4_zero();
      }
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const float wgt = j0 + jj < top_k ? c.sm->r_gate[j0 + jj] : 0.f;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        x.v[u].x = fmaf(wgt, t[jj][u].x, x.v[u].x); x.v[u].y = fmaf(wgt, t[jj][u].y, x.v[u].y);
        x.v[u].z = fmaf(wgt, t[jj][u].z, x.v[u].z); x.v[u].w = fmaf(wgt, t[jj][u].w, x.v[u].w);
      }
    }
  }
  if (hout) {
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int i = c.tid + u * kMegaConsThreads;
      if (i < n4) reinterpret_cast<float4 *>(hout)[i] = x.v[u];
    }
  }
}

// ---- consumer: router of one layer ----------------------------------------------------------
// The CTAs that produced h1 (the o-projection) left, per CTA, the partial
// sums  p[cta][e] = sum_r Wr[e][r] ln2[r] h1[r]  over their rows
// (consume_dense, kind 1).  After the grid barrier every CTA adds the
// partial sums in the same fixed order (warp w: CTAs w, w + 15, ...; then the
// warps in order), so all agree bit for bit:
//   logit_e = inv * total_e + br[e],  inv = 1 / sqrt(mean(h1^2) + eps),
// stages xn = h1 * inv * ln2 in xs and selects the top k itself (logit
// descending, ties to the lower expert id; softmax over the selected logits).
constexpr int kMegaRouteCtas = 10;      // partial-sum rows per warp kept in flight: grids up to 150 CTAs in one round

B200_DEVICE int mega_rpart_stride(int E) { return (E + 31) & ~31; }

B200_DEVICE void mega_route(MegaCtx &c, const MegaArgs &a, const MegaLayer &ly, const XVec &x) {
  const MegaGlobals &g = *c.g;
  const int E = a.E, n4 = a.H >> 2, lane = c.lane;
  const int grid = int(gridDim.x), rstride = mega_rpart_stride(E);
  float(*rsum)[128] = reinterpret_cast<float(*)[128]>(&c.sm->part[0][0][0]);    // [15][128], idle between the phases
  // ln2 and the router bias do not depend on the barrier: first in flight
  float4 gg[2];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int i = c.tid + u * kMegaConsThreads;
    gg[u] = i < n4 ? __ldg(reinterpret_cast<const float4 *>(ly.ln2) + i) : f4_zero();
  }
  float brv[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) brv[i] = (c.warp == 0 && lane + 32 * i < E) ? __ldg(ly.br + lane + 32 * i) : 0.f;
  // ---- this warp's share of the partial sums: lane = expert within a group of 32
#pragma unroll 1
  for (int e0 = 0; e0 < E; e0 += 32) {
    const bool have = e0 + lane < E;
    float tot = 0.f;
#pragma unroll 1
    for (int c0 = c.warp; c0 < grid; c0 += kMegaConsumers * kMegaRouteCtas) {
      float pv[kMegaRouteCtas];
#pragma unroll
      for (int q = 0; q < kMegaRouteCtas; ++q) {
        const int cta = c0 + kMegaConsumers * q;
        pv[q] = (have && cta < grid) ? __ldcg(g.rpart + size_t(cta) * rstride + e0 + lane) : 0.f;
      }
#pragma unroll
      for (int q = 0; q < kMegaRouteCtas; ++q) tot += pv[q];
    }
    if (have) rsum[c.warp][e0 + lane] = tot;
  }
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    ss = fmaf(x.v[u].x, x.v[u].x, ss); ss = fmaf(x.v[u].y, x.v[u].y, ss);
    ss = fmaf(x.v[u].z, x.v[u].z, ss); ss = fmaf(x.v[u].w, x.v[u].w, ss);
  }
  ss = warp_sum(ss);
  if (lane == 0) c.sm->red[c.warp] = ss;
  cons_sync();
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < kMegaConsumers; ++i) sq += c.sm->red[i];
  const float inv = 1.0f / sqrtf(sq / float(a.H) + a.eps);
  mega_stamp(c);
  {
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int i = c.tid + u * kMegaConsThreads;
      if (i < n4) {
        float4 o = x.v[u];
        o.x = o.x * inv * gg[u].x; o.y = o.y * inv * gg[u].y; o.z = o.z * inv * gg[u].z; o.w = o.w * inv * gg[u].w;
        reinterpret_cast<float4 *>(c.sm->u.xs)[i] = o;
        if (blockIdx.x == 0) reinterpret_cast<float4 *>(g.xn)[i] = o;
      }
    }
  }
  if (c.warp == 0) {
    const int k = a.top_k;
    float v[4];
    bool taken[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int ee = lane + 32 * i;
      float l = -INFINITY;
      if (ee < E) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < kMegaConsumers; ++w) t += rsum[w][ee];
        l = fmaf(t, inv, brv[i]);
        if (blockIdx.x == 0) g.rlogits[ee] = l;
      }
      v[i] = (l == l) ? l : -INFINITY;
      taken[i] = ee >= E;
    }
    // k rounds of arg-max; lane j keeps the j-th choice
    float my_v = -INFINITY;
    int my_e = 0;
#pragma unroll 1
    for (int j = 0; j < k; ++j) {
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
      if (lane == j) { my_v = bv; my_e = (be == 0x7fffffff) ? 0 : be; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (lane + 32 * i == be) taken[i] = true;
    }
    // softmax over the selected logits (summed in selection order) and each choice's slot in
    // ascending expert order (one token: every selected expert has one assignment)
    const float top = __shfl_sync(0xffffffffu, my_v, 0);
    const float ex = lane < k ? __expf(my_v - top) : 0.f;
    float sum = 0.f;
    int slot = 0;
#pragma unroll
    for (int j = 0; j < kMegaMaxTopK; ++j) {
      const float oex = __shfl_sync(0xffffffffu, ex, j);
      const int oe = __shfl_sync(0xffffffffu, my_e, j);
      if (j < k) {
        sum += oex;
        slot += (oe < my_e) || (oe == my_e && j < lane);
      }
    }
    if (lane < k) {
      c.sm->r_sel[lane] = my_e;
      c.sm->r_gate[lane] = ex / sum;
      c.sm->r_active[slot] = my_e;
      c.sm->r_assign[slot] = lane;
    }
    __syncwarp();
    if (blockIdx.x == 0) {
      // the routing tables and gates in global memory, in the layout of moe_route_tables
      int *route = g.route;
      int *count = route + 1, *offset = route + 1 + E, *active = offset + E + 1, *perm = active + E;
      if (lane == 0) route[0] = k;
#pragma unroll 1
      for (int ee = lane; ee < E; ee += 32) {
        int cnt = 0, before = 0;
#pragma unroll 1
        for (int j = 0; j < k; ++j) { cnt += (c.sm->r_sel[j] == ee); before += (c.sm->r_sel[j] < ee); }
        count[ee] = cnt;
        offset[ee] = before;
        active[ee] = ee < k ? c.sm->r_active[ee] : -1;
      }
      if (lane == 0) offset[E] = k;
      if (lane < k) {
        perm[lane] = c.sm->r_assign[lane];
        g.topk_idx[lane] = c.sm->r_sel[lane];
        g.topk_w[lane] = c.sm->r_gate[lane];
      }
    }
  }
  cons_sync();
  if (c.tid == 0) mbar_arrive(&c.sm->route_bar);       // the producer may start on the experts
}

// Plain copy of an f32 vector (K <= 4096) from global memory (through L2) into xs.
B200_DEVICE void mega_stage_plain(MegaCtx &c, const float *src, int K) {
  const int n4 = K >> 2;
  float4 v[3];
#pragma unroll
  for (int u = 0; u < 3; ++u) {
    const int i = c.tid + u * kMegaConsThreads;
    v[u] = i < n4 ? __ldcg(reinterpret_cast<const float4 *>(src) + i) : f4_zero();
  }
  cons_sync();
#pragma unroll
  for (int u = 0; u < 3; ++u) {
    const int i = c.tid + u * kMegaConsThreads;
    if (i < n4) reinterpret_cast<float4 *>(c.sm->u.xs)[i] = v[u];
  }
  cons_sync();
}

// ---- consumer: attention of one (slice, kv head) unit from shared memory ---------------------
// Same definition as attn_decode.cuh (RoPE, cache append, sinks, sliding
// window, slices of kAttnSplit positions merged by the last CTA to finish),
// written for a small code footprint: the unit's K and V rows are copied to
// shared memory with cp.async (before the grid barrier that waits for q, k, v:
// they depend only on the position), and every loop over positions or
// dimensions is rolled.  256 threads (warps 0..7), bf16 cache.
struct AttnGeom { int nsplit, split, kvh, j0, nj, owns_new; size_t head_base; };

B200_DEVICE AttnGeom mega_attn_geom(int u, int nsplit, int pos, int window, int cache_len, int NKV) {
  AttnGeom ge;
  ge.nsplit = nsplit;
  ge.split = u % nsplit;
  ge.kvh = u / nsplit;
  const int lo_vis = window > 0 ? max(0, pos + 1 - window) : 0;
  ge.j0 = lo_vis + ge.split * kAttnSplit;
  ge.nj = min(kAttnSplit, pos + 1 - ge.j0);
  ge.owns_new = ge.split == nsplit - 1;
  ge.head_base = size_t(ge.kvh) * cache_len;
  (void)NKV;
  return ge;
}

// Request the unit's cache rows (threads 0..255).  The row of the token being
// appended is not in the cache yet; it is overwritten in shared memory later.
B200_DEVICE void mega_attn_prefetch(MegaAttnSmem &as, const AttnGeom &ge, int tid, const uint16_t *kcache,
                                    const uint16_t *vcache, int cache_len) {
  for (int idx = tid; idx < ge.nj * 8; idx += kMegaAttnWarps * 32) {
    const int row = idx >> 3, ch = idx & 7;
    const size_t src = (ge.head_base + size_t((ge.j0 + row) % cache_len)) * 64 + ch * 8;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(&as.k[row][ch * 8])), "l"(kcache + src) : "memory");
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(&as.v[row][ch * 8])), "l"(vcache + src) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

B200_DEVICE void mega_attn_unit(MegaCtx &c, MegaAttnSmem &as, const AttnGeom &ge, int pos, const MegaArgs &a,
                                const MegaLayer &ly, int cache_len) {
  constexpr int HD = 64, HALF = 32, NT = kMegaAttnWarps * 32;
  const MegaGlobals &g = *c.g;
  const int tid = c.tid, lane = c.lane, warp = c.warp;
  const int G = a.NQ / a.NKV, QD = a.NQ * HD;
  uint16_t *kcache = reinterpret_cast<uint16_t *>(ly.kcache), *vcache = reinterpret_cast<uint16_t *>(ly.vcache);

  // ---- q (rotated, scaled) and, in the slice that owns it, the new K/V row
  const int rp = min(pos, a.max_seq - 1);
  const float *sinp = g.rope + size_t(rp) * HALF;
  const float *cosp = g.rope + size_t(a.max_seq) * HALF + size_t(rp) * HALF;
  {
    const int gq = tid >> 5, d = tid & 31;          // 8 warps = up to 8 q heads of the group
    float rlo = 0.f, rhi = 0.f;
    if (gq < G) {
      const float *q = g.qkv + size_t(ge.kvh * G + gq) * HD;
      const float lo = __ldcg(q + d), hi = __ldcg(q + d + HALF), s = __ldg(sinp + d), cs = __ldg(cosp + d);
      rlo = __fmul_rn(__fsub_rn(__fmul_rn(lo, cs), __fmul_rn(hi, s)), a.attn_scale);
      rhi = __fmul_rn(__fadd_rn(__fmul_rn(lo, s), __fmul_rn(hi, cs)), a.attn_scale);
    }
    as.q[gq][d] = rlo;
    as.q[gq][d + HALF] = rhi;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  attn_sync<2, NT>();                               // cache rows have landed for every thread
  if (ge.owns_new) {
    const size_t slot = (ge.head_base + size_t(pos % cache_len)) * HD;
    const int row = pos - ge.j0;
    if (tid < HALF) {
      const float *k = g.qkv + QD + size_t(ge.kvh) * HD;
      const float lo = __ldcg(k + tid), hi = __ldcg(k + tid + HALF), s = __ldg(sinp + tid), cs = __ldg(cosp + tid);
      const uint16_t blo = f32_to_bf16_rne(__fsub_rn(__fmul_rn(lo, cs), __fmul_rn(hi, s)));
      const uint16_t bhi = f32_to_bf16_rne(__fadd_rn(__fmul_rn(lo, s), __fmul_rn(hi, cs)));
      kcache[slot + tid] = blo;
      kcache[slot + tid + HALF] = bhi;
      as.k[row][tid] = blo;
      as.k[row][tid + HALF] = bhi;
    } else if (tid >= 64 && tid < 128) {
      const int d = tid - 64;
      const uint16_t bv = f32_to_bf16_rne(__ldcg(g.qkv + QD + size_t(a.NKV) * HD + size_t(ge.kvh) * HD + d));
      vcache[slot + d] = bv;
      as.v[row][d] = bv;
    }
  }
  attn_sync<2, NT>();

  // ---- scores: thread = (position, half of the q heads)
  {
    const int p = tid >> 1, h0 = (tid & 1) * 4;
    if (p < ge.nj) {
      float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
      for (int ch = 0; ch < 8; ++ch) {
        const uint4 kw = *reinterpret_cast<const uint4 *>(&as.k[p][ch * 8]);
        const float kf[8] = {bf16_lo(kw.x), bf16_hi(kw.x), bf16_lo(kw.y), bf16_hi(kw.y),
                             bf16_lo(kw.z), bf16_hi(kw.z), bf16_lo(kw.w), bf16_hi(kw.w)};
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const float4 q0 = *reinterpret_cast<const float4 *>(&as.q[h0 + h][ch * 8]);
          const float4 q1 = *reinterpret_cast<const float4 *>(&as.q[h0 + h][ch * 8 + 4]);
          float t = s[h];
          t = fmaf(q0.x, kf[0], t); t = fmaf(q0.y, kf[1], t); t = fmaf(q0.z, kf[2], t); t = fmaf(q0.w, kf[3], t);
          t = fmaf(q1.x, kf[4], t); t = fmaf(q1.y, kf[5], t); t = fmaf(q1.z, kf[6], t); t = fmaf(q1.w, kf[7], t);
          s[h] = t;
        }
      }
#pragma unroll
      for (int h = 0; h < 4; ++h) as.s[h0 + h][p] = s[h];
    }
  }
  attn_sync<2, NT>();

  // ---- softmax over the slice: warp = q head
  float m = -INFINITY, l = 0.f;
  {
    float v[kAttnSplit / 32];
#pragma unroll
    for (int i = 0; i < kAttnSplit / 32; ++i) {
      const int p = lane + 32 * i;
      v[i] = p < ge.nj ? as.s[warp][p] : -INFINITY;
      m = fmaxf(m, v[i]);
    }
    m = warp_max(m);
#pragma unroll
    for (int i = 0; i < kAttnSplit / 32; ++i) {
      const int p = lane + 32 * i;
      const float e = p < ge.nj ? __expf(v[i] - m) : 0.f;
      as.s[warp][p] = e;
      l += e;
    }
    l = warp_sum(l);
  }
  __syncwarp();

  // ---- P V: warp = q head, lane = two dimensions
  float acc0 = 0.f, acc1 = 0.f;
#pragma unroll 4
  for (int p = 0; p < ge.nj; ++p) {
    const float pv = as.s[warp][p];
    const uint32_t vv = *reinterpret_cast<const uint32_t *>(&as.v[p][2 * lane]);
    acc0 = fmaf(pv, bf16_lo(vv), acc0);
    acc1 = fmaf(pv, bf16_hi(vv), acc1);
  }
  const int qh = ge.kvh * G + warp;
  if (warp < G) {
    if (ge.nsplit == 1) {
      // single slice: finish here (the sink joins the denominator only)
      const float sk = __ldg(ly.sinks + qh);
      const float Mf = fmaxf(m, sk), f = __expf(m - Mf);
      const float Lf = fmaf(l, f, __expf(sk - Mf));
      *reinterpret_cast<float2 *>(g.attn + size_t(qh) * HD + 2 * lane) = make_float2(acc0 * f / Lf, acc1 * f / Lf);
    } else {
      *reinterpret_cast<float2 *>(g.part_o + (size_t(qh) * a.max_splits + ge.split) * HD + 2 * lane) =
          make_float2(acc0, acc1);
      if (lane == 0)
        *reinterpret_cast<float2 *>(g.part_ml + (size_t(qh) * a.max_splits + ge.split) * 2) = make_float2(m, l);
    }
  }
  if (ge.nsplit == 1) return;

  // ---- the last slice of this kv head to finish merges all slices, in slice order
  __threadfence();
  attn_sync<2, NT>();
  if (tid == 0) {
    const int done = atomicAdd(&g.counters[ge.kvh], 1);
    as.is_last = (done == ge.nsplit - 1);
    if (as.is_last) g.counters[ge.kvh] = 0;
  }
  attn_sync<2, NT>();
  if (!as.is_last) return;
  __threadfence();
  if (warp < G) {
    const float2 *pm = reinterpret_cast<const float2 *>(g.part_ml + size_t(qh) * a.max_splits * 2);
    const float *po = g.part_o + size_t(qh) * a.max_splits * HD + 2 * lane;
    float M = __ldg(ly.sinks + qh), L = 0.f, o0 = 0.f, o1 = 0.f;
#pragma unroll 1
    for (int s0 = 0; s0 < ge.nsplit; s0 += 8) {
      float2 ml[8], pv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int s = min(s0 + u, ge.nsplit - 1);
        ml[u] = __ldcg(pm + s);
        pv[u] = __ldcg(reinterpret_cast<const float2 *>(po + size_t(s) * HD));
      }
      float Mn = M;
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (s0 + u < ge.nsplit) Mn = fmaxf(Mn, ml[u].x);
      const float f = __expf(M - Mn);
      L *= f; o0 *= f; o1 *= f;
      M = Mn;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (s0 + u < ge.nsplit) {
          const float w = __expf(ml[u].x - M);
          L = fmaf(ml[u].y, w, L);
          o0 = fmaf(pv[u].x, w, o0);
          o1 = fmaf(pv[u].y, w, o1);
        }
      }
    }
    L += __expf(__ldg(ly.sinks + qh) - M);
    *reinterpret_cast<float2 *>(g.attn + size_t(qh) * HD + 2 * lane) = make_float2(o0 / L, o1 / L);
  }
}

// ---- consumer: dense bf16 GEMV over this CTA's rows ------------------------------------
// The kernel's code has to stay resident in the SM's instruction cache across
// the layers, so there is ONE copy of each consumer loop; what differs between
// the operations that share it is data (this struct), not code.
struct DenseJob {
  int kind;              // 0: out = W x + bias; 1: out = (W x + bias) + res; 2: out = W x, running argmax
  int rows, K;
  const float *bias;     // immutable
  const float *res;      // written earlier in this launch: read through L2
  float *out;
  // kind 1 also accumulates the router's partial sums over this CTA's rows (the rows of h1 it has just
  // produced): racc[e] += Wr[e][r] * ln2[r] * h1[r]
  const float *wr, *ln2;
  int E, H;
};

// The 15 warps split K into slices of vpw 16-byte vectors; a lane keeps its 8
// (or, for K > 3840, 16) activations in registers.  A ring slot holds `rps`
// rows (4, or 3 when K > 3072).  Two slots form a group whose per-lane sums are
// transposed-reduced with 8 shuffles; eight groups form a super group that meets
// in shared memory, where threads 0..63 finish one row each.
B200_DEVICE void consume_dense(MegaCtx &c, const DenseJob &job, float &bv, int &bi) {
  const int K = job.K, rps = dense_rps(K);
  int r0, r1;
  cta_range(job.rows, &r0, &r1);
  const int nslots = (r1 - r0 + rps - 1) / rps;
  const int nvec = K >> 3, vpw = (nvec + kMegaConsumers - 1) / kMegaConsumers;
  const int myvec = c.warp * vpw + c.lane;
  const bool active = c.lane < vpw && myvec < nvec;
  // K > 3840: a warp's slice has n2 = vpw - 32 more vectors; lane j < rps * n2 takes (row j / n2, vector 32 + j % n2)
  const int n2 = max(vpw - 32, 1), row2 = c.lane / n2, myvec2 = c.warp * vpw + 32 + c.lane % n2;
  const bool active2 = vpw > 32 && row2 < rps && myvec2 < nvec;
  float x[8], x2[8];
  {
    const float4 *xs4 = reinterpret_cast<const float4 *>(c.sm->u.xs);
    const float4 a0 = active ? xs4[2 * myvec] : f4_zero(), a1 = active ? xs4[2 * myvec + 1] : f4_zero();
    x[0] = a0.x; x[1] = a0.y; x[2] = a0.z; x[3] = a0.w; x[4] = a1.x; x[5] = a1.y; x[6] = a1.z; x[7] = a1.w;
    const float4 b0 = active2 ? xs4[2 * myvec2] : f4_zero(), b1 = active2 ? xs4[2 * myvec2 + 1] : f4_zero();
    x2[0] = b0.x; x2[1] = b0.y; x2[2] = b0.z; x2[3] = b0.w; x2[4] = b1.x; x2[5] = b1.y; x2[6] = b1.z; x2[7] = b1.w;
  }
  // thread t < 64 finishes value t of a super group: group t / 8, slot (t % 8) / 4, row (t % 4) of the slot
  const int my_off = (c.tid >> 3) * 2 * rps + ((c.tid >> 2) & 1) * rps + (c.tid & 3);
  const bool my_valid = c.tid < 64 && (c.tid & 3) < rps;
  // bias / residual of the first super group travel while the weights are consumed
  float pre_b = 0.f, pre_r = 0.f;
  if (my_valid && r0 + my_off < r1) {
    if (job.kind != 2) pre_b = __ldg(job.bias + r0 + my_off);
    if (job.kind == 1) pre_r = __ldcg(job.res + r0 + my_off);
  }
  const int row_bytes = K * 2;
  // router weights (x norm weight) of the first super group's rows for this warp's first three
  // experts (w, w + 15, w + 30): the rows that threads lane and lane + 32 finish
  float wpre[3][2], lpre[2] = {0.f, 0.f};
  float rown = 0.f;      // lanes 0..2: the running sum of expert warp + 15 lane; later experts use racc (lane 0)
  if (job.kind == 1) {
    for (int e = c.warp + kMegaConsumers * 3 + kMegaConsumers * c.lane; e < job.E; e += kMegaConsumers * 32) c.sm->racc[e] = 0.f;
#pragma unroll
    for (int i = 0; i < 3; ++i)
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int e = c.warp + kMegaConsumers * i, tq = c.lane + 32 * q;
        const int row = r0 + (tq >> 3) * 2 * rps + ((tq >> 2) & 1) * rps + (tq & 3);
        wpre[i][q] = 0.f;
        if (e < job.E && (tq & 3) < rps && row < r1) {
          wpre[i][q] = __ldg(job.wr + size_t(e) * job.H + row);       // multiplied at use: nothing waits for these loads here
          if (i == 0) lpre[q] = __ldg(job.ln2 + row);
        }
      }
  }
  int sg_row0 = r0, grp = 0;
#pragma unroll 1
  for (int s = 0; s < nslots; s += 2) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
    for (int hlf = 0; hlf < 2; ++hlf) {
      if (s + hlf < nslots) {
        const uint32_t slot = c.seq % kMegaSlots;
        mega_wait(&c.sm->full[slot], (c.seq / kMegaSlots) & 1, c.sm, c.g->status, 20);
        const uint8_t *base = c.ring + size_t(slot) * kMegaSlotBytes + size_t(myvec) * 16;
        if (active) {
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            if (r < rps) {
              const uint4 w = *reinterpret_cast<const uint4 *>(base + r * row_bytes);
              float t = acc[hlf * 4 + r];
              t = fmaf(bf16_lo(w.x), x[0], t); t = fmaf(bf16_hi(w.x), x[1], t);
              t = fmaf(bf16_lo(w.y), x[2], t); t = fmaf(bf16_hi(w.y), x[3], t);
              t = fmaf(bf16_lo(w.z), x[4], t); t = fmaf(bf16_hi(w.z), x[5], t);
              t = fmaf(bf16_lo(w.w), x[6], t); t = fmaf(bf16_hi(w.w), x[7], t);
              acc[hlf * 4 + r] = t;
            }
          }
        }
        if (active2) {
          const uint4 w = *reinterpret_cast<const uint4 *>(c.ring + size_t(slot) * kMegaSlotBytes + size_t(myvec2) * 16 + row2 * row_bytes);
          float t = 0.f;
          t = fmaf(bf16_lo(w.x), x2[0], t); t = fmaf(bf16_hi(w.x), x2[1], t);
          t = fmaf(bf16_lo(w.y), x2[2], t); t = fmaf(bf16_hi(w.y), x2[3], t);
          t = fmaf(bf16_lo(w.z), x2[4], t); t = fmaf(bf16_hi(w.z), x2[5], t);
          t = fmaf(bf16_lo(w.w), x2[6], t); t = fmaf(bf16_hi(w.w), x2[7], t);
#pragma unroll
          for (int r = 0; r < 3; ++r) acc[hlf * 4 + r] += row2 == r ? t : 0.f;
        }
        __syncwarp();
        if (c.lane == 0) mbar_arrive(&c.sm->empty[slot]);
        c.seq++;
      }
    }
    warp_reduce8(acc, c.lane);
    if ((c.lane & 3) == 0) c.sm->part[c.pbuf][c.warp][grp * 8 + row_of_lane8(c.lane)] = acc[0];
    ++grp;
    if (grp == 8 || s + 2 >= nslots) {
      // ---- the super group meets: one row per thread
      cons_sync();
      const int row = sg_row0 + my_off;
      if (my_valid && (c.tid >> 3) < grp && row < r1) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kMegaConsumers; ++w) v += c.sm->part[c.pbuf][w][c.tid];
        if (sg_row0 != r0) {
          if (job.kind != 2) pre_b = __ldg(job.bias + row);
          if (job.kind == 1) pre_r = __ldcg(job.res + row);
        }
        if (job.kind == 2) argmax_combine(bv, bi, v, row);
        else v = (v + pre_b) + pre_r;
        job.out[row] = v;
        if (job.kind == 1) c.sm->rrow[c.tid] = v;
      } else if (job.kind == 1 && c.tid < 64) {
        c.sm->rrow[c.tid] = 0.f;
      }
      if (job.kind == 1) {
        // ---- router partial sums over the rows just finished: warp w serves experts w, w + 15, ...
        cons_sync();
        float val[2];
        int rowq[2];
        bool okq[2];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int tq = c.lane + 32 * q;
          rowq[q] = sg_row0 + (tq >> 3) * 2 * rps + ((tq >> 2) & 1) * rps + (tq & 3);
          okq[q] = (tq >> 3) < grp && (tq & 3) < rps && rowq[q] < r1;
          val[q] = okq[q] ? c.sm->rrow[tq] : 0.f;
        }
        const bool first_sg = sg_row0 == r0;
        float s3[3];
#pragma unroll
        for (int i = 0; i < 3; ++i) {
          const int e = c.warp + kMegaConsumers * i;
          float sacc = 0.f;
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            float w = wpre[i][q] * lpre[q];
            if (!first_sg) w = (okq[q] && e < job.E) ? __ldg(job.wr + size_t(e) * job.H + rowq[q]) * __ldg(job.ln2 + rowq[q]) : 0.f;
            sacc = fmaf(w, val[q], sacc);
          }
          s3[i] = sacc;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
          for (int i = 0; i < 3; ++i) s3[i] += __shfl_xor_sync(0xffffffffu, s3[i], o);
        rown += c.lane == 0 ? s3[0] : c.lane == 1 ? s3[1] : s3[2];
#pragma unroll 1
        for (int e = c.warp + kMegaConsumers * 3; e < job.E; e += kMegaConsumers) {
          float sacc = 0.f;
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const float w = okq[q] ? __ldg(job.wr + size_t(e) * job.H + rowq[q]) * __ldg(job.ln2 + rowq[q]) : 0.f;
            sacc = fmaf(w, val[q], sacc);
          }
          sacc = warp_sum(sacc);
          if (c.lane == 0) c.sm->racc[e] += sacc;
        }
      }
      sg_row0 += 16 * rps;
      grp = 0;
      c.pbuf ^= 1;
    }
  }
  if (job.kind == 1) {
    // publish this CTA's partial sums: rpart[cta][e] (each by the thread that summed it)
    float *dst = c.g->rpart + size_t(blockIdx.x) * mega_rpart_stride(job.E);
    if (c.lane < 3 && c.warp + kMegaConsumers * c.lane < job.E) dst[c.warp + kMegaConsumers * c.lane] = rown;
    if (c.lane == 0)
      for (int e = c.warp + kMegaConsumers * 3; e < job.E; e += kMegaConsumers) dst[e] = c.sm->racc[e];
  }
}

// ---- consumer: MXFP4 expert GEMV over this CTA's (slot, tile) units ------------------------
// One ring slot = one 16-row tile (codes then scale words).  Warp w takes
// chunks [w * cpw, (w + 1) * cpw) of every tile; its B fragments (f16 hi/lo
// columns of the activations, as in moe_tiled.cuh) stay in registers while
// the expert slot does not change.  Four tiles form a super group (64 rows).
constexpr int kMegaMaxCpw = 3;     // K <= 15 * 3 * 64 = 2880 (a tile of 45 chunks also fills a ring slot)

struct ExpertJob {
  int kind;                 // 0: gate_up (+ clamped SwiGLU, activations already staged in xs); 1: down (stages act[rank])
  int R, K;
  const float *bias;        // [E][R]
  const float *xsrc;        // kind 1: act [top_k][K], written earlier in this launch
  float *out;               // kind 0: act [top_k][R / 2]; kind 1: o [top_k][R]
  float alpha, limit;
  int kc;                   // block-scaled path: K blocks per chunk (ring slot)
};

B200_DEVICE uint32_t pack_half2(float lo, float hi, bool want_lo_part) {
  __half a = __float2half_rn(lo), b = __float2half_rn(hi);
  if (want_lo_part) {
    a = __float2half_rn(lo - __half2float(a));
    b = __float2half_rn(hi - __half2float(b));
  }
  return uint32_t(__half_as_ushort(a)) | (uint32_t(__half_as_ushort(b)) << 16);
}

B200_DEVICE void consume_experts(MegaCtx &c, const ExpertJob &job, int n_act) {
  const int R = job.R, K = job.K;
  const int tiles = R / kTileRows, chunks = K / kChunkK;
  const int cpw = (chunks + kMegaConsumers - 1) / kMegaConsumers;
  int u0, u1;
  cta_range(n_act * tiles, &u0, &u1);
  const int g = c.lane >> 2, t = c.lane & 3;
  uint4 xa[kMegaMaxCpw], xb[kMegaMaxCpw];
  int cur_slot = -1, sg_u0 = u0, tig = 0;
  // thread t < 32 finishes rows 2p, 2p+1 (p = t % 8) of tile t / 8 of a super group
  auto bias_of = [&](int u) {
    const int s = u / tiles, r0 = (u % tiles) * kTileRows;
    return __ldg(reinterpret_cast<const float2 *>(job.bias + size_t(c.sm->r_active[s]) * R + r0) + (c.tid & 7));
  };
  float2 pre = make_float2(0.f, 0.f);
  if (c.tid < 32 && u0 + (c.tid >> 3) < u1) pre = bias_of(u0 + (c.tid >> 3));
#pragma unroll 1
  for (int u = u0; u < u1; ++u) {
    const int slot_e = u / tiles;
    if (slot_e != cur_slot) {
      // ---- fragments of this expert slot's activations: column 0 = f16(x), column 1 = f16(x - hi)
      if (job.kind == 1) mega_stage_plain(c, job.xsrc + size_t(c.sm->r_assign[slot_e]) * K, K);
#pragma unroll
      for (int i = 0; i < kMegaMaxCpw; ++i) {
        xa[i] = make_uint4(0, 0, 0, 0);
        xb[i] = make_uint4(0, 0, 0, 0);
        const int ch = c.warp * cpw + i;
        if (i < cpw && ch < chunks && g < 2) {
          const float4 *p = reinterpret_cast<const float4 *>(c.sm->u.xs + ch * kChunkK + 8 * t);
          const float4 a0 = p[0], a1 = p[1], b0 = p[8], b1 = p[9];
          const bool lo = g == 1;
          xa[i] = make_uint4(pack_half2(a0.x, a0.y, lo), pack_half2(a0.z, a0.w, lo), pack_half2(a1.x, a1.y, lo),
                             pack_half2(a1.z, a1.w, lo));
          xb[i] = make_uint4(pack_half2(b0.x, b0.y, lo), pack_half2(b0.z, b0.w, lo), pack_half2(b1.x, b1.y, lo),
                             pack_half2(b1.z, b1.w, lo));
        }
      }
      cur_slot = slot_e;
    }
    const uint32_t slot = c.seq % kMegaSlots;
    mega_wait(&c.sm->full[slot], (c.seq / kMegaSlots) & 1, c.sm, c.g->status, 21);
    if (u == u0) mega_stamp(c);        // time to the first tile of the phase
    const uint8_t *base = c.ring + size_t(slot) * kMegaSlotBytes;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < kMegaMaxCpw; ++i) {
      const int ch = c.warp * cpw + i;
      if (i < cpw && ch < chunks) {
        const uint4 w = reinterpret_cast<const uint4 *>(base)[ch * 32 + c.lane];
        const uint32_t sw = reinterpret_cast<const uint32_t *>(base + chunks * 512)[ch * 8 + g];
        block_mma2(w.x, w.y, xa[i], scale_fast<0>(sw), scale_fast<1>(sw), acc);
        block_mma2(w.z, w.w, xb[i], scale_fast<2>(sw), scale_fast<3>(sw), acc);
      }
    }
    __syncwarp();
    if (c.lane == 0) mbar_arrive(&c.sm->empty[slot]);
    c.seq++;
    if (t == 0) {
      c.sm->part[c.pbuf][c.warp][tig * 16 + g] = acc[0] + acc[1];
      c.sm->part[c.pbuf][c.warp][tig * 16 + g + 8] = acc[2] + acc[3];
    }
    ++tig;
    if (tig == 4 || u + 1 == u1) {
      cons_sync();
      if (c.tid < 32 && (c.tid >> 3) < tig) {
        const int uu = sg_u0 + (c.tid >> 3), p = c.tid & 7;
        float v0 = 0.f, v1 = 0.f;
#pragma unroll
        for (int w = 0; w < kMegaConsumers; ++w) {
          v0 += c.sm->part[c.pbuf][w][2 * c.tid];
          v1 += c.sm->part[c.pbuf][w][2 * c.tid + 1];
        }
        if (sg_u0 != u0) pre = bias_of(uu);
        const int s = uu / tiles, r0 = (uu % tiles) * kTileRows, rank = c.sm->r_assign[s];
        if (job.kind == 0) {
          job.out[size_t(rank) * (R >> 1) + (r0 >> 1) + p] = swiglu_clamped(v0 + pre.x, v1 + pre.y, job.alpha, job.limit);
        } else {
          *reinterpret_cast<float2 *>(job.out + size_t(rank) * R + r0 + 2 * p) = make_float2(v0 + pre.x, v1 + pre.y);
        }
      }
      sg_u0 += tig;
      tig = 0;
      c.pbuf ^= 1;
    }
  }
  if (u0 >= u1) mega_stamp(c);      // keeps the stamp count the same for CTAs without a unit
}

// ---- consumer: the same expert GEMVs on the block-scaled tensor cores ------------------------
// A CTA owns a range of 8-row groups of one expert slot (mxw_range) and runs
// them as ONE instruction of N = 8 x groups (<= 160) rows per K step: 45
// instructions per phase, issued by one lane of warp 0.  All 15 warps expand
// the slot's activation vector into E2M1 digit rows (the A operand) and warp 0
// moves their scales into tensor memory; then, per chunk of 8 K blocks (one
// ring slot: codes + scale words), warp 0 stores the scale words, issues four
// instructions and lets tcgen05.commit free the slot.  At the end the 8 x N
// results are read back, added up over the digit rows and finished (bias,
// clamped SwiGLU).
// Tensor-memory columns: [0, 96) the digits' scales, [96, 288) the weights'
// scales (8 columns per group of 4 K blocks, at most 23 groups), [288, 448) the accumulator.
B200_DEVICE void mbar_arrive_n(uint64_t *bar, uint32_t n) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(n) : "memory");
}

B200_DEVICE void consume_experts_mx(MegaCtx &c, const ExpertJob &job, int n_act) {
  const int R = job.R, K = job.K;
  const int mkc = max(job.kc, 4), kblocks = K >> 5, nchunks = (kblocks + mkc - 1) / mkc;
  int slot_e, g0, g1;
  mxw_range(n_act, R >> 3, &slot_e, &g0, &g1);
  const int ng = g1 - g0, N = 8 * ng;
  const bool work = ng > 0 && N <= 160 && kblocks <= 92 && (mkc & 3) == 0 && ng * mxw_group_bytes(min(mkc, kblocks)) <= kMegaSlotBytes;
  if (ng > 0 && !work && c.tid == 0) atomicCAS(c.g->status, 0, 55);
  MegaMxSmem &mx = c.sm->u.mx;
  // ---- digit rows of the activation vector (gate_up: xn, staged in xs by the router; down: act of the slot)
  if (work) {
    const int kb = c.tid >> 2, sub = c.tid & 3;
    const bool valid = kb < kblocks;
    float x[8];
    float4 v0 = f4_zero(), v1 = f4_zero();
    if (valid) {
      if (job.kind == 0) {
        v0 = *reinterpret_cast<const float4 *>(mx.xs + kb * 32 + sub * 8);
        v1 = *reinterpret_cast<const float4 *>(mx.xs + kb * 32 + sub * 8 + 4);
      } else {
        const float *src = job.xsrc + size_t(c.sm->r_assign[slot_e]) * K + kb * 32 + sub * 8;
        v0 = __ldcg(reinterpret_cast<const float4 *>(src));
        v1 = __ldcg(reinterpret_cast<const float4 *>(src + 4));
      }
    }
    x[0] = v0.x; x[1] = v0.y; x[2] = v0.z; x[3] = v0.w; x[4] = v1.x; x[5] = v1.y; x[6] = v1.z; x[7] = v1.w;
    mx_expand_radix8(x, mx.a[0], mx.sf[0], kb, sub, valid);
    for (int i = c.tid; i < 2048 / 4; i += kMegaConsThreads) reinterpret_cast<uint32_t *>(mx.a[0] + kblocks * 128)[i] = 0;
    fence_async_smem();
  }
  cons_sync();
  const uint32_t tmem = c.sm->tmem_base;
  if (work && c.warp == 4) {
    // ---- the weights' scale words of every chunk -> tensor memory, as the chunks land (this warp shares
    // warp 0's tensor-memory lanes); warp 0 issues a chunk's instructions when its `sready` completes
    const uint32_t tSFB = tmem + 96;
#pragma unroll 1
    for (int ch = 0; ch < nchunks; ++ch) {
      const uint32_t q = c.seq + uint32_t(ch), s = q % kMegaSlots;
      if (!mega_wait(&c.sm->full[s], (q / kMegaSlots) & 1, c.sm, c.g->status, 24)) break;
      const int kc = min(mkc, kblocks - ch * mkc), gb = mxw_group_bytes(kc);
      // this lane's rows l, l + 32, ...: row n sits in group n / 8, its scale words after the group's codes
      const uint8_t *sw = c.ring + size_t(s) * kMegaSlotBytes + size_t(c.lane >> 3) * gb + kc * 128 + (c.lane & 7) * 4;
#pragma unroll 1
      for (int j = 0; j < (kc + 3) / 4; ++j) {                // 4 K blocks: columns c, c + 1, ... for rows 32 i + l
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          w[i] = c.lane + 32 * i < N ? *reinterpret_cast<const uint32_t *>(sw + size_t(4 * i) * gb + j * 32) : 0u;
        tc_st_words8(tSFB + uint32_t(ch * (mkc >> 2) + j) * 8, w);
      }
      tc_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (c.lane == 0) mbar_arrive(&c.sm->sready[(c.nmx + uint32_t(ch)) % kMegaSlots]);
    }
  }
  if (work && c.warp == 0) {
    const uint32_t tSFA = tmem, tSFB = tmem + 96, tD = tmem + 288;
    const int ngroups = (kblocks + 3) / 4;
    for (int g = 0; g < ngroups; g += 4) {
      const uint32_t *w = reinterpret_cast<const uint32_t *>(mx.sf[0] + (c.lane & 7) * 96) + g;
      tc_st_words4(tSFA + 4 * g, w[0], ngroups - g > 1 ? w[1] : 0u, ngroups - g > 2 ? w[2] : 0u, ngroups - g > 3 ? w[3] : 0u);
    }
    // this lane's biases travel while the weights stream (lane l < 8 finishes columns 32 i + 4 l .. + 3)
    const float *bias = job.bias + size_t(c.sm->r_active[slot_e]) * R + size_t(g0) * 8;
    float4 bpre[5];
#pragma unroll
    for (int i = 0; i < 5; ++i)
      bpre[i] = (c.lane < 8 && 32 * i + 4 * c.lane < N) ? __ldg(reinterpret_cast<const float4 *>(bias + 32 * i + 4 * c.lane)) : f4_zero();
    const uint32_t a_base = smem_u32(mx.a[0]);
    const uint32_t id0 = mx_idesc(128, N, 0, 0), id2 = mx_idesc(128, N, 2, 2);
    bool ok = true;
#pragma unroll 1
    for (int ch = 0; ch < nchunks && ok; ++ch) {
      const uint32_t q = c.seq + uint32_t(ch), s = q % kMegaSlots;
      const uint32_t qs = c.nmx + uint32_t(ch);
      ok = mega_wait(&c.sm->sready[qs % kMegaSlots], (qs / kMegaSlots) & 1, c.sm, c.g->status, 22);   // data landed, scales stored (warp 4)
      if (!ok) break;
      if (ch == 0) mega_stamp(c);                             // time to the first data of the phase
      const int kc = min(mkc, kblocks - ch * mkc);
      const uint8_t *slot = c.ring + size_t(s) * kMegaSlotBytes;
      tc_fence_after_sync();
      {
        // 2 K blocks per instruction: 256 B further in A, 256 B further in this slot's B (16-byte units);
        // B: K blocks of a group 128 B apart, groups mxw_group_bytes apart.  The whole (converged) warp runs
        // this; an elected lane issues (mx_mma_pair_warp), so the warp-uniform operands need no divergent code.
        uint64_t da = tc_smem_desc(a_base + uint32_t(ch * mkc) * 128, 128, 128);
        uint64_t db = tc_smem_desc(smem_u32(slot), 128, uint32_t(mxw_group_bytes(kc)));
        uint32_t sfa = tSFA + 4 * uint32_t(ch * (mkc >> 2)), sfb = tSFB + 8 * uint32_t(ch * (mkc >> 2));   // first group of 4 K blocks
#pragma unroll 1
        for (int st = 0; st < kc / 2; st += 2) {              // 4 K blocks = one group of scale columns = two instructions
          mx_mma_pair_warp(tD, da, db, id0, id2, sfa, sfb, !(ch == 0 && st == 0), st + 1 < kc / 2);
          da += 32; db += 32; sfa += 4; sfb += 8;
        }
        // the slot's `empty` barrier expects the 15 consumer warps: 14 arrivals now, the 15th when the
        // tensor core has read the slot
        mbar_arrive_n_warp(&c.sm->empty[s], kMegaConsumers - 1);
        tc_commit_warp(&c.sm->empty[s], true);
        tc_commit_warp(&c.sm->done[0], ch == nchunks - 1);
      }
      __syncwarp();
    }
    if (ok && mega_wait(&c.sm->done[0], c.ndone & 1, c.sm, c.g->status, 23)) {
      c.ndone++;
      tc_fence_after_sync();
      const int rank = c.sm->r_assign[slot_e];
#pragma unroll
      for (int ci = 0; ci < 5; ++ci) {
        const int c0 = 32 * ci;
        if (c0 >= N) break;
        // lanes 0..7 hold the digit rows of D[.][c0..c0+31]: add them up, lane l keeps columns c0 + 4l..4l+3
        float v[32];
        {
          float lo[16], hi16[16];
          tc_ld16(tD + c0, lo);
          tc_ld16(tD + c0 + 16, hi16);
#pragma unroll
          for (int i = 0; i < 16; ++i) { v[i] = c.lane < 8 ? lo[i] : 0.f; v[16 + i] = c.lane < 8 ? hi16[i] : 0.f; }
        }
        float r16[16], r8[8], r4[4];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float mine = (c.lane & 4) ? v[16 + i] : v[i], other = (c.lane & 4) ? v[i] : v[16 + i];
          r16[i] = mine + __shfl_xor_sync(0xffffffffu, other, 4);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float mine = (c.lane & 2) ? r16[8 + i] : r16[i], other = (c.lane & 2) ? r16[i] : r16[8 + i];
          r8[i] = mine + __shfl_xor_sync(0xffffffffu, other, 2);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float mine = (c.lane & 1) ? r8[4 + i] : r8[i], other = (c.lane & 1) ? r8[i] : r8[4 + i];
          r4[i] = mine + __shfl_xor_sync(0xffffffffu, other, 1);
        }
        const int col = c0 + 4 * c.lane;
        if (c.lane < 8 && col < N) {
          const int row = g0 * 8 + col;
          const float4 b = bpre[ci];
          if (job.kind == 0) {
            *reinterpret_cast<float2 *>(job.out + size_t(rank) * (R >> 1) + (row >> 1)) =
                make_float2(swiglu_clamped(r4[0] + b.x, r4[1] + b.y, job.alpha, job.limit),
                            swiglu_clamped(r4[2] + b.z, r4[3] + b.w, job.alpha, job.limit));
          } else {
            *reinterpret_cast<float4 *>(job.out + size_t(rank) * R + row) =
                make_float4(r4[0] + b.x, r4[1] + b.y, r4[2] + b.z, r4[3] + b.w);
          }
        }
      }
      tc_fence_before_sync();
    }
  }
  if (ng > 0) c.seq += uint32_t(nchunks);
  if (work) c.nmx += uint32_t(nchunks);
  if (!(work && c.warp == 0)) mega_stamp(c);      // thread 0 stamps in the loop above when it has work
}

// grid = one CTA per SM (cooperative launch), 512 threads, dynamic shared
// memory mega_smem_bytes().  g->sync (2 KB) must be zero at launch.
//
// Consumers run a phase loop: per layer 0 = qkv, 1 = attention, 2 = o-proj,
// 3 = router + experts' gate_up, 4 = experts' down; after the last layer one
// more phase 0 = lm_head + argmax.  Every phase ends with a grid barrier.
extern "C" __global__ void __launch_bounds__(kMegaThreads, 1)
mega_decode(const MegaGlobals *__restrict__ gp, MegaArgs a) {
  MegaSmem *sm = reinterpret_cast<MegaSmem *>(dyn_smem + size_t(kMegaSlots) * kMegaSlotBytes);
  MegaCtx c;
  c.sm = sm;
  c.ring = dyn_smem;
  c.g = gp;
  c.nbar = 0;
  c.seq = 0;
  c.pbuf = 0;
  c.nstamp = 0;
  c.ndone = 0;
  c.nmx = 0;
  c.skip_fill = uint32_t(a.test_skip_fill);
  c.tid = threadIdx.x;
  c.lane = threadIdx.x & 31;
  c.warp = threadIdx.x >> 5;
  if (c.tid == 0) {
    for (int i = 0; i < kMegaSlots; ++i) {
      mbar_init(&sm->full[i], 1);
      mbar_init(&sm->empty[i], kMegaConsumers);
    }
    mbar_init(&sm->route_bar, 1);
    for (int i = 0; i < 3; ++i) mbar_init(&sm->done[i], 1);
    for (int i = 0; i < kMegaSlots; ++i) mbar_init(&sm->sready[i], 1);
    sm->abort = 0;
    sm->spin = a.spin ? a.spin : kMegaSpin;
  }
  fence_barrier_init();
  if (a.mx && c.warp == 0) tc_alloc(&sm->tmem_base, 512);       // the only CTA on this SM: all of tensor memory
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (c.warp == kMegaConsumers) {
    if (c.lane == 0) mega_producer(c, a);
    return;
  }

  mega_stamp(c);
  const MegaGlobals &g = *gp;
  const int H = a.H, I = a.I, QD = a.NQ * 64, QKV = QD + 2 * a.NKV * 64;
  const int n4 = H >> 2;
  const int tok = min(max(g.meta[0], 0), a.V - 1), pos = g.meta[1];
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  int nsplit = 1;

#pragma unroll 1
  for (int l = 0; l <= a.layers; ++l) {
    const bool last = l == a.layers;
    const MegaLayer &ly = g.layers[last ? 0 : l];
    const int n_phases = last ? 1 : 5;
#pragma unroll 1
    for (int ph = 0; ph < n_phases; ++ph) {
      if (ph == 0 || ph == 2) {
        // ---- dense: (embedding | experts' combine + residual) -> RMSNorm -> qkv or lm_head; attention -> o-proj
        DenseJob job;
        if (ph == 0) {
          XVec x;
          if (l == 0) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int i = c.tid + u * kMegaConsThreads;
              x.v[u] = f4_zero();
              if (i < n4) {
                const uint2 e = __ldg(reinterpret_cast<const uint2 *>(g.embed + size_t(tok) * H) + i);
                x.v[u] = make_float4(bf16_lo(e.x), bf16_hi(e.x), bf16_lo(e.y), bf16_hi(e.y));
                if (blockIdx.x == 0) reinterpret_cast<float4 *>(g.hA)[i] = x.v[u];
              }
            }
          } else {
            mega_load_combined(c, x, g.hB, g.o, H, a.top_k, (blockIdx.x == 0 && !last) ? g.hA : nullptr);
          }
          mega_norm_to_xs(c, x, last ? g.lnf : ly.ln1, H, a.eps, nullptr);
          mega_stamp(c);
          job.kind = last ? 2 : 0;
          job.rows = last ? a.V : QKV;
          job.K = H;
          job.bias = ly.bqkv;
          job.res = nullptr;
          job.out = last ? g.logits : g.qkv;
          job.wr = nullptr; job.ln2 = nullptr; job.E = 0; job.H = H;
        } else {
          mega_stage_plain(c, g.attn, QD);
          job.kind = 1;
          job.rows = H;
          job.K = QD;
          job.bias = ly.bo;
          job.res = g.hA;
          job.out = g.hB;
          job.wr = ly.wr; job.ln2 = ly.ln2; job.E = a.E; job.H = H;
        }
        consume_dense(c, job, bv, bi);
        if (ph == 0 && !last) {
          // attention's cache rows of this CTA's first unit depend only on the position:
          // request them before the barrier that waits for q, k and v
          const int window = int(ly.window);
          const int lo_vis = window > 0 ? max(0, pos + 1 - window) : 0;
          nsplit = (pos + 1 - lo_vis + kAttnSplit - 1) / kAttnSplit;
          cons_sync();            // every warp has taken its activations out of xs (same storage)
          if (c.warp < kMegaAttnWarps && int(blockIdx.x) < nsplit * a.NKV) {
            const AttnGeom ge = mega_attn_geom(blockIdx.x, nsplit, pos, window, int(ly.cache_len), a.NKV);
            mega_attn_prefetch(sm->u.attn, ge, c.tid, reinterpret_cast<const uint16_t *>(ly.kcache),
                               reinterpret_cast<const uint16_t *>(ly.vcache), int(ly.cache_len));
          }
        }
      } else if (ph == 1) {
        // ---- attention (warps 0..7; one (slice, kv head) unit at a time)
        if (c.warp < kMegaAttnWarps) {
#pragma unroll 1
          for (int u = blockIdx.x; u < nsplit * a.NKV; u += gridDim.x) {
            const AttnGeom ge = mega_attn_geom(u, nsplit, pos, int(ly.window), int(ly.cache_len), a.NKV);
            if (u != int(blockIdx.x))
              mega_attn_prefetch(sm->u.attn, ge, c.tid, reinterpret_cast<const uint16_t *>(ly.kcache),
                                 reinterpret_cast<const uint16_t *>(ly.vcache), int(ly.cache_len));
            mega_attn_unit(c, sm->u.attn, ge, pos, a, ly, int(ly.cache_len));
            attn_sync<2, kMegaAttnWarps * 32>();
          }
        }
      } else {
        // ---- experts: (RMSNorm -> router -> top-k ->) gate_up + clamped SwiGLU -> act; down -> o
        ExpertJob job;
        job.kind = ph == 3 ? 0 : 1;
        job.alpha = a.alpha;
        job.limit = a.limit;
        if (ph == 3) {
          XVec x;
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int i = c.tid + u * kMegaConsThreads;
            x.v[u] = i < n4 ? __ldcg(reinterpret_cast<const float4 *>(g.hB) + i) : f4_zero();
          }
          mega_route(c, a, ly, x);
          mega_stamp(c);
          job.R = 2 * I; job.K = H; job.bias = ly.gu_bias; job.xsrc = nullptr; job.out = g.act; job.kc = a.kc_gu;
        } else {
          job.R = H; job.K = I; job.bias = ly.dn_bias; job.xsrc = g.act; job.out = g.o; job.kc = a.kc_dn;
        }
        if (a.mx) consume_experts_mx(c, job, a.top_k);
        else consume_experts(c, job, a.top_k);
      }
      if (!last) grid_barrier(c);
    }
  }

  // ---- greedy argmax over the CTAs' candidates, fed back into meta
  if (c.warp < 2) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      argmax_combine(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if (c.lane == 0) { sm->am_v[c.warp] = bv; sm->am_i[c.warp] = bi; }
  }
  cons_sync();
  if (c.tid == 0) {
    argmax_combine(bv, bi, sm->am_v[1], sm->am_i[1]);
    g.am_v[blockIdx.x] = bv;
    g.am_i[blockIdx.x] = bi;
  }
  grid_barrier(c);
  if (blockIdx.x == 0 && c.warp == 0) {
    bv = -INFINITY;
    bi = 0x7fffffff;
    for (int q = c.lane; q < int(gridDim.x); q += 32) argmax_combine(bv, bi, __ldcg(g.am_v + q), __ldcg(g.am_i + q));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      argmax_combine(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if (c.lane == 0) {
      if (bi == 0x7fffffff) bi = 0;
      g.next_tok[0] = bi;
      g.meta[0] = bi;
      g.meta[1] = pos + 1;
    }
  }
  if (a.mx && c.warp == 0) {           // every engine finished before the barriers above
    tc_fence_after_sync();
    tc_dealloc(sm->tmem_base, 512);
  }
}
