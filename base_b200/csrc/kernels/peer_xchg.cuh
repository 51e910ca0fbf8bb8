// Dispatch and combine of the expert-parallel decode step, done by the producing kernels themselves over peer
// memory (NVLink stores into the other ranks' buffers), in place of an all-gather and an all-to-all:
//
//   rows_to_peers          RMSNorm of this rank's sequences -> the rows [rank * B, (rank + 1) * B) of EVERY rank's
//                          xn_all (the experts' input; the reference has one device and no dispatch,
//                          lean/lib/AlgorithmLib/ML/Compose.lean:1812-1828 is the per-token expert loop this shards)
//   moe_router_many_peer   waits for every rank's rows, then the router of moe_router_many
//   moe_combine_peers      this rank's partial expert sums of sequence t -> slot `rank` of y_recv on the rank that
//                          owns t
//   rows_to_a_peer         waits for every rank's partial sums, then rows_to_a (mode 1 adds them in rank order, so
//                          the result does not depend on arrival order)
//
// Flags: every rank has a block of 32-bit words (its `flags` buffer): word 0 the step count (peer_epoch_bump, first
// kernel of a step), word 128 + 32 r the dispatch counter of source rank r, word 128 + 32 (8 + r) its combine counter.
// A producer CTA stores its rows, meets (bar.sync), and one thread per destination adds 1 to its counter there with
// red.release.sys (the release covers the whole CTA's stores: they happen before it through the barrier; a fence per
// storing thread and a last-CTA ticket, the first version of this file, cost 15 us per exchange).  Counters only grow:
// a consumer waits until the counter has reached (rounds so far) x (CTAs per round and source), rounds = (step - 1) x
// layers + layer + 1 (ranks run the same steps; a producer cannot get a layer ahead, because each exchange needs the
// one before it from every rank).  Every wait is bounded in time (about 1.5 s) and in iterations; when it runs out
// the kernel stores a code in *status and carries on with what is there, so the step ends and the host reports the
// failure.
#pragma once
#include "batch_dense.cuh"
#include "moe_prefill.cuh"

constexpr int kPeerMax = 8;
constexpr int kPeerWordEpoch = 0, kPeerWordFlags = 128;
constexpr int kPeerCodeDispatch = 4001, kPeerCodeCombine = 4002;

struct PeerTable {
  unsigned long long xn_all[kPeerMax], y_recv[kPeerMax], flags[kPeerMax];   // addresses in this process; own entries local
  int rank, world;
};

B200_DEVICE uint32_t peer_ld_acquire(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

B200_DEVICE void peer_red_release(uint32_t *p) {
  asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p) : "memory");
}

// What a counter reaches when the round (step, layer `tag`) is complete: per_round arrivals per round and source.
B200_DEVICE uint32_t peer_target(const uint32_t *my_flags, int tag, int layers, int per_round) {
  const uint32_t step = *reinterpret_cast<const volatile uint32_t *>(my_flags + kPeerWordEpoch);      // >= 1
  return ((step - 1u) * uint32_t(layers) + uint32_t(tag) + 1u) * uint32_t(per_round);
}

// Threads 0 .. world-1 of the CTA each wait for one source rank's counter; then the CTA meets.
B200_DEVICE void peer_wait_all(const PeerTable *pt, const uint32_t *my_flags, int slot0, uint32_t target, int *status, int code) {
  // a wait that ran out earlier in the step is not repeated by every kernel after it
  if (int(threadIdx.x) < pt->world && *reinterpret_cast<volatile int *>(status) == 0) {
    const uint32_t *f = my_flags + kPeerWordFlags + 32 * (slot0 + int(threadIdx.x));
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    bool ok = false;
    for (uint32_t it = 0; it < (1u << 26); ++it) {
      if (int(peer_ld_acquire(f) - target) >= 0) { ok = true; break; }
      if ((it & 63u) == 63u) {
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > 1500000000ull) break;
      }
      __nanosleep(40);
    }
    if (!ok) atomicCAS(status, 0, code);
  }
  __syncthreads();
}

// Time stamps of the last step (ns, %globaltimer), for reading where a sharded step spends its time: 8 per layer tag
// at byte 8192 of the flags buffer: 0 rows_to_peers start, 1 router start, 2 router after its wait, 3 combine start,
// 4 the next normalisation's start, 5 after its wait.  Written by one thread per kernel.
constexpr int kPeerTraceWord = 2048;
B200_DEVICE void peer_stamp(uint32_t *my_flags, int tag, int slot) {
  if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    reinterpret_cast<unsigned long long *>(my_flags + kPeerTraceWord)[tag * 8 + slot] = t;
  }
}

extern "C" __global__ void peer_epoch_bump(uint32_t *my_flags, int) {
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x == 0 && blockIdx.x == 0) my_flags[kPeerWordEpoch] += 1u;
}

// One CTA of 256 threads per sequence of this rank: x = h * inv * w (as rows_to_a mode 2), stored to every rank.
struct RowsToPeersArgs { int K, B, tag, layers; float eps; };

extern "C" __global__ void __launch_bounds__(256)
rows_to_peers(const float *__restrict__ in, const float *__restrict__ w, const PeerTable *__restrict__ pt,
              uint32_t *__restrict__ my_flags, RowsToPeersArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  peer_stamp(my_flags, a.tag, 0);
  __shared__ float red[8];
  const int t = blockIdx.x, tid = threadIdx.x, K = a.K;
  float4 v[4];
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int i4 = tid + 256 * u;
    v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i4 * 4 < K) v[u] = __ldcg(reinterpret_cast<const float4 *>(in + size_t(t) * K) + i4);
    ss = fmaf(v[u].x, v[u].x, ss); ss = fmaf(v[u].y, v[u].y, ss); ss = fmaf(v[u].z, v[u].z, ss); ss = fmaf(v[u].w, v[u].w, ss);
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float inv = 1.0f / sqrtf(tot / float(K) + a.eps);
  const int world = pt->world, row = pt->rank * a.B + t;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int i4 = tid + 256 * u;
    if (i4 * 4 < K) {
      const float4 g = __ldg(reinterpret_cast<const float4 *>(w) + i4);
      const float4 x = make_float4(v[u].x * inv * g.x, v[u].y * inv * g.y, v[u].z * inv * g.z, v[u].w * inv * g.w);
      for (int r = 0; r < world; ++r)
        reinterpret_cast<float4 *>(reinterpret_cast<float *>(pt->xn_all[r]) + size_t(row) * K)[i4] = x;
    }
  }
  __syncthreads();
  if (tid < world) peer_red_release(reinterpret_cast<uint32_t *>(pt->flags[tid]) + kPeerWordFlags + 32 * pt->rank);
}

// per_round = the sequences per rank: every source rank's rows_to_peers has that many CTAs.
struct RouterPeerArgs { RouterManyArgs r; int tag, layers, per_round; };

extern "C" __global__ void __launch_bounds__(256)
moe_router_many_peer(const float *__restrict__ Wr, const float *__restrict__ br, const float *__restrict__ x,
                     float *__restrict__ logits, const PeerTable *__restrict__ pt, uint32_t *__restrict__ my_flags,
                     int *__restrict__ status, RouterPeerArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  peer_stamp(my_flags, a.tag, 1);
  peer_wait_all(pt, my_flags, 0, peer_target(my_flags, a.tag, a.layers, a.per_round), status, kPeerCodeDispatch);
  peer_stamp(my_flags, a.tag, 2);
  router_many_body(Wr, br, x, logits, a.r);
}

// grid = all sequences of all ranks, one CTA of 256 threads each: y of sequence t, summed over this rank's experts in
// slot order (as moe_combine_range), goes to the rank that holds t, which counts one arrival per sequence and source.
struct CombinePeersArgs { int H, top_k, lo, n, B, tag, layers; };

extern "C" __global__ void __launch_bounds__(256)
moe_combine_peers(const float *__restrict__ o, const float *__restrict__ topk_w, const int *__restrict__ topk_idx,
                  const PeerTable *__restrict__ pt, uint32_t *__restrict__ my_flags, CombinePeersArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  peer_stamp(my_flags, a.tag, 3);
  const int t = blockIdx.x, tid = threadIdx.x;
  const int owner = t / a.B, local = t - owner * a.B;
  float w[8];
  bool mine[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    mine[j] = false;
    w[j] = 0.f;
    if (j < a.top_k) {
      const int e = __ldcg(topk_idx + t * a.top_k + j);
      mine[j] = e >= a.lo && e < a.lo + a.n;
      w[j] = __ldcg(topk_w + t * a.top_k + j);
    }
  }
  float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(pt->y_recv[owner]) + (size_t(pt->rank) * a.B + local) * a.H);
  for (int i4 = tid; i4 * 4 < a.H; i4 += 256) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (mine[j]) {
        const float4 p = __ldcg(reinterpret_cast<const float4 *>(o + size_t(t * a.top_k + j) * a.H) + i4);
        v.x = fmaf(w[j], p.x, v.x); v.y = fmaf(w[j], p.y, v.y); v.z = fmaf(w[j], p.z, v.z); v.w = fmaf(w[j], p.w, v.w);
      }
    dst[i4] = v;
  }
  __syncthreads();
  if (tid == 0) peer_red_release(reinterpret_cast<uint32_t *>(pt->flags[owner]) + kPeerWordFlags + 32 * (kPeerMax + pt->rank));
}

struct RowsToAPeerArgs { RowsToAArgs r; int tag, layers; };

extern "C" __global__ void __launch_bounds__(256)
rows_to_a_peer(const float *__restrict__ in, const float *__restrict__ parts, const float *__restrict__ w,
               float *__restrict__ hout, float *__restrict__ xn, uint16_t *__restrict__ a_tiled,
               const PeerTable *__restrict__ pt, uint32_t *__restrict__ my_flags, int *__restrict__ status,
               RowsToAPeerArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  peer_stamp(my_flags, a.tag, 4);
  // every source rank's moe_combine_peers signals once per sequence of this rank
  peer_wait_all(pt, my_flags, kPeerMax, peer_target(my_flags, a.tag, a.layers, a.r.B), status, kPeerCodeCombine);
  peer_stamp(my_flags, a.tag, 5);
  rows_to_a_body(in, parts, w, hout, xn, a_tiled, a.r);
}
