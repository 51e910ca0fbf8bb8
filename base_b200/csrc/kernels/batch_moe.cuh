// MXFP4 expert GEMVs for a BATCH of tokens on the block-scaled tensor cores (tcgen05.mma.kind::mxf4): every
// expert's weights are read once for all the tokens routed to it.
//
// Same arithmetic as the one-token path (moe_mx.cuh, the expert phases of mega_decode.cuh): the weights are the
// B operand as stored (codes + UE8M0 scales, "wide" layout of mxfp4_retile_wide with 8 K blocks per chunk), the
// activations are the A operand written in balanced radix 8 (mx_expand_radix8: 8 E2M1 digit rows per token with
// block scales 8^(7-t), exact to 2^-22 of each 32-element block's maximum), y = sum of the 8 digit rows.  Here a
// token takes 8 of the 128 A rows, so ONE instruction serves up to 16 tokens of an expert; an expert with more
// tokens is run in passes of 16 (its weights are then served from L2).
//
//   moe_expand_digits   f32 rows -> digits, in the order of the routing permutation (an expert's tokens contiguous):
//                       dig [chunk of 8 K blocks][position][K block of the chunk][8 digit rows x 16 B] (the tokens of an
//                       expert are ONE contiguous piece per chunk), em [position][96] block exponents
//   mxfp4_retile_seg16  checkpoint layout -> per chunk of 8 K blocks and segment of 16 eight-row groups: the segment's codes
//                       ([group][K block][8 rows x 16 B]) followed by its scale words laid out for tcgen05.cp
//                       ([4-block group][32 lanes][16 B]: lane l = the words of rows l, 32 + l, 64 + l, 96 + l)
//   moe_batch_mx_*      units = (expert, pass of <= 16 tokens, segment): N <= 128 rows per instruction; producer warp
//                       (two bulk copies per ring slot: the segment's piece and the tokens' digits of one chunk), issuer
//                       (per 4 K blocks: one tcgen05.cp of the weights' scale words, two instructions), four epilogue
//                       warps (each reads the accumulator rows of four tokens, adds the digit rows, bias, clamped SwiGLU).
// Scale factors in tensor memory: the tensor core's lane quarter q (accumulator rows 32 q ..) takes BOTH operands' scales
// from its own 32 lanes, so every quarter needs a copy.  tcgen05.cp ... 32x128b.warpx4 writes all four by itself (the
// weights' scales); the tokens' scales are computed here and written with tcgen05.st by one warp per quarter.  With one
// token only quarter 0 carries results, which is why the one-token kernels write a single copy.
// Routing tables are those of moe_route_tables_many (count / offset / perm).  Every wait is bounded.
#pragma once
#include "moe_mx.cuh"

constexpr int kBmTok = 16;                   // tokens per pass
constexpr int kBmGroups = 16;                // 8-row groups per unit (N = 128)
constexpr int kBmKc = 8;                     // K blocks per chunk
constexpr int kBmSlots = 8;                  // at most; the ring holds as many slots as fit
constexpr int kBmBBytes = kBmGroups * (kBmKc * 128 + 64);      // 17408: codes + scale words of a chunk
constexpr int kBmRingBytes = 8 * (kBmBBytes + 8 * kBmKc * 128);  // 204800: eight slots when no pass has more than 8 tokens
// A ring slot = [digits of the unit's tokens for one chunk: 1 KB per token, sized for the most tokens any of this CTA's
// units has][the segment's piece, kBmBBytes reserved].  The tensor core reads 128 A rows = 16 KB from the digits' base
// whatever the token count: what lies beyond the tokens is this slot's own weight piece (results of those rows are
// never read).  Fewer tokens per pass = smaller slots = more weight bytes in flight.
constexpr int kBmThreads = 192;              // warps 0..3 epilogue, 4 issuer, 5 producer
constexpr int kBmEmStride = 96;
constexpr int kBmMaxUnits = 192;             // units one CTA can take

// ---- activations -> digits -----------------------------------------------------------------------------
// grid = positions [pos0, pos0 + n) of the permutation, 384 threads (4 per K block).  Position p holds assignment
// a = perm[p]; its source row is x[a / top_k] (gate_up: the token's normalised hidden state) or x[a] (down: the
// assignment's activation).  P = total positions (the stride of the digit array).
struct ExpandArgs { int K, P, pos0, n, top_k, per_token, E; };

extern "C" __global__ void __launch_bounds__(384)
moe_expand_digits(const float *__restrict__ x, const int *__restrict__ route, uint8_t *__restrict__ dig,
                  uint8_t *__restrict__ em, ExpandArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  const int E = a.E;
  const int *perm = route + 1 + E + (E + 1) + E;
  const int *offset = route + 1 + E;
  // pos0 < 0: the range is the one of experts [-pos0 - 1, -pos0 - 1 + n) (read from the tables on the device)
  int p0 = a.pos0, cnt = a.n;
  if (a.pos0 < 0) { const int lo = -a.pos0 - 1; p0 = offset[lo]; cnt = offset[lo + a.n] - p0; }
  const int kblocks = a.K >> 5;
  for (int pi = blockIdx.x; pi < cnt; pi += gridDim.x) {
    const int p = p0 + pi, asg = perm[p];
    const float *src = x + size_t(a.per_token ? asg / a.top_k : asg) * a.K;
    const int kb = threadIdx.x >> 2, sub = threadIdx.x & 3;
    const bool valid = kb < kblocks;
    float v[8];
    const float4 v0 = valid ? __ldcg(reinterpret_cast<const float4 *>(src + kb * 32 + sub * 8)) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 v1 = valid ? __ldcg(reinterpret_cast<const float4 *>(src + kb * 32 + sub * 8 + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
    v[0] = v0.x; v[1] = v0.y; v[2] = v0.z; v[3] = v0.w; v[4] = v1.x; v[5] = v1.y; v[6] = v1.z; v[7] = v1.w;
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
    uint32_t e8 = (__float_as_uint(m) >> 23) & 0xffu;
    int X[8];
    if (e8 >= 40 && e8 < 255) {
      const float up = __uint_as_float((275u - e8) << 23);
#pragma unroll
      for (int i = 0; i < 8; ++i) X[i] = __float2int_rn(v[i] * up);
    } else {
      e8 = 40;
#pragma unroll
      for (int i = 0; i < 8; ++i) X[i] = 0;
    }
    if (valid) {
      uint8_t *d = dig + ((size_t(kb / kBmKc) * a.P + p) * kBmKc + (kb % kBmKc)) * 128 + sub * 4;
#pragma unroll
      for (int q = 0; q < 8; ++q) {                       // digit q (weight 8^q) is digit row 7 - q
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int t1 = X[i] + 4;
          word |= ((kMxDigitLut >> ((t1 & 7) << 2)) & 15u) << (4 * i);
          X[i] = t1 >> 3;
        }
        *reinterpret_cast<uint32_t *>(d + (7 - q) * 16) = word;
      }
      if (sub == 0) em[size_t(p) * kBmEmStride + kb] = uint8_t(e8);
    }
    // K blocks past the end of the row (padding of the last 4-block group): exponent 127
    if (threadIdx.x < kBmEmStride - kblocks) em[size_t(p) * kBmEmStride + kblocks + threadIdx.x] = 127;
  }
}

// ---- weights: checkpoint layout -> segments of 16 groups ---------------------------------------------------
B200_DEVICE size_t seg16_bytes(int kcc, int ng) { return size_t(ng) * kcc * 128 + size_t((kcc + 3) / 4) * 512; }
B200_DEVICE size_t seg16_chunk_bytes(int kcc, int G) {
  const int nseg = (G + kBmGroups - 1) / kBmGroups;
  return size_t(G) * kcc * 128 + size_t(nseg) * ((kcc + 3) / 4) * 512;
}
B200_DEVICE size_t seg16_matrix_bytes(int kblocks, int G) {
  const int full = kblocks / kBmKc, tail = kblocks - full * kBmKc;
  return size_t(full) * seg16_chunk_bytes(kBmKc, G) + (tail ? seg16_chunk_bytes(tail, G) : 0);
}
// start of segment `seg` of chunk c (every earlier chunk and segment is a full one)
B200_DEVICE size_t seg16_offset(int c, int seg, int kcc, int G) {
  return size_t(c) * seg16_chunk_bytes(kBmKc, G) + size_t(seg) * seg16_bytes(kcc, kBmGroups);
}

struct RetileSegArgs { int R, K, n_mat; };

// codes [n_mat][R][K / 2], scales [n_mat][R][K / 32]; one thread per 16 bytes of codes, and per scale word.
extern "C" __global__ void __launch_bounds__(256)
mxfp4_retile_seg16(const uint8_t *__restrict__ codes, const uint8_t *__restrict__ scales, uint8_t *__restrict__ out, RetileSegArgs a) {
  const int kblocks = a.K >> 5, G = a.R >> 3, nch = (kblocks + kBmKc - 1) / kBmKc, nseg = (G + kBmGroups - 1) / kBmGroups;
  const size_t mbytes = seg16_matrix_bytes(kblocks, G);
  const size_t gid = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t total = size_t(a.n_mat) * a.R * kblocks;
  if (gid < total) {
    const int kb = int(gid % kblocks);
    const size_t row_all = gid / kblocks;
    const int row = int(row_all % a.R);
    const size_t mat = row_all / a.R;
    const int c = kb / kBmKc, kbl = kb % kBmKc, kcc = min(kBmKc, kblocks - c * kBmKc), g = row >> 3, seg = g / kBmGroups;
    uint8_t *dst = out + mat * mbytes + seg16_offset(c, seg, kcc, G) + (size_t(g % kBmGroups) * kcc + kbl) * 128 + (row & 7) * 16;
    *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(codes + row_all * (a.K >> 1) + size_t(kb) * 16);
  }
  // scale words: (matrix, chunk, segment, 4-block group j, lane l, row group q)
  const size_t stotal = size_t(a.n_mat) * nch * nseg * 2 * 128;
  if (gid < stotal) {
    const int q = int(gid & 3), l = int((gid >> 2) & 31), j = int((gid >> 7) & 1);
    size_t rest = gid >> 8;
    const int seg = int(rest % nseg);
    rest /= nseg;
    const int c = int(rest % nch);
    const size_t mat = rest / nch;
    const int kcc = min(kBmKc, kblocks - c * kBmKc), ng = min(kBmGroups, G - seg * kBmGroups);
    if (j < (kcc + 3) / 4) {
      const int g = 4 * q + (l >> 3);                       // group of row 32 q + l within the segment
      uint32_t w = 0x7f7f7f7fu;
      if (g < ng) {
        w = 0;
        const size_t row = mat * a.R + size_t(seg * kBmGroups + g) * 8 + (l & 7);
        for (int b = 0; b < 4; ++b) {
          const int kb = c * kBmKc + 4 * j + b;
          w |= (kb < kblocks ? uint32_t(scales[row * kblocks + kb]) : 127u) << (8 * b);
        }
      }
      uint8_t *dst = out + mat * mbytes + seg16_offset(c, seg, kcc, G) + size_t(ng) * kcc * 128 + j * 512 + l * 16 + q * 4;
      *reinterpret_cast<uint32_t *>(dst) = w;
    }
  }
}

// ---- the expert kernel -----------------------------------------------------------------------------------
struct BatchMxArgs {
  MoeDims d;
  int lo, n;            // experts [lo, lo + n) are resident here; the weight array starts at expert lo, the biases at expert 0
  int P;                // positions of the digit array (all assignments of the step)
};

struct BmUnit { int16_t e, pass, g0, ng; };

struct BmBars {
  uint64_t full[kBmSlots], empty[kBmSlots], done[2], uready[2];
  uint32_t tmem_base;
  int abort, n_units, u_base, max_nt;
  uint32_t em_s[2][kBmTok * (kBmEmStride / 4)];      // block exponents of the tokens of two units in flight
};

B200_DEVICE bool bm_wait(uint64_t *bar, uint32_t parity, BmBars *b, int *status, int code) {
  const uint32_t lim = *reinterpret_cast<volatile int *>(&b->abort) ? 4096u : kTcSpin;
  for (uint32_t i = 0; i < lim; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  *reinterpret_cast<volatile int *>(&b->abort) = 1;
  atomicCAS(status, 0, code);
  return false;
}

B200_DEVICE int bm_smem_bytes() { return kBmRingBytes + kBmMaxUnits * int(sizeof(BmUnit)) + int(sizeof(BmBars)) + 64; }

// Two instructions over four consecutive K blocks (scale bytes 0,1 then 2,3 of one column group), issued by an
// elected lane of the converged warp; the second one's operands are a_step / b_step descriptor units further.
// Before them the same lane copies the weights' scale words of these four K blocks from shared memory (32 lanes x 16 B)
// into the four columns at sfb_tmem of every lane quarter; copies and instructions of one thread execute in order.
B200_DEVICE void bm_mma_pair_warp(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc01, uint32_t idesc23,
                                  uint32_t sfa_tmem, uint32_t sfb_tmem, bool accumulate_first, bool second, uint32_t a_step,
                                  uint32_t b_step, uint64_t sf_desc) {
  asm volatile(
      "{\n.reg .pred p, q, e, e2;\n.reg .b64 a2, b2, sa, sb;\n"
      "elect.sync _|e, 0xffffffff;\n"
      "@e tcgen05.cp.cta_group::1.32x128b.warpx4 [%7], %11;\n"
      "setp.ne.b32 p, %5, 0;\nsetp.eq.b32 q, %5, %5;\nsetp.ne.b32 e2, %8, 0;\nand.pred e2, e2, e;\n"
      "@e tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%6], [%7], p;\n"
      "cvt.u64.u32 sa, %9;\ncvt.u64.u32 sb, %10;\nadd.u64 a2, %1, sa;\nadd.u64 b2, %2, sb;\n"
      "@e2 tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], a2, b2, %4, [%6], [%7], q;\n}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc01), "r"(idesc23), "r"(uint32_t(accumulate_first)), "r"(sfa_tmem), "r"(sfb_tmem),
      "r"(uint32_t(second)), "r"(a_step), "r"(b_step), "l"(sf_desc)
      : "memory");
}

// Four words per lane -> four consecutive columns.
B200_DEVICE void tc_st_cols4(uint32_t taddr, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3) {      // whole warp
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(w0), "r"(w1), "r"(w2), "r"(w3)
               : "memory");
}

template <bool GATE_UP>
B200_DEVICE void batch_mx_body(const uint8_t *__restrict__ W, const float *__restrict__ bias, const uint8_t *__restrict__ dig,
                               const uint8_t *__restrict__ em, const int *__restrict__ route, float *__restrict__ out,
                               int *__restrict__ status, const BatchMxArgs &a) {
  const MoeDims &d = a.d;
  const int K = GATE_UP ? d.H : d.I, R = GATE_UP ? 2 * d.I : d.H, E = d.E;
  const int kblocks = K >> 5, nch = (kblocks + kBmKc - 1) / kBmKc, G = R >> 3, nseg = (G + kBmGroups - 1) / kBmGroups;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint8_t *ring = dyn_smem;
  BmUnit *units = reinterpret_cast<BmUnit *>(dyn_smem + kBmRingBytes);
  BmBars *bars = reinterpret_cast<BmBars *>(dyn_smem + kBmRingBytes + kBmMaxUnits * sizeof(BmUnit));
  const int *count = route + 1, *offset = route + 1 + E, *perm = route + 1 + E + (E + 1) + E;

  if (tid == 0) {
    for (int i = 0; i < kBmSlots; ++i) { mbar_init(&bars->full[i], 1); mbar_init(&bars->empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars->done[i], 1); mbar_init(&bars->uready[i], 4); }
    bars->abort = 0;
  }
  fence_barrier_init();
  if (warp == 0) tc_alloc(&bars->tmem_base, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  // columns: the tokens' scales of two units in flight [0, 192), the weights' scales per ring slot (16 columns each) [192, 256), two accumulators [256, 512)
  const uint32_t tSFA = tmem, tSFB = tmem + 192, tD = tmem + 256;
  // What the kernel before this one wrote (moe_expand_digits: the digits and the tokens' exponents) is not touched before
  // pdl_wait() below.  The routing tables are older: moe_expand_digits itself waited for their kernel before it let this
  // one start, so the units and the first weight copies do not wait (they overlap the digit expansion).
  pdl_launch_dependents();

  // ---- this CTA's units: all (expert, segment, pass) triples in that order, cut evenly over the grid
  if (tid == 0) {
    int total = 0;
    for (int e = a.lo; e < a.lo + a.n; ++e) total += ((count[e] + kBmTok - 1) / kBmTok) * nseg;
    const int u0 = int((long long)total * blockIdx.x / gridDim.x), u1 = int((long long)total * (blockIdx.x + 1) / gridDim.x);
    bars->u_base = u0;
    bars->n_units = u1 - u0;
    bars->max_nt = 0;
    if (u1 - u0 > kBmMaxUnits) { bars->n_units = 0; atomicCAS(status, 0, 71); }
  }
  __syncthreads();
  const int n_units = bars->n_units;
  for (int i = tid; i < n_units; i += kBmThreads) {
    int idx = bars->u_base + i, e = a.lo;
    for (; e < a.lo + a.n; ++e) {
      const int ue = ((count[e] + kBmTok - 1) / kBmTok) * nseg;
      if (idx < ue) break;
      idx -= ue;
    }
    const int passes = (count[min(e, a.lo + a.n - 1)] + kBmTok - 1) / kBmTok;
    const int seg = idx / max(passes, 1), pass = idx % max(passes, 1);
    BmUnit u;
    u.e = int16_t(e); u.pass = int16_t(pass); u.g0 = int16_t(seg * kBmGroups); u.ng = int16_t(min(kBmGroups, G - seg * kBmGroups));
    units[i] = u;
    atomicMax(&bars->max_nt, min(kBmTok, count[min(e, a.lo + a.n - 1)] - pass * kBmTok));
  }
  __syncthreads();
  const size_t mbytes = seg16_matrix_bytes(kblocks, G);
  // a ring slot holds TWO consecutive chunks ([digits 0][digits 1][piece 0][piece 1]): handing a slot from the producer to
  // the tensor core and back costs about as much as streaming half a chunk, so it is paid once per two
  const uint32_t a_bytes = uint32_t(max(bars->max_nt, 1)) * (kBmKc * 128), slot_bytes = 2u * (a_bytes + kBmBBytes);
  const uint32_t n_slots = min(4u, uint32_t(kBmRingBytes) / slot_bytes);       // 3 or 4: each owns 16 of the 64 scale columns
  const int npair = (nch + 1) >> 1;

  if (warp == 5) {
    // ---- producer
    if (lane == 0) {
      auto emit = [&](uint32_t q, bool weights, bool digits) {
        const BmUnit u = units[q / uint32_t(npair)];
        const int p = int(q % uint32_t(npair));
        const int off = offset[u.e] + u.pass * kBmTok, nt = min(kBmTok, count[u.e] - u.pass * kBmTok);
        const uint8_t *wexp = W + size_t(u.e - a.lo) * mbytes;
        const uint32_t s = q % n_slots;
        const int c0 = 2 * p, nck = c0 + 1 < nch ? 2 : 1;
        const int kc0 = min(kBmKc, kblocks - c0 * kBmKc), kc1 = nck == 2 ? min(kBmKc, kblocks - (c0 + 1) * kBmKc) : 0;
        const uint32_t bb0 = uint32_t(seg16_bytes(kc0, u.ng)), bb1 = nck == 2 ? uint32_t(seg16_bytes(kc1, u.ng)) : 0u;
        const uint32_t ab = uint32_t(nt * kBmKc * 128);
        uint8_t *dst = ring + size_t(s) * slot_bytes;
        if (weights) {
          mbar_expect_tx(&bars->full[s], bb0 + bb1 + uint32_t(nck) * ab);
          bulk_g2s(dst + 2 * a_bytes, wexp + seg16_offset(c0, u.g0 / kBmGroups, kc0, G), bb0, &bars->full[s]);
          if (nck == 2) bulk_g2s(dst + 2 * a_bytes + kBmBBytes, wexp + seg16_offset(c0 + 1, u.g0 / kBmGroups, kc1, G), bb1, &bars->full[s]);
        }
        if (digits) {
          bulk_g2s(dst, dig + (size_t(c0) * a.P + off) * (kBmKc * 128), ab, &bars->full[s]);
          if (nck == 2) bulk_g2s(dst + a_bytes, dig + (size_t(c0 + 1) * a.P + off) * (kBmKc * 128), ab, &bars->full[s]);
        }
      };
      const uint32_t total = uint32_t(n_units) * uint32_t(npair), head = min(n_slots, total);
      for (uint32_t q = 0; q < head; ++q) emit(q, true, false);       // the first ring fill's weights: before the digits exist
      pdl_wait();
      for (uint32_t q = 0; q < head; ++q) emit(q, false, true);
      // the steady state: plain nested loops (this one thread's instruction count is part of the kernel's pace)
      uint32_t q = head;
      int p = int(head % uint32_t(npair));
      for (int ui = int(head / uint32_t(npair)); ui < n_units; ++ui, p = 0) {
        const BmUnit u = units[ui];
        const int off = offset[u.e] + u.pass * kBmTok, nt = min(kBmTok, count[u.e] - u.pass * kBmTok);
        const uint8_t *wexp = W + size_t(u.e - a.lo) * mbytes;
        const uint32_t ab = uint32_t(nt * kBmKc * 128);
        for (; p < npair; ++p, ++q) {
          const uint32_t s = q % n_slots;
          if (!bm_wait(&bars->empty[s], ((q / n_slots) - 1) & 1, bars, status, 72)) { ui = n_units; break; }
          const int c0 = 2 * p, nck = c0 + 1 < nch ? 2 : 1;
          const int kc0 = min(kBmKc, kblocks - c0 * kBmKc), kc1 = nck == 2 ? min(kBmKc, kblocks - (c0 + 1) * kBmKc) : 0;
          const uint32_t bb0 = uint32_t(seg16_bytes(kc0, u.ng)), bb1 = nck == 2 ? uint32_t(seg16_bytes(kc1, u.ng)) : 0u;
          uint8_t *dst = ring + size_t(s) * slot_bytes;
          mbar_expect_tx(&bars->full[s], bb0 + bb1 + uint32_t(nck) * ab);
          bulk_g2s(dst + 2 * a_bytes, wexp + seg16_offset(c0, u.g0 / kBmGroups, kc0, G), bb0, &bars->full[s]);
          bulk_g2s(dst, dig + (size_t(c0) * a.P + off) * (kBmKc * 128), ab, &bars->full[s]);
          if (nck == 2) {
            bulk_g2s(dst + 2 * a_bytes + kBmBBytes, wexp + seg16_offset(c0 + 1, u.g0 / kBmGroups, kc1, G), bb1, &bars->full[s]);
            bulk_g2s(dst + a_bytes, dig + (size_t(c0 + 1) * a.P + off) * (kBmKc * 128), ab, &bars->full[s]);
          }
        }
      }
    }
  } else if (warp == 4) {
    // ---- issuer (whole warp, an elected lane issues)
    uint32_t q = 0;
    for (int ui = 0; ui < n_units; ++ui) {
      const BmUnit u = units[ui];
      const int N = u.ng * 8;
      if (!bm_wait(&bars->uready[ui & 1], (ui >> 1) & 1, bars, status, 74)) break;      // this unit's token scales are in place, its accumulator is free
      const uint32_t tDu = tD + uint32_t(ui & 1) * 128u, tSFAu = tSFA + uint32_t(ui & 1) * 96u;
      tc_fence_after_sync();
      const uint32_t id0 = mx_idesc(128, N, 0, 0), id2 = mx_idesc(128, N, 2, 2);
      bool ok = true;
      for (int p = 0; p < npair && ok; ++p, ++q) {
        const uint32_t s = q % n_slots;
        ok = bm_wait(&bars->full[s], (q / n_slots) & 1, bars, status, 75);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t base = smem_u32(ring + size_t(s) * slot_bytes);
        for (int kk = 0; kk < 2 && 2 * p + kk < nch; ++kk) {
          const int c = 2 * p + kk, kcc = min(kBmKc, kblocks - c * kBmKc);
          const uint32_t sa = base + uint32_t(kk) * a_bytes, sb = base + 2 * a_bytes + uint32_t(kk) * kBmBBytes;
          const uint32_t ssf = sb + uint32_t(u.ng * kcc * 128);
          for (int pp = 0; 4 * pp < kcc; ++pp) {
            // A in the slot: [token][K block of the chunk][8 digit rows x 16 B]: K blocks 128 B apart, tokens 1 KB apart
            // B in the slot: [group][K block][8 rows x 16 B]: K blocks 128 B apart, groups kcc x 128 B apart
            const uint64_t da = tc_smem_desc(sa + uint32_t(4 * pp) * 128, 128, kBmKc * 128);
            const uint64_t db = tc_smem_desc(sb + uint32_t(4 * pp) * 128, 128, uint32_t(kcc * 128));
            bm_mma_pair_warp(tDu, da, db, id0, id2, tSFAu + 4 * uint32_t(c * (kBmKc >> 2) + pp),
                             tSFB + s * 16 + uint32_t(kk) * 8 + uint32_t(pp) * 4, !(c == 0 && pp == 0), 4 * pp + 2 < kcc, 256u >> 4,
                             256u >> 4, tc_smem_desc(ssf + uint32_t(pp) * 512, 16, 128));
          }
        }
        tc_commit_warp(&bars->empty[s], true);
        tc_commit_warp(&bars->done[ui & 1], p == npair - 1);
        __syncwarp();
      }
      if (!ok) break;
    }
  } else if (warp < 4) {
    // ---- the tokens' scales (every warp writes its own lane quarter's copy, one unit ahead of the issuer) and the epilogue
    auto stage_scales = [&](int ui) {
      const BmUnit u = units[ui];
      const int off = offset[u.e] + u.pass * kBmTok, nt = min(kBmTok, count[u.e] - u.pass * kBmTok);
      // row 32 q + lane of A = digit row (lane & 7) of token 4 q + (lane >> 3); scale byte = exponent - 21 + 3 (7 - digit row)
      const uint32_t adj = 0x01010101u * uint32_t(3 * (7 - (lane & 7)));
      const uint32_t base = tSFA + uint32_t(ui & 1) * 96u + (uint32_t(warp * 32) << 16);
      // the tokens' exponent rows are one contiguous piece: all loads in flight at once, then shared memory
      uint32_t *es = bars->em_s[ui & 1];
      const uint32_t *src = reinterpret_cast<const uint32_t *>(em + size_t(off) * kBmEmStride);
      for (int i = tid; i < nt * (kBmEmStride / 4); i += 128) es[i] = __ldcg(src + i);
      asm volatile("bar.sync 2, 128;" ::: "memory");
      for (int gg = 0; gg < (kblocks + 3) / 4; ++gg) {
        uint32_t w[4];
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
          const int t = 4 * qd + (lane >> 3);
          w[qd] = t < nt ? es[t * (kBmEmStride / 4) + gg] + adj - 0x15151515u : 0x7f7f7f7fu;
        }
        tc_st_cols4(base + 4 * gg, w[0], w[1], w[2], w[3]);
      }
      tc_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->uready[ui & 1]);
    };
    pdl_wait();                                  // the tokens' exponents come from the kernel before
    if (n_units > 0) stage_scales(0);
    for (int ui = 0; ui < n_units; ++ui) {
      const BmUnit u = units[ui];
      const int N = u.ng * 8;
      const int off = offset[u.e] + u.pass * kBmTok, nt = min(kBmTok, count[u.e] - u.pass * kBmTok);
      // the next unit's scales go into the other buffer (its instructions, two units back, are complete: their
      // accumulator was read in the last iteration), so the issuer never waits for this warp
      if (ui + 1 < n_units) stage_scales(ui + 1);
      const uint32_t tDu = tD + uint32_t(ui & 1) * 128u;
      const int tt = 4 * warp + (lane >> 3);
      const int asg = tt < nt ? perm[off + tt] : 0;
      // this lane's biases travel while the weights stream
      float4 bpre[kBmGroups * 8 / 32];
#pragma unroll
      for (int i = 0; i < kBmGroups * 8 / 32; ++i) {
        const int col = 32 * i + 4 * (lane & 7);
        bpre[i] = (tt < nt && col < N) ? __ldg(reinterpret_cast<const float4 *>(bias + size_t(u.e) * R + u.g0 * 8 + col))
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      if (!bm_wait(&bars->done[ui & 1], (ui >> 1) & 1, bars, status, 76)) break;
      tc_fence_after_sync();
#pragma unroll
      for (int ci = 0; ci < kBmGroups * 8 / 32; ++ci) {
        const int c0 = 32 * ci;
        if (c0 >= N) break;
        float v[32];
        {
          float lo16[16], hi16[16];
          tc_ld16(tDu + (uint32_t(warp * 32) << 16) + uint32_t(c0), lo16);
          tc_ld16(tDu + (uint32_t(warp * 32) << 16) + uint32_t(c0 + 16), hi16);
#pragma unroll
          for (int i = 0; i < 16; ++i) { v[i] = lo16[i]; v[16 + i] = hi16[i]; }
        }
        float r16[16], r8[8], r4[4];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float mine = (lane & 4) ? v[16 + i] : v[i], other = (lane & 4) ? v[i] : v[16 + i];
          r16[i] = mine + __shfl_xor_sync(0xffffffffu, other, 4);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float mine = (lane & 2) ? r16[8 + i] : r16[i], other = (lane & 2) ? r16[i] : r16[8 + i];
          r8[i] = mine + __shfl_xor_sync(0xffffffffu, other, 2);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float mine = (lane & 1) ? r8[4 + i] : r8[i], other = (lane & 1) ? r8[i] : r8[4 + i];
          r4[i] = mine + __shfl_xor_sync(0xffffffffu, other, 1);
        }
        const int col = c0 + 4 * (lane & 7);
        if (tt < nt && col < N) {
          const int row = u.g0 * 8 + col;
          const float4 b = bpre[ci];
          if (GATE_UP) {
            *reinterpret_cast<float2 *>(out + size_t(asg) * (R >> 1) + (row >> 1)) =
                make_float2(swiglu_clamped(r4[0] + b.x, r4[1] + b.y, d.alpha, d.limit),
                            swiglu_clamped(r4[2] + b.z, r4[3] + b.w, d.alpha, d.limit));
          } else {
            *reinterpret_cast<float4 *>(out + size_t(asg) * R + row) = make_float4(r4[0] + b.x, r4[1] + b.y, r4[2] + b.z, r4[3] + b.w);
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tc_dealloc(tmem, 512);
  }
}

// grid = one CTA per SM (any number works), kBmThreads threads, dynamic shared memory bm_smem_bytes().
extern "C" __global__ void __launch_bounds__(kBmThreads, 1)
moe_batch_mx_gate_up(const uint8_t *__restrict__ W, const float *__restrict__ bias, const uint8_t *__restrict__ dig,
                     const uint8_t *__restrict__ em, const int *__restrict__ route, float *__restrict__ act,
                     int *__restrict__ status, BatchMxArgs a) {
  batch_mx_body<true>(W, bias, dig, em, route, act, status, a);
}

extern "C" __global__ void __launch_bounds__(kBmThreads, 1)
moe_batch_mx_down(const uint8_t *__restrict__ W, const float *__restrict__ bias, const uint8_t *__restrict__ dig,
                  const uint8_t *__restrict__ em, const int *__restrict__ route, float *__restrict__ o,
                  int *__restrict__ status, BatchMxArgs a) {
  batch_mx_body<false>(W, bias, dig, em, route, o, status, a);
}
