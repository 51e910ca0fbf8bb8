// MXFP4 weights on the block-scaled 5th-generation tensor cores
// (tcgen05.mma.kind::mxf4.block_scale): the E2M1 codes and UE8M0 scales are
// consumed as they are stored, no dequantisation instructions at all.
//
// D[128 x N] (f32, tensor memory) += A[128 x 64] * B[N x 64]^T per instruction,
// both operands E2M1 with one UE8M0 scale per 32 elements of K.
//   * B = N rows of the weight matrix (codes in shared memory, K-major core
//     matrices of 8 rows x 16 bytes = 8 x 32 codes);
//   * A = the activation vector, expanded into T "terms": row t holds the E2M1
//     rounding (with its own block scales) of what rows 0..t-1 left over, so
//     that x = sum_t term_t to about 4^-T of each block's largest element.
//     Only rows 0..T-1 of A carry data; the tensor core reads 128 rows, the
//     other rows alias the same shared memory and their results are ignored.
//   * y[n] = sum_t D[t][n].
// Scale factors live in tensor memory: for rows 32 g + l of an operand, lane l,
// column c + g holds the four scale bytes of four consecutive K blocks; a
// tcgen05.cp of 32 lanes x 16 bytes fills such a group of four columns
// (replicated to lanes l+32, l+64, l+96).  One instruction (K = 64) uses two of
// the four bytes: c (a multiple of 4) is the scale address, the byte pair
// (0 or 2) goes into the instruction descriptor.
//
// Every wait is bounded; on timeout the kernel stores a code in *status, frees
// its tensor memory and returns.
#pragma once
#include "tc_gemm.cuh"


// Instruction descriptor of kind::mxf4: E2M1 x E2M1, UE8M0 scales, K-major operands, f32 accumulator.
B200_DEVICE uint32_t mx_idesc(int M, int N, uint32_t a_sf_byte, uint32_t b_sf_byte) {
  return (b_sf_byte << 4)              // which byte pair of the 32-bit scale column B uses
         | (1u << 7)                   // A format: E2M1
         | (1u << 10)                  // B format: E2M1
         | (uint32_t(N >> 3) << 17)
         | (1u << 23)                  // scale format: UE8M0
         | (uint32_t(M >> 4) << 24)
         | (a_sf_byte << 29);
}

B200_DEVICE void mx_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                        bool accumulate) {                                 // one thread
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(uint32_t(accumulate)), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

// Two instructions over four consecutive K blocks that share one group of scale columns (bytes 0,1 then 2,3):
// the second one's operands are 2 K blocks = 256 bytes further (descriptor address field +16).  One asm block, so
// that the single issuing thread spends as few instructions as possible per tensor-core instruction.
B200_DEVICE void mx_mma_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc01, uint32_t idesc23, uint32_t sfa_tmem,
                             uint32_t sfb_tmem, bool accumulate_first) {                    // one thread
  asm volatile(
      "{\n.reg .pred p, q;\n.reg .b64 a2, b2;\n"
      "setp.ne.b32 p, %5, 0;\nsetp.eq.b32 q, %5, %5;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%6], [%7], p;\n"
      "add.u64 a2, %1, 16;\nadd.u64 b2, %2, 16;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], a2, b2, %4, [%6], [%7], q;\n}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc01), "r"(idesc23), "r"(uint32_t(accumulate_first)), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

// The same pair, executed by a whole converged warp: one elected lane issues, every lane carries the (warp-uniform)
// operands, so that the compiler can keep them in uniform registers and no branch diverges the warp.
B200_DEVICE void mx_mma_pair_warp(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc01, uint32_t idesc23,
                                  uint32_t sfa_tmem, uint32_t sfb_tmem, bool accumulate_first, bool second) {      // whole warp
  asm volatile(
      "{\n.reg .pred p, q, e, e2;\n.reg .b64 a2, b2;\n"
      "elect.sync _|e, 0xffffffff;\n"
      "setp.ne.b32 p, %5, 0;\nsetp.eq.b32 q, %5, %5;\nsetp.ne.b32 e2, %8, 0;\nand.pred e2, e2, e;\n"
      "@e tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%6], [%7], p;\n"
      "add.u64 a2, %1, 16;\nadd.u64 b2, %2, 16;\n"
      "@e2 tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], a2, b2, %4, [%6], [%7], q;\n}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc01), "r"(idesc23), "r"(uint32_t(accumulate_first)), "r"(sfa_tmem), "r"(sfb_tmem),
      "r"(uint32_t(second))
      : "memory");
}
// tcgen05.commit / mbarrier.arrive by the elected lane of a converged warp.
B200_DEVICE void tc_commit_warp(uint64_t *bar, bool on) {
  asm volatile("{\n.reg .pred e, o;\nelect.sync _|e, 0xffffffff;\nsetp.ne.b32 o, %1, 0;\nand.pred e, e, o;\n"
               "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}\n" ::"r"(smem_u32(bar)),
               "r"(uint32_t(on))
               : "memory");
}
B200_DEVICE void mbar_arrive_n_warp(uint64_t *bar, uint32_t n) {
  asm volatile("{\n.reg .pred e;\nelect.sync _|e, 0xffffffff;\n@e mbarrier.arrive.shared::cta.b64 _, [%0], %1;\n}\n" ::"r"(smem_u32(bar)),
               "r"(n)
               : "memory");
}

// Shared memory (32 rows x 16 bytes, rows 16 bytes apart) -> four 32-bit columns of tensor-memory lanes 0..31,
// replicated to the other three lane quarters.
B200_DEVICE void tc_cp_32x128b(uint32_t taddr, uint32_t smem_addr) {       // one thread
  const uint64_t sdesc = tc_smem_desc(smem_addr, 16, 128);
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// Two f32 -> one byte of two E2M1 codes (round to nearest even, saturating): `lo` in the low nibble.
B200_DEVICE uint32_t f32x2_to_e2m1x2(float lo, float hi) {
  uint32_t r;
  asm("{\n.reg .b8 b;\ncvt.rn.satfinite.e2m1x2.f32 b, %1, %2;\ncvt.u32.u8 %0, b;\n}\n" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
