// 5th-generation tensor-core (tcgen05) building blocks for sm_100a:
// D[128 x N] (f32, in tensor memory) = A[128 x K] (bf16, K-major in shared
// memory) x B[N x K]^T (bf16, K-major).  A one-CTA GEMM that exercises them
// lives with the tests (tests/kernels/probe_kernels.cu).
//
// What is used:
//   * tensor memory (TMEM): allocated by one warp (tcgen05.alloc), accumulator
//     row i lives in TMEM lane i, column j in 32-bit column j;
//   * tcgen05.mma.cta_group::1.kind::f16 issued by ONE thread, operands named
//     by 64-bit shared-memory matrix descriptors, shape and types by a 32-bit
//     instruction descriptor;
//   * tcgen05.commit -> mbarrier for completion, tcgen05.ld (32 lanes x 32
//     bit) to read the accumulator back: warp w of the CTA reads lanes
//     32 (w % 4) .. 32 (w % 4) + 31.
// Shared-memory operand layout (no swizzle, K-major): "core matrices" of 8 rows
// x 16 bytes stored as 128 contiguous bytes.  A tile of R rows x 64 columns
// (bf16) is stored as [8 column groups of 16 B][R rows][16 B]: the next 8-row
// group is 128 B further (stride byte offset), the next column group R * 16 B
// further (leading byte offset).  One MMA consumes K = 16, i.e. two column groups.
//
// Every wait is bounded; on timeout the kernel stores a code in *status, frees
// its tensor memory and returns.
#pragma once
#include "moe_stream.cuh"

constexpr uint32_t kTcSpin = 1u << 22;

// ---- descriptors ---------------------------------------------------------------------------
// Shared-memory matrix descriptor: start address, leading and stride byte offsets in units of
// 16 bytes, descriptor version 1 (sm_100), no swizzle.
B200_DEVICE uint64_t tc_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr >> 4) & 0x3fffu);
  d |= uint64_t((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= uint64_t(1) << 46;
  return d;
}

// Instruction descriptor of kind::f16 with bf16 inputs, f32 accumulator, both operands K-major.
B200_DEVICE uint32_t tc_idesc_bf16(int M, int N) {
  return (1u << 4)            // D format: f32
         | (1u << 7)          // A format: bf16
         | (1u << 10)         // B format: bf16
         | (uint32_t(N >> 3) << 17) | (uint32_t(M >> 4) << 24);
}

// ---- instructions ----------------------------------------------------------------------------
B200_DEVICE void tc_alloc(uint32_t *smem_result, uint32_t ncols) {       // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
B200_DEVICE void tc_dealloc(uint32_t taddr, uint32_t ncols) {             // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
B200_DEVICE void tc_mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, bool accumulate) {  // one thread
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
               "l"(adesc), "l"(bdesc), "r"(idesc), "r"(uint32_t(accumulate))
               : "memory");
}
B200_DEVICE void tc_commit(uint64_t *bar) {                               // one thread
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
B200_DEVICE void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
B200_DEVICE void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
B200_DEVICE void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 16 consecutive 32-bit columns of this thread's TMEM lane (whole warp; taddr = lane base << 16 | column).
B200_DEVICE void tc_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                 "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Bounded mbarrier wait for the tensor-core kernels.
B200_DEVICE bool tc_wait(uint64_t *bar, uint32_t parity) {
  for (uint32_t i = 0; i < kTcSpin; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

// ---- operand staging ---------------------------------------------------------------------------
// Byte offset of element (row r, column c) of an R-row x 64-column bf16 tile in the layout above.
B200_DEVICE uint32_t tc_tile_off(int R, int r, int c) { return uint32_t(c >> 3) * uint32_t(R) * 16 + uint32_t(r) * 16 + uint32_t(c & 7) * 2; }
