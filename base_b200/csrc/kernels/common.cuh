// Shared device helpers for the sm_100a kernels.
#pragma once
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define B200_DEVICE __device__ __forceinline__

// ---- MXFP4 ------------------------------------------------------------------
// Element format (reference: lean/lib/AlgorithmLib/ML/QuantMX.lean:56-74):
// 4-bit code, sign in bit 3, magnitude index in bits 2..0 into
// {0, .5, 1, 1.5, 2, 3, 4, 6}.  Block format (QuantMX.lean:131-147): 32
// codes share one power-of-two scale.  The reference leaves the byte layout
// open; this library fixes: low nibble = even element, high nibble = odd
// element, scale byte s = 2^(s-127) (s = 0 -> 2^-127, s = 255 -> NaN).

B200_DEVICE float ue8m0_to_f32(uint32_t s) {
  uint32_t bits = s << 23;
  if (s == 0) bits = 0x00400000u;        // 2^-127, an f32 subnormal
  if (s == 255) bits = 0x7fc00000u;      // NaN
  return __uint_as_float(bits);
}

// One byte (two codes) -> two f16 values, element 2i in .x, 2i+1 in .y.
// cvt.rn.f16x2.e2m1x2 is exact: every E2M1 value is an f16 value.
B200_DEVICE void e2m1x8_to_f16x2(uint32_t w, __half2 (&h)[4]) {
  uint32_t r0, r1, r2, r3;
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "mov.b32 {b0, b1, b2, b3}, %4;\n"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
      "}\n"
      : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
      : "r"(w));
  h[0] = *reinterpret_cast<__half2 *>(&r0);
  h[1] = *reinterpret_cast<__half2 *>(&r1);
  h[2] = *reinterpret_cast<__half2 *>(&r2);
  h[3] = *reinterpret_cast<__half2 *>(&r3);
}

// Eight codes (one 32-bit word, element 0 in the lowest nibble) -> f32.
B200_DEVICE void e2m1x8_to_f32(uint32_t w, float (&v)[8]) {
  __half2 h[4];
  e2m1x8_to_f16x2(w, h);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __half22float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

// ---- warp helpers -------------------------------------------------------------

B200_DEVICE float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

B200_DEVICE float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum each of 16 per-lane values over the 32 lanes of a warp with 16
// shuffles (instead of 80).  On return v[0] of lane l holds the total of
// value index row_of_lane16(l); the summation tree is fixed, so the result
// does not depend on scheduling.
B200_DEVICE int row_of_lane16(int lane) {
  return ((lane >> 4) & 1) * 8 + ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2 + ((lane >> 1) & 1);
}

B200_DEVICE void warp_reduce16(float (&v)[16], int lane) {
#pragma unroll
  for (int half = 8, off = 16; half >= 1; half >>= 1, off >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      float a = v[i], b = v[i + half];
      float send = upper ? a : b;
      float keep = upper ? b : a;
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
  v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
}

// Same for 8 values (8 shuffles).  v[0] of lane l: value index
// ((l>>4)&1)*4 + ((l>>3)&1)*2 + ((l>>2)&1), summed over all 32 lanes.
B200_DEVICE int row_of_lane8(int lane) {
  return ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
}

B200_DEVICE void warp_reduce8(float (&v)[8], int lane) {
#pragma unroll
  for (int half = 4, off = 16; half >= 1; half >>= 1, off >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      float a = v[i], b = v[i + half];
      float send = upper ? a : b;
      float keep = upper ? b : a;
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
  v[0] += __shfl_xor_sync(0xffffffffu, v[0], 2);
  v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
}

// ---- activation ---------------------------------------------------------------
// Clamped SwiGLU of the gpt-oss experts: gate is clamped from above, the
// linear branch on both sides, the sigmoid runs on alpha * gate, and the
// linear branch is offset by one before the product.
B200_DEVICE float swiglu_clamped(float gate, float up, float alpha, float limit) {
  gate = fminf(gate, limit);
  up = fminf(fmaxf(up, -limit), limit);
  float glu = gate / (1.0f + __expf(-alpha * gate));
  return (up + 1.0f) * glu;
}

B200_DEVICE float silu(float g) { return g / (1.0f + __expf(-g)); }

// ---- programmatic dependent launch --------------------------------------------
B200_DEVICE void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
B200_DEVICE void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
