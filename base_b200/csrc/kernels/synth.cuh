// Seeded synthetic tensors, generated on the device.
//
// The reference ships no quantised checkpoints and none can be downloaded in
// the build environment, so the model-sized workloads run on random-init
// weights with the shapes and value distributions the benchmark configs name.
// Every element is a pure function of (seed, tensor id, element index) built
// from 32-bit integer arithmetic only, so the CPU oracle regenerates the very
// same bytes (oracle/synth.py, oracle/model_oracle.c) without any transfer:
//   h(i)     = fmix32(i * 0x9E3779B1 + tensor * 0x85EBCA77 + seed * 0xC2B2AE3D)
//   byte i   = (h(i >> 2) >> 8 (i & 3)) & 255              uniform codes, two per byte
//   scale i  = lo + h(i) % span                            UE8M0 exponent bytes
//   normal i = (sum of the 8 bytes of h(2i), h(2i+1) - 1020) * c,  c = sigma / 209.0232
//              (Irwin-Hall approximation of N(0, sigma); exact in f32: an
//              integer times one constant)
#pragma once
#include "dense_decode.cuh"

B200_DEVICE uint32_t synth_hash(uint32_t i, uint32_t tensor, uint32_t seed) {
  uint32_t h = i * 0x9E3779B1u + tensor * 0x85EBCA77u + seed * 0xC2B2AE3Du;
  h ^= h >> 16; h *= 0x85EBCA6Bu; h ^= h >> 13; h *= 0xC2B2AE35u; h ^= h >> 16;
  return h;
}

B200_DEVICE float synth_normal(uint32_t i, uint32_t tensor, uint32_t seed, float c) {
  const uint32_t a = synth_hash(2 * i, tensor, seed), b = synth_hash(2 * i + 1, tensor, seed);
  const int s = int((a & 255) + ((a >> 8) & 255) + ((a >> 16) & 255) + (a >> 24) + (b & 255) + ((b >> 8) & 255) +
                    ((b >> 16) & 255) + (b >> 24)) - 1020;
  return __fmul_rn(float(s), c);
}

struct SynthArgs {
  unsigned long long n;   // elements
  uint32_t tensor, seed;
  int kind;               // 0 bytes, 1 scales, 2 normal f32, 3 normal bf16, 4 f32 1 + normal
  float c;                // sigma / 209.0232 for the normal kinds
  int lo, span;           // scales
  unsigned long long first;   // index of element 0 of dst within the tensor (a slice of a larger tensor)
};

extern "C" __global__ void __launch_bounds__(256)
synth_fill(void *__restrict__ dst, SynthArgs a) {
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += stride) {
    const uint32_t i32 = uint32_t(a.first + i);
    switch (a.kind) {
      case 0: {
        const uint32_t h = synth_hash(i32 >> 2, a.tensor, a.seed);
        reinterpret_cast<uint8_t *>(dst)[i] = uint8_t(h >> (8 * (i32 & 3)));
        break;
      }
      case 1:
        reinterpret_cast<uint8_t *>(dst)[i] = uint8_t(a.lo + synth_hash(i32, a.tensor, a.seed) % uint32_t(a.span));
        break;
      case 2:
        reinterpret_cast<float *>(dst)[i] = synth_normal(i32, a.tensor, a.seed, a.c);
        break;
      case 3:
        reinterpret_cast<uint16_t *>(dst)[i] = f32_to_bf16_rne(synth_normal(i32, a.tensor, a.seed, a.c));
        break;
      default:
        reinterpret_cast<float *>(dst)[i] = __fadd_rn(1.0f, synth_normal(i32, a.tensor, a.seed, a.c));
        break;
    }
  }
}
