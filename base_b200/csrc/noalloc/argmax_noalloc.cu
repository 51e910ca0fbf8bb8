// Greedy argmax that allocates nothing.
//
// Who needs this: callers that hold device pointers but must not allocate —
// code running inside a pre-sized memory pool or an arena handed out by
// another runtime, a latency-critical serving loop where cudaMalloc would
// stall every stream of the device, or a host program that has already given
// all device memory away.  The regular path (cl_b200_launch of
// `argmax_first`) needs three small scratch buffers that the caller creates
// with cl_cuda_create_buffer; here that scratch is a fixed array inside the
// library image instead.
//
// The scratch lives in device memory for as long as the library is loaded on
// a device (about 66 KB per GPU).  It is shared by every call and keeps the
// previous call's contents, so the part that must start at zero (the arrival
// tickets) is cleared on the caller's stream at the start of each call, and
// two calls that overlap on the GPU (different streams, no ordering) race.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>

#include "../kernels/dense_decode.cuh"

namespace {

constexpr int kNoAllocParts = 128;      // slices per token, as the regular path uses
constexpr int kNoAllocMaxTokens = 64;   // largest B this entry point accepts
constexpr int kNoAllocMaxDevices = 64;
constexpr size_t kPartVBytes = sizeof(float) * kNoAllocParts * kNoAllocMaxTokens;
constexpr size_t kPartIBytes = sizeof(int) * kNoAllocParts * kNoAllocMaxTokens;
constexpr size_t kTicketBytes = sizeof(int) * kNoAllocMaxTokens;

// [part values][part indices][tickets]
static __device__ __align__(256) unsigned char g_argmax_scratch[kPartVBytes + kPartIBytes + kTicketBytes];

// Device address of the scratch, per device ordinal.  In host code the name
// g_argmax_scratch is only a handle for the runtime, never a device address.
// The address belongs to the device's primary context; if the host program
// resets the device it goes stale, which shows as an error of the first
// operation on it: the entry point then looks it up again, once.
std::atomic<unsigned char *> g_scratch_ptr[kNoAllocMaxDevices];

unsigned char *resolve_scratch(int dev, cudaError_t *e) {
  unsigned char *p = nullptr;
  *e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_argmax_scratch);
  if (*e != cudaSuccess || !p) return nullptr;
  g_scratch_ptr[dev].store(p, std::memory_order_release);
  return p;
}

thread_local char t_noalloc_err[256] = "";

int fail(const char *what, cudaError_t e) {
  snprintf(t_noalloc_err, sizeof(t_noalloc_err), "%s: %s", what, e == cudaSuccess ? "invalid argument" : cudaGetErrorString(e));
  return -1;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) const char *cl_b200_argmax_noalloc_error(void) {
  return t_noalloc_err;
}

// out_dev[b] = smallest index of the maximum of logits_dev[b * stride .. + vocab), b < tokens.
// All pointers are device pointers on the current device; `stream` is a
// cudaStream_t / CUstream (null = the legacy default stream).  Everything
// runs on that stream: to order the call after logits this library produced,
// pass the producing stream's handle (cl_b200_stream_handle), because the
// library's streams do not synchronise with the default stream.
// The first call on a device looks up the scratch address (one
// cudaGetSymbolAddress); make that first call outside any stream capture.
extern "C" __attribute__((visibility("default"))) int32_t
cl_b200_argmax_noalloc(const float *logits_dev, int32_t vocab, int32_t tokens, int32_t stride, int32_t *out_dev,
                       void *stream) {
  t_noalloc_err[0] = 0;
  if (!logits_dev || !out_dev || vocab <= 0 || tokens <= 0 || stride < vocab) return fail("argmax_noalloc", cudaSuccess);
  if (tokens > kNoAllocMaxTokens) {
    snprintf(t_noalloc_err, sizeof(t_noalloc_err), "argmax_noalloc: %d tokens exceed the built-in scratch (max %d)",
             tokens, kNoAllocMaxTokens);
    return -1;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail("cudaGetDevice", e);
  if (dev < 0 || dev >= kNoAllocMaxDevices) return fail("device ordinal out of range", cudaSuccess);
  unsigned char *base = g_scratch_ptr[dev].load(std::memory_order_acquire);
  if (!base && !(base = resolve_scratch(dev, &e))) return fail("cudaGetSymbolAddress", e);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  e = cudaMemsetAsync(base + kPartVBytes + kPartIBytes, 0, kTicketBytes, st);
  if (e != cudaSuccess) {
    // a remembered address from before a device reset: look it up again, once
    (void)cudaGetLastError();
    cudaError_t e2;
    if (!(base = resolve_scratch(dev, &e2))) return fail("cudaGetSymbolAddress", e2);
    e = cudaMemsetAsync(base + kPartVBytes + kPartIBytes, 0, kTicketBytes, st);
    if (e != cudaSuccess) return fail("cudaMemsetAsync", e);
  }
  float *part_v = reinterpret_cast<float *>(base);
  int *part_i = reinterpret_cast<int *>(base + kPartVBytes);
  int *tickets = reinterpret_cast<int *>(base + kPartVBytes + kPartIBytes);
  ArgmaxArgs a{vocab, tokens, stride, kNoAllocParts};
  argmax_first<<<dim3(kNoAllocParts, tokens, 1), 256, 0, st>>>(logits_dev, out_dev, nullptr, nullptr, part_v, part_i,
                                                               tickets, a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail("argmax_first launch", e);
  return 0;
}
