// Driver-API entry points resolved at run time.
//
// The reference reaches libcuda through cudarc, which dlopens it
// (base/Cargo.toml:10, cudarc features "driver"); doing the same here keeps
// the shared library loadable on hosts without a GPU driver, where only the
// symbol table is inspected.
#pragma once
#include <cuda.h>
#include <dlfcn.h>

#define B200_DRIVER_FNS(X)                                                      \
  X(cuInit) X(cuDeviceGet) X(cuDeviceGetCount) X(cuDeviceGetAttribute)          \
  X(cuDevicePrimaryCtxRetain) X(cuDevicePrimaryCtxRelease) X(cuCtxSetCurrent)   \
  X(cuCtxGetCurrent) X(cuCtxSynchronize) X(cuMemAlloc) X(cuMemFree)             \
  X(cuMemsetD8Async) X(cuMemcpyHtoD) X(cuMemcpyDtoH) X(cuMemcpyHtoDAsync)       \
  X(cuMemcpyDtoHAsync) X(cuMemcpyDtoDAsync) X(cuMemGetInfo) X(cuStreamCreate)   \
  X(cuStreamSynchronize) X(cuStreamDestroy) X(cuStreamWaitEvent)                \
  X(cuEventCreate) X(cuEventRecord) X(cuEventElapsedTime) X(cuEventDestroy)     \
  X(cuEventQuery) X(cuEventSynchronize) X(cuStreamBeginCapture) X(cuStreamEndCapture)                 \
  X(cuGraphInstantiateWithFlags) X(cuGraphUpload) X(cuGraphLaunch)              \
  X(cuGraphExecDestroy) X(cuGraphDestroy) X(cuMemAllocHost) X(cuMemFreeHost)    \
  X(cuModuleLoadData) X(cuModuleGetFunction) X(cuModuleUnload)                  \
  X(cuLaunchKernel) X(cuLaunchKernelEx) X(cuFuncSetAttribute)                   \
  X(cuGetErrorString) X(cuMemHostRegister) X(cuMemHostUnregister)          \
  X(cuIpcGetMemHandle) X(cuIpcOpenMemHandle) X(cuIpcCloseMemHandle)

// cuda.h maps the unversioned names to their current _vN symbols with
// macros; stringify AFTER that expansion so dlsym asks for the right one.
#define B200_STR2(x) #x
#define B200_STR(x) B200_STR2(x)

struct CudaDriver {
#define X(name) decltype(&name) p_##name = nullptr;
  B200_DRIVER_FNS(X)
#undef X
  void *handle = nullptr;
  bool ok = false;

  bool load() {
    if (ok) return true;
    const char *names[] = {"libcuda.so.1", "libcuda.so"};
    for (const char *n : names) {
      handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (handle) break;
    }
    if (!handle) return false;
    bool all = true;
#define X(name)                                                          \
    p_##name = reinterpret_cast<decltype(&name)>(dlsym(handle, B200_STR(name))); \
    if (!p_##name) all = false;
    B200_DRIVER_FNS(X)
#undef X
    ok = all;
    return ok;
  }
};
