// NCCL entry points resolved at run time (libnccl.so.2), so that the library loads on hosts without NCCL
// and single-GPU users never touch it.  Only what the expert-parallel decode step needs: communicator set-up
// from a unique id, all-gather, grouped send/recv (all-to-all).  The reference has no collective of any kind.
#pragma once
#include <dlfcn.h>
#include <stddef.h>

typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;                 // 0 = ncclSuccess
enum { kNcclUint8 = 1, kNcclFloat32 = 7 };

struct NcclLib {
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllGather)(const void *, void *, size_t, int, ncclComm_t, void *) = nullptr;
  ncclResult_t (*Send)(const void *, size_t, int, int, ncclComm_t, void *) = nullptr;
  ncclResult_t (*Recv)(void *, size_t, int, int, ncclComm_t, void *) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
  void *handle = nullptr;
  bool ok = false;

  bool load() {
    if (ok) return true;
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
      handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (handle) break;
    }
    if (!handle) return false;
    bool all = true;
#define X(field, sym)                                                         \
    field = reinterpret_cast<decltype(field)>(dlsym(handle, sym));            \
    if (!field) all = false;
    X(GetUniqueId, "ncclGetUniqueId") X(CommInitRank, "ncclCommInitRank") X(CommDestroy, "ncclCommDestroy")
    X(AllGather, "ncclAllGather") X(Send, "ncclSend") X(Recv, "ncclRecv") X(GroupStart, "ncclGroupStart")
    X(GroupEnd, "ncclGroupEnd") X(GetErrorString, "ncclGetErrorString")
#undef X
    ok = all;
    return ok;
  }
};
