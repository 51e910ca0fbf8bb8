// Native stage programs: what replaces the JIT'd CLIF functions of the
// reference (base/src/jit.rs:134-231).  A plugin is a table of
// `void(uint8_t *mem)` functions; stage code talks to the device only through
// the cl_cuda_* / cl_b200_* ABI, as generated code does in the reference.
#pragma once
#include <cstdint>
#include <cstring>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "b200abi.h"

namespace b200 {

using StageFn = void (*)(uint8_t *mem);

struct StageEntry {
  const char *name;   // "" for the no-op stub at index 0
  StageFn fn;
};

struct Plugin {
  const char *name;
  std::vector<StageEntry> stages;
  StageFn destroy;    // called by b200_base_free; may be null
};

void register_plugin(const Plugin &p);
const Plugin *find_plugin(const std::string &name);
const std::vector<Plugin> &all_plugins();

// Fixed memory map of native plugins (offsets as the reference's generated
// programs use: lean/lib/AlgorithmLib/Core.lean:23-28, 53-62).
constexpr uint64_t kOffCudaCtx = 0x10;
constexpr uint64_t kOffDataPtr = 0x18;
constexpr uint64_t kOffDataLen = 0x20;
constexpr uint64_t kOffOutPtr = 0x28;
constexpr uint64_t kOffOutLen = 0x30;
constexpr uint64_t kOffStatus = 0x40;   // i64, 0 = ok
constexpr uint64_t kOffState = 0x48;    // plugin-private heap pointer
constexpr uint64_t kMinNativeMemory = 0x100;

template <typename T>
inline T rd(const uint8_t *mem, uint64_t off) {
  T v;
  memcpy(&v, mem + off, sizeof(T));
  return v;
}
template <typename T>
inline void wr(uint8_t *mem, uint64_t off, T v) {
  memcpy(mem + off, &v, sizeof(T));
}

struct StageIO {
  uint8_t *mem;
  const uint8_t *data;
  uint64_t data_len;
  uint8_t *out;
  uint64_t out_len;
  explicit StageIO(uint8_t *m)
      : mem(m),
        data(reinterpret_cast<const uint8_t *>(rd<uint64_t>(m, kOffDataPtr))),
        data_len(rd<uint64_t>(m, kOffDataLen)),
        out(reinterpret_cast<uint8_t *>(rd<uint64_t>(m, kOffOutPtr))),
        out_len(rd<uint64_t>(m, kOffOutLen)) {}
  B200CudaContext *ctx() const { return reinterpret_cast<B200CudaContext *>(rd<uint64_t>(mem, kOffCudaCtx)); }
  B200CudaContext **ctx_slot() const { return reinterpret_cast<B200CudaContext **>(mem + kOffCudaCtx); }
  template <typename S>
  S *state() const { return reinterpret_cast<S *>(rd<uint64_t>(mem, kOffState)); }
  void set_state(void *p) const { wr<uint64_t>(mem, kOffState, reinterpret_cast<uint64_t>(p)); }
};

// Record a stage failure: status word + thread-local message.
void stage_fail(uint8_t *mem, int64_t code, const std::string &msg);

// What a `load` stage creates, so that a failed load leaves nothing behind and a
// later destroy frees exactly what this stage made.  The CUDA context at
// mem+0x10 may belong to the caller (it was there before `load`): then only the
// buffers created between begin() and seal() are this stage's, identified by
// their ids (ids are sequential and never reused, base/src/ffi/cuda.rs:360-381).
struct LoadScope {
  uint8_t *mem;
  bool created_ctx = false;
  int first_buf = -1, last_buf = -2;      // inclusive id range of this load's buffers
  std::vector<int> pinned, events, graphs;

  static int probe_id(B200CudaContext *ctx) {
    const int id = cl_cuda_create_buffer(ctx, 4);
    if (id >= 0) cl_cuda_free_buffer(ctx, id);
    return id;
  }
  // Context (created when the slot is empty) and the id watermark.  False: nothing to undo.
  bool begin(uint8_t *m) {
    mem = m;
    StageIO io(m);
    if (!io.ctx()) {
      cl_cuda_init(io.ctx_slot());
      if (!io.ctx()) return false;
      created_ctx = true;
    }
    first_buf = probe_id(io.ctx()) + 1;
    return first_buf > 0;
  }
  void seal() { last_buf = probe_id(StageIO(mem).ctx()) - 1; }
  // Free everything made since begin(): the whole context when this stage created it.
  void release() {
    StageIO io(mem);
    B200CudaContext *ctx = io.ctx();
    if (!ctx) return;
    if (created_ctx) { cl_cuda_cleanup(io.ctx_slot()); return; }
    cl_cuda_stream_sync(ctx, -1);
    if (last_buf < first_buf) seal();
    for (int g : graphs) cl_cuda_graph_destroy(ctx, g);
    for (int id = first_buf; id <= last_buf; ++id) cl_cuda_free_buffer(ctx, id);   // ids freed earlier just answer -1
    for (int p : pinned) cl_cuda_pinned_free(ctx, p);
    for (int e : events) cl_cuda_event_destroy(ctx, e);
  }
  void fail(int64_t code, const std::string &msg) {
    release();
    stage_fail(mem, code, msg);
  }
};

// Launch helper over cl_b200_launch with the built-in module.
struct Launcher {
  B200CudaContext *ctx;
  int module;
  int stream = -1;
  bool ok = true;
  std::string err;
  int issued = 0;
  int limit = -1;     // >= 0: only the first `limit` launches are issued (launch-ladder profiling)
  int count = 0;      // launches asked for so far
  // Timing ablation only: B200_SKIP="first:period[,first:period...]" drops launch number
  // first, first+period, ... of this launcher; the step's results are then meaningless.
  bool skipped() {
    static const char *e = getenv("B200_SKIP");
    if (!e) return false;
    const int i = issued++;
    for (const char *p = e; p && *p; p = strchr(p, ',') ? strchr(p, ',') + 1 : nullptr) {
      int first = 0, period = 1 << 30;
      if (sscanf(p, "%d:%d", &first, &period) < 1) break;
      if (i >= first && period > 0 && (i - first) % period == 0) return true;
    }
    return false;
  }
  template <typename S>
  void operator()(const char *name, std::initializer_list<int32_t> bufs, const S &scalars, int gx, int gy,
                  int gz, int bx, int smem = 0, int flags = 0) {
    if (!ok || skipped()) return;
    if (limit >= 0 && count >= limit) { ++count; return; }
    ++count;
    std::vector<int32_t> ids(bufs);
    int rc = cl_b200_launch(ctx, module, reinterpret_cast<const uint8_t *>(name), int32_t(ids.size()),
                            reinterpret_cast<const uint8_t *>(ids.data()),
                            reinterpret_cast<const uint8_t *>(&scalars), int32_t(sizeof(S)), gx, gy, gz, bx,
                            1, 1, smem, stream, flags);
    if (rc != 0) {
      ok = false;
      err = std::string(name) + ": " + cl_b200_last_error();
    }
  }
};

}  // namespace b200
