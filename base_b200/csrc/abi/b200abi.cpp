// Device-primitive layer: the `cl_cuda_*` ABI of the reference
// (base/src/ffi/cuda.rs) re-implemented over the CUDA driver API, plus the
// `cl_b200_*` additions declared in include/b200abi.h.
//
// State model, as in the reference (cuda.rs:6-9, 126-128): one heap context
// per `cl_cuda_init`, tables of buffers / streams / events / graphs / pinned
// blocks / modules indexed by sequential ids, all behind one mutex.  A freed
// id leaves a tombstone so ids are never reused (cuda.rs:1222-1243).
#include "b200abi.h"
#include "cuda_dyn.h"
#include "nccl_dyn.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

extern "C" {
extern const unsigned char b200_kernels_image_start[];
extern const unsigned char b200_kernels_image_end[];
}

namespace {

CudaDriver g_drv;
NcclLib g_nccl;
std::mutex g_drv_mu;
thread_local std::string t_err;

void set_err(const std::string &s) {
  t_err = s;
  if (const char *e = getenv("B200_LOG")) {
    if (e[0] && e[0] != '0') fprintf(stderr, "[b200abi] %s\n", s.c_str());
  }
}

std::string cu_err(CUresult r) {
  const char *s = nullptr;
  if (g_drv.ok && g_drv.p_cuGetErrorString(r, &s) == CUDA_SUCCESS && s) return s;
  return "CUDA error " + std::to_string(int(r));
}

struct Buffer { CUdeviceptr ptr = 0; int64_t size = 0; bool live = false; };
struct Event  { CUevent ev = nullptr; bool live = false; bool recorded = false; };
struct Stream { CUstream st = nullptr; bool live = false; };
struct Graph  { CUgraphExec ex = nullptr; bool live = false; };
struct Pinned { void *p = nullptr; int64_t size = 0; bool live = false; };
struct Module {
  CUmodule mod = nullptr; bool live = false;
  std::unordered_map<std::string, CUfunction> fns;
};

}  // namespace

struct B200CudaContext {
  std::mutex mu;
  int ordinal = 0;
  CUdevice dev = 0;
  CUcontext cuctx = nullptr;
  CUstream main_stream = nullptr;
  int sm_count = 0;
  std::vector<Buffer> buffers;
  std::vector<Stream> streams;
  std::vector<Event> events;
  std::vector<Graph> graphs;
  std::vector<Pinned> pinned;
  std::vector<Module> modules;
  std::unordered_map<const void *, int> text_modules;  // PTX text address -> module id
  int builtin_module = -1;
  ncclComm_t comm = nullptr;      // expert-parallel communicator (cl_b200_comm_init), else null
  int comm_rank = 0, comm_world = 1;
};

namespace {

#define CU_TRY(ctx_expr, call)                                   \
  do {                                                           \
    CUresult _r = (call);                                        \
    if (_r != CUDA_SUCCESS) {                                    \
      set_err(std::string(#call) + ": " + cu_err(_r));           \
      return -1;                                                 \
    }                                                            \
  } while (0)

// The driver context is bound to the calling thread on every entry, as the
// reference does lazily per thread (cuda.rs:85-97).
bool bind(const B200CudaContext *c) {
  if (!c || !c->cuctx) { set_err("null context"); return false; }
  CUcontext cur = nullptr;
  if (g_drv.p_cuCtxGetCurrent(&cur) == CUDA_SUCCESS && cur == c->cuctx) return true;
  CUresult r = g_drv.p_cuCtxSetCurrent(c->cuctx);
  if (r != CUDA_SUCCESS) { set_err("cuCtxSetCurrent: " + cu_err(r)); return false; }
  return true;
}

Buffer *get_buf(B200CudaContext *c, int32_t id) {
  if (id < 0 || size_t(id) >= c->buffers.size() || !c->buffers[id].live) return nullptr;
  return &c->buffers[id];
}

bool get_stream(B200CudaContext *c, int32_t id, CUstream *out) {
  if (id < 0) { *out = c->main_stream; return true; }
  if (size_t(id) >= c->streams.size() || !c->streams[id].live) return false;
  *out = c->streams[id].st;
  return true;
}

int32_t do_upload(B200CudaContext *c, int32_t id, int64_t off, const uint8_t *src, int64_t size,
                  bool async, int32_t stream_id) {
  if (!c) { set_err("null context"); return -1; }
  if (size < 0 || off < 0 || (size > 0 && !src)) { set_err("upload: bad size/offset/pointer"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  Buffer *b = get_buf(c, id);
  if (!b) { set_err("upload: bad buffer id"); return -1; }
  if (off > b->size || size > b->size - off) { set_err("upload: out of bounds"); return -1; }
  if (size == 0) return 0;
  CUstream st;
  if (!get_stream(c, stream_id, &st)) { set_err("upload: bad stream id"); return -1; }
  if (async) {
    CU_TRY(c, g_drv.p_cuMemcpyHtoDAsync(b->ptr + off, src, size_t(size), st));
  } else {
    // Synchronous with respect to work already queued on the main stream.
    CU_TRY(c, g_drv.p_cuMemcpyHtoDAsync(b->ptr + off, src, size_t(size), c->main_stream));
    CU_TRY(c, g_drv.p_cuStreamSynchronize(c->main_stream));
  }
  return 0;
}

int32_t do_download(B200CudaContext *c, int32_t id, int64_t off, uint8_t *dst, int64_t size,
                    bool async, int32_t stream_id) {
  if (!c) { set_err("null context"); return -1; }
  if (size < 0 || off < 0 || (size > 0 && !dst)) { set_err("download: bad size/offset/pointer"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  Buffer *b = get_buf(c, id);
  if (!b) { set_err("download: bad buffer id"); return -1; }
  if (off > b->size || size > b->size - off) { set_err("download: out of bounds"); return -1; }
  if (size == 0) return 0;
  CUstream st;
  if (!get_stream(c, stream_id, &st)) { set_err("download: bad stream id"); return -1; }
  if (async) {
    CU_TRY(c, g_drv.p_cuMemcpyDtoHAsync(dst, b->ptr + off, size_t(size), st));
  } else {
    CU_TRY(c, g_drv.p_cuMemcpyDtoHAsync(dst, b->ptr + off, size_t(size), c->main_stream));
    CU_TRY(c, g_drv.p_cuStreamSynchronize(c->main_stream));
  }
  return 0;
}

int32_t load_module_locked(B200CudaContext *c, const void *image) {
  CUmodule m = nullptr;
  CU_TRY(c, g_drv.p_cuModuleLoadData(&m, image));
  Module mod;
  mod.mod = m;
  mod.live = true;
  c->modules.push_back(std::move(mod));
  return int32_t(c->modules.size() - 1);
}

CUfunction get_fn_locked(B200CudaContext *c, int32_t module_id, const char *name) {
  if (module_id < 0 || size_t(module_id) >= c->modules.size() || !c->modules[module_id].live) {
    set_err("launch: bad module id");
    return nullptr;
  }
  Module &m = c->modules[module_id];
  auto it = m.fns.find(name);
  if (it != m.fns.end()) return it->second;
  CUfunction f = nullptr;
  CUresult r = g_drv.p_cuModuleGetFunction(&f, m.mod, name);
  if (r != CUDA_SUCCESS) {
    set_err(std::string("cuModuleGetFunction(") + name + "): " + cu_err(r));
    return nullptr;
  }
  m.fns.emplace(name, f);
  return f;
}

int32_t launch_common(B200CudaContext *c, CUfunction f, int32_t n_bufs, const uint8_t *bind_ids,
                      const uint8_t *scalars, int32_t scalar_bytes, int32_t gx, int32_t gy, int32_t gz,
                      int32_t bx, int32_t by, int32_t bz, int32_t smem, CUstream st, int32_t flags) {
  constexpr int kMaxPtrs = 64;
  if (n_bufs > kMaxPtrs) { set_err("launch: too many buffers"); return -1; }
  CUdeviceptr ptrs[kMaxPtrs];
  void *params[kMaxPtrs + 1];
  for (int i = 0; i < n_bufs; ++i) {
    int32_t id;
    memcpy(&id, bind_ids + 4 * i, 4);
    if (id == -1 && scalars != nullptr) {
      ptrs[i] = 0;  // optional operand of a cl_b200_launch kernel
    } else {
      Buffer *b = get_buf(c, id);
      if (!b) { set_err("launch: bad buffer id in bind table"); return -1; }
      ptrs[i] = b->ptr;
    }
    params[i] = &ptrs[i];
  }
  int np = n_bufs;
  if (scalar_bytes > 0) params[np++] = const_cast<uint8_t *>(scalars);
  if (smem > 32 * 1024) {     // (dynamic + static may exceed the 48 KB default even when dynamic alone does not)
    CU_TRY(c, g_drv.p_cuFuncSetAttribute(f, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, smem));
  }
  // One shared-memory carveout for every kernel of this library: an SM must
  // drain before it can change its L1/shared split, which would serialise
  // back-to-back kernels with different footprints and defeat programmatic
  // dependent launch.  (B200_CARVEOUT=-1 leaves the driver's default.)
  {
    static const int carve = [] { const char *e = getenv("B200_CARVEOUT"); return e ? atoi(e) : 100; }();
    if (carve >= 0) g_drv.p_cuFuncSetAttribute(f, CU_FUNC_ATTRIBUTE_PREFERRED_SHARED_MEMORY_CARVEOUT, carve);
  }
  if (flags & 3) {
    CUlaunchConfig cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDimX = gx; cfg.gridDimY = gy; cfg.gridDimZ = gz;
    cfg.blockDimX = bx; cfg.blockDimY = by; cfg.blockDimZ = bz;
    cfg.sharedMemBytes = smem;
    cfg.hStream = st;
    CUlaunchAttribute attr[2];
    memset(attr, 0, sizeof(attr));
    unsigned n = 0;
    if (flags & 1) {
      attr[n].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
      attr[n].value.programmaticStreamSerializationAllowed = 1;
      ++n;
    }
    if (flags & 2) {
      // every CTA of the grid resident at once (kernels with grid-wide barriers)
      attr[n].id = CU_LAUNCH_ATTRIBUTE_COOPERATIVE;
      attr[n].value.cooperative = 1;
      ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    CU_TRY(c, g_drv.p_cuLaunchKernelEx(&cfg, f, params, nullptr));
  } else {
    CU_TRY(c, g_drv.p_cuLaunchKernel(f, gx, gy, gz, bx, by, bz, smem, st, params, nullptr));
  }
  return 0;
}

int32_t launch_text(B200CudaContext *c, const uint8_t *text, const uint8_t *name, int32_t n_bufs,
                    const uint8_t *bind_ids, int32_t gx, int32_t gy, int32_t gz, int32_t bx, int32_t by,
                    int32_t bz, int32_t stream_id) {
  if (!c) { set_err("null context"); return -1; }
  if (!text || n_bufs < 0 || (n_bufs > 0 && !bind_ids)) { set_err("launch: bad arguments"); return -1; }
  if (gx <= 0 || gy <= 0 || gz <= 0 || bx <= 0 || by <= 0 || bz <= 0) {
    set_err("launch: non-positive grid/block dimension");
    return -1;
  }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  CUstream st;
  if (!get_stream(c, stream_id, &st)) { set_err("launch: bad stream id"); return -1; }
  int mid;
  auto it = c->text_modules.find(text);
  if (it != c->text_modules.end()) {
    mid = it->second;
  } else {
    mid = load_module_locked(c, text);
    if (mid < 0) return -1;
    c->text_modules.emplace(text, mid);
  }
  CUfunction f = get_fn_locked(c, mid, name ? reinterpret_cast<const char *>(name) : "main");
  if (!f) return -1;
  return launch_common(c, f, n_bufs, bind_ids, nullptr, 0, gx, gy, gz, bx, by, bz, 0, st, 0);
}

}  // namespace

extern "C" {

const char *cl_b200_last_error(void) { return t_err.c_str(); }

void cl_cuda_init(B200CudaContext **slot) {
  if (!slot) return;
  *slot = nullptr;
  {
    std::lock_guard<std::mutex> g(g_drv_mu);
    if (!g_drv.load()) { set_err("libcuda.so.1 not available"); return; }
  }
  if (g_drv.p_cuInit(0) != CUDA_SUCCESS) { set_err("cuInit failed (no GPU?)"); return; }
  int ordinal = 0;
  if (const char *e = getenv("B200_DEVICE")) ordinal = atoi(e);
  else if (const char *e2 = getenv("LOCAL_RANK")) ordinal = atoi(e2);
  int count = 0;
  if (g_drv.p_cuDeviceGetCount(&count) != CUDA_SUCCESS || count <= 0) { set_err("no CUDA device"); return; }
  if (ordinal < 0 || ordinal >= count) ordinal = ordinal % count;
  B200CudaContext *c = new B200CudaContext();
  c->ordinal = ordinal;
  CUresult r = g_drv.p_cuDeviceGet(&c->dev, ordinal);
  if (r == CUDA_SUCCESS) r = g_drv.p_cuDevicePrimaryCtxRetain(&c->cuctx, c->dev);
  if (r == CUDA_SUCCESS) r = g_drv.p_cuCtxSetCurrent(c->cuctx);
  if (r == CUDA_SUCCESS) r = g_drv.p_cuStreamCreate(&c->main_stream, CU_STREAM_NON_BLOCKING);
  if (r != CUDA_SUCCESS) {
    set_err("context setup: " + cu_err(r));
    if (c->cuctx) g_drv.p_cuDevicePrimaryCtxRelease(c->dev);
    delete c;
    return;
  }
  g_drv.p_cuDeviceGetAttribute(&c->sm_count, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT, c->dev);
  *slot = c;
}

void cl_cuda_cleanup(B200CudaContext **slot) {
  if (!slot || !*slot) return;
  B200CudaContext *c = *slot;
  {
    std::lock_guard<std::mutex> g(c->mu);
    if (bind(c)) {
      g_drv.p_cuCtxSynchronize();
      for (auto &gph : c->graphs) if (gph.live) g_drv.p_cuGraphExecDestroy(gph.ex);
      for (auto &e : c->events) if (e.live) g_drv.p_cuEventDestroy(e.ev);
      for (auto &s : c->streams) if (s.live) g_drv.p_cuStreamDestroy(s.st);
      for (auto &b : c->buffers) if (b.live) g_drv.p_cuMemFree(b.ptr);
      for (auto &p : c->pinned) if (p.live) g_drv.p_cuMemFreeHost(p.p);
      for (auto &m : c->modules) if (m.live) g_drv.p_cuModuleUnload(m.mod);
      if (c->comm && g_nccl.ok) g_nccl.CommDestroy(c->comm);
      if (c->main_stream) g_drv.p_cuStreamDestroy(c->main_stream);
      g_drv.p_cuDevicePrimaryCtxRelease(c->dev);
    }
  }
  delete c;
  *slot = nullptr;
}

int32_t cl_cuda_create_buffer(B200CudaContext *c, int64_t size) {
  if (!c) { set_err("null context"); return -1; }
  if (size <= 0) { set_err("create_buffer: size <= 0"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  CUdeviceptr p = 0;
  CU_TRY(c, g_drv.p_cuMemAlloc(&p, size_t(size)));
  CUresult r = g_drv.p_cuMemsetD8Async(p, 0, size_t(size), c->main_stream);
  if (r != CUDA_SUCCESS) {
    g_drv.p_cuMemFree(p);
    set_err("create_buffer memset: " + cu_err(r));
    return -1;
  }
  Buffer b;
  b.ptr = p; b.size = size; b.live = true;
  c->buffers.push_back(b);
  return int32_t(c->buffers.size() - 1);
}

int32_t cl_cuda_free_buffer(B200CudaContext *c, int32_t id) {
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  Buffer *b = get_buf(c, id);
  if (!b) { set_err("free_buffer: bad or already freed id"); return -1; }
  g_drv.p_cuStreamSynchronize(c->main_stream);
  g_drv.p_cuMemFree(b->ptr);
  b->live = false; b->ptr = 0; b->size = 0;
  return 0;
}

int32_t cl_cuda_upload(B200CudaContext *c, int32_t id, const uint8_t *src, int64_t size) {
  return do_upload(c, id, 0, src, size, false, -1);
}
int32_t cl_cuda_upload_ptr(B200CudaContext *c, int32_t id, const uint8_t *src, int64_t size) {
  return do_upload(c, id, 0, src, size, false, -1);
}
int32_t cl_cuda_upload_ptr_offset(B200CudaContext *c, int32_t id, int64_t off, const uint8_t *src, int64_t size) {
  return do_upload(c, id, off, src, size, false, -1);
}
int32_t cl_cuda_download(B200CudaContext *c, int32_t id, uint8_t *dst, int64_t size) {
  return do_download(c, id, 0, dst, size, false, -1);
}
int32_t cl_cuda_download_ptr(B200CudaContext *c, int32_t id, uint8_t *dst, int64_t size) {
  return do_download(c, id, 0, dst, size, false, -1);
}
int32_t cl_cuda_download_ptr_offset(B200CudaContext *c, int32_t id, int64_t off, uint8_t *dst, int64_t size) {
  return do_download(c, id, off, dst, size, false, -1);
}
int32_t cl_cuda_upload_ptr_async(B200CudaContext *c, int32_t id, const uint8_t *src, int64_t size, int32_t sid) {
  return do_upload(c, id, 0, src, size, true, sid);
}
int32_t cl_cuda_upload_ptr_offset_async(B200CudaContext *c, int32_t id, int64_t off, const uint8_t *src,
                                        int64_t size, int32_t sid) {
  return do_upload(c, id, off, src, size, true, sid);
}
int32_t cl_cuda_download_ptr_async(B200CudaContext *c, int32_t id, uint8_t *dst, int64_t size, int32_t sid) {
  return do_download(c, id, 0, dst, size, true, sid);
}

int32_t cl_cuda_stream_create(B200CudaContext *c) {
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  CUstream st = nullptr;
  CU_TRY(c, g_drv.p_cuStreamCreate(&st, CU_STREAM_NON_BLOCKING));
  // Order the new stream after the work already queued on the main stream.
  CUevent fence = nullptr;
  if (g_drv.p_cuEventCreate(&fence, CU_EVENT_DISABLE_TIMING) != CUDA_SUCCESS ||
      g_drv.p_cuEventRecord(fence, c->main_stream) != CUDA_SUCCESS ||
      g_drv.p_cuStreamWaitEvent(st, fence, 0) != CUDA_SUCCESS) {
    if (fence) g_drv.p_cuEventDestroy(fence);
    g_drv.p_cuStreamDestroy(st);
    set_err("stream_create: fence failed");
    return -1;
  }
  g_drv.p_cuEventDestroy(fence);
  Stream s;
  s.st = st; s.live = true;
  c->streams.push_back(s);
  return int32_t(c->streams.size() - 1);
}

int32_t cl_cuda_stream_sync(B200CudaContext *c, int32_t sid) {
  if (!c) { set_err("null context"); return -1; }
  CUstream st;
  {
    std::lock_guard<std::mutex> g(c->mu);
    if (!bind(c)) return -1;
    if (!get_stream(c, sid, &st)) { set_err("stream_sync: bad stream id"); return -1; }
  }
  CU_TRY(c, g_drv.p_cuStreamSynchronize(st));
  return 0;
}

int32_t cl_cuda_stream_destroy(B200CudaContext *c, int32_t sid) {
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  if (sid < 0 || size_t(sid) >= c->streams.size() || !c->streams[sid].live) {
    set_err("stream_destroy: bad stream id");
    return -1;
  }
  g_drv.p_cuStreamSynchronize(c->streams[sid].st);
  g_drv.p_cuStreamDestroy(c->streams[sid].st);
  c->streams[sid].live = false;
  c->streams[sid].st = nullptr;
  return 0;
}

int32_t cl_cuda_event_create(B200CudaContext *c) {
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  CUevent ev = nullptr;
  CU_TRY(c, g_drv.p_cuEventCreate(&ev, CU_EVENT_DEFAULT));
  Event e;
  e.ev = ev; e.live = true;
  c->events.push_back(e);
  return int32_t(c->events.size() - 1);
}

int32_t cl_cuda_event_record(B200CudaContext *c, int32_t eid, int32_t sid) {
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  if (eid < 0 || size_t(eid) >= c->events.size() || !c->events[eid].live) {
    set_err("event_record: bad event id");
    return -1;
  }
  CUstream st;
  if (!get_stream(c, sid, &st)) { set_err("event_record: bad stream id"); return -1; }
  CU_TRY(c, g_drv.p_cuEventRecord(c->events[eid].ev, st));
  c->events[eid].recorded = true;
  return 0;
}

int32_t cl_cuda_stream_wait_event(B200CudaContext *c, int32_t sid, int32_t eid) {
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  if (eid < 0 || size_t(eid) >= c->events.size() || !c->events[eid].live) {
    set_err("stream_wait_event: bad event id");
    return -1;
  }
  CUstream st;
  if (!get_stream(c, sid, &st)) { set_err("stream_wait_event: bad stream id"); return -1; }
  CU_TRY(c, g_drv.p_cuStreamWaitEvent(st, c->events[eid].ev, 0));
  return 0;
}

int32_t cl_cuda_event_elapsed_ms_bits(B200CudaContext *c, int32_t a, int32_t b) {
  if (!c) { set_err("null context"); return -1; }
  CUevent ea, eb;
  {
    std::lock_guard<std::mutex> g(c->mu);
    if (!bind(c)) return -1;
    auto ok = [&](int32_t id) {
      return id >= 0 && size_t(id) < c->events.size() && c->events[id].live && c->events[id].recorded;
    };
    if (!ok(a) || !ok(b)) { set_err("event_elapsed: bad or unrecorded event"); return -1; }
    ea = c->events[a].ev;
    eb = c->events[b].ev;
  }
  float ms = 0.f;
  // cuEventElapsedTime needs both events complete.
  CU_TRY(c, g_drv.p_cuEventSynchronize(eb));
  CU_TRY(c, g_drv.p_cuEventElapsedTime(&ms, ea, eb));
  int32_t bits;
  memcpy(&bits, &ms, 4);
  return bits;
}

int32_t cl_cuda_event_destroy(B200CudaContext *c, int32_t eid) {
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  if (eid < 0 || size_t(eid) >= c->events.size() || !c->events[eid].live) {
    set_err("event_destroy: bad event id");
    return -1;
  }
  g_drv.p_cuEventDestroy(c->events[eid].ev);
  c->events[eid].live = false;
  c->events[eid].ev = nullptr;
  return 0;
}

int32_t cl_cuda_graph_begin_capture(B200CudaContext *c, int32_t sid) {
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  CUstream st;
  if (!get_stream(c, sid, &st)) { set_err("graph_begin_capture: bad stream id"); return -1; }
  CU_TRY(c, g_drv.p_cuStreamBeginCapture(st, CU_STREAM_CAPTURE_MODE_RELAXED));
  return 0;
}

int32_t cl_cuda_graph_end_capture(B200CudaContext *c, int32_t sid) {
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  CUstream st;
  if (!get_stream(c, sid, &st)) { set_err("graph_end_capture: bad stream id"); return -1; }
  CUgraph graph = nullptr;
  CUresult r = g_drv.p_cuStreamEndCapture(st, &graph);
  if (r != CUDA_SUCCESS || !graph) { set_err("cuStreamEndCapture: " + cu_err(r)); return -1; }
  CUgraphExec ex = nullptr;
  r = g_drv.p_cuGraphInstantiateWithFlags(&ex, graph, 0);
  g_drv.p_cuGraphDestroy(graph);
  if (r != CUDA_SUCCESS || !ex) { set_err("cuGraphInstantiate: " + cu_err(r)); return -1; }
  Graph gr;
  gr.ex = ex; gr.live = true;
  c->graphs.push_back(gr);
  return int32_t(c->graphs.size() - 1);
}

static int32_t graph_op(B200CudaContext *c, int32_t gid, int32_t sid, bool launch) {
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  if (gid < 0 || size_t(gid) >= c->graphs.size() || !c->graphs[gid].live) {
    set_err("graph: bad graph id");
    return -1;
  }
  CUstream st;
  if (!get_stream(c, sid, &st)) { set_err("graph: bad stream id"); return -1; }
  if (launch) CU_TRY(c, g_drv.p_cuGraphLaunch(c->graphs[gid].ex, st));
  else CU_TRY(c, g_drv.p_cuGraphUpload(c->graphs[gid].ex, st));
  return 0;
}
int32_t cl_cuda_graph_upload(B200CudaContext *c, int32_t gid, int32_t sid) { return graph_op(c, gid, sid, false); }
int32_t cl_cuda_graph_launch(B200CudaContext *c, int32_t gid, int32_t sid) { return graph_op(c, gid, sid, true); }

int32_t cl_cuda_graph_destroy(B200CudaContext *c, int32_t gid) {
  if (gid < 0) { set_err("graph_destroy: bad graph id"); return -1; }
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  if (size_t(gid) >= c->graphs.size() || !c->graphs[gid].live) { set_err("graph_destroy: bad graph id"); return -1; }
  g_drv.p_cuGraphExecDestroy(c->graphs[gid].ex);
  c->graphs[gid].live = false;
  c->graphs[gid].ex = nullptr;
  return 0;
}

int32_t cl_cuda_pinned_alloc(B200CudaContext *c, int64_t size) {
  if (size <= 0) { set_err("pinned_alloc: size <= 0"); return -1; }
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  void *p = nullptr;
  CU_TRY(c, g_drv.p_cuMemAllocHost(&p, size_t(size)));
  memset(p, 0, size_t(size));
  Pinned pn;
  pn.p = p; pn.size = size; pn.live = true;
  c->pinned.push_back(pn);
  return int32_t(c->pinned.size() - 1);
}

int64_t cl_cuda_pinned_ptr(B200CudaContext *c, int32_t pid) {
  if (!c) { set_err("null context"); return 0; }
  std::lock_guard<std::mutex> g(c->mu);
  if (pid < 0 || size_t(pid) >= c->pinned.size() || !c->pinned[pid].live) {
    set_err("pinned_ptr: bad id");
    return 0;
  }
  return int64_t(reinterpret_cast<intptr_t>(c->pinned[pid].p));
}

int32_t cl_cuda_pinned_free(B200CudaContext *c, int32_t pid) {
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  if (pid < 0 || size_t(pid) >= c->pinned.size() || !c->pinned[pid].live) {
    set_err("pinned_free: bad id");
    return -1;
  }
  g_drv.p_cuStreamSynchronize(c->main_stream);
  g_drv.p_cuMemFreeHost(c->pinned[pid].p);
  c->pinned[pid].live = false;
  c->pinned[pid].p = nullptr;
  return 0;
}

int32_t cl_cuda_launch(B200CudaContext *c, const uint8_t *text, int32_t n_bufs, const uint8_t *bind_ids,
                       int32_t gx, int32_t gy, int32_t gz, int32_t bx, int32_t by, int32_t bz) {
  return launch_text(c, text, nullptr, n_bufs, bind_ids, gx, gy, gz, bx, by, bz, -1);
}
int32_t cl_cuda_launch_named(B200CudaContext *c, const uint8_t *text, const uint8_t *name, int32_t n_bufs,
                             const uint8_t *bind_ids, int32_t gx, int32_t gy, int32_t gz, int32_t bx,
                             int32_t by, int32_t bz) {
  if (!name) { set_err("launch_named: null name"); return -1; }
  return launch_text(c, text, name, n_bufs, bind_ids, gx, gy, gz, bx, by, bz, -1);
}
int32_t cl_cuda_launch_on_stream(B200CudaContext *c, const uint8_t *text, int32_t n_bufs,
                                 const uint8_t *bind_ids, int32_t gx, int32_t gy, int32_t gz, int32_t bx,
                                 int32_t by, int32_t bz, int32_t sid) {
  return launch_text(c, text, nullptr, n_bufs, bind_ids, gx, gy, gz, bx, by, bz, sid);
}
int32_t cl_cuda_launch_named_on_stream(B200CudaContext *c, const uint8_t *text, const uint8_t *name,
                                       int32_t n_bufs, const uint8_t *bind_ids, int32_t gx, int32_t gy,
                                       int32_t gz, int32_t bx, int32_t by, int32_t bz, int32_t sid) {
  if (!name) { set_err("launch_named: null name"); return -1; }
  return launch_text(c, text, name, n_bufs, bind_ids, gx, gy, gz, bx, by, bz, sid);
}

int32_t cl_cuda_sync(const B200CudaContext *cc) {
  B200CudaContext *c = const_cast<B200CudaContext *>(cc);
  if (!c) { set_err("null context"); return -1; }
  {
    std::lock_guard<std::mutex> g(c->mu);
    if (!bind(c)) return -1;
  }
  CUresult r = g_drv.p_cuCtxSynchronize();
  if (r != CUDA_SUCCESS) {
    set_err("cuCtxSynchronize: " + cu_err(r));
    fprintf(stderr, "cl_cuda_sync: %s\n", cu_err(r).c_str());
    return -1;
  }
  return 0;
}

// ---- additions -------------------------------------------------------------

int32_t cl_b200_load_module(B200CudaContext *c, const uint8_t *image, int64_t len) {
  if (!c) { set_err("null context"); return -1; }
  if (!image || len <= 0) { set_err("load_module: empty image"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  // The driver reads the image's own header for its size; a private copy
  // with a trailing NUL makes PTX text safe too.
  std::vector<uint8_t> copy(image, image + len);
  copy.push_back(0);
  return load_module_locked(c, copy.data());
}

int32_t cl_b200_builtin_module(B200CudaContext *c) {
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  if (c->builtin_module >= 0) return c->builtin_module;
  if (b200_kernels_image_end - b200_kernels_image_start < 64) {
    set_err("built-in kernel image is missing from this build");
    return -1;
  }
  int m = load_module_locked(c, b200_kernels_image_start);
  if (m >= 0) c->builtin_module = m;
  return m;
}

int32_t cl_b200_launch(B200CudaContext *c, int32_t module_id, const uint8_t *name, int32_t n_bufs,
                       const uint8_t *bind_ids, const uint8_t *scalars, int32_t scalar_bytes,
                       int32_t gx, int32_t gy, int32_t gz, int32_t bx, int32_t by, int32_t bz,
                       int32_t smem, int32_t sid, int32_t flags) {
  if (!c) { set_err("null context"); return -1; }
  if (!name || n_bufs < 0 || (n_bufs > 0 && !bind_ids) || scalar_bytes < 0 ||
      (scalar_bytes > 0 && !scalars) || smem < 0) {
    set_err("b200_launch: bad arguments");
    return -1;
  }
  if (gx <= 0 || gy <= 0 || gz <= 0 || bx <= 0 || by <= 0 || bz <= 0) {
    set_err("b200_launch: non-positive grid/block dimension");
    return -1;
  }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  CUstream st;
  if (!get_stream(c, sid, &st)) { set_err("b200_launch: bad stream id"); return -1; }
  CUfunction f = get_fn_locked(c, module_id, reinterpret_cast<const char *>(name));
  if (!f) return -1;
  static const uint8_t dummy = 0;
  return launch_common(c, f, n_bufs, bind_ids, scalars ? scalars : &dummy, scalar_bytes, gx, gy, gz, bx,
                       by, bz, smem, st, flags);
}

int64_t cl_b200_buffer_ptr(B200CudaContext *c, int32_t id) {
  if (!c) { set_err("null context"); return 0; }
  std::lock_guard<std::mutex> g(c->mu);
  Buffer *b = get_buf(c, id);
  if (!b) { set_err("buffer_ptr: bad id"); return 0; }
  return int64_t(b->ptr);
}

int64_t cl_b200_buffer_size(B200CudaContext *c, int32_t id) {
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  Buffer *b = get_buf(c, id);
  if (!b) { set_err("buffer_size: bad id"); return -1; }
  return b->size;
}

int32_t cl_b200_memset_async(B200CudaContext *c, int32_t id, int64_t off, int32_t value, int64_t size,
                             int32_t sid) {
  if (!c) { set_err("null context"); return -1; }
  if (off < 0 || size < 0) { set_err("memset: bad range"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  Buffer *b = get_buf(c, id);
  if (!b) { set_err("memset: bad buffer id"); return -1; }
  if (off > b->size || size > b->size - off) { set_err("memset: out of bounds"); return -1; }
  CUstream st;
  if (!get_stream(c, sid, &st)) { set_err("memset: bad stream id"); return -1; }
  if (size == 0) return 0;
  CU_TRY(c, g_drv.p_cuMemsetD8Async(b->ptr + off, (unsigned char)value, size_t(size), st));
  return 0;
}

int32_t cl_b200_copy_to_device_ptr(B200CudaContext *c, int32_t src_buf, int64_t src_offset, uint64_t dst_device_ptr,
                                   int64_t size, int32_t stream_id) {
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  Buffer *b = get_buf(c, src_buf);
  if (!b) { set_err("copy_to_device_ptr: bad buffer id"); return -1; }
  if (src_offset < 0 || size <= 0 || src_offset + size > int64_t(b->size) || dst_device_ptr == 0) {
    set_err("copy_to_device_ptr: range out of bounds or null destination");
    return -1;
  }
  CUstream st;
  if (!get_stream(c, stream_id, &st)) { set_err("copy_to_device_ptr: bad stream id"); return -1; }
  CU_TRY(c, g_drv.p_cuMemcpyDtoDAsync(CUdeviceptr(dst_device_ptr), b->ptr + src_offset, size_t(size), st));
  return 0;
}

int32_t cl_b200_copy_async(B200CudaContext *c, int32_t dst, int64_t doff, int32_t src, int64_t soff,
                           int64_t size, int32_t sid) {
  if (!c) { set_err("null context"); return -1; }
  if (doff < 0 || soff < 0 || size < 0) { set_err("copy: bad range"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  Buffer *d = get_buf(c, dst), *s = get_buf(c, src);
  if (!d || !s) { set_err("copy: bad buffer id"); return -1; }
  if (doff > d->size || size > d->size - doff || soff > s->size || size > s->size - soff) {
    set_err("copy: out of bounds");
    return -1;
  }
  CUstream st;
  if (!get_stream(c, sid, &st)) { set_err("copy: bad stream id"); return -1; }
  if (size == 0) return 0;
  CU_TRY(c, g_drv.p_cuMemcpyDtoDAsync(d->ptr + doff, s->ptr + soff, size_t(size), st));
  return 0;
}

int32_t cl_b200_device_ordinal(B200CudaContext *c) { return c ? c->ordinal : -1; }
int32_t cl_b200_sm_count(B200CudaContext *c) { return c ? c->sm_count : -1; }
// The CUstream behind a stream id (-1 = the main stream), as an integer; 0 for a bad id.
int64_t cl_b200_stream_handle(B200CudaContext *c, int32_t stream_id) {
  if (!c) { set_err("null context"); return 0; }
  std::lock_guard<std::mutex> g(c->mu);
  CUstream st = nullptr;
  if (!get_stream(c, stream_id, &st)) { set_err("stream_handle: bad stream id"); return 0; }
  return int64_t(reinterpret_cast<uintptr_t>(st));
}

// ---- collectives over NCCL (expert-parallel decode) --------------------------------------------
int32_t cl_b200_comm_unique_id(uint8_t *out128) {
  if (!out128) { set_err("comm_unique_id: null pointer"); return -1; }
  std::lock_guard<std::mutex> g(g_drv_mu);
  if (!g_nccl.load()) { set_err("libnccl.so.2 not available"); return -1; }
  ncclUniqueId id;
  const ncclResult_t r = g_nccl.GetUniqueId(&id);
  if (r != 0) { set_err(std::string("ncclGetUniqueId: ") + g_nccl.GetErrorString(r)); return -1; }
  memcpy(out128, id.internal, 128);
  return 0;
}

int32_t cl_b200_comm_init(B200CudaContext *c, const uint8_t *id128, int32_t rank, int32_t world) {
  if (!c) { set_err("null context"); return -1; }
  if (!id128 || world < 1 || rank < 0 || rank >= world) { set_err("comm_init: bad arguments"); return -1; }
  {
    std::lock_guard<std::mutex> g(g_drv_mu);
    if (!g_nccl.load()) { set_err("libnccl.so.2 not available"); return -1; }
  }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  if (c->comm) { set_err("comm_init: already initialised"); return -1; }
  ncclUniqueId id;
  memcpy(id.internal, id128, 128);
  const ncclResult_t r = g_nccl.CommInitRank(&c->comm, world, id, rank);
  if (r != 0) { c->comm = nullptr; set_err(std::string("ncclCommInitRank: ") + g_nccl.GetErrorString(r)); return -1; }
  c->comm_rank = rank;
  c->comm_world = world;
  return 0;
}

int32_t cl_b200_ipc_export(B200CudaContext *c, int32_t buf_id, uint8_t *out64) {
  if (!c || !out64) { set_err("ipc_export: null argument"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  Buffer *b = get_buf(c, buf_id);
  if (!b) { set_err("ipc_export: bad buffer"); return -1; }
  CUipcMemHandle h;
  static_assert(sizeof(h) == 64, "the handle is 64 bytes");
  CU_TRY(c, g_drv.p_cuIpcGetMemHandle(&h, b->ptr));
  memcpy(out64, &h, 64);
  return 0;
}

int64_t cl_b200_ipc_open(B200CudaContext *c, const uint8_t *handle64) {
  if (!c || !handle64) { set_err("ipc_open: null argument"); return 0; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return 0;
  CUipcMemHandle h;
  memcpy(&h, handle64, 64);
  CUdeviceptr p = 0;
  const CUresult r = g_drv.p_cuIpcOpenMemHandle(&p, h, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS);
  if (r != CUDA_SUCCESS) { set_err("cuIpcOpenMemHandle: " + cu_err(r)); return 0; }
  return int64_t(p);
}

int32_t cl_b200_ipc_close(B200CudaContext *c, int64_t address) {
  if (!c || address == 0) { set_err("ipc_close: null argument"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  CU_TRY(c, g_drv.p_cuIpcCloseMemHandle(CUdeviceptr(address)));
  return 0;
}

int32_t cl_b200_comm_world(B200CudaContext *c) { return c && c->comm ? c->comm_world : 1; }

// recv[r * bytes .. (r + 1) * bytes) on every rank = rank r's send[send_offset .. + bytes).
int32_t cl_b200_comm_all_gather(B200CudaContext *c, int32_t send_buf, int64_t send_offset, int32_t recv_buf, int64_t bytes,
                                int32_t stream_id) {
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  if (!c->comm) { set_err("all_gather: no communicator"); return -1; }
  Buffer *s = get_buf(c, send_buf), *d = get_buf(c, recv_buf);
  CUstream st;
  if (!s || !d || bytes <= 0 || send_offset < 0 || send_offset + bytes > s->size || bytes * c->comm_world > d->size ||
      !get_stream(c, stream_id, &st)) {
    set_err("all_gather: bad buffer, size or stream");
    return -1;
  }
  const ncclResult_t r = g_nccl.AllGather(reinterpret_cast<const void *>(s->ptr + send_offset), reinterpret_cast<void *>(d->ptr),
                                          size_t(bytes), kNcclUint8, c->comm, st);
  if (r != 0) { set_err(std::string("ncclAllGather: ") + g_nccl.GetErrorString(r)); return -1; }
  return 0;
}

// Rank r receives send[r * bytes .. + bytes) of every rank q into recv[q * bytes .. + bytes) (grouped send/recv).
int32_t cl_b200_comm_all_to_all(B200CudaContext *c, int32_t send_buf, int32_t recv_buf, int64_t bytes, int32_t stream_id) {
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  if (!c->comm) { set_err("all_to_all: no communicator"); return -1; }
  Buffer *s = get_buf(c, send_buf), *d = get_buf(c, recv_buf);
  CUstream st;
  if (!s || !d || bytes <= 0 || bytes * c->comm_world > s->size || bytes * c->comm_world > d->size || !get_stream(c, stream_id, &st)) {
    set_err("all_to_all: bad buffer, size or stream");
    return -1;
  }
  ncclResult_t r = g_nccl.GroupStart();
  for (int q = 0; q < c->comm_world && r == 0; ++q) {
    r = g_nccl.Send(reinterpret_cast<const void *>(s->ptr + size_t(q) * bytes), size_t(bytes), kNcclUint8, q, c->comm, st);
    if (r == 0) r = g_nccl.Recv(reinterpret_cast<void *>(d->ptr + size_t(q) * bytes), size_t(bytes), kNcclUint8, q, c->comm, st);
  }
  const ncclResult_t r2 = g_nccl.GroupEnd();
  if (r != 0 || r2 != 0) { set_err(std::string("all_to_all: ") + g_nccl.GetErrorString(r != 0 ? r : r2)); return -1; }
  return 0;
}

int64_t cl_b200_mem_free(B200CudaContext *c) {
  if (!c) { set_err("null context"); return -1; }
  std::lock_guard<std::mutex> g(c->mu);
  if (!bind(c)) return -1;
  size_t fr = 0, tot = 0;
  CU_TRY(c, g_drv.p_cuMemGetInfo(&fr, &tot));
  return int64_t(fr);
}

}  // extern "C"

// ---- cl_cublas_* on this library's own kernels ---------------------------------

namespace {

struct SgemvArgs { int rows, cols; float alpha, beta; };
struct SgemmArgs {
  int transa, transb, m, n, k;
  float alpha, beta;
  long long stride_a, stride_b, stride_c;
  int lda, ldb, ldc;
};

float bits_f32(int32_t b) { float f; memcpy(&f, &b, 4); return f; }

bool buf_holds(B200CudaContext *c, int32_t id, int64_t floats) {
  int64_t sz = cl_b200_buffer_size(c, id);
  return sz >= 0 && floats >= 0 && floats * 4 <= sz;
}

int32_t sgemv_impl(B200CudaContext *c, int32_t trans, int32_t m, int32_t n, int32_t alpha_bits,
                   int32_t a_buf, int32_t x_buf, int32_t beta_bits, int32_t y_buf, int32_t sid) {
  if (!c) { set_err("null context"); return -1; }
  if (m <= 0 || n <= 0) { set_err("sgemv: non-positive dimension"); return -1; }
  const int64_t xlen = trans ? m : n, ylen = trans ? n : m;
  if (!buf_holds(c, a_buf, int64_t(m) * n) || !buf_holds(c, x_buf, xlen) || !buf_holds(c, y_buf, ylen)) {
    set_err("sgemv: bad buffer id or buffer too small");
    return -1;
  }
  int mod = cl_b200_builtin_module(c);
  if (mod < 0) return -1;
  int32_t ids[3] = {a_buf, x_buf, y_buf};
  // Column-major A (m x n, lda = m) is row-major W[n][m].
  SgemvArgs a{n, m, bits_f32(alpha_bits), bits_f32(beta_bits)};
  if (trans) {
    const int rows_per_cta = 8 * 4;
    return cl_b200_launch(c, mod, reinterpret_cast<const uint8_t *>("sgemv_t_f32"), 3,
                          reinterpret_cast<const uint8_t *>(ids), reinterpret_cast<const uint8_t *>(&a),
                          sizeof(a), (n + rows_per_cta - 1) / rows_per_cta, 1, 1, 256, 1, 1, 0, sid, 0);
  }
  return cl_b200_launch(c, mod, reinterpret_cast<const uint8_t *>("sgemv_n_f32"), 3,
                        reinterpret_cast<const uint8_t *>(ids), reinterpret_cast<const uint8_t *>(&a),
                        sizeof(a), (m + 255) / 256, 1, 1, 256, 1, 1, 0, sid, 0);
}

int32_t sgemm_impl(B200CudaContext *c, int32_t transa, int32_t transb, int32_t m, int32_t n, int32_t k,
                   int32_t alpha_bits, int32_t a_buf, int64_t sa, int32_t b_buf, int64_t sb,
                   int32_t beta_bits, int32_t c_buf, int64_t sc, int32_t batch, int32_t sid) {
  if (!c) { set_err("null context"); return -1; }
  if (m <= 0 || n <= 0 || k <= 0 || batch <= 0 || sa < 0 || sb < 0 || sc < 0) {
    set_err("sgemm: non-positive dimension or negative stride");
    return -1;
  }
  if (batch > 65535) { set_err("sgemm: batch_count too large"); return -1; }
  const int64_t need_a = sa * (batch - 1) + int64_t(m) * k;
  const int64_t need_b = sb * (batch - 1) + int64_t(k) * n;
  const int64_t need_c = sc * (batch - 1) + int64_t(m) * n;
  if (!buf_holds(c, a_buf, need_a) || !buf_holds(c, b_buf, need_b) || !buf_holds(c, c_buf, need_c)) {
    set_err("sgemm: bad buffer id or buffer too small");
    return -1;
  }
  int mod = cl_b200_builtin_module(c);
  if (mod < 0) return -1;
  int32_t ids[3] = {a_buf, b_buf, c_buf};
  SgemmArgs g{transa != 0, transb != 0, m, n, k, bits_f32(alpha_bits), bits_f32(beta_bits),
              sa, sb, sc, transa ? k : m, transb ? n : k, m};
  const int64_t outs = int64_t(m) * n;
  return cl_b200_launch(c, mod, reinterpret_cast<const uint8_t *>("sgemm_naive_f32"), 3,
                        reinterpret_cast<const uint8_t *>(ids), reinterpret_cast<const uint8_t *>(&g),
                        sizeof(g), int32_t((outs + 255) / 256), batch, 1, 256, 1, 1, 0, sid, 0);
}

}  // namespace

extern "C" {

int32_t cl_cublas_sgemv(B200CudaContext *c, int32_t trans, int32_t m, int32_t n, int32_t alpha_bits,
                        int32_t a_buf, int32_t x_buf, int32_t beta_bits, int32_t y_buf) {
  return sgemv_impl(c, trans, m, n, alpha_bits, a_buf, x_buf, beta_bits, y_buf, -1);
}
int32_t cl_cublas_sgemv_on_stream(B200CudaContext *c, int32_t trans, int32_t m, int32_t n, int32_t alpha_bits,
                                  int32_t a_buf, int32_t x_buf, int32_t beta_bits, int32_t y_buf, int32_t sid) {
  return sgemv_impl(c, trans, m, n, alpha_bits, a_buf, x_buf, beta_bits, y_buf, sid);
}
int32_t cl_cublas_sgemm(B200CudaContext *c, int32_t transa, int32_t transb, int32_t m, int32_t n, int32_t k,
                        int32_t alpha_bits, int32_t a_buf, int32_t b_buf, int32_t beta_bits, int32_t c_buf) {
  return sgemm_impl(c, transa, transb, m, n, k, alpha_bits, a_buf, 0, b_buf, 0, beta_bits, c_buf, 0, 1, -1);
}
int32_t cl_cublas_sgemm_strided_batched(B200CudaContext *c, int32_t transa, int32_t transb, int32_t m, int32_t n,
                                        int32_t k, int32_t alpha_bits, int32_t a_buf, int64_t sa, int32_t b_buf,
                                        int64_t sb, int32_t beta_bits, int32_t c_buf, int64_t sc, int32_t batch) {
  return sgemm_impl(c, transa, transb, m, n, k, alpha_bits, a_buf, sa, b_buf, sb, beta_bits, c_buf, sc, batch, -1);
}
int32_t cl_cublas_sgemm_strided_batched_on_stream(B200CudaContext *c, int32_t transa, int32_t transb, int32_t m,
                                                  int32_t n, int32_t k, int32_t alpha_bits, int32_t a_buf,
                                                  int64_t sa, int32_t b_buf, int64_t sb, int32_t beta_bits,
                                                  int32_t c_buf, int64_t sc, int32_t batch, int32_t sid) {
  return sgemm_impl(c, transa, transb, m, n, k, alpha_bits, a_buf, sa, b_buf, sb, beta_bits, c_buf, sc, batch, sid);
}

}  // extern "C"
