// Stage program `native:qwen2` — greedy decode of a Qwen2-architecture model
// with f32 weights, the path the reference ships
// (lean/algorithms/Qwen2Common.lean, Qwen2Algorithm.lean, Qwen2Proven.lean).
// Same decode protocol: data = [token_id:u32][pos:u32], out = [next_token:u32]
// (Qwen2Common.lean:30, 830-864).
//
// The reference issues 2 + 24*22 + 3 = 533 device operations per token
// (Qwen2Common.lean:1755-1756: rmsnorm, 3 sgemv, 3 bias adds, 2 rope, 2
// kvstore, sgemm, softmax, sgemm, sgemv, add, rmsnorm, 2 sgemv, silu, sgemv,
// add per layer).  Here a layer is 5 launches inside one replayed CUDA graph:
//   norm + fused q/k/v GEMV + bias      (rows NQ*64 + 2*NKV*64)
//   attention (RoPE, KV append, split-KV softmax, P^T V)
//   o-proj GEMV + residual
//   norm + stacked gate/up GEMV         (rows 2*Dff)
//   SiLU(gate)*up + down GEMV + residual
// then final norm + tied lm_head GEMV, and the first-index argmax.
// Weights are synthetic (kernels/synth.cuh), f32 ~ N(0, 0.02), tied embeddings.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <memory>
#include <vector>

#include "plugin.h"

namespace {

using namespace b200;

struct QwenHeader {
  uint32_t magic;        // 'QW21'
  uint32_t layers, hidden, inter, n_q, n_kv, head_dim, vocab, max_seq, batch;
  float rope_theta, eps;
  uint32_t seed, flags;  // flags bit 0: programmatic dependent launch; bit 3: weights and KV cache stay on disk (openFiles)
  uint32_t reserved[2];
};
static_assert(sizeof(QwenHeader) == 64, "header is 64 bytes");
constexpr uint32_t kMagic = 0x31325751;  // "QW21"

struct GemvArgs { int rows, K, B, top_k; float eps; int w_is_f32, prologue, in_stride, out_stride, row_iters; };
struct DenseStreamArgs { GemvArgs g; int stages; };
struct EmbedArgs { int H, B, is_f32, vocab; };
struct ArgmaxArgs { int V, B, stride, parts; };
struct AttnArgs {
  int NQ, NKV, HD, B, cache_len, window, max_pos, qkv_stride, has_sinks, kv_is_f32;
  float scale;
  int max_splits;
};
struct SynthArgs { unsigned long long n; uint32_t tensor, seed; int kind; float c; int lo, span; unsigned long long first; };

// tensor id = layer * 32 + kind; globals use layer 1000
enum Kind : uint32_t { kLn1 = 0, kWqkv, kBqkv, kWo, kLn2, kWgu, kWdn, kEmbed = 16, kLnF };

struct Layer { int ln1, wqkv, bqkv, wo, ln2, wgu, wdn, kcache, vcache; };

struct State {
  QwenHeader h;
  int module = -1;
  std::vector<Layer> layers;
  int embed = -1, lnf = -1, rope = -1;
  int meta = -1, hA = -1, hB = -1, qkv = -1, attn = -1, gu = -1, part_o = -1, part_ml = -1, counters = -1;
  int logits = -1, next_tok = -1, tokens_out = -1, status = -1, am_v = -1, am_i = -1, am_ticket = -1;
  int pin_in = -1, pin_out = -1, graph = -1, ev0 = -1, ev1 = -1;
  int max_splits = 1, max_decode = 4096;
  int dense_stream = 1;
  LoadScope scope;
  std::vector<int64_t> next_pos;     // per sequence: the position the next step runs at
  // on-disk mode (header flags bit 3): ONE layer's weights and ONE K/V pair live on the device (layers[0]); every step
  // streams each layer's weights from the weight file and its K/V rows from the cache file, and writes the new row back
  int on_disk = 0, wfd = -1, kvfd = -1;
  std::vector<uint8_t> host;
};

constexpr int kArgmaxParts = 128;

int alloc(B200CudaContext *ctx, uint64_t bytes, bool *ok) {
  int id = cl_cuda_create_buffer(ctx, int64_t(bytes));
  if (id < 0) *ok = false;
  return id;
}

void synth(Launcher &L, int buf, uint64_t n, uint32_t layer, uint32_t kind, uint32_t seed, int gen, double sigma) {
  SynthArgs a{};
  a.n = n; a.tensor = layer * 32 + kind; a.seed = seed; a.kind = gen; a.c = float(sigma / 209.0232); a.span = 1;
  L("synth_fill", {buf}, a, int(std::max<uint64_t>(1, std::min<uint64_t>((n + 255) / 256, 148 * 32))), 1, 1, 256);
}

void launch_gemv(State *s, Launcher &L, std::initializer_list<int32_t> bufs9, GemvArgs g, int pdl) {
  std::vector<int32_t> b(bufs9);
  const int row_bytes = g.K * 4;
  const int xbytes = g.B * g.K * 4 + 160;
  const int stages = std::min(4, (112000 - xbytes) / (4 * row_bytes));
  if (!s->dense_stream || stages < 1) {
    L("gemv_fused", {b[0], b[1], b[2], b[3], b[4], b[5], b[6], b[7], b[8]}, g, (g.rows + 7) / 8, 1, 1, 128,
      xbytes, pdl);
    return;
  }
  DenseStreamArgs da{g, stages};
  const int grid = std::min((g.rows + 3) / 4, 296);
  L("gemv_stream", {b[0], b[1], b[2], b[3], b[4], b[5], b[6], b[7], b[8], s->status}, da, grid, 1, 1, 128,
    xbytes + 4 * stages * row_bytes + 4 * stages * 8, pdl);
}

void enqueue_layer(State *s, Launcher &L, const Layer &ly);
void enqueue_tail(State *s, Launcher &L);

void enqueue_head(State *s, Launcher &L) {
  const QwenHeader &h = s->h;
  const int pdl = (h.flags & 1) ? 1 : 0;
  EmbedArgs ea{int(h.hidden), int(h.batch), 1, int(h.vocab)};
  L("embed_gather", {s->embed, s->meta, s->hA}, ea, (int(h.hidden) + 255) / 256, int(h.batch), 1, 256, 0, pdl);
}

void enqueue_step(State *s, Launcher &L) {
  const QwenHeader &h = s->h;
  enqueue_head(s, L);
  for (uint32_t l = 0; l < h.layers; ++l) enqueue_layer(s, L, s->layers[l]);
  enqueue_tail(s, L);
}

void enqueue_layer(State *s, Launcher &L, const Layer &ly) {
  const QwenHeader &h = s->h;
  const int H = h.hidden, F = h.inter, B = h.batch;
  const int QD = h.n_q * 64, KVD = h.n_kv * 64, QKV = QD + 2 * KVD;
  const int pdl = (h.flags & 1) ? 1 : 0;
  {
    GemvArgs gq{QKV, H, B, 0, h.eps, 1, 1, H, QKV, 1};
    launch_gemv(s, L, {ly.wqkv, ly.bqkv, s->hA, ly.ln1, -1, -1, -1, -1, s->qkv}, gq, pdl);
    AttnArgs aa{int(h.n_q), int(h.n_kv), 64, B, int(h.max_seq), 0, int(h.max_seq), QKV, 0, 1, 0.125f, s->max_splits};
    L("attn_decode_f32", {s->qkv, s->rope, s->meta, ly.kcache, ly.vcache, -1, s->part_o, s->part_ml, s->counters, s->attn},
      aa, s->max_splits, int(h.n_kv), B, 128, 0, pdl);
    GemvArgs go{H, QD, B, 0, h.eps, 1, 0, QD, H, 1};
    launch_gemv(s, L, {ly.wo, -1, s->attn, -1, -1, -1, -1, s->hA, s->hB}, go, pdl);           // hB = hA + Wo attn
    GemvArgs gg{2 * F, H, B, 0, h.eps, 1, 1, H, 2 * F, 1};
    launch_gemv(s, L, {ly.wgu, -1, s->hB, ly.ln2, -1, -1, -1, -1, s->gu}, gg, pdl);           // [gate; up]
    GemvArgs gd{H, F, B, 0, h.eps, 1, 3, 2 * F, H, 1};
    launch_gemv(s, L, {ly.wdn, -1, s->gu, -1, -1, -1, -1, s->hB, s->hA}, gd, pdl);            // hA = hB + Wd act
  }
}

void enqueue_tail(State *s, Launcher &L) {
  const QwenHeader &h = s->h;
  const int H = h.hidden, B = h.batch, V = h.vocab;
  const int pdl = (h.flags & 1) ? 1 : 0;
  GemvArgs gl{V, H, B, 0, h.eps, 1, 1, H, V, std::max(1, (V + 8 * 1184 - 1) / (8 * 1184))};
  launch_gemv(s, L, {s->embed, -1, s->hA, s->lnf, -1, -1, -1, -1, s->logits}, gl, pdl);       // tied lm_head
  ArgmaxArgs am{V, B, V, kArgmaxParts};
  L("argmax_first", {s->logits, s->next_tok, s->meta, s->meta, s->am_v, s->am_i, s->am_ticket}, am, kArgmaxParts, B, 1,
    256, 0, pdl);
}

void stage_noop(uint8_t *) {}

void destroy(uint8_t *mem);

// load on a loaded instance releases what the earlier load made and loads anew.
void stage_load(uint8_t *mem) {
  StageIO io(mem);
  if (io.data_len != sizeof(QwenHeader)) return stage_fail(mem, 1, "load: payload must be the 64-byte header");
  QwenHeader h;
  memcpy(&h, io.data, sizeof(h));
  if (h.magic != kMagic) return stage_fail(mem, 1, "load: bad magic");
  if (h.head_dim != 64 || h.n_kv == 0 || h.n_q % h.n_kv || h.n_q / h.n_kv > 8)
    return stage_fail(mem, 1, "load: head_dim must be 64 and n_q = 1..8 x n_kv");
  if (h.hidden == 0 || h.hidden % 8 || h.hidden > 5120 || h.inter == 0 || h.inter % 8 || h.inter > 5120 ||
      h.n_q * 64 > 5120)
    return stage_fail(mem, 1, "load: hidden/inter must be multiples of 8, at most 5120");
  if (h.batch == 0 || h.batch > 4 || h.layers == 0 || h.layers > 128 || h.vocab == 0 || h.max_seq == 0 ||
      h.max_seq > (1u << 20))
    return stage_fail(mem, 1, "load: batch 1..4, layers/vocab/max_seq in range");
  if (io.state<State>()) destroy(mem);          // a valid request on a loaded instance: reload
  LoadScope scope;
  if (!scope.begin(mem)) return stage_fail(mem, 2, std::string("load: no CUDA device: ") + cl_b200_last_error());
  B200CudaContext *ctx = io.ctx();
  std::unique_ptr<State> s(new State());
  s->h = h;
  s->module = cl_b200_builtin_module(ctx);
  if (s->module < 0) return scope.fail(2, std::string("load: kernel image: ") + cl_b200_last_error());
  if (const char *e = getenv("B200_DENSE_STREAM")) s->dense_stream = atoi(e);
  const uint64_t H = h.hidden, F = h.inter, B = h.batch, V = h.vocab;
  const uint64_t QD = uint64_t(h.n_q) * 64, KVD = uint64_t(h.n_kv) * 64, QKV = QD + 2 * KVD;
  bool ok = true;
  Launcher L{ctx, s->module};
  s->embed = alloc(ctx, V * H * 4, &ok);
  s->lnf = alloc(ctx, H * 4, &ok);
  if (!ok) return scope.fail(2, std::string("load: allocation failed: ") + cl_b200_last_error());
  synth(L, s->embed, V * H, 1000, kEmbed, h.seed, 2, 0.02);
  synth(L, s->lnf, H, 1000, kLnF, h.seed, 4, 0.02);
  s->on_disk = (h.flags & 8) ? 1 : 0;
  const uint32_t resident = s->on_disk ? 1u : h.layers;      // on-disk mode: one working set, filled per layer from the file
  s->layers.resize(resident);
  for (uint32_t l = 0; l < resident && ok && L.ok; ++l) {
    Layer &ly = s->layers[l];
    ly.ln1 = alloc(ctx, H * 4, &ok);
    ly.wqkv = alloc(ctx, QKV * H * 4, &ok);
    ly.bqkv = alloc(ctx, QKV * 4, &ok);
    ly.wo = alloc(ctx, H * QD * 4, &ok);
    ly.ln2 = alloc(ctx, H * 4, &ok);
    ly.wgu = alloc(ctx, 2 * F * H * 4, &ok);
    ly.wdn = alloc(ctx, H * F * 4, &ok);
    ly.kcache = alloc(ctx, B * KVD * h.max_seq * 4, &ok);
    ly.vcache = alloc(ctx, B * KVD * h.max_seq * 4, &ok);
    if (!ok) break;
    if (s->on_disk) continue;
    synth(L, ly.ln1, H, l, kLn1, h.seed, 4, 0.02);
    synth(L, ly.wqkv, QKV * H, l, kWqkv, h.seed, 2, 0.02);
    synth(L, ly.bqkv, QKV, l, kBqkv, h.seed, 2, 0.02);
    synth(L, ly.wo, H * QD, l, kWo, h.seed, 2, 0.02);
    synth(L, ly.ln2, H, l, kLn2, h.seed, 4, 0.02);
    synth(L, ly.wgu, 2 * F * H, l, kWgu, h.seed, 2, 0.02);
    synth(L, ly.wdn, H * F, l, kWdn, h.seed, 2, 0.02);
  }
  if (!ok || !L.ok || cl_cuda_stream_sync(ctx, -1) != 0)
    return scope.fail(2, "load: weight generation failed: " + (L.ok ? std::string(cl_b200_last_error()) : L.err));
  {
    const int half = 32;
    std::vector<float> tab(size_t(2) * h.max_seq * half);
    for (uint32_t p = 0; p < h.max_seq; ++p)
      for (int i = 0; i < half; ++i) {
        const float inv = powf(h.rope_theta, -(float(i) / float(half)));
        const float ang = float(p) * inv;
        tab[size_t(p) * half + i] = sinf(ang);
        tab[size_t(h.max_seq) * half + size_t(p) * half + i] = cosf(ang);
      }
    s->rope = alloc(ctx, tab.size() * 4, &ok);
    if (ok) ok = cl_cuda_upload_ptr(ctx, s->rope, reinterpret_cast<const uint8_t *>(tab.data()), int64_t(tab.size() * 4)) == 0;
  }
  s->max_splits = int((h.max_seq + 127) / 128);
  s->meta = alloc(ctx, B * 8, &ok);
  s->hA = alloc(ctx, B * H * 4, &ok);
  s->hB = alloc(ctx, B * H * 4, &ok);
  s->qkv = alloc(ctx, B * QKV * 4, &ok);
  s->attn = alloc(ctx, B * QD * 4, &ok);
  s->gu = alloc(ctx, B * 2 * F * 4, &ok);
  s->part_o = alloc(ctx, B * h.n_q * uint64_t(s->max_splits) * 64 * 4, &ok);
  s->part_ml = alloc(ctx, B * h.n_q * uint64_t(s->max_splits) * 2 * 4, &ok);
  s->counters = alloc(ctx, B * h.n_kv * 4, &ok);
  s->logits = alloc(ctx, B * V * 4, &ok);
  s->next_tok = alloc(ctx, B * 4, &ok);
  s->tokens_out = alloc(ctx, uint64_t(s->max_decode) * B * 4, &ok);
  s->status = alloc(ctx, 4, &ok);
  s->am_v = alloc(ctx, B * kArgmaxParts * 4, &ok);
  s->am_i = alloc(ctx, B * kArgmaxParts * 4, &ok);
  s->am_ticket = alloc(ctx, B * 4, &ok);
  s->pin_in = cl_cuda_pinned_alloc(ctx, 64);
  s->pin_out = cl_cuda_pinned_alloc(ctx, 64);
  s->ev0 = cl_cuda_event_create(ctx);
  s->ev1 = cl_cuda_event_create(ctx);
  if (!ok || s->pin_in < 0 || s->pin_out < 0)
    return scope.fail(2, std::string("load: allocation failed: ") + cl_b200_last_error());
  scope.pinned = {s->pin_in, s->pin_out};
  scope.events = {s->ev0, s->ev1};
  scope.seal();
  s->scope = scope;
  io.set_state(s.release());
}

bool ensure_graph(State *s, B200CudaContext *ctx, std::string *err) {
  if (s->graph >= 0) return true;
  if (cl_cuda_graph_begin_capture(ctx, -1) != 0) { *err = cl_b200_last_error(); return false; }
  Launcher L{ctx, s->module};
  enqueue_step(s, L);
  const int g = cl_cuda_graph_end_capture(ctx, -1);
  if (!L.ok) { *err = L.err; if (g >= 0) cl_cuda_graph_destroy(ctx, g); return false; }
  if (g < 0) { *err = cl_b200_last_error(); return false; }
  cl_cuda_graph_upload(ctx, g, -1);
  s->graph = g;
  return true;
}

// ---- on-disk mode (the reference's qwen2_on_disk variant, lean/algorithms/Qwen2OnDiskAlgorithm.lean:18-42: one layer's
// weight buffers and one K/V pair on the device, reused by all layers; "only the storage strategy differs") ------------
// Weight file: the reference's flat f32 layout (tools/qwen2_convert.py:12-28).  Cache file: f32
// [layer][K, V][sequence][kv head][position][64], created by openFiles.
struct FlatLayout {
  uint64_t embed, layer0, per_layer, lnf, lm_head, total;            // float offsets
  uint64_t ln1, wq, bq, wk, bk, wv, bv, wo, ln2, wgate, wup, wdn;    // float offsets inside a layer
};

FlatLayout flat_layout(const QwenHeader &h) {
  const uint64_t H = h.hidden, F = h.inter, V = h.vocab, QD = uint64_t(h.n_q) * 64, KVD = uint64_t(h.n_kv) * 64;
  FlatLayout f{};
  uint64_t at = 0;
  f.ln1 = at; at += H;
  f.wq = at; at += QD * H;
  f.bq = at; at += QD;
  f.wk = at; at += KVD * H;
  f.bk = at; at += KVD;
  f.wv = at; at += KVD * H;
  f.bv = at; at += KVD;
  f.wo = at; at += H * QD;
  f.ln2 = at; at += H;
  f.wgate = at; at += F * H;
  f.wup = at; at += F * H;
  f.wdn = at; at += H * F;
  f.per_layer = at;
  f.embed = 0;
  f.layer0 = V * H;
  f.lnf = f.layer0 + uint64_t(h.layers) * f.per_layer;
  f.lm_head = f.lnf + H;
  f.total = f.lm_head + V * H;
  return f;
}

bool read_all(int fd, void *dst, uint64_t bytes, uint64_t off) {
  uint8_t *p = static_cast<uint8_t *>(dst);
  while (bytes) {
    const ssize_t n = pread(fd, p, size_t(std::min<uint64_t>(bytes, 1u << 30)), off_t(off));
    if (n <= 0) return false;
    p += n; off += uint64_t(n); bytes -= uint64_t(n);
  }
  return true;
}

bool write_all(int fd, const void *src, uint64_t bytes, uint64_t off) {
  const uint8_t *p = static_cast<const uint8_t *>(src);
  while (bytes) {
    const ssize_t n = pwrite(fd, p, size_t(bytes), off_t(off));
    if (n <= 0) return false;
    p += n; off += uint64_t(n); bytes -= uint64_t(n);
  }
  return true;
}

void close_files(State *s) {
  if (s->wfd >= 0) close(s->wfd);
  if (s->kvfd >= 0) close(s->kvfd);
  s->wfd = s->kvfd = -1;
}

// openFiles: data = "weights_path\0cache_path\0".  Checks the weight file's size against the header's shapes, loads the
// embedding (it doubles as lm_head: a file whose lm_head differs is refused) and the final norm, creates the cache file.
void stage_open_files(uint8_t *mem) {
  StageIO io(mem);
  State *s = io.state<State>();
  if (!s || !s->on_disk) return stage_fail(mem, 1, "openFiles: needs a load with flags bit 3");
  const char *d = reinterpret_cast<const char *>(io.data);
  const size_t n = size_t(io.data_len);
  const size_t l1 = n ? strnlen(d, n) : 0;
  if (l1 == 0 || l1 + 1 >= n || d[n - 1] != 0) return stage_fail(mem, 1, "openFiles: data must be two NUL-terminated paths");
  const char *wpath = d, *kvpath = d + l1 + 1;
  B200CudaContext *ctx = io.ctx();
  const QwenHeader &h = s->h;
  const FlatLayout f = flat_layout(h);
  close_files(s);
  s->wfd = open(wpath, O_RDONLY);
  if (s->wfd < 0) return stage_fail(mem, 2, std::string("openFiles: cannot open ") + wpath);
  struct stat st;
  if (fstat(s->wfd, &st) != 0 || uint64_t(st.st_size) != f.total * 4) {
    close_files(s);
    return stage_fail(mem, 1, "openFiles: the weight file's size does not match the header's shapes");
  }
  const uint64_t H = h.hidden, V = h.vocab, emb = V * H * 4;
  const uint64_t kv_bytes = uint64_t(h.layers) * 2 * h.batch * h.n_kv * h.max_seq * 64 * 4;
  s->host.resize(size_t(std::max<uint64_t>(f.per_layer * 4, 1u << 20)));
  // embedding and lm_head, a piece at a time: equal, or the file is not for this (tied) stage program
  std::vector<uint8_t> other(s->host.size());
  for (uint64_t off = 0; off < emb; off += s->host.size()) {
    const uint64_t nb = std::min<uint64_t>(s->host.size(), emb - off);
    if (!read_all(s->wfd, s->host.data(), nb, f.embed * 4 + off) || !read_all(s->wfd, other.data(), nb, f.lm_head * 4 + off)) {
      close_files(s);
      return stage_fail(mem, 2, "openFiles: short read");
    }
    if (memcmp(s->host.data(), other.data(), size_t(nb)) != 0) {
      close_files(s);
      return stage_fail(mem, 1, "openFiles: lm_head differs from embed_tokens (this stage program ties them)");
    }
    if (cl_cuda_upload_ptr_offset(ctx, s->embed, int64_t(off), s->host.data(), int64_t(nb)) != 0) {
      close_files(s);
      return stage_fail(mem, 2, std::string("openFiles: ") + cl_b200_last_error());
    }
  }
  if (!read_all(s->wfd, s->host.data(), H * 4, f.lnf * 4) || cl_cuda_upload_ptr(ctx, s->lnf, s->host.data(), int64_t(H * 4)) != 0) {
    close_files(s);
    return stage_fail(mem, 2, "openFiles: final norm");
  }
  s->kvfd = open(kvpath, O_RDWR | O_CREAT | O_TRUNC, 0600);
  if (s->kvfd < 0 || ftruncate(s->kvfd, off_t(kv_bytes)) != 0) {
    close_files(s);
    return stage_fail(mem, 2, std::string("openFiles: cannot create ") + kvpath);
  }
}

// One decode step with the weights and the cache on disk.  Nothing is captured: the host reads a layer's bytes, the
// synchronous copies (which run on the main stream, after the layer before) fill the working set, the layer's kernels
// follow, and the stream is drained before the new cache row is read back.
bool step_on_disk(State *s, B200CudaContext *ctx, std::string *err) {
  const QwenHeader &h = s->h;
  if (s->wfd < 0 || s->kvfd < 0) { *err = "openFiles has not run"; return false; }
  const FlatLayout f = flat_layout(h);
  const uint64_t H = h.hidden, F = h.inter, QD = uint64_t(h.n_q) * 64, KVD = uint64_t(h.n_kv) * 64;
  const uint64_t region = uint64_t(h.batch) * h.n_kv * h.max_seq * 64;          // floats of one layer's K (or V)
  const Layer &ws = s->layers[0];
  Launcher L{ctx, s->module};
  enqueue_head(s, L);
  float *w = reinterpret_cast<float *>(s->host.data());
  auto up = [&](int buf, uint64_t dst_floats, uint64_t src_floats, uint64_t count) {
    return cl_cuda_upload_ptr_offset(ctx, buf, int64_t(dst_floats * 4), reinterpret_cast<const uint8_t *>(w + src_floats),
                                     int64_t(count * 4)) == 0;
  };
  std::vector<float> row(64);
  for (uint32_t l = 0; l < h.layers; ++l) {
    if (!read_all(s->wfd, w, f.per_layer * 4, (f.layer0 + uint64_t(l) * f.per_layer) * 4)) { *err = "weight file: short read"; return false; }
    if (cl_cuda_stream_sync(ctx, -1) != 0) { *err = cl_b200_last_error(); return false; }     // the layer before is done with the working set
    bool ok = up(ws.ln1, 0, f.ln1, H) && up(ws.wqkv, 0, f.wq, QD * H) && up(ws.wqkv, QD * H, f.wk, KVD * H) &&
              up(ws.wqkv, (QD + KVD) * H, f.wv, KVD * H) && up(ws.bqkv, 0, f.bq, QD) && up(ws.bqkv, QD, f.bk, KVD) &&
              up(ws.bqkv, QD + KVD, f.bv, KVD) && up(ws.wo, 0, f.wo, H * QD) && up(ws.ln2, 0, f.ln2, H) &&
              up(ws.wgu, 0, f.wgate, F * H) && up(ws.wgu, F * H, f.wup, F * H) && up(ws.wdn, 0, f.wdn, H * F);
    // this layer's K/V rows of the positions before the current one
    const uint64_t kbase = uint64_t(l) * 2 * region, vbase = kbase + region;
    std::vector<float> past;
    for (uint32_t b = 0; b < h.batch && ok; ++b) {
      const uint64_t pos = uint64_t(s->next_pos[b]);
      if (pos == 0) continue;
      past.resize(size_t(pos) * 64);
      for (uint32_t kh = 0; kh < h.n_kv && ok; ++kh) {
        const uint64_t at = (uint64_t(b) * h.n_kv + kh) * h.max_seq * 64;
        ok = read_all(s->kvfd, past.data(), pos * 256, (kbase + at) * 4) &&
             cl_cuda_upload_ptr_offset(ctx, ws.kcache, int64_t(at * 4), reinterpret_cast<const uint8_t *>(past.data()), int64_t(pos * 256)) == 0 &&
             read_all(s->kvfd, past.data(), pos * 256, (vbase + at) * 4) &&
             cl_cuda_upload_ptr_offset(ctx, ws.vcache, int64_t(at * 4), reinterpret_cast<const uint8_t *>(past.data()), int64_t(pos * 256)) == 0;
      }
    }
    if (!ok) { *err = std::string("streaming layer ") + std::to_string(l) + ": " + cl_b200_last_error(); return false; }
    enqueue_layer(s, L, ws);
    if (!L.ok) { *err = L.err; return false; }
    if (cl_cuda_stream_sync(ctx, -1) != 0) { *err = cl_b200_last_error(); return false; }
    // the row this step appended goes back to the file
    for (uint32_t b = 0; b < h.batch && ok; ++b)
      for (uint32_t kh = 0; kh < h.n_kv && ok; ++kh) {
        const uint64_t at = ((uint64_t(b) * h.n_kv + kh) * h.max_seq + uint64_t(s->next_pos[b])) * 64;
        ok = cl_cuda_download_ptr_offset(ctx, ws.kcache, int64_t(at * 4), reinterpret_cast<uint8_t *>(row.data()), 256) == 0 &&
             write_all(s->kvfd, row.data(), 256, (kbase + at) * 4) &&
             cl_cuda_download_ptr_offset(ctx, ws.vcache, int64_t(at * 4), reinterpret_cast<uint8_t *>(row.data()), 256) == 0 &&
             write_all(s->kvfd, row.data(), 256, (vbase + at) * 4);
      }
    if (!ok) { *err = "cache file: write failed"; return false; }
  }
  enqueue_tail(s, L);
  if (!L.ok) { *err = L.err; return false; }
  return true;
}

void stage_prep(uint8_t *mem) {
  StageIO io(mem);
  State *s = io.state<State>();
  if (!s) return stage_fail(mem, 1, "prep: load has not run");
  if (io.data_len != uint64_t(s->h.batch) * 8) return stage_fail(mem, 1, "prep: data must be [token,pos] per sequence");
  for (uint32_t b = 0; b < s->h.batch; ++b) {
    uint32_t tok, pos;
    memcpy(&tok, io.data + 8 * b, 4);
    memcpy(&pos, io.data + 8 * b + 4, 4);
    if (tok >= s->h.vocab || pos >= s->h.max_seq) return stage_fail(mem, 1, "prep: token or position out of range");
  }
  uint8_t *pin = reinterpret_cast<uint8_t *>(cl_cuda_pinned_ptr(io.ctx(), s->pin_in));
  memcpy(pin, io.data, io.data_len);
  if (cl_cuda_upload_ptr_async(io.ctx(), s->meta, pin, int64_t(io.data_len), -1) != 0)
    return stage_fail(mem, 2, std::string("prep: upload: ") + cl_b200_last_error());
  s->next_pos.assign(s->h.batch, -1);
  for (uint32_t b = 0; b < s->h.batch; ++b) {
    uint32_t pos;
    memcpy(&pos, io.data + 8 * b + 4, 4);
    s->next_pos[b] = pos;
  }
}

// The device advances the positions itself; the host mirrors them so that a step past the end of the
// cache and of the RoPE table is refused.
bool room_for(State *s, uint32_t n, std::string *why) {
  if (s->next_pos.size() != s->h.batch) { *why = "prep has not run"; return false; }
  for (int64_t p : s->next_pos)
    if (p < 0 || p + int64_t(n) > int64_t(s->h.max_seq)) {
      *why = "position " + std::to_string(p) + " + " + std::to_string(n) + " steps is out of range (max_seq " +
             std::to_string(s->h.max_seq) + ")";
      return false;
    }
  return true;
}

void stage_infer(uint8_t *mem) {
  StageIO io(mem);
  State *s = io.state<State>();
  if (!s) return stage_fail(mem, 1, "infer: load has not run");
  B200CudaContext *ctx = io.ctx();
  if (io.data_len != 0) {
    stage_prep(mem);
    if (rd<int64_t>(mem, kOffStatus) != 0) return;
  }
  const uint64_t ob = uint64_t(s->h.batch) * 4;
  if (io.out_len != 0 && io.out_len != ob) return stage_fail(mem, 1, "infer: out must be one u32 per sequence");
  std::string err;
  if (!room_for(s, 1, &err)) return stage_fail(mem, 1, "infer: " + err);
  if (s->on_disk) {
    if (!step_on_disk(s, ctx, &err)) return stage_fail(mem, 2, "infer: " + err);
  } else {
    if (!ensure_graph(s, ctx, &err)) return stage_fail(mem, 2, "infer: graph capture: " + err);
    if (cl_cuda_graph_launch(ctx, s->graph, -1) != 0)
      return stage_fail(mem, 2, std::string("infer: graph launch: ") + cl_b200_last_error());
  }
  for (int64_t &p : s->next_pos) p += 1;
  uint8_t *pout = reinterpret_cast<uint8_t *>(cl_cuda_pinned_ptr(ctx, s->pin_out));
  cl_cuda_download_ptr_async(ctx, s->status, pout + 32, 4, -1);
  if (io.out_len) cl_cuda_download_ptr_async(ctx, s->next_tok, pout, int64_t(ob), -1);
  if (cl_cuda_stream_sync(ctx, -1) != 0) return stage_fail(mem, 3, std::string("infer: sync: ") + cl_b200_last_error());
  int32_t st;
  memcpy(&st, pout + 32, 4);
  if (st != 0) return stage_fail(mem, 4, "infer: a kernel gave up waiting for a bulk copy");
  if (io.out_len) memcpy(io.out, pout, ob);
}

void stage_decode(uint8_t *mem) {
  StageIO io(mem);
  State *s = io.state<State>();
  if (!s) return stage_fail(mem, 1, "decode: load has not run");
  B200CudaContext *ctx = io.ctx();
  uint32_t n = 0;
  if (io.data_len != 4) return stage_fail(mem, 1, "decode: data must be one u32 step count");
  memcpy(&n, io.data, 4);
  if (n == 0 || n > uint32_t(s->max_decode)) return stage_fail(mem, 1, "decode: step count out of range");
  const uint64_t tb = uint64_t(n) * s->h.batch * 4;
  if (io.out_len != 0 && io.out_len != tb && io.out_len != tb + 4)
    return stage_fail(mem, 1, "decode: out must be empty, tokens, or tokens + 4 bytes");
  std::string err;
  if (!room_for(s, n, &err)) return stage_fail(mem, 1, "decode: " + err);
  if (!s->on_disk && !ensure_graph(s, ctx, &err)) return stage_fail(mem, 2, "decode: graph capture: " + err);
  const int64_t row = int64_t(s->h.batch) * 4;
  cl_cuda_event_record(ctx, s->ev0, -1);
  for (uint32_t i = 0; i < n; ++i) {
    if (s->on_disk) {
      if (!step_on_disk(s, ctx, &err)) return stage_fail(mem, 2, "decode: " + err);
      for (int64_t &p : s->next_pos) p += 1;                 // the next step's cache rows depend on it
    } else if (cl_cuda_graph_launch(ctx, s->graph, -1) != 0) {
      return stage_fail(mem, 2, std::string("decode: launch: ") + cl_b200_last_error());
    }
    if (cl_b200_copy_async(ctx, s->tokens_out, int64_t(i) * row, s->next_tok, 0, row, -1) != 0)
      return stage_fail(mem, 2, std::string("decode: launch: ") + cl_b200_last_error());
  }
  cl_cuda_event_record(ctx, s->ev1, -1);
  if (!s->on_disk)
    for (int64_t &p : s->next_pos) p += n;
  if (cl_cuda_stream_sync(ctx, -1) != 0) return stage_fail(mem, 3, std::string("decode: sync: ") + cl_b200_last_error());
  int32_t st = 0;
  if (cl_cuda_download_ptr(ctx, s->status, reinterpret_cast<uint8_t *>(&st), 4) != 0 || st != 0)
    return stage_fail(mem, 4, "decode: a kernel gave up waiting for a bulk copy");
  if (io.out_len >= tb && cl_cuda_download_ptr(ctx, s->tokens_out, io.out, int64_t(tb)) != 0)
    return stage_fail(mem, 2, std::string("decode: download: ") + cl_b200_last_error());
  if (io.out_len == tb + 4) {
    const int32_t bits = cl_cuda_event_elapsed_ms_bits(ctx, s->ev0, s->ev1);
    memcpy(io.out + tb, &bits, 4);
  }
}

void stage_fetch_logits(uint8_t *mem) {
  StageIO io(mem);
  State *s = io.state<State>();
  if (!s) return stage_fail(mem, 1, "fetchLogits: load has not run");
  const uint64_t n = uint64_t(s->h.batch) * s->h.vocab * 4;
  if (io.out_len != n) return stage_fail(mem, 1, "fetchLogits: wrong out size");
  if (cl_cuda_download_ptr(io.ctx(), s->logits, io.out, int64_t(n)) != 0)
    return stage_fail(mem, 2, std::string("fetchLogits: ") + cl_b200_last_error());
}

// fetchTensor: data = [layer:u32][kind:u32] (layer 1000 = globals); out = raw f32 bytes.
void stage_fetch_tensor(uint8_t *mem) {
  StageIO io(mem);
  State *s = io.state<State>();
  if (!s) return stage_fail(mem, 1, "fetchTensor: load has not run");
  if (io.data_len != 8) return stage_fail(mem, 1, "fetchTensor: data must be [layer, kind]");
  uint32_t q[2];
  memcpy(q, io.data, 8);
  int buf = -1;
  if (q[0] == 1000) buf = q[1] == kEmbed ? s->embed : q[1] == kLnF ? s->lnf : -1;
  else if (q[0] < s->layers.size()) {      // on-disk mode: only the working set (layer 0) is resident
    const Layer &ly = s->layers[q[0]];
    const int t[] = {ly.ln1, ly.wqkv, ly.bqkv, ly.wo, ly.ln2, ly.wgu, ly.wdn};
    if (q[1] < 7) buf = t[q[1]];
  }
  if (buf < 0) return stage_fail(mem, 1, "fetchTensor: no such tensor");
  if (int64_t(io.out_len) != cl_b200_buffer_size(io.ctx(), buf)) return stage_fail(mem, 1, "fetchTensor: wrong out size");
  if (cl_cuda_download_ptr(io.ctx(), buf, io.out, int64_t(io.out_len)) != 0)
    return stage_fail(mem, 2, std::string("fetchTensor: ") + cl_b200_last_error());
}

// setTensor: data = [layer:u32][kind:u32] (as fetchTensor) followed by the tensor's f32 bytes in the layout fetchTensor
// returns (row-major [out][in]; wqkv = [q; k; v] rows, wgu = [gate; up] rows, the embedding doubles as lm_head): real
// weights replace the seeded ones (the reference's flat weight file, tools/qwen2_convert.py:12-28, is such tensors in a
// fixed order; base_b200/convert.py reads it).  The step's captured graph stays valid: the buffers do not move.
void stage_set_tensor(uint8_t *mem) {
  StageIO io(mem);
  State *s = io.state<State>();
  if (!s) return stage_fail(mem, 1, "setTensor: load has not run");
  if (io.data_len < 8) return stage_fail(mem, 1, "setTensor: data must be [layer, kind] + bytes");
  uint32_t q[2];
  memcpy(q, io.data, 8);
  int buf = -1;
  if (q[0] == 1000) buf = q[1] == kEmbed ? s->embed : q[1] == kLnF ? s->lnf : -1;
  else if (q[0] < s->layers.size()) {      // on-disk mode: only the working set (layer 0) is resident
    const Layer &ly = s->layers[q[0]];
    const int t[] = {ly.ln1, ly.wqkv, ly.bqkv, ly.wo, ly.ln2, ly.wgu, ly.wdn};
    if (q[1] < 7) buf = t[q[1]];
  }
  if (buf < 0) return stage_fail(mem, 1, "setTensor: no such tensor");
  const int64_t bytes = int64_t(io.data_len) - 8;
  if (bytes != cl_b200_buffer_size(io.ctx(), buf)) return stage_fail(mem, 1, "setTensor: wrong size for this tensor");
  if (cl_cuda_sync(io.ctx()) != 0 || cl_cuda_upload_ptr(io.ctx(), buf, io.data + 8, bytes) != 0)
    return stage_fail(mem, 2, std::string("setTensor: ") + cl_b200_last_error());
}

void destroy(uint8_t *mem) {
  StageIO io(mem);
  State *s = io.state<State>();
  if (s) {
    if (s->graph >= 0) s->scope.graphs.push_back(s->graph);
    close_files(s);
    s->scope.release();
    delete s;
    io.set_state(nullptr);
  }
}

struct Registrar {
  Registrar() {
    Plugin p;
    p.name = "qwen2";
    p.stages = {{"", stage_noop},       {"load", stage_load},     {"prep", stage_prep},
                {"infer", stage_infer}, {"decode", stage_decode}, {"fetchLogits", stage_fetch_logits},
                {"fetchTensor", stage_fetch_tensor}, {"setTensor", stage_set_tensor},
                {"openFiles", stage_open_files}};
    p.destroy = destroy;
    register_plugin(p);
  }
} registrar;

}  // namespace
