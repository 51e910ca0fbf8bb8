// Stage program `native:gptoss` — greedy decode of a gpt-oss-architecture
// model (MXFP4 mixture-of-experts FFN, GQA attention with sinks and an
// alternating sliding window, RoPE, RMSNorm) behind the reference's decode
// protocol: per `infer` call data = [token_id:u32][pos:u32] per sequence,
// out = [next_token:u32] per sequence (reference:
// lean/algorithms/Qwen2Common.lean:30, 830-864; one device sync per token,
// :1028-1055).  Stages follow the reference's load -> prep -> infer split
// (lean/algorithms/CudaGemvPersistAlgorithm.lean:34-100).
//
// What is different from the reference's Qwen2 program, by design:
//   * one CUDA graph per decode step, captured once and replayed (the
//     reference issues 533 launches per token from generated host code,
//     Qwen2Common.lean:1755-1756); position and token live in a device `meta`
//     buffer as in the reference (:658-671), so the graph never changes;
//   * six kernels per layer: norm+qkv GEMV, attention (RoPE, KV append,
//     split-KV, sinks), o-proj+residual, norm+router+top-k+permutation,
//     gate_up+SwiGLU, down.  The weighted combine of the experts and the
//     residual add ride in the next layer's first kernel.
//   * `decode` runs N steps with the argmax fed back on the device.
//
// Weights are synthetic (kernels/synth.cuh): `load` takes only the header.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <vector>

#include "plugin.h"

namespace {

using namespace b200;

struct GptOssHeader {
  uint32_t magic;        // 'GOS1'
  uint32_t layers, hidden, inter, experts, top_k;
  uint32_t n_q, n_kv, head_dim, vocab, window, max_seq, batch;
  float rope_theta, eps, alpha, limit;
  uint32_t seed;
  uint32_t flags;        // bit 0: programmatic dependent launch; bit 2: one f16 column per token in the experts;
                         // bit 5: the whole step as one persistent kernel (batch 1)
                         // bit 6: with bit 5, the experts run on the block-scaled tensor cores (mx tiles, moe_mx.cuh)
                         // bit 7: batched mode (up to 256 sequences per GPU): dense layers and experts on the tcgen05
                         //        tensor cores, weights read once per step for all sequences (batch_dense.cuh, batch_moe.cuh)
  uint32_t expert_lo, expert_n;   // experts resident on this rank (expert_n = 0: all)
  // Failure-path test hooks of the persistent step kernel (0 in production): 1 + the ring fill its producers
  // leave out, and the iteration limit of its waits (0: the default).  With a fill left out the consumers'
  // bounded wait runs out, the kernel stores a status code and ends, and `infer` reports it.
  uint32_t test_skip_fill, test_spin;
  // Batched mode (flags bit 7) over several GPUs: this process is rank ep_rank of ep_world (0 or 1: one GPU).
  // It holds `batch` of the ep_world * batch sequences (their KV caches; dense weights are replicated) and the
  // experts [ep_rank * experts / ep_world, ...) of every layer.
  uint32_t ep_rank, ep_world;
  uint32_t reserved[7];
};
static_assert(sizeof(GptOssHeader) == 128, "header is 128 bytes");
constexpr uint32_t kMagic = 0x31534f47;  // "GOS1"

// ---- kernel argument structs (must match the .cuh files) ---------------------------
struct MoeDims { int H, I, E, top_k, T; float alpha, limit; };
struct StreamArgs { MoeDims d; int exact, xcols, stages; };
struct RouteArgs { MoeDims d; int norm; float eps; };
struct RetileArgs { int R, K, n_mat; };
struct DequantArgs { int K, R, expert, row0, nrows; };
struct GemvArgs { int rows, K, B, top_k; float eps; int w_is_f32, prologue, in_stride, out_stride, row_iters; };
struct EmbedArgs { int H, B, is_f32, vocab; };
struct ArgmaxArgs { int V, B, stride, parts; };
struct AttnArgs {
  int NQ, NKV, HD, B, cache_len, window, max_pos, qkv_stride, has_sinks, kv_is_f32;
  float scale;
  int max_splits;
};
struct MegaArgs {
  int layers, H, I, E, top_k, NQ, NKV, V, max_seq;
  float eps, alpha, limit, attn_scale;
  int max_splits;
  int mx, kc_gu, kc_dn;
  int test_skip_fill;
  unsigned spin;
};
constexpr int kMegaThreads = 512;
constexpr int kMegaSmemBytes = 7 * 25088 + 56832;   // ring + MegaSmem (mega_decode.cuh): all 227 KB
constexpr int kMxSlotBytes = 25088;
struct RetileWideArgs { int R, K, n_mat, kc; };
struct AttnBatchArgs { int NQ, NKV, B, cache_len, window, max_pos, qkv_stride; float scale; int max_splits, S; };
constexpr int kAbThreads = 256, kAbSmemBytes = 2 * 2 * 128 * 72 * 2 + 8 * 64 * 4 + 8 * 128 * 4 + 32;
struct DenseRetileArgs { int rows, K; };
struct RowsToAArgs { int K, B, mode, n_parts; long long part_stride; float eps; };
struct DenseTcArgs { int rows, K, B, kind, m64_rows16, out_stride; };
struct ExpandArgs { int K, P, pos0, n, top_k, per_token, E; };
struct BatchMxArgs { MoeDims d; int lo, n, P; };
struct RouterManyArgs { int T, H, E; };
struct TablesManyArgs { int A, E, lo, n; };
struct CombineRangeArgs { int H, top_k, lo, n; };
struct TopkTablesArgs { MoeDims d; TablesManyArgs t; int do_topk; };
// peer_xchg.cuh: the exchange done by the kernels themselves over peer memory
constexpr int kPeerMax = 8;
struct PeerTable { unsigned long long xn_all[kPeerMax], y_recv[kPeerMax], flags[kPeerMax]; int rank, world; };
struct RowsToPeersArgs { int K, B, tag, layers; float eps; };
struct RouterPeerArgs { RouterManyArgs r; int tag, layers, per_round; };
struct CombinePeersArgs { int H, top_k, lo, n, B, tag, layers; };
struct RowsToAPeerArgs { RowsToAArgs r; int tag, layers; };
struct RetileSegArgs { int R, K, n_mat; };
constexpr int kBdThreads = 192, kBdSmemBytes = 8 * (8192 + 16 * 1024) + 64 * 129 * 4 + 512;
constexpr int kBmThreads = 192, kBmSmemBytes = 8 * (16 * (8 * 128 + 64) + 8 * 8 * 128) + 192 * 8 + 4096;
struct SynthArgs { unsigned long long n; uint32_t tensor, seed; int kind; float c; int lo, span; unsigned long long first; };

// Tensor kinds (tensor id = layer * 32 + kind; globals use layer = 1000).
enum Kind : uint32_t {
  kLn1 = 0, kWqkv, kBqkv, kSinks, kWo, kBo, kLn2, kWr, kBr, kGuCodes, kGuScales, kGuBias, kDnCodes, kDnScales,
  kDnBias, kEmbed = 16, kLmHead, kLnF
};

struct Layer {
  int ln1, wqkv, bqkv, sinks, wo, bo, ln2, wr, br;
  int gu_codes, gu_scales, gu_bias, dn_codes, dn_scales, dn_bias;
  int gu_mx = -1, dn_mx = -1;      // header flags bit 6: the wide block-scaled tensor-core layout (mxfp4_retile_wide)
  int wqkv_t = -1, wo_t = -1;      // batched mode: the dense weights tiled for the tensor cores (dense_tc_retile)
  int kcache, vcache;
  int cache_len, window;
};

struct State {
  GptOssHeader h;
  int module = -1;
  std::vector<Layer> layers;
  int embed = -1, lm_head = -1, lnf = -1, rope = -1;
  int meta = -1, hA = -1, hB = -1, qkv = -1, attn = -1, part_o = -1, part_ml = -1, counters = -1;
  int xn = -1, rlogits = -1, topk_idx = -1, topk_w = -1, route = -1, ticket = -1, act = -1, act_h = -1, o = -1;
  int logits = -1, next_tok = -1, tokens_out = -1, status = -1, zero_w = -1, scratch = -1;
  int pin_in = -1, pin_out = -1, am_v = -1, am_i = -1, am_ticket = -1;
  int graph = -1;
  int ev0 = -1, ev1 = -1;
  int max_splits = 1;
  int warps_gu = 4, warps_dn = 4, ring_stages = 2, cta_target = 100000;
  int max_decode = 4096;
  int dense_stream = 1, dense_stages = 4, dense_ctas = 296;
  int mega = 0, mega_tab = -1, mega_sync = -1, mega_am_v = -1, mega_am_i = -1, mega_grid = 0, mega_trace = -1, mega_rpart = -1, mega_mx = 0, mega_kc_gu = 8, mega_kc_dn = 8;
  // batched mode
  int batched = 0, lm_head_t = -1, a_tiled = -1, xn_all = -1, dig = -1, em = -1, y_part = -1, y_recv = -1, tiles = -1;
  int ep_rank = 0, ep_world = 1, expert_lo = 0, expert_n = 0, m64_rows16 = 1;
  int peer = 0, peer_tab = -1, xflags = -1;      // peerInit: the kernels exchange over peer memory (no NCCL in the step)
  std::vector<int64_t> peer_maps;               // addresses cl_b200_ipc_open returned
  LoadScope scope;
  int fail_after = -1;
  std::vector<int64_t> next_pos;     // per sequence: the position the next step will run at (-1: prep has not run)
};

bool synth(B200CudaContext *ctx, Launcher &L, int buf, uint64_t n, uint32_t layer, uint32_t kind, uint32_t seed,
           int gen, double sigma, int lo = 0, int span = 1, uint64_t first = 0) {
  SynthArgs a{};
  a.n = n;
  a.tensor = layer * 32 + kind;
  a.seed = seed;
  a.kind = gen;
  a.c = float(sigma / 209.0232);
  a.lo = lo;
  a.span = span;
  a.first = first;
  const int blocks = int(std::min<uint64_t>((n + 255) / 256, 148 * 32));
  L("synth_fill", {buf}, a, std::max(1, blocks), 1, 1, 256);
  (void)ctx;
  return L.ok;
}

int alloc(B200CudaContext *ctx, uint64_t bytes, bool *ok) {
  int id = cl_cuda_create_buffer(ctx, int64_t(bytes));
  if (id < 0) *ok = false;
  return id;
}

}  // namespace

#include "gptoss_impl.inc"
