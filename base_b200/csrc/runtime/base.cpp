// Runtime: Artifact readers, Base, native stage dispatch.
// Reference behaviour being mirrored: base/src/lib.rs:36-148 (Base),
// base-types/src/lib.rs:25-60 (types), py-base/src/lib.rs:126-178 (JSON).
#include "b200base.h"
#include "plugin.h"

#include <sys/mman.h>

#include <algorithm>
#include <cctype>
#include <cerrno>
#include <climits>
#include <cstdlib>
#include <map>
#include <memory>
#include <mutex>

namespace b200 {

static thread_local std::string t_error;
static void set_error(const std::string &s) { t_error = s; }

static std::vector<Plugin> &registry() {
  static std::vector<Plugin> r;
  return r;
}
void register_plugin(const Plugin &p) { registry().push_back(p); }
const Plugin *find_plugin(const std::string &name) {
  for (auto &p : registry())
    if (name == p.name) return &p;
  return nullptr;
}
const std::vector<Plugin> &all_plugins() { return registry(); }

void stage_fail(uint8_t *mem, int64_t code, const std::string &msg) {
  wr<int64_t>(mem, kOffStatus, code ? code : -1);
  set_error(msg);
}

// ---- minimal JSON reader (objects, arrays, strings, integers, bool, null) ------
struct JVal {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  bool b = false;
  double num = 0;
  int64_t inum = 0;
  uint64_t unum = 0;
  bool neg = false;
  bool is_int = false;
  std::string str;
  std::vector<JVal> arr;
  std::vector<std::pair<std::string, JVal>> obj;
  const JVal *get(const char *k) const {
    for (auto &kv : obj)
      if (kv.first == k) return &kv.second;
    return nullptr;
  }
};

struct JParser {
  const char *p, *end;
  std::string err;
  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool fail(const char *m) { if (err.empty()) err = m; return false; }
  bool parse_string(std::string &out) {
    if (p >= end || *p != '"') return fail("expected string");
    ++p;
    while (p < end && *p != '"') {
      if (*p == '\\') {
        if (++p >= end) return fail("bad escape");
        switch (*p) {
          case 'n': out.push_back('\n'); break;
          case 't': out.push_back('\t'); break;
          case 'r': out.push_back('\r'); break;
          case 'b': out.push_back('\b'); break;
          case 'f': out.push_back('\f'); break;
          case 'u': {
            if (end - p < 5) return fail("bad \\u escape");
            unsigned cp = unsigned(strtoul(std::string(p + 1, p + 5).c_str(), nullptr, 16));
            p += 4;
            if (cp < 0x80) out.push_back(char(cp));
            else if (cp < 0x800) { out.push_back(char(0xC0 | (cp >> 6))); out.push_back(char(0x80 | (cp & 0x3F))); }
            else { out.push_back(char(0xE0 | (cp >> 12))); out.push_back(char(0x80 | ((cp >> 6) & 0x3F))); out.push_back(char(0x80 | (cp & 0x3F))); }
            break;
          }
          default: out.push_back(*p);
        }
        ++p;
      } else {
        out.push_back(*p++);
      }
    }
    if (p >= end) return fail("unterminated string");
    ++p;
    return true;
  }
  // Containers nest at most kMaxDepth deep (an artifact needs 5): the parser recurses once per level.
  static constexpr int kMaxDepth = 64;
  int depth = 0;
  bool parse(JVal &v) {
    if (depth >= kMaxDepth) return fail("nesting too deep");
    ++depth;
    const bool ok = parse_inner(v);
    --depth;
    return ok;
  }
  bool parse_inner(JVal &v) {
    ws();
    if (p >= end) return fail("unexpected end");
    char c = *p;
    if (c == '{') {
      v.kind = JVal::Obj;
      ++p; ws();
      if (p < end && *p == '}') { ++p; return true; }
      while (true) {
        ws();
        std::string k;
        if (!parse_string(k)) return false;
        ws();
        if (p >= end || *p != ':') return fail("expected ':'");
        ++p;
        JVal child;
        if (!parse(child)) return false;
        v.obj.emplace_back(std::move(k), std::move(child));
        ws();
        if (p < end && *p == ',') { ++p; continue; }
        if (p < end && *p == '}') { ++p; return true; }
        return fail("expected ',' or '}'");
      }
    }
    if (c == '[') {
      v.kind = JVal::Arr;
      ++p; ws();
      if (p < end && *p == ']') { ++p; return true; }
      while (true) {
        JVal child;
        if (!parse(child)) return false;
        v.arr.push_back(std::move(child));
        ws();
        if (p < end && *p == ',') { ++p; continue; }
        if (p < end && *p == ']') { ++p; return true; }
        return fail("expected ',' or ']'");
      }
    }
    if (c == '"') { v.kind = JVal::Str; return parse_string(v.str); }
    if (!strncmp(p, "true", std::min<size_t>(4, end - p)) && end - p >= 4) { v.kind = JVal::Bool; v.b = true; p += 4; return true; }
    if (!strncmp(p, "false", std::min<size_t>(5, end - p)) && end - p >= 5) { v.kind = JVal::Bool; v.b = false; p += 5; return true; }
    if (!strncmp(p, "null", std::min<size_t>(4, end - p)) && end - p >= 4) { v.kind = JVal::Null; p += 4; return true; }
    if (c == '-' || isdigit((unsigned char)c)) {
      const char *s = p;
      bool is_int = true;
      if (*p == '-') ++p;
      while (p < end && (isdigit((unsigned char)*p) || *p == '.' || *p == 'e' || *p == 'E' || *p == '+' || *p == '-')) {
        if (*p == '.' || *p == 'e' || *p == 'E') is_int = false;
        ++p;
      }
      std::string t(s, p);
      v.kind = JVal::Num;
      v.is_int = is_int;
      v.num = strtod(t.c_str(), nullptr);
      if (is_int) {
        // unsigned fields (memory_size, offsets) may exceed 2^63 - 1: keep the exact value or reject
        errno = 0;
        if (t[0] == '-') { v.inum = strtoll(t.c_str(), nullptr, 10); v.neg = true; }
        else v.unum = strtoull(t.c_str(), nullptr, 10);
        if (errno == ERANGE) return fail("integer out of range");
        if (!v.neg) v.inum = v.unum > uint64_t(INT64_MAX) ? INT64_MAX : int64_t(v.unum);
      }
      return true;
    }
    return fail("unexpected character");
  }
};

}  // namespace b200

using namespace b200;

struct AlgorithmRec { uint32_t fn_idx = 0; };

struct B200Artifact {
  std::string cranelift_ir;
  uint64_t memory_size = 0;
  uint64_t io[4] = {0, 0, 0, 0};
  std::vector<uint8_t> initial_memory;
  AlgorithmRec main;
  std::vector<std::pair<std::string, AlgorithmRec>> extras;
};

struct B200Base {
  uint8_t *mem = nullptr;
  uint64_t mem_len = 0;
  uint64_t io[4];
  const Plugin *plugin = nullptr;   // null: no functions
  bool locked = false;
  std::mutex mu;
};

namespace {

bool get_u64(const JVal *v, uint64_t *out) {
  if (!v || v->kind != JVal::Num || !v->is_int || v->neg) return false;
  *out = v->unum;
  return true;
}

bool parse_algorithm(const JVal *v, AlgorithmRec *a, std::string *err) {
  if (!v || v->kind != JVal::Obj) { *err = "algorithm: expected object"; return false; }
  uint64_t idx;
  if (!get_u64(v->get("fn_idx"), &idx) || idx > 0xffffffffull) { *err = "algorithm: missing or invalid fn_idx"; return false; }
  const JVal *o = v->get("output");
  if (!o || o->kind != JVal::Arr) { *err = "algorithm: missing field `output`"; return false; }
  a->fn_idx = uint32_t(idx);
  return true;
}

// bincode 1.x default options: little-endian fixed ints, u64 lengths.
struct BinReader {
  const uint8_t *p, *end;
  bool ok = true;
  uint64_t u64() { if (end - p < 8) { ok = false; return 0; } uint64_t v; memcpy(&v, p, 8); p += 8; return v; }
  uint32_t u32() { if (end - p < 4) { ok = false; return 0; } uint32_t v; memcpy(&v, p, 4); p += 4; return v; }
  bool bytes(uint64_t n, const uint8_t **out) { if (uint64_t(end - p) < n) { ok = false; return false; } *out = p; p += n; return true; }
  std::string str() { uint64_t n = u64(); const uint8_t *s; if (!ok || !bytes(n, &s)) return ""; return std::string(reinterpret_cast<const char *>(s), n); }
  void skip_output() {  // Vec<OutputBatchSchema>
    uint64_t nb = u64();
    for (uint64_t i = 0; ok && i < nb; ++i) {
      uint64_t nc = u64();
      for (uint64_t j = 0; ok && j < nc; ++j) { str(); u32(); u64(); u64(); }
      u64();
    }
  }
};

}  // namespace

extern "C" {

const char *b200_last_error(void) { return t_error.c_str(); }

B200Artifact *b200_artifact_from_json(const char *text, uint64_t len) {
  if (!text) { set_error("null text"); return nullptr; }
  JParser jp{text, text + len, ""};
  JVal root;
  if (!jp.parse(root) || root.kind != JVal::Obj) { set_error("artifact JSON: " + (jp.err.empty() ? std::string("expected object") : jp.err)); return nullptr; }
  std::unique_ptr<B200Artifact> a(new B200Artifact());
  const JVal *setup = root.get("setup");
  if (!setup || setup->kind != JVal::Obj) { set_error("artifact JSON: missing field `setup`"); return nullptr; }
  const JVal *ir = setup->get("cranelift_ir");
  if (!ir || ir->kind != JVal::Str) { set_error("setup: missing field `cranelift_ir`"); return nullptr; }
  a->cranelift_ir = ir->str;
  if (!get_u64(setup->get("memory_size"), &a->memory_size)) { set_error("setup: missing field `memory_size`"); return nullptr; }
  const JVal *io = setup->get("io_offsets");
  if (!io || io->kind != JVal::Obj) { set_error("setup: missing field `io_offsets`"); return nullptr; }
  const char *names[4] = {"data_ptr", "data_len", "out_ptr", "out_len"};
  for (int i = 0; i < 4; ++i)
    if (!get_u64(io->get(names[i]), &a->io[i])) { set_error(std::string("io_offsets: missing field `") + names[i] + "`"); return nullptr; }
  if (const JVal *im = setup->get("initial_memory")) {
    if (im->kind != JVal::Arr) { set_error("setup: initial_memory must be an array of bytes"); return nullptr; }
    a->initial_memory.reserve(im->arr.size());
    for (auto &e : im->arr) {
      if (e.kind != JVal::Num || !e.is_int || e.inum < 0 || e.inum > 255) { set_error("setup: initial_memory element out of range"); return nullptr; }
      a->initial_memory.push_back(uint8_t(e.inum));
    }
  }
  std::string err;
  if (!parse_algorithm(root.get("main"), &a->main, &err)) { set_error("main: " + err); return nullptr; }
  if (const JVal *ex = root.get("extras")) {
    if (ex->kind != JVal::Obj) { set_error("extras: expected object"); return nullptr; }
    for (auto &kv : ex->obj) {
      AlgorithmRec r;
      if (!parse_algorithm(&kv.second, &r, &err)) { set_error("extras." + kv.first + ": " + err); return nullptr; }
      a->extras.emplace_back(kv.first, r);
    }
  }
  return a.release();
}

B200Artifact *b200_artifact_from_bytes(const uint8_t *bytes, uint64_t len) {
  if (!bytes) { set_error("null bytes"); return nullptr; }
  BinReader r{bytes, bytes + len};
  std::unique_ptr<B200Artifact> a(new B200Artifact());
  a->cranelift_ir = r.str();
  a->memory_size = r.u64();
  for (int i = 0; i < 4; ++i) a->io[i] = r.u64();
  uint64_t n = r.u64();
  const uint8_t *im = nullptr;
  if (r.ok && r.bytes(n, &im)) a->initial_memory.assign(im, im + n);
  a->main.fn_idx = r.u32();
  r.skip_output();
  uint64_t ne = r.u64();
  for (uint64_t i = 0; r.ok && i < ne; ++i) {
    std::string k = r.str();
    AlgorithmRec rec;
    rec.fn_idx = r.u32();
    r.skip_output();
    a->extras.emplace_back(k, rec);
  }
  if (!r.ok) { set_error("failed to deserialize artifact (truncated bincode)"); return nullptr; }
  return a.release();
}

void b200_artifact_free(B200Artifact *a) { delete a; }
const char *b200_artifact_cranelift_ir(const B200Artifact *a) { return a ? a->cranelift_ir.c_str() : ""; }
uint64_t b200_artifact_memory_size(const B200Artifact *a) { return a ? a->memory_size : 0; }
void b200_artifact_io_offsets(const B200Artifact *a, uint64_t out[4]) { if (a) memcpy(out, a->io, 32); }
const uint8_t *b200_artifact_initial_memory(const B200Artifact *a, uint64_t *len) {
  if (!a) { if (len) *len = 0; return nullptr; }
  if (len) *len = a->initial_memory.size();
  return a->initial_memory.data();
}
uint32_t b200_artifact_main_fn(const B200Artifact *a) { return a ? a->main.fn_idx : 0; }
uint32_t b200_artifact_extras_count(const B200Artifact *a) { return a ? uint32_t(a->extras.size()) : 0; }
const char *b200_artifact_extra_name(const B200Artifact *a, uint32_t i) {
  return (a && i < a->extras.size()) ? a->extras[i].first.c_str() : "";
}
uint32_t b200_artifact_extra_fn(const B200Artifact *a, uint32_t i) {
  return (a && i < a->extras.size()) ? a->extras[i].second.fn_idx : 0;
}

B200Base *b200_base_new(const char *cranelift_ir, uint64_t memory_size, const uint64_t io_offsets[4],
                        const uint8_t *initial_memory, uint64_t initial_len, int32_t *err_kind) {
  auto fail = [&](int32_t kind, const std::string &m) -> B200Base * {
    if (err_kind) *err_kind = kind;
    set_error(m);
    return nullptr;
  };
  if (err_kind) *err_kind = B200_OK;
  if (!io_offsets) return fail(B200_ERR_EXECUTION, "null io_offsets");
  std::string ir = cranelift_ir ? cranelift_ir : "";
  const Plugin *plugin = nullptr;
  if (!ir.empty()) {
    // trim
    size_t b = ir.find_first_not_of(" \t\r\n"), e = ir.find_last_not_of(" \t\r\n");
    std::string t = (b == std::string::npos) ? "" : ir.substr(b, e - b + 1);
    if (t.rfind("native:", 0) != 0)
      return fail(B200_ERR_CLIF_PARSE,
                  "cranelift_ir is CLIF text; this runtime has no Cranelift and accepts only "
                  "\"\" or \"native:<plugin>\"");
    plugin = find_plugin(t.substr(7));
    if (!plugin) return fail(B200_ERR_CLIF_PARSE, "unknown native plugin `" + t.substr(7) + "`");
    if (io_offsets[0] != kOffDataPtr || io_offsets[1] != kOffDataLen || io_offsets[2] != kOffOutPtr ||
        io_offsets[3] != kOffOutLen)
      return fail(B200_ERR_CLIF_PARSE, "native plugins require io_offsets 0x18/0x20/0x28/0x30");
  }
  uint64_t header_end = io_offsets[3] + 8;
  if (header_end < io_offsets[3]) header_end = UINT64_MAX;  // saturating, base/src/lib.rs:37-40
  uint64_t needed = std::max(std::max(memory_size, initial_len), header_end);
  if (plugin) needed = std::max(needed, kMinNativeMemory);
  // The reference aborts when such a resize cannot be served (base/src/lib.rs:36-52); here it is an error.
  // The cap also keeps the rounding below from wrapping.
  if (needed > (uint64_t(1) << 40)) return fail(B200_ERR_EXECUTION, "memory_size beyond 1 TiB");
  for (int i = 0; i < 4; ++i)
    if (io_offsets[i] > needed - 8) return fail(B200_ERR_EXECUTION, "io offset outside memory");
  // Page-locked for the life of the Base, like the reference's pinned box.
  uint8_t *mem = static_cast<uint8_t *>(aligned_alloc(64, (needed + 63) / 64 * 64));
  if (!mem) return fail(B200_ERR_EXECUTION, "out of host memory");
  memset(mem, 0, (needed + 63) / 64 * 64);
  if (initial_len && initial_memory) memcpy(mem, initial_memory, initial_len);
  B200Base *base = new B200Base();
  base->mem = mem;
  base->mem_len = needed;
  memcpy(base->io, io_offsets, 32);
  base->plugin = plugin;
  base->locked = mlock(mem, needed) == 0;
  return base;
}

B200Base *b200_base_from_artifact(const B200Artifact *a, int32_t *err_kind) {
  if (!a) { if (err_kind) *err_kind = B200_ERR_EXECUTION; set_error("null artifact"); return nullptr; }
  return b200_base_new(a->cranelift_ir.c_str(), a->memory_size, a->io, a->initial_memory.data(),
                       a->initial_memory.size(), err_kind);
}

void b200_base_free(B200Base *base) {
  if (!base) return;
  if (base->plugin && base->plugin->destroy) base->plugin->destroy(base->mem);
  if (base->locked) munlock(base->mem, base->mem_len);
  free(base->mem);
  delete base;
}

int32_t b200_base_execute_into(B200Base *base, uint32_t fn_idx, const uint8_t *data, uint64_t data_len,
                               uint8_t *out, uint64_t out_len) {
  if (!base) { set_error("null base"); return B200_ERR_EXECUTION; }
  std::lock_guard<std::mutex> g(base->mu);   // `&mut self` in the reference
  wr<uint64_t>(base->mem, base->io[0], reinterpret_cast<uint64_t>(data));
  wr<uint64_t>(base->mem, base->io[1], data_len);
  wr<uint64_t>(base->mem, base->io[2], reinterpret_cast<uint64_t>(out));
  wr<uint64_t>(base->mem, base->io[3], out_len);
  if (base->plugin) {
    if (fn_idx >= base->plugin->stages.size()) {
      set_error("fn_idx " + std::to_string(fn_idx) + " out of range (have " +
                std::to_string(base->plugin->stages.size()) + " fns)");
      return B200_ERR_EXECUTION;
    }
    wr<int64_t>(base->mem, kOffStatus, 0);
    base->plugin->stages[fn_idx].fn(base->mem);
    int64_t st = rd<int64_t>(base->mem, kOffStatus);
    if (st != 0) {
      set_error("stage `" + std::string(base->plugin->stages[fn_idx].name) + "` failed (" +
                std::to_string(st) + "): " + t_error);
      return B200_ERR_EXECUTION;
    }
  }
  return B200_OK;
}

uint8_t *b200_base_memory(B200Base *base, uint64_t *len) {
  if (!base) { if (len) *len = 0; return nullptr; }
  if (len) *len = base->mem_len;
  return base->mem;
}

uint32_t b200_base_fn_count(B200Base *base) {
  return (base && base->plugin) ? uint32_t(base->plugin->stages.size()) : 0;
}

uint32_t b200_plugin_count(void) { return uint32_t(all_plugins().size()); }
const char *b200_plugin_name(uint32_t i) { return i < all_plugins().size() ? all_plugins()[i].name : ""; }
uint32_t b200_plugin_fn_count(const char *plugin) {
  const Plugin *p = plugin ? find_plugin(plugin) : nullptr;
  return p ? uint32_t(p->stages.size()) : 0;
}
const char *b200_plugin_fn_name(const char *plugin, uint32_t fn_idx) {
  const Plugin *p = plugin ? find_plugin(plugin) : nullptr;
  return (p && fn_idx < p->stages.size()) ? p->stages[fn_idx].name : "";
}

}  // extern "C"
