// Error slot, JSON parser, safetensors reader, config loading and weight validation (host only).
#include <cerrno>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>

#include "common.h"

namespace pg {

static thread_local std::string g_error;

int set_error(int code, const std::string& msg) {
  g_error = msg;
  return code;
}
void clear_error() { g_error.clear(); }
const char* last_error_cstr() { return g_error.c_str(); }

// ------------------------------------------------------------------ JSON
const Json* Json::get(const std::string& key) const {
  if (kind != Object) return nullptr;
  for (auto& kv : obj)
    if (kv.first == key) return &kv.second;
  return nullptr;
}

namespace {
struct Parser {
  const char* p;
  const char* end;
  std::string err;
  int depth = 0;

  void ws() {
    while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
  }
  bool fail(const std::string& m) {
    if (err.empty()) err = m;
    return false;
  }
  bool lit(const char* s) {
    size_t n = strlen(s);
    if ((size_t)(end - p) < n || memcmp(p, s, n) != 0) return fail(std::string("expected ") + s);
    p += n;
    return true;
  }
  static void utf8(std::string& o, unsigned cp) {
    if (cp < 0x80) o += (char)cp;
    else if (cp < 0x800) { o += (char)(0xC0 | (cp >> 6)); o += (char)(0x80 | (cp & 0x3F)); }
    else if (cp < 0x10000) {
      o += (char)(0xE0 | (cp >> 12)); o += (char)(0x80 | ((cp >> 6) & 0x3F)); o += (char)(0x80 | (cp & 0x3F));
    } else {
      o += (char)(0xF0 | (cp >> 18)); o += (char)(0x80 | ((cp >> 12) & 0x3F));
      o += (char)(0x80 | ((cp >> 6) & 0x3F)); o += (char)(0x80 | (cp & 0x3F));
    }
  }
  bool hex4(unsigned* out) {
    if (end - p < 4) return fail("short \\u escape");
    unsigned v = 0;
    for (int i = 0; i < 4; ++i) {
      char c = *p++;
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else return fail("bad \\u escape");
    }
    *out = v;
    return true;
  }
  bool string(std::string* out) {
    if (p >= end || *p != '"') return fail("expected string");
    ++p;
    while (p < end && *p != '"') {
      if (*p == '\\') {
        ++p;
        if (p >= end) return fail("bad escape");
        char c = *p++;
        switch (c) {
          case '"': *out += '"'; break;
          case '\\': *out += '\\'; break;
          case '/': *out += '/'; break;
          case 'b': *out += '\b'; break;
          case 'f': *out += '\f'; break;
          case 'n': *out += '\n'; break;
          case 'r': *out += '\r'; break;
          case 't': *out += '\t'; break;
          case 'u': {
            unsigned cp;
            if (!hex4(&cp)) return false;
            if (cp >= 0xD800 && cp < 0xDC00 && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {
              p += 2;
              unsigned lo;
              if (!hex4(&lo)) return false;
              cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            }
            utf8(*out, cp);
            break;
          }
          default: return fail("bad escape");
        }
      } else {
        *out += *p++;
      }
    }
    if (p >= end) return fail("unterminated string");
    ++p;
    return true;
  }
  bool value(Json* out) {
    if (++depth > 64) return fail("nesting too deep");
    ws();
    if (p >= end) return fail("unexpected end of input");
    bool ok = true;
    char c = *p;
    if (c == '{') {
      out->kind = Json::Object;
      ++p;
      ws();
      if (p < end && *p == '}') { ++p; }
      else {
        for (;;) {
          ws();
          std::string key;
          if (!string(&key)) { ok = false; break; }
          ws();
          if (p >= end || *p != ':') { ok = fail("expected ':'"); break; }
          ++p;
          Json v;
          if (!value(&v)) { ok = false; break; }
          out->obj.emplace_back(std::move(key), std::move(v));
          ws();
          if (p < end && *p == ',') { ++p; continue; }
          if (p < end && *p == '}') { ++p; break; }
          ok = fail("expected ',' or '}'");
          break;
        }
      }
    } else if (c == '[') {
      out->kind = Json::Array;
      ++p;
      ws();
      if (p < end && *p == ']') { ++p; }
      else {
        for (;;) {
          Json v;
          if (!value(&v)) { ok = false; break; }
          out->arr.push_back(std::move(v));
          ws();
          if (p < end && *p == ',') { ++p; continue; }
          if (p < end && *p == ']') { ++p; break; }
          ok = fail("expected ',' or ']'");
          break;
        }
      }
    } else if (c == '"') {
      out->kind = Json::String;
      ok = string(&out->str);
    } else if (c == 't') {
      out->kind = Json::Bool; out->b = true; ok = lit("true");
    } else if (c == 'f') {
      out->kind = Json::Bool; out->b = false; ok = lit("false");
    } else if (c == 'n') {
      out->kind = Json::Null; ok = lit("null");
    } else if (c == '-' || (c >= '0' && c <= '9')) {
      const char* s = p;
      bool integer = true;
      if (*p == '-') ++p;
      while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '+' || *p == '-')) {
        if (*p == '.' || *p == 'e' || *p == 'E') integer = false;
        ++p;
      }
      std::string tok(s, p);
      char* e = nullptr;
      out->kind = Json::Number;
      out->num = strtod(tok.c_str(), &e);
      out->num_is_integer = integer;
      if (e == tok.c_str() || *e != 0) ok = fail("bad number '" + tok + "'");
    } else {
      ok = fail(std::string("unexpected character '") + c + "'");
    }
    --depth;
    return ok;
  }
};
}  // namespace

bool parse_json(const char* data, size_t len, Json* out, std::string* err) {
  Parser ps{data, data + len, {}, 0};
  if (!ps.value(out)) {
    if (err) *err = ps.err + " at byte " + std::to_string(ps.p - data);
    return false;
  }
  ps.ws();
  if (ps.p != ps.end) {
    if (err) *err = "trailing characters at byte " + std::to_string(ps.p - data);
    return false;
  }
  return true;
}

// ------------------------------------------------------------------ safetensors
static bool read_file(const std::string& path, std::vector<uint8_t>* out, std::string* err) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) {
    *err = std::string(strerror(errno));
    return false;
  }
  fseek(f, 0, SEEK_END);
  long n = ftell(f);
  fseek(f, 0, SEEK_SET);
  if (n < 0) {
    fclose(f);
    *err = "cannot size file";
    return false;
  }
  out->resize((size_t)n);
  size_t got = n ? fread(out->data(), 1, (size_t)n, f) : 0;
  fclose(f);
  if (got != (size_t)n) {
    *err = "short read";
    return false;
  }
  return true;
}

static uint64_t dtype_size(const std::string& d) {
  if (d == "F64" || d == "I64" || d == "U64") return 8;
  if (d == "F32" || d == "I32" || d == "U32") return 4;
  if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 2;
  if (d == "I8" || d == "U8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2") return 1;
  return 0;
}

int read_safetensors(const std::string& path, SafeTensorsFile* out) {
  std::string err;
  if (!read_file(path, &out->bytes, &err))
    return set_error(PG_ASSET, "failed to read safetensors file " + path + ": " + err);
  auto bad = [&](const std::string& m) {
    return set_error(PG_ASSET, "failed to parse safetensors file " + path + ": " + m);
  };
  const auto& b = out->bytes;
  if (b.size() < 8) return bad("header too small");
  uint64_t n = 0;
  for (int i = 7; i >= 0; --i) n = (n << 8) | b[i];
  if (n > 100000000ULL) return bad("header too large");
  if (n > b.size() - 8) return bad("invalid header length");
  Json hdr;
  if (!parse_json((const char*)b.data() + 8, (size_t)n, &hdr, &err)) return bad("invalid header: " + err);
  if (hdr.kind != Json::Object) return bad("header is not an object");
  out->data_start = 8 + (size_t)n;
  uint64_t data_len = b.size() - out->data_start;
  for (auto& kv : hdr.obj) {
    if (kv.first == "__metadata__") continue;
    const Json& t = kv.second;
    const Json *dt = t.get("dtype"), *sh = t.get("shape"), *off = t.get("data_offsets");
    if (!dt || dt->kind != Json::String || !sh || sh->kind != Json::Array || !off ||
        off->kind != Json::Array || off->arr.size() != 2)
      return bad("invalid tensor entry " + kv.first);
    TensorEntry e;
    e.dtype = dt->str;
    uint64_t count = 1;
    for (auto& d : sh->arr) {
      if (d.kind != Json::Number || d.num < 0) return bad("invalid shape for " + kv.first);
      e.shape.push_back((uint64_t)d.num);
      count *= (uint64_t)d.num;
    }
    e.begin = (uint64_t)off->arr[0].num;
    e.end = (uint64_t)off->arr[1].num;
    if (e.begin > e.end || e.end > data_len) return bad("invalid offsets for tensor " + kv.first);
    uint64_t es = dtype_size(e.dtype);
    if (es == 0) return bad("unknown dtype " + e.dtype + " for tensor " + kv.first);
    if (count * es != e.end - e.begin) return bad("tensor " + kv.first + " byte length does not match its shape");
    out->tensors.emplace(kv.first, std::move(e));
  }
  return PG_OK;
}

// ------------------------------------------------------------------ config
int validate_config(const pg_gpt2_config& c) {
  if (c.vocab_size == 0) return set_error(PG_INVALID_CONFIG, "vocab_size must be > 0");
  if (c.n_positions == 0) return set_error(PG_INVALID_CONFIG, "n_positions must be > 0");
  if (c.n_embd == 0) return set_error(PG_INVALID_CONFIG, "n_embd must be > 0");
  if (c.n_layer == 0) return set_error(PG_INVALID_CONFIG, "n_layer must be > 0");
  if (c.n_head == 0) return set_error(PG_INVALID_CONFIG, "n_head must be > 0");
  if (c.n_inner == 0) return set_error(PG_INVALID_CONFIG, "n_inner must be > 0");
  if (c.n_embd % c.n_head != 0)
    return set_error(PG_INVALID_CONFIG, "n_embd " + std::to_string(c.n_embd) +
                                            " must be divisible by n_head " + std::to_string(c.n_head));
  if (!(c.layer_norm_epsilon > 0.0f)) return set_error(PG_INVALID_CONFIG, "layer_norm_epsilon must be > 0");
  return PG_OK;
}

int load_config_json(const std::string& path, pg_gpt2_config* out) {
  std::vector<uint8_t> bytes;
  std::string err;
  if (!read_file(path, &bytes, &err))
    return set_error(PG_ASSET, "failed to read config file " + path + ": " + err);
  Json j;
  if (!parse_json((const char*)bytes.data(), bytes.size(), &j, &err) || j.kind != Json::Object)
    return set_error(PG_ASSET, "failed to parse config file " + path + ": " + (err.empty() ? "not an object" : err));
  auto req = [&](const char* key, uint64_t* v) -> int {
    const Json* f = j.get(key);
    if (!f || f->kind != Json::Number || f->num < 0 || !f->num_is_integer)
      return set_error(PG_ASSET, "failed to parse config file " + path + ": missing field `" + key + "`");
    *v = (uint64_t)f->num;
    return PG_OK;
  };
  auto opt = [&](const char* key, uint64_t* v, bool* present) -> int {
    const Json* f = j.get(key);
    *present = false;
    if (!f || f->kind == Json::Null) return PG_OK;
    if (f->kind != Json::Number || f->num < 0 || !f->num_is_integer)
      return set_error(PG_ASSET, "failed to parse config file " + path + ": invalid field `" + key + "`");
    *v = (uint64_t)f->num;
    *present = true;
    return PG_OK;
  };
  pg_gpt2_config c{};
  if (int r = req("vocab_size", &c.vocab_size)) return r;
  if (int r = req("n_embd", &c.n_embd)) return r;
  if (int r = req("n_layer", &c.n_layer)) return r;
  if (int r = req("n_head", &c.n_head)) return r;
  bool has_pos = false, has_ctx = false, has_inner = false;
  uint64_t n_ctx = 0;
  if (int r = opt("n_positions", &c.n_positions, &has_pos)) return r;
  if (int r = opt("n_ctx", &n_ctx, &has_ctx)) return r;
  if (!has_pos) {
    if (!has_ctx) return set_error(PG_INVALID_CONFIG, "config must contain n_positions or n_ctx");
    c.n_positions = n_ctx;
  }
  c.n_inner = 4 * c.n_embd;
  uint64_t inner = 0;
  if (int r = opt("n_inner", &inner, &has_inner)) return r;
  if (has_inner) c.n_inner = inner;
  c.layer_norm_epsilon = 1e-5f;
  if (const Json* e = j.get("layer_norm_epsilon")) {
    if (e->kind == Json::Number) c.layer_norm_epsilon = (float)e->num;
    else if (e->kind != Json::Null)
      return set_error(PG_ASSET, "failed to parse config file " + path + ": invalid field `layer_norm_epsilon`");
  }
  if (int r = validate_config(c)) return r;
  *out = c;
  return PG_OK;
}

// ------------------------------------------------------------------ weights
static const char* kBlockFields[12] = {"ln_1_g", "ln_1_b", "c_attn_w", "c_attn_b", "c_proj_w", "c_proj_b",
                                       "ln_2_g", "ln_2_b", "c_fc_w", "c_fc_b", "c_proj_mlp_w", "c_proj_mlp_b"};

static int expect_len(const std::string& name, uint64_t actual, uint64_t expected) {
  if (actual != expected)
    return set_error(PG_INVALID_WEIGHTS, name + " len " + std::to_string(actual) +
                                             " does not match expected " + std::to_string(expected));
  return PG_OK;
}

int validate_weight_lens(const pg_gpt2_config& cfg, const uint64_t* lens, uint64_t n) {
  uint64_t c = cfg.n_embd, f = cfg.n_inner, L = cfg.n_layer;
  if (n < PG_GLOBAL_TENSORS)
    return set_error(PG_INVALID_WEIGHTS, "blocks len 0 does not match n_layer " + std::to_string(L));
  if (int r = expect_len("wte", lens[0], cfg.vocab_size * c)) return r;
  if (int r = expect_len("wpe", lens[1], cfg.n_positions * c)) return r;
  if (int r = expect_len("ln_f_g", lens[2], c)) return r;
  if (int r = expect_len("ln_f_b", lens[3], c)) return r;
  uint64_t nb = (n - PG_GLOBAL_TENSORS) / PG_TENSORS_PER_LAYER;
  if (nb != L || (n - PG_GLOBAL_TENSORS) % PG_TENSORS_PER_LAYER != 0)
    return set_error(PG_INVALID_WEIGHTS, "blocks len " + std::to_string(nb) + " does not match n_layer " + std::to_string(L));
  for (uint64_t i = 0; i < L; ++i) {
    uint64_t expect[12] = {c, c, c * 3 * c, 3 * c, c * c, c, c, c, c * f, f, f * c, c};
    for (int k = 0; k < 12; ++k)
      if (int r = expect_len("blocks[" + std::to_string(i) + "]." + kBlockFields[k], lens[4 + 12 * i + k], expect[k]))
        return r;
  }
  return PG_OK;
}

static std::string shape_str(const std::vector<uint64_t>& s) {
  std::string o = "[";
  for (size_t i = 0; i < s.size(); ++i) o += (i ? ", " : "") + std::to_string(s[i]);
  return o + "]";
}

int load_weights_safetensors(const std::string& path, const pg_gpt2_config& cfg, HostWeights* out) {
  auto file = std::make_shared<SafeTensorsFile>();
  if (int r = read_safetensors(path, file.get())) return r;
  uint64_t c = cfg.n_embd, f = cfg.n_inner;
  struct Want { std::string name; std::vector<uint64_t> shape; };
  std::vector<Want> wants = {{"wte.weight", {cfg.vocab_size, c}}, {"wpe.weight", {cfg.n_positions, c}},
                             {"ln_f.weight", {c}}, {"ln_f.bias", {c}}};
  for (uint64_t i = 0; i < cfg.n_layer; ++i) {
    std::string p = "h." + std::to_string(i) + ".";
    wants.push_back({p + "ln_1.weight", {c}});
    wants.push_back({p + "ln_1.bias", {c}});
    wants.push_back({p + "attn.c_attn.weight", {c, 3 * c}});
    wants.push_back({p + "attn.c_attn.bias", {3 * c}});
    wants.push_back({p + "attn.c_proj.weight", {c, c}});
    wants.push_back({p + "attn.c_proj.bias", {c}});
    wants.push_back({p + "ln_2.weight", {c}});
    wants.push_back({p + "ln_2.bias", {c}});
    wants.push_back({p + "mlp.c_fc.weight", {c, f}});
    wants.push_back({p + "mlp.c_fc.bias", {f}});
    wants.push_back({p + "mlp.c_proj.weight", {f, c}});
    wants.push_back({p + "mlp.c_proj.bias", {c}});
  }
  out->ptrs.clear();
  out->lens.clear();
  out->owned.clear();
  out->owned.reserve(wants.size());
  for (auto& w : wants) {
    // bare name first, then the "transformer." prefix (the reference's tensor_f32 fallback)
    std::string name = w.name;
    auto it = file->tensors.find(name);
    if (it == file->tensors.end()) {
      name = "transformer." + w.name;
      it = file->tensors.find(name);
      if (it == file->tensors.end()) return set_error(PG_ASSET, "tensor " + name + " not found");
    }
    const TensorEntry& e = it->second;
    if (e.dtype != "F32")
      return set_error(PG_ASSET, "tensor " + name + " has dtype " + e.dtype + ", expected F32");
    if (e.shape != w.shape)
      return set_error(PG_INVALID_WEIGHTS, "tensor " + name + " shape " + shape_str(e.shape) +
                                               " does not match expected " + shape_str(w.shape));
    uint64_t count = (e.end - e.begin) / 4;
    // little-endian bytes -> f32 (the data section has no alignment guarantee, so copy)
    std::vector<float> v(count);
    memcpy(v.data(), file->data(e), count * 4);
    out->owned.push_back(std::move(v));
    out->ptrs.push_back(out->owned.back().data());
    out->lens.push_back(count);
  }
  return PG_OK;
}

}  // namespace pg
