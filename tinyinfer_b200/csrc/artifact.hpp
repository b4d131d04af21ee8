// Weight artifact reader: manifest.json (strict ASCII JSON) + weights.bin, fully verified
// before any byte reaches the GPU.
//
// Accepts exactly what the reference loader accepts (llm/src/artifact.hpp:153-199) for the
// GPT-2 124M artifact written by llm/export_weights.py:163-205 -- schema 1, 256-byte alignment,
// sibling "weights.bin", the pinned identity strings, whole-file and per-tensor SHA-256,
// dtype/extent/alignment/overlap checks, finite fp16, finite positive fp32 scales, no int8
// value -128 -- and, additionally, other GPT-2 shapes with 64-wide heads (the manifest's
// architecture block is then authoritative), which the reference rejects.
// Own JSON parser and SHA-256: no third-party dependency, no allocation proportional to input
// beyond the file contents themselves.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace tib {

struct InvalidInput : std::runtime_error { using std::runtime_error::runtime_error; };
struct IoFailure : std::runtime_error { using std::runtime_error::runtime_error; };

// ---------------------------------------------------------------- JSON
struct JsonValue {
  enum Type { kNull, kBool, kNumber, kString, kArray, kObject } type = kNull;
  std::string text;                                   // number literal, string contents or true/false
  std::vector<JsonValue> items;
  std::vector<std::pair<std::string, JsonValue>> members;

  const JsonValue& get(const char* key) const {
    if (type == kObject)
      for (const auto& m : members) if (m.first == key) return m.second;
    throw InvalidInput(std::string("missing manifest field: ") + key);
  }
  const std::string& as_string() const { if (type != kString) throw InvalidInput("expected JSON string"); return text; }
  uint64_t as_uint() const {
    if (type != kNumber || text.empty()) throw InvalidInput("expected unsigned exact JSON integer");
    uint64_t v = 0;
    for (char c : text) {
      if (c < '0' || c > '9') throw InvalidInput("expected unsigned exact JSON integer");
      if (v > (UINT64_MAX - uint64_t(c - '0')) / 10) throw InvalidInput("integer overflow");
      v = v * 10 + uint64_t(c - '0');
    }
    return v;
  }
  double as_double() const {
    if (type != kNumber) throw InvalidInput("expected JSON number");
    char* end = nullptr; const double v = std::strtod(text.c_str(), &end);
    if (!end || *end != '\0' || !std::isfinite(v)) throw InvalidInput("invalid JSON number");
    return v;
  }
};

class JsonReader {
 public:
  explicit JsonReader(const std::string& s) : s_(s) {}
  JsonValue parse() {
    JsonValue v = value(0);
    blanks();
    if (at_ != s_.size()) throw InvalidInput("trailing JSON");
    return v;
  }

 private:
  const std::string& s_;
  size_t at_ = 0;
  void blanks() { while (at_ < s_.size() && (s_[at_] == ' ' || s_[at_] == '\t' || s_[at_] == '\n' || s_[at_] == '\r')) ++at_; }
  char next() { if (at_ >= s_.size()) throw InvalidInput("truncated JSON"); return s_[at_++]; }
  bool digits() { const size_t from = at_; while (at_ < s_.size() && s_[at_] >= '0' && s_[at_] <= '9') ++at_; return at_ > from; }
  std::string quoted() {
    if (next() != '"') throw InvalidInput("invalid JSON punctuation");
    std::string out;
    for (;;) {
      char c = next();
      if (c == '"') return out;
      if (c == '\\') {
        switch (c = next()) {
          case '"': case '\\': case '/': out += c; break;
          case 'b': out += '\b'; break; case 'f': out += '\f'; break; case 'n': out += '\n'; break;
          case 'r': out += '\r'; break; case 't': out += '\t'; break;
          default: throw InvalidInput("manifest strings must use ASCII (unicode escapes unsupported)");
        }
      } else if (static_cast<unsigned char>(c) < 32 || static_cast<unsigned char>(c) > 126) throw InvalidInput("non-ASCII manifest string");
      else out += c;
    }
  }
  JsonValue value(int depth) {
    if (depth > 32) throw InvalidInput("JSON nesting limit");
    blanks();
    if (at_ >= s_.size()) throw InvalidInput("empty JSON");
    JsonValue v;
    const char c = s_[at_];
    if (c == '{') {
      ++at_; v.type = JsonValue::kObject; blanks();
      if (at_ < s_.size() && s_[at_] == '}') { ++at_; return v; }
      for (;;) {
        blanks();
        std::string key = quoted();
        blanks();
        if (next() != ':') throw InvalidInput("invalid JSON punctuation");
        for (const auto& m : v.members) if (m.first == key) throw InvalidInput("duplicate JSON key");
        v.members.emplace_back(std::move(key), value(depth + 1));
        blanks();
        const char d = next();
        if (d == '}') break;
        if (d != ',') throw InvalidInput("object delimiter");
      }
    } else if (c == '[') {
      ++at_; v.type = JsonValue::kArray; blanks();
      if (at_ < s_.size() && s_[at_] == ']') { ++at_; return v; }
      for (;;) {
        v.items.push_back(value(depth + 1));
        blanks();
        const char d = next();
        if (d == ']') break;
        if (d != ',') throw InvalidInput("array delimiter");
      }
    } else if (c == '"') { v.type = JsonValue::kString; v.text = quoted(); }
    else if (c == 't' || c == 'f' || c == 'n') {
      const char* word = c == 't' ? "true" : c == 'f' ? "false" : "null";
      const size_t n = std::strlen(word);
      if (s_.compare(at_, n, word) != 0) throw InvalidInput("invalid JSON literal");
      at_ += n; v.type = c == 'n' ? JsonValue::kNull : JsonValue::kBool; v.text = word;
    } else {
      const size_t from = at_;
      if (s_[at_] == '-') ++at_;
      if (at_ >= s_.size()) throw InvalidInput("number expected");
      if (s_[at_] == '0') ++at_;
      else if (s_[at_] >= '1' && s_[at_] <= '9') digits();
      else throw InvalidInput("number expected");
      if (at_ < s_.size() && s_[at_] == '.') { ++at_; if (!digits()) throw InvalidInput("invalid fraction"); }
      if (at_ < s_.size() && (s_[at_] == 'e' || s_[at_] == 'E')) {
        ++at_;
        if (at_ < s_.size() && (s_[at_] == '+' || s_[at_] == '-')) ++at_;
        if (!digits()) throw InvalidInput("invalid exponent");
      }
      v.type = JsonValue::kNumber; v.text = s_.substr(from, at_ - from);
    }
    return v;
  }
};

// ---------------------------------------------------------------- SHA-256 (FIPS 180-4)
class Sha256 {
 public:
  void update(const void* data, size_t n) {
    const uint8_t* p = static_cast<const uint8_t*>(data);
    total_ += n;
    if (fill_) {
      const size_t take = std::min(n, size_t(64) - fill_);
      std::memcpy(buf_ + fill_, p, take); fill_ += take; p += take; n -= take;
      if (fill_ == 64) { compress(buf_); fill_ = 0; }
    }
    for (; n >= 64; p += 64, n -= 64) compress(p);
    if (n) { std::memcpy(buf_, p, n); fill_ = n; }
  }
  std::string hex() {
    const uint64_t bits = total_ * 8;
    uint8_t pad[72] = {0x80};
    const size_t pad_len = (fill_ < 56 ? 56 : 120) - fill_;
    for (int i = 0; i < 8; ++i) pad[pad_len + i] = uint8_t(bits >> (56 - 8 * i));
    update(pad, pad_len + 8);
    char out[65];
    for (int i = 0; i < 8; ++i) std::snprintf(out + 8 * i, 9, "%08x", h_[i]);
    return std::string(out, 64);
  }
  static std::string of(const void* data, size_t n) { Sha256 s; s.update(data, n); return s.hex(); }

 private:
  uint32_t h_[8] = {0x6a09e667u, 0xbb67ae85u, 0x3c6ef372u, 0xa54ff53au, 0x510e527fu, 0x9b05688cu, 0x1f83d9abu, 0x5be0cd19u};
  uint8_t buf_[64];
  size_t fill_ = 0;
  uint64_t total_ = 0;
  static uint32_t ror(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
  void compress(const uint8_t* p) {
    static const uint32_t K[64] = {
        0x428a2f98u, 0x71374491u, 0xb5c0fbcfu, 0xe9b5dba5u, 0x3956c25bu, 0x59f111f1u, 0x923f82a4u, 0xab1c5ed5u, 0xd807aa98u,
        0x12835b01u, 0x243185beu, 0x550c7dc3u, 0x72be5d74u, 0x80deb1feu, 0x9bdc06a7u, 0xc19bf174u, 0xe49b69c1u, 0xefbe4786u,
        0x0fc19dc6u, 0x240ca1ccu, 0x2de92c6fu, 0x4a7484aau, 0x5cb0a9dcu, 0x76f988dau, 0x983e5152u, 0xa831c66du, 0xb00327c8u,
        0xbf597fc7u, 0xc6e00bf3u, 0xd5a79147u, 0x06ca6351u, 0x14292967u, 0x27b70a85u, 0x2e1b2138u, 0x4d2c6dfcu, 0x53380d13u,
        0x650a7354u, 0x766a0abbu, 0x81c2c92eu, 0x92722c85u, 0xa2bfe8a1u, 0xa81a664bu, 0xc24b8b70u, 0xc76c51a3u, 0xd192e819u,
        0xd6990624u, 0xf40e3585u, 0x106aa070u, 0x19a4c116u, 0x1e376c08u, 0x2748774cu, 0x34b0bcb5u, 0x391c0cb3u, 0x4ed8aa4au,
        0x5b9cca4fu, 0x682e6ff3u, 0x748f82eeu, 0x78a5636fu, 0x84c87814u, 0x8cc70208u, 0x90befffau, 0xa4506cebu, 0xbef9a3f7u,
        0xc67178f2u};
    uint32_t w[64];
    for (int i = 0; i < 16; ++i) w[i] = uint32_t(p[4 * i]) << 24 | uint32_t(p[4 * i + 1]) << 16 | uint32_t(p[4 * i + 2]) << 8 | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = ror(w[i - 15], 7) ^ ror(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = ror(w[i - 2], 17) ^ ror(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t v[8];
    std::memcpy(v, h_, sizeof v);
    for (int i = 0; i < 64; ++i) {
      const uint32_t t1 = v[7] + (ror(v[4], 6) ^ ror(v[4], 11) ^ ror(v[4], 25)) + ((v[4] & v[5]) ^ (~v[4] & v[6])) + K[i] + w[i];
      const uint32_t t2 = (ror(v[0], 2) ^ ror(v[0], 13) ^ ror(v[0], 22)) + ((v[0] & v[1]) ^ (v[0] & v[2]) ^ (v[1] & v[2]));
      v[7] = v[6]; v[6] = v[5]; v[5] = v[4]; v[4] = v[3] + t1; v[3] = v[2]; v[2] = v[1]; v[1] = v[0]; v[0] = t1 + t2;
    }
    for (int i = 0; i < 8; ++i) h_[i] += v[i];
  }
};

// ---------------------------------------------------------------- artifact
struct TensorEntry { std::string dtype; std::vector<int> shape; uint64_t offset = 0, nbytes = 0; };

struct ModelShape { int layers = 12, heads = 12, hidden = 768, vocab = 50257, positions = 1024; };

inline std::vector<uint8_t> slurp(const std::string& path, uint64_t limit) {
  std::FILE* f = std::fopen(path.c_str(), "rb");
  if (!f) throw IoFailure("cannot open artifact: " + path);
  std::unique_ptr<std::FILE, int (*)(std::FILE*)> guard(f, &std::fclose);
  if (std::fseek(f, 0, SEEK_END) != 0) throw IoFailure("cannot size artifact: " + path);
  const long size = std::ftell(f);
  if (size < 0 || uint64_t(size) > limit) throw InvalidInput("artifact exceeds size limit");
  std::rewind(f);
  std::vector<uint8_t> data(static_cast<size_t>(size));
  if (!data.empty() && std::fread(data.data(), 1, data.size(), f) != data.size()) throw IoFailure("short artifact read");
  return data;
}

class Artifact {
 public:
  std::vector<uint8_t> blob;
  std::map<std::string, TensorEntry> tensors;
  std::string precision;
  ModelShape shape;

  explicit Artifact(const std::string& manifest_path) {
    const std::vector<uint8_t> raw = slurp(manifest_path, 1u << 20);
    const size_t cut = manifest_path.find_last_of("/\\");
    const std::string dir = cut == std::string::npos ? std::string() : manifest_path.substr(0, cut + 1);
    load(std::string(raw.begin(), raw.end()), slurp(dir + "weights.bin", 8ull << 30));
  }
  Artifact(const std::string& manifest_text, std::vector<uint8_t> weights) { load(manifest_text, std::move(weights)); }

  const TensorEntry& need(const std::string& name, const std::vector<int>& dims, const char* dtype) const {
    const auto it = tensors.find(name);
    if (it == tensors.end() || it->second.shape != dims || it->second.dtype != dtype) throw InvalidInput("tensor schema mismatch: " + name);
    return it->second;
  }

 private:
  void load(const std::string& text, std::vector<uint8_t> weights) {
    if (text.size() > (1u << 20)) throw InvalidInput("artifact exceeds size limit");
    const JsonValue doc = JsonReader(text).parse();
    if (doc.get("schema_version").as_uint() != 1 || doc.get("alignment").as_uint() != 256 || doc.get("binary").as_string() != "weights.bin" ||
        doc.get("model_id").as_string() != "openai-community/gpt2" ||
        doc.get("revision").as_string() != "607a30d783dfa663caf39e06633721c8d4cfcd7e" ||
        doc.get("source_sha256").as_string() != "248dfc3911869ec493c76e65bf2fcf7f615828b0254c12b473182f0f81d3a707")
      throw InvalidInput("unrecognized artifact identity");
    const JsonValue& arch = doc.get("architecture");
    shape.layers = int(std::min<uint64_t>(arch.get("layers").as_uint(), 1u << 20));
    shape.heads = int(std::min<uint64_t>(arch.get("heads").as_uint(), 1u << 20));
    shape.hidden = int(std::min<uint64_t>(arch.get("hidden").as_uint(), 1u << 20));
    shape.vocab = int(std::min<uint64_t>(arch.get("vocab").as_uint(), 1u << 20));
    shape.positions = int(std::min<uint64_t>(arch.get("capacity").as_uint(), 1u << 20));
    if (shape.layers < 1 || shape.layers > 64 || shape.heads < 1 || shape.heads > 64 || shape.hidden != shape.heads * 64 ||
        shape.vocab != 50257 || shape.positions < 2 || shape.positions > 1024 || arch.get("gelu").as_string() != "gelu_new" ||
        arch.get("layer_norm_eps").as_double() != 1e-5)
      throw InvalidInput("unsupported architecture (GPT-2 family with 64-wide heads, vocab 50257, gelu_new, eps 1e-5)");
    precision = doc.get("precision").as_string();
    if (precision != "fp16" && precision != "int8") throw InvalidInput("unknown precision");

    blob = std::move(weights);
    if (blob.size() != doc.get("binary_bytes").as_uint() || Sha256::of(blob.data(), blob.size()) != doc.get("binary_sha256").as_string())
      throw InvalidInput("weights binary SHA256/length mismatch");
    const JsonValue& list = doc.get("tensors");
    if (list.type != JsonValue::kArray || list.items.size() > 1024) throw InvalidInput("invalid tensor list");
    std::vector<std::pair<uint64_t, uint64_t>> spans;
    for (const JsonValue& item : list.items) {
      TensorEntry t;
      t.dtype = item.get("dtype").as_string(); t.offset = item.get("offset").as_uint(); t.nbytes = item.get("nbytes").as_uint();
      const JsonValue& dims = item.get("shape");
      if (dims.type != JsonValue::kArray || dims.items.empty() || dims.items.size() > 2) throw InvalidInput("tensor rank");
      uint64_t count = 1;
      for (const JsonValue& d : dims.items) {
        const uint64_t n = d.as_uint();
        if (!n || n > 50257) throw InvalidInput("tensor dimension");
        count *= n; t.shape.push_back(int(n));
      }
      const uint64_t width = t.dtype == "float16" ? 2 : t.dtype == "float32" ? 4 : t.dtype == "int8" ? 1 : 0;
      if (!width || t.nbytes != count * width || t.offset % 256 || t.offset > blob.size() || t.nbytes > blob.size() - t.offset)
        throw InvalidInput("tensor extent/dtype/alignment");
      const uint8_t* data = blob.data() + t.offset;
      if (Sha256::of(data, t.nbytes) != item.get("sha256").as_string()) throw InvalidInput("tensor SHA256 mismatch");
      if (width == 2) {
        for (uint64_t i = 0; i < t.nbytes; i += 2) if ((data[i + 1] & 0x7c) == 0x7c) throw InvalidInput("nonfinite half weight");
      } else if (width == 4) {
        for (uint64_t i = 0; i < t.nbytes; i += 4) { float v; std::memcpy(&v, data + i, 4); if (!std::isfinite(v) || v <= 0) throw InvalidInput("nonpositive/nonfinite scale"); }
      } else if (std::memchr(data, 0x80, t.nbytes)) throw InvalidInput("unsupported INT8 -128 weight");
      if (!tensors.emplace(item.get("name").as_string(), t).second) throw InvalidInput("duplicate tensor name");
      spans.emplace_back(t.offset, t.offset + t.nbytes);
    }
    std::sort(spans.begin(), spans.end());
    for (size_t i = 1; i < spans.size(); ++i) if (spans[i - 1].second > spans[i].first) throw InvalidInput("overlapping weights");
  }
};

}  // namespace tib
