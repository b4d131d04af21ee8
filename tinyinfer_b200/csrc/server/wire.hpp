// Wire protocol v1 of the batching server: big-endian, u32 body-length prefix, binary token ids.
// Byte-compatible with the reference (server/include/protocol.hpp:7-45, server/protocol.py:5-40,
// server/README.md "Protocol and limits"):
//   request body   !HHQII  version=1, kind (1 generate / 2 cancel), id != 0, max_new, count; then count x u32 ids
//   response body  !HHQIIIIQQQQ  version, kind (0x8002 FIRST / 0x8001 FINAL), id, status, count, batch, 0,
//                  queue_ns, first_ns, infer_ns, server_ns; then count x u32 ids
// Status: 0 ok, 1 invalid, 2 overloaded, 3 cancelled, 4 internal.  Malformed frames throw; the
// connection is then closed by the caller.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <utility>
#include <vector>

namespace tib::server {

constexpr uint16_t kVersion = 1, kGenerate = 1, kCancel = 2, kFinal = 0x8001, kFirst = 0x8002;
enum Status : uint32_t { kOk = 0, kInvalid = 1, kOverloaded = 2, kCancelled = 3, kInternal = 4 };
constexpr uint32_t kVocab = 50257;
constexpr size_t kRequestHeader = 20;

using Bytes = std::vector<uint8_t>;

inline uint64_t load_be(const uint8_t* p, int bytes) {
  uint64_t v = 0;
  for (int i = 0; i < bytes; ++i) v = (v << 8) | p[i];
  return v;
}
inline void store_be(Bytes& out, uint64_t v, int bytes) {
  for (int shift = 8 * (bytes - 1); shift >= 0; shift -= 8) out.push_back(uint8_t(v >> shift));
}

struct Request {
  uint16_t kind = 0;
  uint64_t id = 0;
  uint32_t max_new = 0;
  std::vector<int32_t> tokens;
};

// Validates one request body against the server's limits (capacity = context positions,
// max_new = largest generation the server accepts).
inline Request decode_request(const Bytes& body, uint32_t capacity, uint32_t max_new) {
  if (body.size() < kRequestHeader || load_be(body.data(), 2) != kVersion) throw std::runtime_error("request version/size");
  Request r;
  r.kind = uint16_t(load_be(body.data() + 2, 2));
  r.id = load_be(body.data() + 4, 8);
  r.max_new = uint32_t(load_be(body.data() + 12, 4));
  const uint64_t count = load_be(body.data() + 16, 4);
  if (r.id == 0 || body.size() != kRequestHeader + 4 * count) throw std::runtime_error("request ID/length");
  if (r.kind == kCancel) {
    if (count || r.max_new) throw std::runtime_error("cancel fields");
    return r;
  }
  if (r.kind != kGenerate || count == 0 || r.max_new == 0 || r.max_new > max_new || count + r.max_new > capacity)
    throw std::runtime_error("token/context limits");
  r.tokens.reserve(size_t(count));
  for (uint64_t i = 0; i < count; ++i) {
    const uint32_t t = uint32_t(load_be(body.data() + kRequestHeader + 4 * i, 4));
    if (t >= kVocab) throw std::runtime_error("token ID");
    r.tokens.push_back(int32_t(t));
  }
  return r;
}

struct Response {
  uint16_t kind = kFinal;
  uint64_t id = 0;
  Status status = kOk;
  uint32_t batch_size = 0;
  uint64_t queue_ns = 0, first_ns = 0, infer_ns = 0, server_ns = 0;
  std::vector<int32_t> tokens;
};

inline Bytes encode_response(const Response& r) {
  Bytes out;
  out.reserve(64 + 4 * r.tokens.size());
  store_be(out, 60 + 4 * r.tokens.size(), 4);
  store_be(out, kVersion, 2); store_be(out, r.kind, 2); store_be(out, r.id, 8); store_be(out, r.status, 4);
  store_be(out, r.tokens.size(), 4); store_be(out, r.batch_size, 4); store_be(out, 0, 4);
  store_be(out, r.queue_ns, 8); store_be(out, r.first_ns, 8); store_be(out, r.infer_ns, 8); store_be(out, r.server_ns, 8);
  for (int32_t t : r.tokens) store_be(out, uint32_t(t), 4);
  return out;
}

// Reassembles length-prefixed frames from arbitrary fragments; a declared length outside
// [20, limit] is rejected as soon as the 4 prefix bytes are known, before the body is buffered.
class FrameAssembler {
 public:
  explicit FrameAssembler(uint32_t limit) : limit_(limit) {}
  template <class OnFrame>
  void feed(const uint8_t* data, size_t n, OnFrame&& on_frame) {
    size_t at = 0;
    while (at < n) {
      if (!have_prefix_) {
        const size_t take = std::min(n - at, 4 - pending_.size());
        pending_.insert(pending_.end(), data + at, data + at + take);
        at += take;
        if (pending_.size() < 4) return;
        want_ = load_be(pending_.data(), 4);
        pending_.clear();
        if (want_ < kRequestHeader || want_ > limit_) throw std::runtime_error("frame length limit");
        body_.clear();
        body_.reserve(size_t(want_));
        have_prefix_ = true;
      }
      const size_t take = std::min<uint64_t>(n - at, want_ - body_.size());
      body_.insert(body_.end(), data + at, data + at + take);
      at += take;
      if (body_.size() == want_) {
        have_prefix_ = false;
        Bytes done;
        done.swap(body_);
        on_frame(std::move(done));
      }
    }
  }

 private:
  uint32_t limit_;
  uint64_t want_ = 0;
  bool have_prefix_ = false;
  Bytes pending_, body_;
};

}  // namespace tib::server
