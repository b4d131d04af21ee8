// tinyinfer_server: TCP batching server in front of the ti_llm model ABI, one model replica per GPU.
//
// Same wire protocol, command-line flags, limits and failure behaviour as the reference server
// (server/src/main.cpp:34-57 flags, :172-252 socket handling, server/README.md) with a different
// execution model behind the socket:
//   * N worker threads, one per entry of --devices (one ti_llm context each: own weights,
//     stream and KV pages; GPT-2 fits one GPU, so GPUs are replicas and nothing crosses NVLink; a GPU
//     listed twice carries two replicas whose decode steps overlap on the device);
//     a router hands every accepted request to the worker with the fewest tokens outstanding;
//   * continuous batching: a worker admits waiting requests into free KV slots between decode
//     steps (the reference forms a batch once and runs it to completion, main.cpp:100-150), so a
//     long generation never blocks short ones queued behind it; --max-wait-us only delays the
//     first admission of an otherwise idle worker, to let a batch gather; a busy worker waits for
//     --admit-batch free slots (default: an eighth of --max-batch) or for as many as there are requests
//     waiting, so that under load prompts are prefilled several at a time in one many-row pass;
//   * up to 64 requests per step and worker (--max-batch; the reference stops at 32).
// One epoll thread owns every socket and all connection state; requests travel to the workers and
// completions back through multi-producer/single-consumer queues plus an eventfd.  epoll events carry
// a never-reused registration number instead of a pointer or file descriptor, so an event collected
// for a closed connection cannot act on a new connection that reuses its descriptor.
// `--model cpu` replaces the GPU model with a deterministic token function for protocol tests
// (next = (last + cached_length + 1) mod 50257, the reference's CPU stand-in, model.hpp:70-75).
#include <arpa/inet.h>
#include <fcntl.h>
#include <sys/epoll.h>
#include <sys/eventfd.h>
#include <sys/resource.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <chrono>
#include <condition_variable>
#include <csignal>
#include <deque>
#include <iostream>
#include <map>
#include <memory>
#include <mutex>
#include <sstream>
#include <string>
#include <thread>
#include <unordered_map>
#include <unordered_set>

#include "queue.hpp"
#include "tinyinfer_llm.h"
#include "wire.hpp"

using namespace tib::server;
using Clock = std::chrono::steady_clock;

namespace {

uint64_t nanos(Clock::duration d) { return uint64_t(std::chrono::duration_cast<std::chrono::nanoseconds>(d).count()); }

volatile std::sig_atomic_t g_stop = 0;
void on_signal(int) { g_stop = 1; }

// ---------------------------------------------------------------------------------- options
struct Config {
  int port = 8091, max_batch = 8, max_wait_us = 1000, capacity = 1024, max_new = 128, max_pending = 256, max_connections = 256;
  int per_connection = 32, max_output = 1 << 20, max_ids = 100000, send_chunk = 65536, gemm = 0, attention = 0;
  // A busy worker admits waiting requests only when this many KV slots are free (or as many as are waiting, if fewer):
  // their prompts then travel in one pass with many rows instead of one small pass per freed slot.  0 = max_batch / 8
  // (measured at --max-batch 64 under saturating load: 1 -> 61.9k, 4 -> 69.8k, 8 -> 71.8k, 16 -> 69.0k, 32 -> 64.1k tokens/s).
  int admit_batch = 0;
  bool native = false;
  // test hook: worker number fail_worker fails its model call number fail_after_steps (0 = never), as a native execution
  // failure would; exercises the poisoned-worker path without touching a GPU
  int fail_worker = 0, fail_after_steps = 0;
  std::vector<int> devices{0};
  std::string manifest, host = "127.0.0.1";
};

Config parse_options(int argc, char** argv) {
  Config c;
  const std::map<std::string, int*> ints{
      {"port", &c.port}, {"max-batch", &c.max_batch}, {"max-wait-us", &c.max_wait_us}, {"capacity", &c.capacity},
      {"max-new-tokens", &c.max_new}, {"max-pending", &c.max_pending}, {"max-connections", &c.max_connections},
      {"per-connection", &c.per_connection}, {"max-output-bytes", &c.max_output}, {"max-ids", &c.max_ids},
      {"send-chunk-bytes", &c.send_chunk}, {"gemm-config", &c.gemm}, {"attention-config", &c.attention},
      {"fail-worker", &c.fail_worker}, {"fail-after-steps", &c.fail_after_steps}, {"admit-batch", &c.admit_batch}};
  auto integer = [](const std::string& text) {
    size_t used = 0;
    const int v = std::stoi(text, &used);
    if (used != text.size()) throw std::runtime_error("noninteger option");
    return v;
  };
  for (int i = 1; i < argc; i += 2) {
    const std::string flag = argv[i];
    if (i + 1 >= argc || flag.rfind("--", 0) != 0) throw std::runtime_error("expected option/value pairs");
    const std::string key = flag.substr(2), value = argv[i + 1];
    if (key == "model") {
      if (value != "cpu" && value != "native") throw std::runtime_error("model must be cpu/native");
      c.native = value == "native";
    } else if (key == "manifest") c.manifest = value;
    else if (key == "host") c.host = value;
    else if (key == "device") c.devices = {integer(value)};
    else if (key == "devices") {
      c.devices.clear();
      std::stringstream list(value);
      for (std::string item; std::getline(list, item, ',');) c.devices.push_back(integer(item));
    } else if (ints.count(key)) *ints.at(key) = integer(value);
    else throw std::runtime_error("unknown option: " + key);
  }
  // A device may be listed more than once: every mention is a replica of its own (weights, KV pages, stream, worker
  // thread).  Decode steps are latency-bound, so two replicas of 32 requests on one B200 generate more tokens per second
  // than one of 64 (measured under saturating load: 79.2k against 74.6k; four replicas of 64: 123.6k).
  bool devices_ok = !c.devices.empty() && c.devices.size() <= 64;
  for (int d : c.devices) devices_ok = devices_ok && d >= 0;
  if (c.port < 1 || c.port > 65535 || c.max_batch < 1 || c.max_batch > 64 || c.max_wait_us < 0 || c.max_wait_us > 1000000 ||
      c.capacity < 2 || c.capacity > 1024 || c.max_new < 1 || c.max_new >= c.capacity || c.max_pending < 1 || c.max_pending > 100000 ||
      c.max_connections < 1 || c.max_connections > 100000 || c.per_connection < 1 || c.per_connection > c.max_pending ||
      c.max_output < 64 || c.max_output > 64 * 1024 * 1024 || c.max_ids < 1 || c.max_ids > 1000000 || c.send_chunk < 1 ||
      c.send_chunk > 1048576 || c.gemm < 0 || c.gemm > 11 || c.attention < 0 || c.attention > 1 || !devices_ok ||
      (c.native && c.manifest.empty()) || c.fail_worker < 0 || c.fail_worker >= int(c.devices.size()) || c.fail_after_steps < 0 ||
      c.admit_batch < 0 || c.admit_batch > 64)
    throw std::runtime_error("option range");
  return c;
}

// ---------------------------------------------------------------------------------- model replica
class Replica {
 public:
  Replica(const Config& c, int device, int fail_after = 0)
      : native_(c.native), capacity_(c.capacity), fail_after_(fail_after), lengths_(size_t(c.max_batch), 0), last_(size_t(c.max_batch), 0) {
    if (!native_) return;
    if (ti_llm_abi_version() != 1) throw std::runtime_error("ti_llm ABI mismatch");
    ti_llm_options o{sizeof(ti_llm_options), device, c.max_batch, c.max_batch, c.capacity, c.gemm, c.attention};
    check(ti_llm_create(c.manifest.c_str(), &o, &model_));
  }
  ~Replica() { if (model_) ti_llm_destroy(model_); }
  Replica(const Replica&) = delete;
  Replica& operator=(const Replica&) = delete;

  void reset(int slot) {
    if (native_) { check(ti_llm_reset(model_, slot)); return; }
    lengths_.at(size_t(slot)) = 0; last_.at(size_t(slot)) = 0;
  }
  // Appends rows[i] to slots[i]; returns the greedy next id of every row.
  std::vector<int32_t> step(const std::vector<int32_t>& slots, const std::vector<const std::vector<int32_t>*>& rows) {
    std::vector<int32_t> next(slots.size());
    if (fail_after_ > 0 && ++calls_ == fail_after_) throw std::runtime_error("injected model failure (test hook)");
    if (native_) {
      size_t stride = 0;
      for (auto* row : rows) stride = std::max(stride, row->size());
      tokens_.assign(rows.size() * stride, 0); lens_.resize(rows.size());
      for (size_t i = 0; i < rows.size(); ++i) {
        std::copy(rows[i]->begin(), rows[i]->end(), tokens_.begin() + long(i * stride));
        lens_[i] = int32_t(rows[i]->size());
      }
      check(ti_llm_forward_batch(model_, slots.data(), tokens_.data(), lens_.data(), int32_t(slots.size()), int32_t(stride), nullptr, next.data()));
      return next;
    }
    for (size_t i = 0; i < slots.size(); ++i) {
      const size_t s = size_t(slots[i]);
      if (rows[i]->empty() || lengths_.at(s) + int(rows[i]->size()) > capacity_) throw std::runtime_error("CPU context limit");
      for (int32_t t : *rows[i]) { last_[s] = t; ++lengths_[s]; }
      next[i] = int32_t((int64_t(last_[s]) + lengths_[s] + 1) % kVocab);
    }
    return next;
  }
  void report(std::ostream& out, int device) {
    if (!native_) { out << "{\"trace_mode\":\"cpu_oracle_no_native_calls\"}\n"; return; }
    ti_llm_trace t{};
    const int status = ti_llm_get_trace(model_, &t);
    out << "{\"device\":" << device << ",\"native_trace_status\":" << status;
    if (status == 0)
      out << ",\"forward_calls\":" << t.forward_calls << ",\"embedding\":" << t.embedding << ",\"gemm_fp16\":" << t.gemm_fp16
          << ",\"gemm_int8\":" << t.gemm_int8 << ",\"layernorm\":" << t.layernorm << ",\"gelu\":" << t.gelu << ",\"attention\":" << t.attention
          << ",\"residual\":" << t.residual << ",\"kv_scatter_gather\":" << t.kv_scatter_gather << ",\"lm_head\":" << t.lm_head
          << ",\"argmax\":" << t.argmax << ",\"nll\":" << t.nll;
    out << "}\n";
  }

 private:
  void check(int status) { if (status) throw std::runtime_error(ti_llm_last_error()); }
  bool native_;
  int capacity_, fail_after_ = 0, calls_ = 0;
  std::vector<int> lengths_;
  std::vector<int32_t> last_, tokens_, lens_;
  ti_llm_model* model_ = nullptr;
};

// ---------------------------------------------------------------------------------- shared records
struct Job {
  int fd = -1;
  uint64_t connection = 0;
  Request wire;
  Clock::time_point accepted;
  std::atomic<bool> cancel{false};
  int worker = 0;
};
struct Completion { std::shared_ptr<Job> job; Response response; };

class Server;

// ---------------------------------------------------------------------------------- GPU worker
class Worker {
 public:
  Worker(Server& server, const Config& c, int index, int device) : server_(server), config_(c), index_(index), device_(device) {}
  void load() { replica_ = std::make_unique<Replica>(config_, device_, index_ == config_.fail_worker ? config_.fail_after_steps : 0); }
  bool healthy() const { return !poisoned_flag_.load(std::memory_order_relaxed); }
  void start() { thread_ = std::thread([this] { run(); }); }
  void join() { if (thread_.joinable()) thread_.join(); }
  void submit(std::shared_ptr<Job> job) {
    load_tokens_.fetch_add(int64_t(job->wire.tokens.size() + job->wire.max_new), std::memory_order_relaxed);
    inbox_.push(std::move(job));
    queued_.fetch_add(1, std::memory_order_release);
    wake();
  }
  void wake() { std::lock_guard<std::mutex> hold(mutex_); signal_.notify_one(); }
  int64_t load_tokens() const { return load_tokens_.load(std::memory_order_relaxed); }
  void report(std::ostream& out) { if (replica_) replica_->report(out, device_); }

 private:
  struct Active {
    std::shared_ptr<Job> job;
    std::vector<int32_t> generated;
    Clock::time_point admitted;
    uint32_t batch_size = 0;
    uint64_t first_ns = 0;
  };
  void run() noexcept;
  void finish(Active& a, Status status);
  bool drain_inbox();

  Server& server_;
  const Config& config_;
  int index_, device_;
  std::unique_ptr<Replica> replica_;
  std::thread thread_;
  MpscQueue<std::shared_ptr<Job>> inbox_;
  std::atomic<size_t> queued_{0};
  std::atomic<int64_t> load_tokens_{0};
  std::mutex mutex_;
  std::condition_variable signal_;
  std::deque<std::shared_ptr<Job>> waiting_;
  bool poisoned_ = false;
  std::atomic<bool> poisoned_flag_{false};           // what the router sees
};

// ---------------------------------------------------------------------------------- socket front end
struct Connection {
  uint64_t token;
  FrameAssembler frames;
  std::deque<Bytes> outbox;
  size_t sent = 0, queued_bytes = 0;
  bool overflowed = false;
  std::unordered_map<uint64_t, std::shared_ptr<Job>> active;
  std::unordered_set<uint64_t> seen_ids;
  Connection(uint64_t t, uint32_t frame_limit) : token(t), frames(frame_limit) {}
};

class Server {
 public:
  explicit Server(Config c) : config_(std::move(c)) {
    for (size_t i = 0; i < config_.devices.size(); ++i) workers_.push_back(std::make_unique<Worker>(*this, config_, int(i), config_.devices[i]));
    // Every replica is loaded (in parallel) before the socket is opened: readiness is never announced early.
    std::vector<std::thread> loaders;
    std::vector<std::string> errors(workers_.size());
    for (size_t i = 0; i < workers_.size(); ++i)
      loaders.emplace_back([this, i, &errors] { try { workers_[i]->load(); } catch (const std::exception& e) { errors[i] = e.what(); } });
    for (auto& t : loaders) t.join();
    for (const auto& e : errors) if (!e.empty()) throw std::runtime_error(e);
  }
  ~Server() {
    stopping_.store(true);
    for (auto& c : connections_) for (auto& a : c.second->active) a.second->cancel.store(true);
    for (auto& w : workers_) w->wake();
    for (auto& w : workers_) w->join();
    for (auto& w : workers_) w->report(std::cerr);
    for (auto& c : connections_) close(c.first);
    if (listener_ >= 0) close(listener_);
    if (event_ >= 0) close(event_);
    if (epoll_ >= 0) close(epoll_);
  }
  bool stopping() const { return stopping_.load(); }

  // Called by workers: hand a response to the socket thread.
  void complete(const std::shared_ptr<Job>& job, Response response) {
    response.id = job->wire.id;
    completions_.push({job, std::move(response)});
    const uint64_t one = 1;
    ssize_t n;
    do { n = write(event_, &one, sizeof one); } while (n < 0 && errno == EINTR);    // EAGAIN: a wake-up is already pending
  }
  void run();

 private:
  enum class Kind { kListener, kCompletions, kClient };
  struct Target { int fd; Kind kind; };
  uint64_t register_fd(int fd, Kind kind) { const uint64_t token = ++next_token_; targets_[token] = {fd, kind}; return token; }
  bool is_live(uint64_t token, int fd) const { auto it = targets_.find(token); return it != targets_.end() && it->second.fd == fd && it->second.kind == Kind::kClient; }

  void arm(int fd, Connection& c) {
    epoll_event e{};
    e.data.u64 = c.token;
    e.events = EPOLLIN | EPOLLRDHUP | (c.outbox.empty() ? 0u : unsigned(EPOLLOUT));
    if (epoll_ctl(epoll_, EPOLL_CTL_MOD, fd, &e) < 0) throw std::runtime_error("epoll MOD");
  }
  void drop(int fd, uint64_t token) {
    auto it = connections_.find(fd);
    if (it == connections_.end() || it->second->token != token) return;
    for (auto& a : it->second->active) a.second->cancel.store(true);
    targets_.erase(token);                                   // retire the registration before the descriptor can be reused
    epoll_ctl(epoll_, EPOLL_CTL_DEL, fd, nullptr);
    close(fd);
    connections_.erase(it);
    for (auto& w : workers_) w->wake();
  }
  bool send_later(int fd, const Response& r) {
    auto it = connections_.find(fd);
    if (it == connections_.end()) return false;
    Connection& c = *it->second;
    Bytes bytes = encode_response(r);
    if (c.queued_bytes + bytes.size() > size_t(config_.max_output)) { c.overflowed = true; return false; }
    c.queued_bytes += bytes.size();
    c.outbox.push_back(std::move(bytes));
    arm(fd, c);
    return true;
  }
  void on_frame(int fd, Bytes body);
  void on_readable(int fd, uint64_t token);
  void on_writable(int fd, uint64_t token);
  void accept_all();
  void drain_completions();

  Config config_;
  int listener_ = -1, epoll_ = -1, event_ = -1;
  uint64_t next_token_ = 0, listener_token_ = 0, event_token_ = 0;
  size_t outstanding_ = 0;
  std::unordered_map<uint64_t, Target> targets_;
  std::unordered_map<int, std::unique_ptr<Connection>> connections_;
  std::vector<std::unique_ptr<Worker>> workers_;
  MpscQueue<Completion> completions_;
  std::atomic<bool> stopping_{false};
};

// ---------------------------------------------------------------------------------- worker loop
bool Worker::drain_inbox() {
  bool any = false;
  std::shared_ptr<Job> job;
  while (queued_.load(std::memory_order_acquire) && inbox_.try_pop(job)) {
    queued_.fetch_sub(1, std::memory_order_acq_rel);
    waiting_.push_back(std::move(job));
    any = true;
  }
  return any;
}

void Worker::finish(Active& a, Status status) {
  Response r;
  r.kind = kFinal; r.status = status; r.batch_size = a.batch_size; r.first_ns = a.first_ns;
  r.queue_ns = nanos(a.admitted - a.job->accepted);
  r.infer_ns = nanos(Clock::now() - a.admitted);
  r.server_ns = nanos(Clock::now() - a.job->accepted);
  if (status == kOk) r.tokens = a.generated;
  load_tokens_.fetch_sub(int64_t(a.job->wire.tokens.size() + a.job->wire.max_new), std::memory_order_relaxed);
  server_.complete(a.job, std::move(r));
}

void Worker::run() noexcept {
  const size_t slots = size_t(config_.max_batch);
  std::vector<std::unique_ptr<Active>> active(slots);          // index = KV slot
  size_t live = 0;
  auto retire = [&](size_t slot, Status status) {
    finish(*active[slot], status);
    active[slot].reset();
    --live;
  };
  for (;;) {
    drain_inbox();
    if (live == 0 && waiting_.empty()) {
      if (server_.stopping() && !queued_.load()) break;
      std::unique_lock<std::mutex> lock(mutex_);
      signal_.wait_for(lock, std::chrono::milliseconds(1), [&] { return server_.stopping() || queued_.load() > 0; });
      continue;
    }
    // An idle worker lets a batch gather for at most max_wait_us after its oldest request arrived.
    if (live == 0 && !waiting_.empty() && waiting_.size() < slots && !server_.stopping()) {
      const auto deadline = waiting_.front()->accepted + std::chrono::microseconds(config_.max_wait_us);
      while (waiting_.size() < slots && Clock::now() < deadline && !server_.stopping()) {
        std::unique_lock<std::mutex> lock(mutex_);
        signal_.wait_until(lock, deadline, [&] { return server_.stopping() || queued_.load() > 0; });
        lock.unlock();
        drain_inbox();
      }
    }
    try {
      // ---- admission: waiting requests take free slots and are prefilled together
      std::vector<int32_t> new_slots;
      std::vector<const std::vector<int32_t>*> new_rows;
      // (a busy worker waits until admit_batch slots are free, or as many as there are requests waiting)
      const size_t group = config_.admit_batch ? std::min(size_t(config_.admit_batch), slots) : std::max<size_t>(1, slots / 8);
      const size_t wanted = std::min(group, waiting_.size());
      const bool admit_now = live == 0 || slots - live >= wanted || server_.stopping() || poisoned_;
      while (admit_now && !waiting_.empty() && live < slots) {
        std::shared_ptr<Job> job = std::move(waiting_.front());
        waiting_.pop_front();
        auto a = std::make_unique<Active>();
        a->job = job; a->admitted = Clock::now();
        if (poisoned_ || job->cancel.load() || server_.stopping()) {
          finish(*a, poisoned_ ? kInternal : kCancelled);
          continue;
        }
        size_t slot = 0;
        while (active[slot]) ++slot;
        replica_->reset(int(slot));
        active[slot] = std::move(a);
        ++live;
        new_slots.push_back(int32_t(slot));
        new_rows.push_back(&active[slot]->job->wire.tokens);
      }
      for (int32_t s : new_slots) active[size_t(s)]->batch_size = uint32_t(live);
      auto absorb = [&](const std::vector<int32_t>& which, const std::vector<int32_t>& next, Clock::time_point returned) {
        for (size_t j = 0; j < which.size(); ++j) {
          const size_t slot = size_t(which[j]);
          Active& a = *active[slot];
          if (a.job->cancel.load() || server_.stopping()) { replica_->reset(int(slot)); retire(slot, kCancelled); continue; }
          a.generated.push_back(next[j]);
          if (a.generated.size() == 1) {
            a.first_ns = nanos(returned - a.admitted);
            Response first;
            first.kind = kFirst; first.batch_size = a.batch_size; first.tokens = {next[j]}; first.first_ns = a.first_ns;
            first.queue_ns = nanos(a.admitted - a.job->accepted); first.infer_ns = a.first_ns; first.server_ns = nanos(returned - a.job->accepted);
            server_.complete(a.job, std::move(first));
          }
          if (a.generated.size() == a.job->wire.max_new) { replica_->reset(int(slot)); retire(slot, kOk); }
        }
      };
      // ---- one pass: the prompts of the requests admitted above together with one decode step for every request
      // that already has its first token (admissions do not cost the running requests a separate pass)
      std::vector<int32_t> pass_slots = new_slots;
      std::vector<const std::vector<int32_t>*> pass_rows = new_rows;
      std::vector<std::vector<int32_t>> last_tokens;
      last_tokens.reserve(slots);
      for (size_t slot = 0; slot < slots; ++slot) {
        if (!active[slot]) continue;
        Active& a = *active[slot];
        if (std::find(new_slots.begin(), new_slots.end(), int32_t(slot)) != new_slots.end()) continue;   // admitted in this pass
        if (a.job->cancel.load() || server_.stopping()) { replica_->reset(int(slot)); retire(slot, kCancelled); continue; }
        last_tokens.push_back({a.generated.back()});
        pass_slots.push_back(int32_t(slot));
      }
      for (auto& row : last_tokens) pass_rows.push_back(&row);
      if (!pass_slots.empty()) absorb(pass_slots, replica_->step(pass_slots, pass_rows), Clock::now());
    } catch (const std::exception& error) {
      // A failed native call leaves the replica unusable: everything outstanding and everything that
      // arrives later on this worker is answered with an internal error; the process stays up.
      std::cerr << "model_poisoned: device " << device_ << ": " << error.what() << '\n';
      poisoned_ = true;
      poisoned_flag_.store(true, std::memory_order_relaxed);
      for (size_t slot = 0; slot < slots; ++slot) if (active[slot]) retire(slot, kInternal);
    }
  }
}

// ---------------------------------------------------------------------------------- socket handling
void Server::on_frame(int fd, Bytes body) {
  auto it = connections_.find(fd);
  if (it == connections_.end()) return;
  Connection& c = *it->second;
  if (c.overflowed) return;
  Request wire = decode_request(body, uint32_t(config_.capacity), uint32_t(config_.max_new));
  if (wire.kind == kCancel) {
    auto found = c.active.find(wire.id);
    if (found != c.active.end()) { found->second->cancel.store(true); workers_[size_t(found->second->worker)]->wake(); }
    return;                                                  // unknown or finished ids: ignored
  }
  if (c.seen_ids.count(wire.id) || c.seen_ids.size() >= size_t(config_.max_ids)) throw std::runtime_error("duplicate/request-ID limit");
  c.seen_ids.insert(wire.id);
  if (outstanding_ >= size_t(config_.max_pending) || c.active.size() >= size_t(config_.per_connection)) {
    Response r;
    r.id = wire.id; r.status = kOverloaded;
    send_later(fd, r);
    return;
  }
  auto job = std::make_shared<Job>();
  job->fd = fd; job->connection = c.token; job->wire = std::move(wire); job->accepted = Clock::now();
  // fewest outstanding tokens among the workers whose model still works; a poisoned worker (it answers everything with an
  // internal error at once, so it always looks idle) only gets requests when no healthy one is left
  size_t best = 0;
  for (size_t i = 1; i < workers_.size(); ++i) {
    const bool better_health = workers_[i]->healthy() && !workers_[best]->healthy();
    const bool same_health = workers_[i]->healthy() == workers_[best]->healthy();
    if (better_health || (same_health && workers_[i]->load_tokens() < workers_[best]->load_tokens())) best = i;
  }
  job->worker = int(best);
  c.active.emplace(job->wire.id, job);
  ++outstanding_;
  workers_[best]->submit(std::move(job));
}

void Server::on_readable(int fd, uint64_t token) {
  // At most 64 KiB per event; every recv asks for no more than what is left of that allowance.
  uint8_t buffer[16384];
  size_t allowance = 65536;
  while (allowance) {
    const size_t want = std::min(sizeof buffer, allowance);
    const ssize_t got = recv(fd, buffer, want, 0);
    if (got > 0) {
      allowance -= size_t(got);
      auto it = connections_.find(fd);
      if (it == connections_.end() || it->second->token != token) return;
      it->second->frames.feed(buffer, size_t(got), [&](Bytes b) { on_frame(fd, std::move(b)); });
      it = connections_.find(fd);
      if (it == connections_.end() || it->second->token != token) return;
      if (it->second->overflowed) { drop(fd, token); return; }
    } else if (got == 0) { drop(fd, token); return; }
    else if (errno == EINTR) continue;
    else if (errno == EAGAIN || errno == EWOULDBLOCK) return;
    else { drop(fd, token); return; }
  }
}

void Server::on_writable(int fd, uint64_t token) {
  auto it = connections_.find(fd);
  if (it == connections_.end() || it->second->token != token) return;
  Connection& c = *it->second;
  size_t budget = 65536;
  while (!c.outbox.empty() && budget) {
    Bytes& head = c.outbox.front();
    const size_t count = std::min({head.size() - c.sent, size_t(config_.send_chunk), budget});
    const ssize_t n = send(fd, head.data() + c.sent, count, MSG_NOSIGNAL);
    if (n > 0) {
      budget -= size_t(n); c.sent += size_t(n); c.queued_bytes -= size_t(n);
      if (c.sent == head.size()) { c.outbox.pop_front(); c.sent = 0; }
    } else if (n < 0 && errno == EINTR) continue;
    else if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) break;
    else { drop(fd, token); return; }
  }
  arm(fd, c);
}

void Server::accept_all() {
  for (int round = 0; round < 64; ++round) {
    const int fd = accept4(listener_, nullptr, nullptr, SOCK_NONBLOCK | SOCK_CLOEXEC);
    if (fd < 0) {
      if (errno == EINTR) continue;
      if (errno == EAGAIN || errno == EWOULDBLOCK) return;
      throw std::runtime_error("accept");
    }
    if (connections_.size() >= size_t(config_.max_connections)) { close(fd); continue; }
    const uint64_t token = register_fd(fd, Kind::kClient);
    connections_.emplace(fd, std::make_unique<Connection>(token, uint32_t(kRequestHeader + 4 * size_t(config_.capacity))));
    epoll_event e{};
    e.data.u64 = token; e.events = EPOLLIN | EPOLLRDHUP;
    if (epoll_ctl(epoll_, EPOLL_CTL_ADD, fd, &e) < 0) { drop(fd, token); throw std::runtime_error("epoll ADD client"); }
  }
}

void Server::drain_completions() {
  uint64_t count;
  while (read(event_, &count, sizeof count) < 0 && errno == EINTR) {}
  Completion done;
  while (completions_.try_pop(done)) {
    const bool terminal = done.response.kind == kFinal;
    if (terminal) --outstanding_;
    auto it = connections_.find(done.job->fd);
    if (it == connections_.end() || it->second->token != done.job->connection) continue;    // the client is gone
    if (terminal) it->second->active.erase(done.job->wire.id);
    if (!send_later(done.job->fd, done.response)) drop(done.job->fd, done.job->connection);
  }
}

void Server::run() {
  // every queued request holds a connection: take as many descriptors as the process may have
  rlimit files{};
  if (getrlimit(RLIMIT_NOFILE, &files) == 0 && files.rlim_cur < files.rlim_max) {
    files.rlim_cur = files.rlim_max;
    setrlimit(RLIMIT_NOFILE, &files);
  }
  listener_ = socket(AF_INET, SOCK_STREAM | SOCK_NONBLOCK | SOCK_CLOEXEC, 0);
  if (listener_ < 0) throw std::runtime_error("socket");
  const int one = 1;
  setsockopt(listener_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in address{};
  address.sin_family = AF_INET;
  address.sin_port = htons(uint16_t(config_.port));
  if (inet_pton(AF_INET, config_.host.c_str(), &address.sin_addr) != 1 ||
      bind(listener_, reinterpret_cast<sockaddr*>(&address), sizeof address) < 0 || listen(listener_, 1024) < 0)
    throw std::runtime_error("bind/listen");
  epoll_ = epoll_create1(EPOLL_CLOEXEC);
  event_ = eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
  if (epoll_ < 0 || event_ < 0) throw std::runtime_error("epoll/eventfd");
  listener_token_ = register_fd(listener_, Kind::kListener);
  event_token_ = register_fd(event_, Kind::kCompletions);
  for (uint64_t token : {listener_token_, event_token_}) {
    epoll_event e{};
    e.data.u64 = token; e.events = EPOLLIN;
    if (epoll_ctl(epoll_, EPOLL_CTL_ADD, targets_.at(token).fd, &e) < 0) throw std::runtime_error("epoll ADD");
  }
  for (auto& w : workers_) w->start();
  std::cout << "{\"ready\":true,\"model\":\"" << (config_.native ? "native" : "cpu_oracle") << "\",\"port\":" << config_.port << ",\"devices\":[";
  for (size_t i = 0; i < config_.devices.size(); ++i) std::cout << (i ? "," : "") << config_.devices[i];
  std::cout << "],\"max_batch\":" << config_.max_batch << "}" << std::endl;

  epoll_event events[128];
  while (!g_stop) {
    const int n = epoll_wait(epoll_, events, 128, 50);
    if (n < 0) { if (errno == EINTR) continue; throw std::runtime_error("epoll wait"); }
    for (int i = 0; i < n; ++i) {
      const uint64_t token = events[i].data.u64;
      const auto target = targets_.find(token);
      if (target == targets_.end()) continue;               // stale entry of this batch: its registration was retired
      const int fd = target->second.fd;
      const Kind kind = target->second.kind;
      if (kind == Kind::kListener) { accept_all(); continue; }
      if (kind == Kind::kCompletions) { drain_completions(); continue; }
      const uint32_t flags = events[i].events;
      try {
        // identity is re-checked before every action: an earlier action may have closed the connection
        if ((flags & EPOLLIN) && is_live(token, fd)) on_readable(fd, token);
        if ((flags & EPOLLOUT) && is_live(token, fd)) on_writable(fd, token);
        if ((flags & (EPOLLERR | EPOLLHUP | EPOLLRDHUP)) && is_live(token, fd)) drop(fd, token);
      } catch (const std::exception&) { drop(fd, token); }
    }
  }
}

}  // namespace

int main(int argc, char** argv) {
  // The workers' batches change composition from pass to pass: the runtime's speculative continuation of
  // step-by-step decoding (see llm_runtime.cpp) would mostly launch steps nobody asks for.
  setenv("TINYINFER_B200_SPECULATE", "0", 0);
  std::signal(SIGINT, on_signal);
  std::signal(SIGTERM, on_signal);
  try {
    Server server(parse_options(argc, argv));
    server.run();
    return 0;
  } catch (const std::exception& e) {
    std::cerr << "server_failed: " << e.what() << '\n';
    return 1;
  }
}
