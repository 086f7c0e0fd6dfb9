// Parameter server: record wire format, the shard object ("CachePS") and an in-box TCP front end
// with a pipelining client.
//
// Wire / record format (kept from the reference, src/grpc_ps/flatc.h:8-29, parameters.h:4-35):
//   [int32 n][int32 end_offset[n]] { uint64 key; int32 dim; float emb[dim] } x n     (packed)
// end_offset[i] is the byte offset, from the start of the buffer, one past record i.  dim == 0 means
// "key missing" in a Get reply.
//
// CachePS (src/grpc_ps/cache_ps_impl.h:34-143): a BaseKV engine plus Put / Get / LoadFakeData /
// Clear, extended with the gradient verb the north star asks for (UpdateParameter: server-side SGD
// or row-wise Adagrad, math of DGL-KE's push handler, src/kg/kg/dgl-ke/python/dglke/kvserver.py:
// 41-51) and with checkpoints in the record format (LoadCkpt is a stub upstream,
// cache_ps_impl.h:75-80).  Each stored value is [emb[dim], adagrad_state].
//
// Transport: the gRPC service (GetParameter / PutParameter / Command, src/grpc_ps/proto/ps.proto:
// 39-43) becomes a framed protocol over a loopback TCP socket: {u32 magic, u32 op, u64 len}
// followed by the payload.  The client splits a request into sub-requests of at most
// max_keys_per_request keys (2000 upstream, grpc_ps_client.h:31), sends them back to back and then
// collects the replies, which is the asynchronous window of the reference client.
#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <unistd.h>

#include "common/rs_common.h"
#include "runtime/base.h"
#include "runtime/json_lite.h"
#include "runtime/kv_engine.h"
#include "runtime/task_provider.h"

namespace rs {

// ---------------------------------------------------------------- wire format
struct WireWriter {
  std::vector<char> buf;
  int n = 0;
  explicit WireWriter(int count) : n(count) { buf.resize(4 + 4 * static_cast<size_t>(count)); memcpy(buf.data(), &n, 4); }
  void add(int i, uint64_t key, int dim, const float* emb) {
    const size_t at = buf.size();
    buf.resize(at + 12 + 4 * static_cast<size_t>(dim));
    memcpy(buf.data() + at, &key, 8);
    memcpy(buf.data() + at + 8, &dim, 4);
    if (dim) memcpy(buf.data() + at + 12, emb, 4 * static_cast<size_t>(dim));
    const int end = static_cast<int>(buf.size());
    memcpy(buf.data() + 4 + 4 * static_cast<size_t>(i), &end, 4);
  }
};

struct WireReader {
  const char* p;
  size_t len;
  int n = 0;
  bool ok = false;
  WireReader(const void* data, size_t bytes) : p(static_cast<const char*>(data)), len(bytes) {
    if (bytes < 4) return;
    memcpy(&n, p, 4);
    ok = n >= 0 && bytes >= 4 + 4 * static_cast<size_t>(n);
  }
  bool item(int i, uint64_t* key, int* dim, const float** emb) const {
    int end, beg = 4 + 4 * n;
    memcpy(&end, p + 4 + 4 * static_cast<size_t>(i), 4);
    if (i > 0) memcpy(&beg, p + 4 + 4 * static_cast<size_t>(i - 1), 4);
    if (beg < 0 || end < beg + 12 || static_cast<size_t>(end) > len) return false;
    memcpy(key, p + beg, 8);
    memcpy(dim, p + beg + 8, 4);
    if (*dim < 0 || beg + 12 + 4 * static_cast<long long>(*dim) != end) return false;
    *emb = reinterpret_cast<const float*>(p + beg + 12);
    return true;
  }
};

// ---------------------------------------------------------------- CachePS
class CachePS {
 public:
  CachePS(const std::string& engine, const std::string& json) {
    JsonLite j(json);
    dim_ = static_cast<int>(j.i64("dim", j.i64("value_size", 128) / 4));
    KVConfig c = ParseKVConfig(json);
    c.value_size = static_cast<uint32_t>(dim_ + 1) * 4;  // embedding + optimizer state
    kv_ = CreateKV(engine, c);
    optimizer_ = j.str("optimizer", "rowwise_adagrad") == "sgd" ? 0 : 1;
    lr_ = static_cast<float>(j.num("lr", 0.01));
    eps_ = static_cast<float>(j.num("eps", 1e-10));
  }
  bool ok() const { return kv_ != nullptr; }
  int dim() const { return dim_; }
  BaseKV* kv() { return kv_.get(); }

  void Put(const uint64_t* keys, size_t n, const float* values) {
    std::vector<float> rec(dim_ + 1);
    for (size_t i = 0; i < n; ++i) {
      // keep an existing optimizer state
      if (!kv_->Get(keys[i], rec.data())) rec[dim_] = 0.f;
      memcpy(rec.data(), values + i * dim_, 4 * static_cast<size_t>(dim_));
      kv_->Put(keys[i], rec.data());
    }
  }
  // out: [n, dim]; found[i] = 1/0 (missing rows are zero)
  void Get(const uint64_t* keys, size_t n, float* out, uint8_t* found) {
    auto body = [&](size_t b, size_t e, int) {
      std::vector<float> rec(dim_ + 1);
      for (size_t i = b; i < e; ++i) {
        const bool ok = kv_->Get(keys[i], rec.data());
        if (ok) memcpy(out + i * dim_, rec.data(), 4 * static_cast<size_t>(dim_));
        else memset(out + i * dim_, 0, 4 * static_cast<size_t>(dim_));
        if (found) found[i] = ok ? 1 : 0;
      }
    };
    if (n >= 2048) ThreadPool::global().parallel_for(n, body);
    else body(0, n, 0);
  }
  // Server-side optimizer.  Duplicate keys: state takes every occurrence's mean(g^2) first, then every
  // occurrence is applied with the post-step state (row-wise Adagrad); SGD sums.  Unknown keys are skipped.
  size_t Update(const uint64_t* keys, size_t n, const float* grads) {
    std::lock_guard<std::mutex> lk(update_mu_);
    std::vector<float> rec(dim_ + 1);
    size_t applied = 0;
    if (optimizer_ == 1) {
      for (size_t i = 0; i < n; ++i) {
        if (!kv_->Get(keys[i], rec.data())) continue;
        double s = 0;
        for (int d = 0; d < dim_; ++d) s += static_cast<double>(grads[i * dim_ + d]) * grads[i * dim_ + d];
        rec[dim_] += static_cast<float>(s / dim_);
        kv_->Put(keys[i], rec.data());
      }
    }
    for (size_t i = 0; i < n; ++i) {
      if (!kv_->Get(keys[i], rec.data())) continue;
      const float scale = optimizer_ == 1 ? lr_ / (std::sqrt(rec[dim_]) + eps_) : lr_;
      for (int d = 0; d < dim_; ++d) rec[d] -= scale * grads[i * dim_ + d];
      kv_->Put(keys[i], rec.data());
      ++applied;
    }
    return applied;
  }
  // Keys 0 .. n-1 with value = key.  A count beyond the engine's capacity (a garbled or hostile request) is cut down
  // to the capacity instead of looping over it; returns how many keys were written.
  uint64_t LoadFakeData(uint64_t n) {
    n = std::min<uint64_t>(n, kv_->config().capacity);
    auto body = [&](size_t b, size_t e, int) {
      std::vector<float> rec(dim_ + 1);
      for (size_t k = b; k < e; ++k) {
        std::fill(rec.begin(), rec.end() - 1, static_cast<float>(k));
        rec[dim_] = 0.f;
        kv_->Put(k, rec.data());
      }
    };
    ThreadPool::global().parallel_for(n, body);
    return n;
  }
  void Clear() { kv_->Clear(); }

  // Checkpoint = one record-format file holding every (key, dim + 1, [emb, state]).
  int SaveCkpt(const std::string& path) {
    const uint64_t n = kv_->Size();
    std::vector<uint64_t> keys(n);
    const size_t m = kv_->Keys(keys.data(), n);
    FILE* f = fopen(path.c_str(), "wb");
    if (!f) return set_error(RS_ERR_IO, "cannot write %s", path.c_str());
    const size_t chunk = 1 << 16;
    std::vector<float> rec(dim_ + 1);
    uint64_t header[2] = {0x52534232434B5054ull, m};
    fwrite(header, 8, 2, f);
    for (size_t b = 0; b < m; b += chunk) {
      const size_t e = std::min(m, b + chunk);
      WireWriter w(static_cast<int>(e - b));
      for (size_t i = b; i < e; ++i) {
        if (!kv_->Get(keys[i], rec.data())) std::fill(rec.begin(), rec.end(), 0.f);
        w.add(static_cast<int>(i - b), keys[i], dim_ + 1, rec.data());
      }
      const uint64_t bytes = w.buf.size();
      fwrite(&bytes, 8, 1, f);
      fwrite(w.buf.data(), 1, w.buf.size(), f);
    }
    fclose(f);
    return RS_OK;
  }
  int LoadCkpt(const std::string& path) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return set_error(RS_ERR_IO, "cannot read %s", path.c_str());
    uint64_t header[2];
    if (fread(header, 8, 2, f) != 2 || header[0] != 0x52534232434B5054ull) {
      fclose(f);
      return set_error(RS_ERR_IO, "%s is not a parameter-server checkpoint", path.c_str());
    }
    fseek(f, 0, SEEK_END);
    const uint64_t file_bytes = static_cast<uint64_t>(ftell(f));
    fseek(f, 16, SEEK_SET);
    uint64_t loaded = 0, bytes;
    std::vector<char> buf;
    while (fread(&bytes, 8, 1, f) == 1) {
      if (bytes > file_bytes) { fclose(f); return set_error(RS_ERR_IO, "%s holds a block longer than the file", path.c_str()); }
      buf.resize(bytes);
      if (fread(buf.data(), 1, bytes, f) != bytes) { fclose(f); return set_error(RS_ERR_IO, "%s is truncated", path.c_str()); }
      WireReader r(buf.data(), bytes);
      if (!r.ok) { fclose(f); return set_error(RS_ERR_IO, "%s holds a corrupt block", path.c_str()); }
      for (int i = 0; i < r.n; ++i) {
        uint64_t key; int dim; const float* emb;
        if (!r.item(i, &key, &dim, &emb) || dim != dim_ + 1) { fclose(f); return set_error(RS_ERR_IO, "%s: bad record", path.c_str()); }
        kv_->Put(key, emb);
        ++loaded;
      }
    }
    fclose(f);
    if (loaded != header[1]) return set_error(RS_ERR_IO, "%s is truncated: %llu of %llu records", path.c_str(),
                                              (unsigned long long)loaded, (unsigned long long)header[1]);
    return RS_OK;
  }

 private:
  std::unique_ptr<BaseKV> kv_;
  int dim_ = 32;
  int optimizer_ = 1;
  float lr_ = 0.01f, eps_ = 1e-10f;
  std::mutex update_mu_;
};

// ---------------------------------------------------------------- framed TCP transport
constexpr uint32_t kPsMagic = 0x52535053;  // "RSPS"
enum PsOp : uint32_t { OP_GET = 1, OP_PUT = 2, OP_UPDATE = 3, OP_CLEAR = 4, OP_FAKE = 5, OP_SAVE = 6, OP_LOAD = 7, OP_STATS = 8, OP_BYE = 9, OP_PRIORITY = 10 };
struct Frame { uint32_t magic, op; uint64_t len; };
// A request larger than this (or naming more keys) is a protocol error: the connection is closed instead of sizing
// buffers from a header that may be garbage.  Clients split their batches far below both (max_per_req).
constexpr uint64_t kMaxFrameBytes = 256ull << 20;
constexpr size_t kMaxKeysPerRequest = size_t{1} << 22;

static bool send_all(int fd, const void* p, size_t n) {
  const char* c = static_cast<const char*>(p);
  while (n) {
    const ssize_t w = ::send(fd, c, n, MSG_NOSIGNAL);
    if (w <= 0) { if (errno == EINTR) continue; return false; }
    c += w; n -= static_cast<size_t>(w);
  }
  return true;
}
static bool recv_all(int fd, void* p, size_t n) {
  char* c = static_cast<char*>(p);
  while (n) {
    const ssize_t r = ::recv(fd, c, n, 0);
    if (r <= 0) { if (r < 0 && errno == EINTR) continue; return false; }
    c += r; n -= static_cast<size_t>(r);
  }
  return true;
}
static bool send_frame(int fd, uint32_t op, const void* payload, uint64_t len) {
  Frame f{kPsMagic, op, len};
  return send_all(fd, &f, sizeof(f)) && (len == 0 || send_all(fd, payload, len));
}

// Two serving modes.  workers == 0: every connection's thread reads a request, executes it and answers (the reference's
// synchronous server, src/grpc_ps/grpc_ps_server.cpp:35-118).  workers > 0: the connection threads are only the front
// end; requests go through a TaskProvider (FIFO or priority levels, keyed by connection) to a pool of worker threads,
// and a per-connection sequencer sends the answers in request order, because clients pipeline their sub-requests
// (the reference's asynchronous server: completion queue -> task queue -> worker coroutines,
// src/grpc_ps/grpc_ps_server_async.cpp:56-96, 246-318).  OP_PRIORITY raises the sender's class by one level.
class PsServer {
 public:
  PsServer(CachePS* ps, int port, int workers = 0, const std::string& scheduler = "fifo", int levels = 7,
           const std::string& bind_host = "127.0.0.1")
      : ps_(ps), port_(port), n_workers_(workers < 0 ? 0 : workers), bind_host_(bind_host == "localhost" ? "127.0.0.1" : bind_host) {
    if (n_workers_ > 0) {
      if (scheduler == "priority") provider_ = std::make_unique<PriorityProvider<Task>>(levels);
      else provider_ = std::make_unique<FifoProvider<Task>>();
    }
  }
  ~PsServer() { Stop(); }
  int Start() {
    lfd_ = ::socket(AF_INET, SOCK_STREAM, 0);
    if (lfd_ < 0) return set_error(RS_ERR_IO, "socket() failed");
    int one = 1;
    setsockopt(lfd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in a{};
    a.sin_family = AF_INET;
    if (inet_pton(AF_INET, bind_host_.c_str(), &a.sin_addr) != 1) {      // loopback by default; "0.0.0.0" serves every interface
      ::close(lfd_);
      lfd_ = -1;
      return set_error(RS_ERR_INVALID, "%s is not an IPv4 address to listen on", bind_host_.c_str());
    }
    a.sin_port = htons(static_cast<uint16_t>(port_));
    if (::bind(lfd_, reinterpret_cast<sockaddr*>(&a), sizeof(a)) != 0 || ::listen(lfd_, 64) != 0) {
      ::close(lfd_);
      lfd_ = -1;
      return set_error(RS_ERR_IO, "cannot listen on %s:%d", bind_host_.c_str(), port_);
    }
    socklen_t sl = sizeof(a);
    getsockname(lfd_, reinterpret_cast<sockaddr*>(&a), &sl);
    port_ = ntohs(a.sin_port);
    running_ = true;
    for (int i = 0; i < n_workers_; ++i) pool_.emplace_back([this] { WorkerLoop(); });
    acceptor_ = std::thread([this] { AcceptLoop(); });
    return RS_OK;
  }
  // Once per period: requests, keys and reply payload served since the last line, to stderr (only while there is
  // traffic) and into `out` for callers that want the last reading.  The reference's asynchronous server prints its
  // MB/s once a second from such a thread (src/grpc_ps/grpc_ps_server_async.cpp:109-117).
  void StartMonitor(int period_ms, bool print) {
    std::lock_guard<std::mutex> lk(mon_mu_);
    if (monitor_.joinable()) return;
    mon_stop_ = false;
    monitor_ = std::thread([this, period_ms, print] {
      uint64_t r0 = requests_.load(), k0 = keys_.load();
      auto t0 = std::chrono::steady_clock::now();
      std::unique_lock<std::mutex> lk(mon_mu_);
      while (!mon_stop_) {
        if (mon_cv_.wait_for(lk, std::chrono::milliseconds(period_ms), [this] { return mon_stop_; })) break;
        const uint64_t r1 = requests_.load(), k1 = keys_.load();
        const auto t1 = std::chrono::steady_clock::now();
        const double sec = std::chrono::duration<double>(t1 - t0).count();
        const double kreq = (r1 - r0) / sec / 1e3, mkeys = (k1 - k0) / sec / 1e6;
        const double mbs = (k1 - k0) * (12.0 + 4.0 * ps_->dim()) / sec / 1e6;       // record bytes per served key
        mon_last_[0] = kreq; mon_last_[1] = mkeys; mon_last_[2] = mbs;
        mon_lines_.fetch_add(1, std::memory_order_relaxed);
        if (print && r1 != r0) fprintf(stderr, "PS throughput: %.3f Kreq/s %.3f Mkeys/s %.1f MB/s\n", kreq, mkeys, mbs);
        r0 = r1; k0 = k1; t0 = t1;
      }
    });
  }
  void StopMonitor() {
    {
      std::lock_guard<std::mutex> lk(mon_mu_);
      mon_stop_ = true;
    }
    mon_cv_.notify_all();
    if (monitor_.joinable()) monitor_.join();
  }
  // out[0..2] = Kreq/s, Mkeys/s, MB/s of the last period; returns how many periods have been measured.
  uint64_t MonitorLast(double* out) {
    std::lock_guard<std::mutex> lk(mon_mu_);
    for (int i = 0; i < 3; ++i) out[i] = mon_last_[i];
    return mon_lines_.load();
  }
  void Stop() {
    StopMonitor();
    if (!running_.exchange(false)) return;
    ::shutdown(lfd_, SHUT_RDWR);
    ::close(lfd_);
    if (acceptor_.joinable()) acceptor_.join();
    std::vector<std::thread> ws;
    {
      std::lock_guard<std::mutex> lk(mu_);
      for (int fd : conns_) ::shutdown(fd, SHUT_RDWR);
      ws.swap(workers_);
    }
    for (auto& t : ws) t.join();
    if (provider_) provider_->Close();
    for (auto& t : pool_) t.join();
    pool_.clear();
  }
  int port() const { return port_; }
  uint64_t requests() const { return requests_.load(); }
  uint64_t keys_served() const { return keys_.load(); }
  uint64_t pooled_requests() const { return pooled_.load(); }

 private:
  struct Conn {
    int fd;
    uint64_t id;
    std::mutex mu;                               // sequencer state and the socket's send side
    uint64_t next_send = 0;
    std::unordered_map<uint64_t, std::pair<uint32_t, std::vector<char>>> ready;
    bool dead = false;
  };
  struct Task {
    std::shared_ptr<Conn> conn;
    uint64_t seq = 0;
    Frame f{};
    std::vector<char> in;
  };
  void AcceptLoop() {
    uint64_t next_id = 1;
    while (running_) {
      const int fd = ::accept(lfd_, nullptr, nullptr);
      if (fd < 0) { if (!running_) break; continue; }
      int one = 1;
      setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      std::lock_guard<std::mutex> lk(mu_);
      conns_.push_back(fd);
      const uint64_t id = next_id++;
      workers_.emplace_back([this, fd, id] { Serve(fd, id); });
    }
  }
  void Serve(int fd, uint64_t id) {
    auto conn = std::make_shared<Conn>();
    conn->fd = fd;
    conn->id = id;
    try {
      ServeLoop(conn);
    } catch (const std::exception&) {
      // e.g. std::bad_alloc on a hostile size: this connection ends, the server and its other connections go on
    }
    {
      // The descriptor leaves the server's list before it is closed (Stop() shuts down what is listed, and a closed
      // number may already belong to somebody else's socket), and it is closed under the connection's lock so that no
      // worker sends on a reused number.  Answers that workers still hold for this connection are dropped.
      std::lock_guard<std::mutex> sl(mu_);
      std::lock_guard<std::mutex> lk(conn->mu);
      conns_.erase(std::remove(conns_.begin(), conns_.end(), fd), conns_.end());
      conn->dead = true;
      ::close(fd);
    }
  }
  // Executes one request.  False: protocol error, the connection must end.
  bool Process(const Frame& f, std::vector<char>& in, uint32_t* rop, std::vector<char>* reply) {
    const int dim = ps_->dim();
    *rop = f.op;
    auto put8 = [&](uint64_t v) {
      reply->resize(8);
      memcpy(reply->data(), &v, 8);
    };
    if (f.op == OP_GET) {
      const size_t n = f.len / 8;
      if (f.len % 8 != 0 || n > kMaxKeysPerRequest) return false;
      const uint64_t* keys = reinterpret_cast<const uint64_t*>(in.data());
      std::vector<float> vals(n * dim);
      std::vector<uint8_t> found(n);
      ps_->Get(keys, n, vals.data(), found.data());
      WireWriter w(static_cast<int>(n));
      for (size_t i = 0; i < n; ++i) w.add(static_cast<int>(i), keys[i], found[i] ? dim : 0, vals.data() + i * dim);
      keys_.fetch_add(n, std::memory_order_relaxed);
      reply->assign(w.buf.begin(), w.buf.end());
    } else if (f.op == OP_PUT || f.op == OP_UPDATE) {
      WireReader r(in.data(), f.len);
      uint64_t done = 0;
      if (r.ok && static_cast<size_t>(r.n) <= kMaxKeysPerRequest) {
        std::vector<uint64_t> keys;
        std::vector<float> vals;
        for (int i = 0; i < r.n; ++i) {
          uint64_t key; int d; const float* emb;
          if (!r.item(i, &key, &d, &emb) || d != dim) continue;
          keys.push_back(key);
          vals.insert(vals.end(), emb, emb + dim);
        }
        if (f.op == OP_PUT) { ps_->Put(keys.data(), keys.size(), vals.data()); done = keys.size(); }
        else done = ps_->Update(keys.data(), keys.size(), vals.data());
        keys_.fetch_add(keys.size(), std::memory_order_relaxed);
      }
      put8(done);
    } else if (f.op == OP_CLEAR) {
      ps_->Clear();
      put8(1);
    } else if (f.op == OP_FAKE) {
      uint64_t n = 0;
      if (f.len >= 8) memcpy(&n, in.data(), 8);
      put8(ps_->LoadFakeData(n));
    } else if (f.op == OP_SAVE || f.op == OP_LOAD) {
      const std::string path(in.data(), in.size());
      put8(f.op == OP_SAVE ? ps_->SaveCkpt(path) : ps_->LoadCkpt(path));
    } else if (f.op == OP_STATS) {
      uint64_t s[4] = {ps_->kv()->Size(), requests_.load(), keys_.load(), pooled_.load()};
      reply->resize(sizeof(s));
      memcpy(reply->data(), s, sizeof(s));
    } else {
      return false;
    }
    return true;
  }
  void ServeLoop(const std::shared_ptr<Conn>& conn) {
    const int fd = conn->fd;
    std::vector<char> in, reply;
    uint64_t seq = 0;
    while (running_) {
      Frame f;
      if (!recv_all(fd, &f, sizeof(f)) || f.magic != kPsMagic || f.len > kMaxFrameBytes) break;
      in.resize(f.len);
      if (f.len && !recv_all(fd, in.data(), f.len)) break;
      requests_.fetch_add(1, std::memory_order_relaxed);
      if (f.op == OP_PRIORITY) {                       // answered by the front end; travels through the sequencer
        uint64_t level = 1;
        if (provider_) {
          provider_->ImprovePriority(conn->id);
          level = static_cast<uint64_t>(provider_->LevelOf(conn->id));
        }
        std::vector<char> r(8);
        memcpy(r.data(), &level, 8);
        if (!Deliver(conn, seq++, f.op, std::move(r))) break;
        continue;
      }
      if (!provider_) {
        uint32_t rop;
        reply.clear();
        if (!Process(f, in, &rop, &reply)) break;
        if (!send_frame(fd, rop, reply.data(), reply.size())) break;
        continue;
      }
      if (f.op < OP_GET || f.op > OP_STATS) break;     // unknown verbs end the connection here, not in a worker
      Task t;
      t.conn = conn;
      t.seq = seq++;
      t.f = f;
      t.in.swap(in);
      provider_->Put(std::move(t), conn->id);
    }
  }
  void WorkerLoop() {
    Task t;
    while (provider_->Get(&t)) {
      uint32_t rop = t.f.op;
      std::vector<char> reply;
      bool ok = false;
      try {
        ok = Process(t.f, t.in, &rop, &reply);
      } catch (const std::exception&) {
        ok = false;
      }
      pooled_.fetch_add(1, std::memory_order_relaxed);
      if (!ok) {
        std::lock_guard<std::mutex> lk(t.conn->mu);
        if (!t.conn->dead) ::shutdown(t.conn->fd, SHUT_RDWR);   // its reader thread sees the end and closes
      } else {
        Deliver(t.conn, t.seq, rop, std::move(reply));
      }
      t = Task();
    }
  }
  // Sends the answer of request `seq` once every earlier answer of the connection has gone out.
  bool Deliver(const std::shared_ptr<Conn>& c, uint64_t seq, uint32_t op, std::vector<char> reply) {
    std::lock_guard<std::mutex> lk(c->mu);
    if (c->dead) return false;
    c->ready.emplace(seq, std::make_pair(op, std::move(reply)));
    while (true) {
      auto it = c->ready.find(c->next_send);
      if (it == c->ready.end()) return true;
      const bool sent = send_frame(c->fd, it->second.first, it->second.second.data(), it->second.second.size());
      c->ready.erase(it);
      ++c->next_send;
      if (!sent) {
        ::shutdown(c->fd, SHUT_RDWR);
        return false;
      }
    }
  }
  CachePS* ps_;
  int port_, lfd_ = -1;
  const int n_workers_;
  const std::string bind_host_;
  std::unique_ptr<TaskProvider<Task>> provider_;
  std::atomic<bool> running_{false};
  std::thread acceptor_;
  std::mutex mu_;
  std::vector<int> conns_;
  std::vector<std::thread> workers_, pool_;
  std::atomic<uint64_t> requests_{0}, keys_{0}, pooled_{0};
  std::mutex mon_mu_;
  std::condition_variable mon_cv_;
  std::thread monitor_;
  bool mon_stop_ = false;
  double mon_last_[3] = {0, 0, 0};
  std::atomic<uint64_t> mon_lines_{0};
};

class PsClient {
 public:
  int Connect(const std::string& host, int port) {
    fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd_ < 0) return set_error(RS_ERR_IO, "socket() failed");
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_port = htons(static_cast<uint16_t>(port));
    if (inet_pton(AF_INET, host == "localhost" ? "127.0.0.1" : host.c_str(), &a.sin_addr) != 1 ||
        ::connect(fd_, reinterpret_cast<sockaddr*>(&a), sizeof(a)) != 0) {
      ::close(fd_);
      fd_ = -1;
      return set_error(RS_ERR_IO, "cannot connect to parameter server %s:%d", host.c_str(), port);
    }
    int one = 1;
    setsockopt(fd_, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    return RS_OK;
  }
  ~PsClient() { if (fd_ >= 0) ::close(fd_); }

  // out [n, dim]; found [n] optional.  Sub-requests are pipelined.
  int Get(const uint64_t* keys, size_t n, int dim, float* out, uint8_t* found, size_t max_per_req) {
    std::lock_guard<std::mutex> lk(mu_);
    const size_t nreq = (n + max_per_req - 1) / max_per_req;
    for (size_t r = 0; r < nreq; ++r) {
      const size_t b = r * max_per_req, e = std::min(n, b + max_per_req);
      if (!send_frame(fd_, OP_GET, keys + b, (e - b) * 8)) return set_error(RS_ERR_IO, "parameter server connection lost");
    }
    std::vector<char> in;
    for (size_t r = 0; r < nreq; ++r) {
      const size_t b = r * max_per_req, e = std::min(n, b + max_per_req);
      Frame f;
      if (!recv_all(fd_, &f, sizeof(f)) || f.magic != kPsMagic) return set_error(RS_ERR_IO, "parameter server connection lost");
      in.resize(f.len);
      if (f.len && !recv_all(fd_, in.data(), f.len)) return set_error(RS_ERR_IO, "parameter server connection lost");
      WireReader w(in.data(), f.len);
      if (!w.ok || static_cast<size_t>(w.n) != e - b) return set_error(RS_ERR_IO, "malformed Get reply");
      for (size_t i = b; i < e; ++i) {
        uint64_t key; int d; const float* emb;
        if (!w.item(static_cast<int>(i - b), &key, &d, &emb) || key != keys[i]) return set_error(RS_ERR_IO, "malformed Get reply");
        if (d == dim) memcpy(out + i * dim, emb, 4 * static_cast<size_t>(dim));
        else memset(out + i * dim, 0, 4 * static_cast<size_t>(dim));   // dim 0 = key missing
        if (found) found[i] = d == dim ? 1 : 0;
      }
    }
    return RS_OK;
  }
  int PutOrUpdate(uint32_t op, const uint64_t* keys, size_t n, int dim, const float* vals, size_t max_per_req, uint64_t* done) {
    std::lock_guard<std::mutex> lk(mu_);
    const size_t nreq = (n + max_per_req - 1) / max_per_req;
    for (size_t r = 0; r < nreq; ++r) {
      const size_t b = r * max_per_req, e = std::min(n, b + max_per_req);
      WireWriter w(static_cast<int>(e - b));
      for (size_t i = b; i < e; ++i) w.add(static_cast<int>(i - b), keys[i], dim, vals + i * dim);
      if (!send_frame(fd_, op, w.buf.data(), w.buf.size())) return set_error(RS_ERR_IO, "parameter server connection lost");
    }
    uint64_t total = 0;
    for (size_t r = 0; r < nreq; ++r) {
      Frame f;
      uint64_t d = 0;
      if (!recv_all(fd_, &f, sizeof(f)) || f.len != 8 || !recv_all(fd_, &d, 8)) return set_error(RS_ERR_IO, "parameter server connection lost");
      total += d;
    }
    if (done) *done = total;
    return RS_OK;
  }
  int Command(uint32_t op, const void* payload, size_t len, void* reply, size_t reply_cap) {
    std::lock_guard<std::mutex> lk(mu_);
    if (!send_frame(fd_, op, payload, len)) return set_error(RS_ERR_IO, "parameter server connection lost");
    Frame f;
    if (!recv_all(fd_, &f, sizeof(f)) || f.len > reply_cap) return set_error(RS_ERR_IO, "parameter server connection lost");
    if (f.len && !recv_all(fd_, reply, f.len)) return set_error(RS_ERR_IO, "parameter server connection lost");
    return RS_OK;
  }

 private:
  int fd_ = -1;
  std::mutex mu_;
};

}  // namespace rs

// ================================================================ C ABI
using rs::CachePS;
using rs::PsClient;
using rs::PsServer;

RS_API long long rs_wire_packed_size(long long n, int dim) { return 4 + 4 * n + n * (12 + 4ll * dim); }
// Packs n records of a common dim (dims may be overridden per item by `dims`, 0 = missing).
RS_API int rs_wire_pack(const unsigned long long* keys, long long n, int dim, const float* values, const int* dims, void* out,
                        long long cap, long long* written) {
  RS_REQUIRE(n >= 0 && (n == 0 || (keys && (values || dim == 0))) && out && written, "rs_wire_pack: null argument");
  if (dims)
    for (long long i = 0; i < n; ++i) RS_REQUIRE(dims[i] >= 0 && dims[i] <= dim, "rs_wire_pack: record %lld has dim %d outside [0, %d]", i, dims[i], dim);
  rs::WireWriter w(static_cast<int>(n));
  for (long long i = 0; i < n; ++i) w.add(static_cast<int>(i), keys[i], dims ? dims[i] : dim, values + i * dim);
  RS_REQUIRE(static_cast<long long>(w.buf.size()) <= cap, "rs_wire_pack: buffer too small (%zu > %lld)", w.buf.size(), cap);
  memcpy(out, w.buf.data(), w.buf.size());
  *written = static_cast<long long>(w.buf.size());
  return RS_OK;
}
RS_API int rs_wire_count(const void* buf, long long len) {
  rs::WireReader r(buf, static_cast<size_t>(len));
  return r.ok ? r.n : -1;
}
// values_out [n, dim] (zero rows where the record's dim != dim), dims_out [n].
RS_API int rs_wire_unpack(const void* buf, long long len, int dim, unsigned long long* keys_out, int* dims_out, float* values_out) {
  rs::WireReader r(buf, static_cast<size_t>(len));
  if (!r.ok) return rs::set_error(RS_ERR_INVALID, "malformed record buffer");
  for (int i = 0; i < r.n; ++i) {
    uint64_t key; int d; const float* emb;
    if (!r.item(i, &key, &d, &emb)) return rs::set_error(RS_ERR_INVALID, "malformed record %d", i);
    keys_out[i] = key;
    if (dims_out) dims_out[i] = d;
    if (values_out) {
      if (d == dim) memcpy(values_out + static_cast<size_t>(i) * dim, emb, 4 * static_cast<size_t>(dim));
      else memset(values_out + static_cast<size_t>(i) * dim, 0, 4 * static_cast<size_t>(dim));
    }
  }
  return RS_OK;
}

RS_API int rs_ps_create(const char* engine, const char* json, void** out) {
  RS_REQUIRE(engine && out, "rs_ps_create: null argument");
  RS_NOEXCEPT_BODY(
    auto* ps = new CachePS(engine, json ? json : "{}");
    if (!ps->ok()) { delete ps; return RS_ERR_INVALID; }
    *out = ps;
    return RS_OK;
  )
}
RS_API int rs_ps_destroy(void* ps) { delete static_cast<CachePS*>(ps); return RS_OK; }
RS_API int rs_ps_dim(void* ps) { return static_cast<CachePS*>(ps)->dim(); }
RS_API unsigned long long rs_ps_size(void* ps) { return static_cast<CachePS*>(ps)->kv()->Size(); }
RS_API int rs_ps_put(void* ps, const unsigned long long* keys, long long n, const float* values) {
  static_cast<CachePS*>(ps)->Put(reinterpret_cast<const uint64_t*>(keys), static_cast<size_t>(n), values);
  return RS_OK;
}
RS_API int rs_ps_get(void* ps, const unsigned long long* keys, long long n, float* out, unsigned char* found) {
  static_cast<CachePS*>(ps)->Get(reinterpret_cast<const uint64_t*>(keys), static_cast<size_t>(n), out, found);
  return RS_OK;
}
RS_API int rs_ps_update(void* ps, const unsigned long long* keys, long long n, const float* grads, long long* applied) {
  const size_t a = static_cast<CachePS*>(ps)->Update(reinterpret_cast<const uint64_t*>(keys), static_cast<size_t>(n), grads);
  if (applied) *applied = static_cast<long long>(a);
  return RS_OK;
}
RS_API int rs_ps_load_fake(void* ps, unsigned long long n) { RS_NOEXCEPT_BODY(static_cast<CachePS*>(ps)->LoadFakeData(n); return RS_OK;) }
RS_API int rs_ps_clear(void* ps) { static_cast<CachePS*>(ps)->Clear(); return RS_OK; }
RS_API int rs_ps_save(void* ps, const char* path) { RS_NOEXCEPT_BODY(return static_cast<CachePS*>(ps)->SaveCkpt(path);) }
RS_API int rs_ps_load(void* ps, const char* path) { RS_NOEXCEPT_BODY(return static_cast<CachePS*>(ps)->LoadCkpt(path);) }

// port 0 picks a free port; *port_out receives the bound port.
RS_API int rs_ps_server_start(void* ps, int port, void** server_out, int* port_out) {
  RS_REQUIRE(ps && server_out, "rs_ps_server_start: null argument");
  auto* s = new PsServer(static_cast<CachePS*>(ps), port);
  const int rc = s->Start();
  if (rc != RS_OK) { delete s; return rc; }
  *server_out = s;
  if (port_out) *port_out = s->port();
  return RS_OK;
}
// workers > 0: front-end threads + a worker pool behind a "fifo" or "priority" task provider.
RS_API int rs_ps_server_start_pool(void* ps, int port, int workers, const char* scheduler, int levels, void** server_out, int* port_out) {
  RS_REQUIRE(ps && server_out, "rs_ps_server_start_pool: null argument");
  const std::string sched = scheduler ? scheduler : "fifo";
  RS_REQUIRE(sched == "fifo" || sched == "priority", "rs_ps_server_start_pool: scheduler must be fifo or priority");
  RS_NOEXCEPT_BODY(
    auto* s = new PsServer(static_cast<CachePS*>(ps), port, workers, sched, levels);
    const int rc = s->Start();
    if (rc != RS_OK) { delete s; return rc; }
    *server_out = s;
    if (port_out) *port_out = s->port();
    return RS_OK;
  )
}
// The general form: listens on `host` (an IPv4 address; the two entry points above listen on 127.0.0.1, the reference's
// server on 0.0.0.0:15000, src/grpc_ps/grpc_ps_server.cpp:129); workers == 0 is the synchronous mode.
RS_API int rs_ps_server_start_on(void* ps, const char* host, int port, int workers, const char* scheduler, int levels,
                                 void** server_out, int* port_out) {
  RS_REQUIRE(ps && server_out && host, "rs_ps_server_start_on: null argument");
  const std::string sched = scheduler ? scheduler : "fifo";
  RS_REQUIRE(sched == "fifo" || sched == "priority", "rs_ps_server_start_on: scheduler must be fifo or priority");
  RS_NOEXCEPT_BODY(
    auto* s = new PsServer(static_cast<CachePS*>(ps), port, workers, sched, levels, host);
    const int rc = s->Start();
    if (rc != RS_OK) { delete s; return rc; }
    *server_out = s;
    if (port_out) *port_out = s->port();
    return RS_OK;
  )
}
RS_API int rs_ps_server_stop(void* server) { delete static_cast<PsServer*>(server); return RS_OK; }
RS_API int rs_ps_server_monitor_start(void* server, int period_ms, int print) {
  RS_REQUIRE(server && period_ms > 0, "rs_ps_server_monitor_start: bad argument");
  RS_NOEXCEPT_BODY(static_cast<PsServer*>(server)->StartMonitor(period_ms, print != 0); return RS_OK;)
}
RS_API int rs_ps_server_monitor_stop(void* server) {
  static_cast<PsServer*>(server)->StopMonitor();
  return RS_OK;
}
RS_API unsigned long long rs_ps_server_monitor_last(void* server, double* out3) {
  return static_cast<PsServer*>(server)->MonitorLast(out3);
}

RS_API int rs_ps_client_connect(const char* host, int port, void** out) {
  RS_REQUIRE(host && out, "rs_ps_client_connect: null argument");
  auto* c = new PsClient();
  const int rc = c->Connect(host, port);
  if (rc != RS_OK) { delete c; return rc; }
  *out = c;
  return RS_OK;
}
RS_API int rs_ps_client_close(void* c) { delete static_cast<PsClient*>(c); return RS_OK; }
RS_API int rs_ps_client_get(void* c, const unsigned long long* keys, long long n, int dim, float* out, unsigned char* found,
                            int max_per_req) {
  return static_cast<PsClient*>(c)->Get(reinterpret_cast<const uint64_t*>(keys), static_cast<size_t>(n), dim, out, found,
                                        static_cast<size_t>(max_per_req > 0 ? max_per_req : 2000));
}
RS_API int rs_ps_client_put(void* c, const unsigned long long* keys, long long n, int dim, const float* values, int max_per_req) {
  return static_cast<PsClient*>(c)->PutOrUpdate(rs::OP_PUT, reinterpret_cast<const uint64_t*>(keys), static_cast<size_t>(n), dim,
                                                values, static_cast<size_t>(max_per_req > 0 ? max_per_req : 2000), nullptr);
}
RS_API int rs_ps_client_update(void* c, const unsigned long long* keys, long long n, int dim, const float* grads, int max_per_req,
                               unsigned long long* applied) {
  uint64_t a = 0;
  const int rc = static_cast<PsClient*>(c)->PutOrUpdate(rs::OP_UPDATE, reinterpret_cast<const uint64_t*>(keys), static_cast<size_t>(n),
                                                        dim, grads, static_cast<size_t>(max_per_req > 0 ? max_per_req : 2000), &a);
  if (applied) *applied = a;
  return rc;
}
// op: 4 clear, 5 load fake data (arg = n), 6 save (path), 7 load (path), 8 stats (reply: size, requests, keys)
// reply4: up to four 64-bit words of the server's answer (unused words are zero).
RS_API int rs_ps_client_command(void* c, int op, const void* payload, long long len, unsigned long long* reply4) {
  unsigned long long tmp[4] = {0, 0, 0, 0};
  const int rc = static_cast<PsClient*>(c)->Command(static_cast<uint32_t>(op), payload, static_cast<size_t>(len), tmp, sizeof(tmp));
  if (reply4) memcpy(reply4, tmp, sizeof(tmp));
  return rc;
}

// Stand-alone task providers over integer task ids (the schedulers can be exercised without sockets).
RS_API int rs_provider_new(const char* kind, int levels, unsigned long long seed, void** out) {
  RS_REQUIRE(kind && out, "rs_provider_new: null argument");
  RS_NOEXCEPT_BODY(
    const std::string k = kind;
    if (k == "fifo") *out = static_cast<rs::TaskProvider<long long>*>(new rs::FifoProvider<long long>());
    else if (k == "priority") *out = static_cast<rs::TaskProvider<long long>*>(new rs::PriorityProvider<long long>(levels, seed));
    else return rs::set_error(RS_ERR_INVALID, "rs_provider_new: kind must be fifo or priority");
    return RS_OK;
  )
}
RS_API int rs_provider_delete(void* p) { delete static_cast<rs::TaskProvider<long long>*>(p); return RS_OK; }
RS_API int rs_provider_put(void* p, long long task, unsigned long long klass) {
  RS_NOEXCEPT_BODY(static_cast<rs::TaskProvider<long long>*>(p)->Put(task, klass); return RS_OK;)
}
// Returns the next task id, or -1 when nothing is queued.
RS_API long long rs_provider_try_get(void* p) {
  long long t = -1;
  return static_cast<rs::TaskProvider<long long>*>(p)->TryGet(&t) ? t : -1;
}
RS_API long long rs_provider_left(void* p) { return static_cast<long long>(static_cast<rs::TaskProvider<long long>*>(p)->Left()); }
RS_API int rs_provider_improve(void* p, unsigned long long klass) {
  RS_NOEXCEPT_BODY(static_cast<rs::TaskProvider<long long>*>(p)->ImprovePriority(klass); return RS_OK;)
}
RS_API int rs_provider_level(void* p, unsigned long long klass) { return static_cast<rs::TaskProvider<long long>*>(p)->LevelOf(klass); }
