// Task schedulers between the front end of a server (threads that read requests off connections) and its worker pool.
//
// The reference's asynchronous parameter server hands requests from its completion-queue front end to worker
// coroutines through a queue, and src/grpc_ps/provider.h:13-201 defines the two policies for that hand-over: a FIFO
// list, and `level` priority lists where a task's class starts at level 1, ImporvePriority raises it, and the next
// task is drawn from level i with probability proportional to i x (tasks waiting at level i).  Same policies here,
// with blocking Get (condition variable), class ids instead of task pointers as the key of the priority map, deques
// instead of vectors erased at the front, and one generator per provider instead of a random_device per draw.
#pragma once
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <mutex>
#include <random>
#include <unordered_map>
#include <vector>

namespace rs {

template <class T>
class TaskProvider {
 public:
  virtual ~TaskProvider() = default;
  virtual void Put(T task, uint64_t klass) = 0;
  // Blocks until a task is there or Close() was called; false = closed and drained.
  virtual bool Get(T* out) = 0;
  // Non-blocking form.
  virtual bool TryGet(T* out) = 0;
  virtual size_t Left() const = 0;
  virtual void ImprovePriority(uint64_t klass) = 0;
  virtual int LevelOf(uint64_t klass) const = 0;
  virtual void Close() = 0;
};

template <class T>
class FifoProvider final : public TaskProvider<T> {
 public:
  void Put(T task, uint64_t) override {
    {
      std::lock_guard<std::mutex> lk(mu_);
      q_.push_back(std::move(task));
    }
    cv_.notify_one();
  }
  bool Get(T* out) override {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [&] { return closed_ || !q_.empty(); });
    return pop(out);
  }
  bool TryGet(T* out) override {
    std::lock_guard<std::mutex> lk(mu_);
    return pop(out);
  }
  size_t Left() const override {
    std::lock_guard<std::mutex> lk(mu_);
    return q_.size();
  }
  void ImprovePriority(uint64_t) override {}
  int LevelOf(uint64_t) const override { return 1; }
  void Close() override {
    {
      std::lock_guard<std::mutex> lk(mu_);
      closed_ = true;
    }
    cv_.notify_all();
  }

 private:
  bool pop(T* out) {
    if (q_.empty()) return false;
    *out = std::move(q_.front());
    q_.pop_front();
    return true;
  }
  mutable std::mutex mu_;
  std::condition_variable cv_;
  std::deque<T> q_;
  bool closed_ = false;
};

template <class T>
class PriorityProvider final : public TaskProvider<T> {
 public:
  explicit PriorityProvider(int levels = 7, uint64_t seed = 0x5EEDull) : q_(levels < 1 ? 1 : levels), rng_(seed) {}
  void Put(T task, uint64_t klass) override {
    {
      std::lock_guard<std::mutex> lk(mu_);
      q_[level_locked(klass) - 1].push_back(std::move(task));
      ++left_;
    }
    cv_.notify_one();
  }
  bool Get(T* out) override {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [&] { return closed_ || left_ > 0; });
    return pop(out);
  }
  bool TryGet(T* out) override {
    std::lock_guard<std::mutex> lk(mu_);
    return pop(out);
  }
  size_t Left() const override {
    std::lock_guard<std::mutex> lk(mu_);
    return left_;
  }
  // Raises the class by one level (tasks already queued keep their place).  When that leaves nobody at level 1, every
  // class moves down one level, so levels stay relative and a class cannot be starved by inflation.
  void ImprovePriority(uint64_t klass) override {
    std::lock_guard<std::mutex> lk(mu_);
    int& l = level_[klass];
    if (l == 0) l = 1;
    if (l < static_cast<int>(q_.size())) ++l;
    bool any_at_one = false;
    for (auto& kv : level_) any_at_one |= kv.second == 1;
    if (!any_at_one)
      for (auto& kv : level_) --kv.second;
  }
  int LevelOf(uint64_t klass) const override {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = level_.find(klass);
    return it == level_.end() ? 1 : it->second;
  }
  void Close() override {
    {
      std::lock_guard<std::mutex> lk(mu_);
      closed_ = true;
    }
    cv_.notify_all();
  }

 private:
  int level_locked(uint64_t klass) {
    int& l = level_[klass];
    if (l == 0) l = 1;
    return l;
  }
  bool pop(T* out) {
    if (left_ == 0) return false;
    double total = 0;
    for (size_t i = 0; i < q_.size(); ++i) total += static_cast<double>(i + 1) * q_[i].size();
    double x = std::uniform_real_distribution<double>(0.0, total)(rng_);
    size_t pick = q_.size();
    for (size_t i = 0; i < q_.size(); ++i) {
      const double w = static_cast<double>(i + 1) * q_[i].size();
      if (w == 0) continue;
      pick = i;                       // the last non-empty level absorbs rounding at the upper end
      if (x < w) break;
      x -= w;
    }
    *out = std::move(q_[pick].front());
    q_[pick].pop_front();
    --left_;
    return true;
  }
  mutable std::mutex mu_;
  std::condition_variable cv_;
  std::vector<std::deque<T>> q_;
  std::unordered_map<uint64_t, int> level_;
  std::mt19937_64 rng_;
  size_t left_ = 0;
  bool closed_ = false;
};

}  // namespace rs
