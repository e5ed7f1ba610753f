// Blocking FIFO (reference: include/ps/internal/threadsafe_queue.h:17-48) with an added
// timed pop so that service threads can notice shutdown.
#ifndef PS_INTERNAL_THREADSAFE_QUEUE_H_
#define PS_INTERNAL_THREADSAFE_QUEUE_H_
#include <chrono>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <utility>

namespace ps {

template <typename T>
class ThreadsafeQueue {
 public:
  void Push(T v) {
    {
      std::lock_guard<std::mutex> lk(mu_);
      q_.push_back(std::move(v));
    }
    cv_.notify_one();
  }
  // Blocks until an element is available.
  void WaitAndPop(T* out) {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [this] { return !q_.empty(); });
    *out = std::move(q_.front());
    q_.pop_front();
  }
  // Waits at most `ms`; returns false on timeout.
  bool WaitAndPopFor(T* out, int ms) {
    std::unique_lock<std::mutex> lk(mu_);
    if (!cv_.wait_for(lk, std::chrono::milliseconds(ms), [this] { return !q_.empty(); }))
      return false;
    *out = std::move(q_.front());
    q_.pop_front();
    return true;
  }
  bool TryPop(T* out) {
    std::lock_guard<std::mutex> lk(mu_);
    if (q_.empty()) return false;
    *out = std::move(q_.front());
    q_.pop_front();
    return true;
  }
  size_t Size() const {
    std::lock_guard<std::mutex> lk(mu_);
    return q_.size();
  }

 private:
  mutable std::mutex mu_;
  std::condition_variable cv_;
  std::deque<T> q_;
};

}  // namespace ps
#endif  // PS_INTERNAL_THREADSAFE_QUEUE_H_
