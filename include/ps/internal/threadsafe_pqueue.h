// Blocking priority queue of messages: highest Meta::priority first, FIFO among equals.
// (The reference's comparator, include/ps/internal/threadsafe_pqueue.h:46-53, uses <= and so
// has no defined order among equal priorities; here ties keep arrival order.)
#ifndef PS_INTERNAL_THREADSAFE_PQUEUE_H_
#define PS_INTERNAL_THREADSAFE_PQUEUE_H_
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <mutex>
#include <queue>
#include <utility>
#include <vector>

#include "ps/internal/message.h"

namespace ps {

class ThreadsafePQueue {
 public:
  void Push(Message msg) {
    {
      std::lock_guard<std::mutex> lk(mu_);
      heap_.push(Entry{msg.meta.priority, seq_++, std::move(msg)});
    }
    cv_.notify_one();
  }
  void WaitAndPop(Message* out) {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [this] { return !heap_.empty(); });
    PopLocked(out);
  }
  bool WaitAndPopFor(Message* out, int ms) {
    std::unique_lock<std::mutex> lk(mu_);
    if (!cv_.wait_for(lk, std::chrono::milliseconds(ms), [this] { return !heap_.empty(); }))
      return false;
    PopLocked(out);
    return true;
  }
  size_t Size() const {
    std::lock_guard<std::mutex> lk(mu_);
    return heap_.size();
  }

 private:
  struct Entry {
    int priority;
    uint64_t seq;
    Message msg;
  };
  struct Later {
    bool operator()(const Entry& a, const Entry& b) const {
      if (a.priority != b.priority) return a.priority < b.priority;
      return a.seq > b.seq;
    }
  };
  void PopLocked(Message* out) {
    *out = std::move(const_cast<Entry&>(heap_.top()).msg);
    heap_.pop();
  }
  mutable std::mutex mu_;
  std::condition_variable cv_;
  std::priority_queue<Entry, std::vector<Entry>, Later> heap_;
  uint64_t seq_ = 0;
};

}  // namespace ps
#endif  // PS_INTERNAL_THREADSAFE_PQUEUE_H_
