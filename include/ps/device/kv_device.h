// DeviceKVWorker: the KVWorker calling convention on top of the device data plane.
//
// A request on device-resident values is a kernel launch instead of messages, but the
// contract of the reference's KVWorker (include/ps/kv_app.h:54-372) is kept: Push / Pull /
// PushPull return an integer timestamp at once, an optional callback runs when the request
// has completed, and Wait(ts) blocks until then.  Completion is observed by a small thread
// that waits on CUDA events in submission order -- the role the Customer's receive thread
// plays for message responses (src/customer.cc:49-64) -- and a request whose kernel gave up
// on a device-side wait makes Wait throw ps::Error instead of hanging.
//
// Header-only; include from a translation unit compiled with the CUDA runtime headers and
// link libpsb200_device and the CUDA runtime.
#ifndef PS_DEVICE_KV_DEVICE_H_
#define PS_DEVICE_KV_DEVICE_H_
#include <cuda_runtime.h>

#include <condition_variable>
#include <deque>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#include "ps/device/psdev.h"
#include "ps/internal/logging.h"

namespace ps {

class DeviceKVWorker {
 public:
  using Callback = std::function<void()>;

  // `world`, `table` describe the symmetric heap and the dense table (see psdev.h); every
  // rank must issue the same sequence of requests on `channel`.
  DeviceKVWorker(const psdev_world_t& world, const psdev_table_t& table, const psdev_opt_t& opt,
                 int channel, uint64_t timeout_ns = 20000000000ull)
      : world_(world), table_(table), opt_(opt), channel_(channel), timeout_ns_(timeout_ns) {
    CHECK_EQ(cudaGetDevice(&device_), cudaSuccess);
    thread_ = std::thread(&DeviceKVWorker::Completing, this);
  }
  ~DeviceKVWorker() {
    {
      std::lock_guard<std::mutex> lk(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    thread_.join();
  }

  // Elements [begin, end) of the table (multiples of 8).  The gradient buffer must hold this
  // worker's values when the kernel runs (stream order), and must not be rewritten before
  // the request has completed -- the zero-copy rule of ZPush (kv_app.h:236-242).
  int Push(int64_t begin, int64_t end, cudaStream_t s, const Callback& cb = nullptr) {
    return Submit(PSDEV_OP_PUSH, begin, end, s, cb);
  }
  int Pull(int64_t begin, int64_t end, cudaStream_t s, const Callback& cb = nullptr) {
    return Submit(PSDEV_OP_PULL, begin, end, s, cb);
  }
  int PushPull(int64_t begin, int64_t end, cudaStream_t s, const Callback& cb = nullptr) {
    return Submit(PSDEV_OP_PUSHPULL, begin, end, s, cb);
  }

  // Blocks until request `timestamp` has completed (its callback has run by then).
  void Wait(int timestamp) {
    std::unique_lock<std::mutex> lk(mu_);
    CHECK(timestamp >= 0 && timestamp < next_ts_) << "unknown timestamp " << timestamp;
    done_cv_.wait(lk, [&] { return completed_ > timestamp; });
    if (first_error_ts_ >= 0 && first_error_ts_ <= timestamp) {
      LOG(FATAL) << "device request " << first_error_ts_ << " failed with status " << error_
                 << " (a peer did not arrive within the deadline)";
    }
  }

  void set_optimizer(const psdev_opt_t& opt) { opt_ = opt; }

 private:
  struct Pending {
    int ts;
    cudaEvent_t ev;
    Callback cb;
  };

  int Submit(int op, int64_t begin, int64_t end, cudaStream_t s, const Callback& cb) {
    int rc = psdev_dense_op(&world_, &table_, op, begin, end, &opt_, channel_, 0, timeout_ns_,
                            /*sync=*/1, s);
    CHECK_EQ(rc, 0) << "psdev_dense_op failed";
    Pending p;
    CHECK_EQ(cudaEventCreateWithFlags(&p.ev, cudaEventDisableTiming), cudaSuccess);
    CHECK_EQ(cudaEventRecord(p.ev, s), cudaSuccess);
    p.cb = cb;
    std::lock_guard<std::mutex> lk(mu_);
    p.ts = next_ts_++;
    queue_.push_back(std::move(p));
    cv_.notify_one();
    return queue_.back().ts;
  }

  void Completing() {
    cudaSetDevice(device_);
    for (;;) {
      Pending p;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [&] { return stop_ || !queue_.empty(); });
        if (queue_.empty()) return;
        p = std::move(queue_.front());
        queue_.pop_front();
      }
      cudaEventSynchronize(p.ev);
      cudaEventDestroy(p.ev);
      int32_t status = 0;
      psdev_channel_status(world_.peer_base[world_.rank], channel_, &status, nullptr);
      if (p.cb) p.cb();  // before the request counts as complete, like the reference
      {
        std::lock_guard<std::mutex> lk(mu_);
        if (status != 0 && first_error_ts_ < 0) {
          first_error_ts_ = p.ts;
          error_ = status;
        }
        completed_ = p.ts + 1;
      }
      done_cv_.notify_all();
    }
  }

  psdev_world_t world_;
  psdev_table_t table_;
  psdev_opt_t opt_;
  int channel_;
  uint64_t timeout_ns_;
  int device_ = 0;
  std::mutex mu_;
  std::condition_variable cv_, done_cv_;
  std::deque<Pending> queue_;
  int next_ts_ = 0;
  int completed_ = 0;
  int first_error_ts_ = -1;
  int error_ = 0;
  bool stop_ = false;
  std::thread thread_;
};

}  // namespace ps
#endif  // PS_DEVICE_KV_DEVICE_H_
