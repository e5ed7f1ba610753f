// Customer: the mailbox of one application endpoint (a KVWorker, KVServer or SimpleApp).
//
// It owns a priority receive queue and a thread that runs the application's handler on each
// delivered message, and it tracks outstanding requests by timestamp so that callers can
// wait for all responses.  Reference: include/ps/internal/customer.h:26-111,
// src/customer.cc:14-64.  Differences: endpoints are tagged worker-side or server-side so a
// process that is worker and server at once can host both with the same (app, customer) ids;
// waits can be bounded; a failed request (device error, dead peer) can be marked so that
// WaitRequest reports it instead of blocking forever.
#ifndef PS_INTERNAL_CUSTOMER_H_
#define PS_INTERNAL_CUSTOMER_H_
#include <deque>
#include <chrono>
#include <atomic>
#include <condition_variable>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <mutex>
#include <thread>
#include <utility>
#include <vector>

#include "ps/internal/message.h"
#include "ps/internal/threadsafe_pqueue.h"

namespace ps {

class Customer {
 public:
  using RecvHandle = std::function<void(const Message& recved)>;
  enum Side { kWorkerSide = 0, kServerSide = 1 };

  // Registers with the Postoffice and starts the handler thread.  With start = false the
  // thread is started by StartReceiving(): an application object that stores the pointer to
  // its Customer needs that store to happen before the first message is handled (messages
  // that arrive earlier wait in the queue).
  Customer(int app_id, int customer_id, const RecvHandle& recv_handle, Side side = kWorkerSide,
           bool start = true);
  void StartReceiving();
  // Unregisters, drains and joins the handler thread.
  ~Customer();

  int app_id() const { return app_id_; }
  int customer_id() const { return customer_id_; }
  Side side() const { return side_; }

  // Opens a request to `recver` (a node id or a group id) and returns its timestamp.  The
  // request completes when every node of `recver` has responded.
  int NewRequest(int recver);
  // Blocks until request `timestamp` completed.
  void WaitRequest(int timestamp);
  // Bounded form: false if `timeout_ms` elapsed first (timeout_ms < 0 waits forever).
  bool WaitRequestFor(int timestamp, int timeout_ms);
  // Responses received so far for `timestamp`.
  int NumResponse(int timestamp);
  // Credits `num` responses (used for recipients that were skipped, and by the handler
  // thread after each response message).
  void AddResponse(int timestamp, int num = 1);
  // Marks request `timestamp` as failed with `why` and completes it: WaitRequest throws
  // ps::Error for it instead of returning.  Used by the device plane when a kernel gave up
  // waiting for a peer; message traffic never fails a request this way.
  void FailRequest(int timestamp, const std::string& why);
  // Hands a received message to this customer (called by the van's receive thread).
  void Accept(const Message& recved) { recv_queue_.Push(recved); }
  // False during the first milliseconds of a customer's life (PS_HANDLE_GRACE_MS, default 20).
  // An application object is constructed first and given its handles afterwards
  // (`SimpleApp app(0, 0); app.set_request_handle(...)`): a request that was already waiting
  // for the customer would otherwise be answered by the default handle.  The van keeps such
  // requests parked until the customer is mature.
  bool Mature() const;

 private:
  void Receiving();

  const std::chrono::steady_clock::time_point created_ = std::chrono::steady_clock::now();
  const int app_id_;
  const int customer_id_;
  const Side side_;
  RecvHandle recv_handle_;
  ThreadsafePQueue recv_queue_;
  std::unique_ptr<std::thread> recv_thread_;

  std::mutex tracker_mu_;
  std::condition_variable tracker_cond_;
  // tracker_[ts - tracker_base_] = (responses expected, responses received).  Requests below
  // tracker_base_ have completed and been forgotten: the table keeps a window of recent
  // requests instead of growing for the life of the process (the reference's never shrinks,
  // src/customer.cc:25-47); timestamps keep counting up.
  std::deque<std::pair<int, int>> tracker_;
  std::map<int, std::string> failed_;  // timestamp -> reason, erased when waited for
  int tracker_base_ = 0;
  static constexpr size_t kTrackerWindow = 4096;
  DISALLOW_COPY_AND_ASSIGN(Customer);
};

}  // namespace ps
#endif  // PS_INTERNAL_CUSTOMER_H_
