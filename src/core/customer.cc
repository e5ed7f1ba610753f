#include "ps/internal/customer.h"

#include <chrono>
#include <climits>

#include "ps/internal/postoffice.h"

namespace ps {

Customer::Customer(int app_id, int customer_id, const RecvHandle& recv_handle, Side side,
                   bool start)
    : app_id_(app_id), customer_id_(customer_id), side_(side), recv_handle_(recv_handle) {
  Postoffice::Get()->AddCustomer(this);
  if (start) StartReceiving();
}

bool Customer::Mature() const {
  static const int grace_ms = GetEnv("PS_HANDLE_GRACE_MS", 20);
  return std::chrono::steady_clock::now() - created_ >= std::chrono::milliseconds(grace_ms);
}

void Customer::StartReceiving() {
  if (!recv_thread_) recv_thread_.reset(new std::thread(&Customer::Receiving, this));
}

Customer::~Customer() {
  Postoffice::Get()->RemoveCustomer(this);
  Message stop;
  stop.meta.control.cmd = Control::TERMINATE;
  // lowest possible priority: everything already queued is handled first
  stop.meta.priority = INT_MIN;
  recv_queue_.Push(stop);
  if (recv_thread_) recv_thread_->join();
}

int Customer::NewRequest(int recver) {
  const int expected = static_cast<int>(Postoffice::Get()->GetNodeIDs(recver).size());
  std::lock_guard<std::mutex> lk(tracker_mu_);
  tracker_.emplace_back(expected, 0);
  return tracker_base_ + static_cast<int>(tracker_.size()) - 1;
}

void Customer::WaitRequest(int timestamp) { WaitRequestFor(timestamp, -1); }

bool Customer::WaitRequestFor(int timestamp, int timeout_ms) {
  std::unique_lock<std::mutex> lk(tracker_mu_);
  CHECK_GE(timestamp, 0);
  CHECK_LT(static_cast<size_t>(timestamp), tracker_base_ + tracker_.size()) << "unknown timestamp";
  auto done = [this, timestamp] {
    if (timestamp < tracker_base_) return true;  // completed long ago
    const auto& e = tracker_[timestamp - tracker_base_];
    return e.first <= e.second;
  };
  bool finished = true;
  if (timeout_ms < 0) {
    tracker_cond_.wait(lk, done);
  } else {
    finished = tracker_cond_.wait_for(lk, std::chrono::milliseconds(timeout_ms), done);
  }
  if (finished) {
    auto it = failed_.find(timestamp);
    if (it != failed_.end()) {
      const std::string why = it->second;
      failed_.erase(it);
      lk.unlock();
      LOG(FATAL) << "request " << timestamp << " failed: " << why;
    }
  }
  return finished;
}

void Customer::FailRequest(int timestamp, const std::string& why) {
  std::lock_guard<std::mutex> lk(tracker_mu_);
  failed_[timestamp] = why;
  if (failed_.size() > kTrackerWindow) failed_.erase(failed_.begin());
  if (timestamp >= tracker_base_) {
    auto& e = tracker_[timestamp - tracker_base_];
    e.second = e.first;
  }
  tracker_cond_.notify_all();  // under the lock: see AddResponse
}

int Customer::NumResponse(int timestamp) {
  std::lock_guard<std::mutex> lk(tracker_mu_);
  // forgotten: complete, and more than anyone expects
  if (timestamp < tracker_base_) return INT_MAX;
  return tracker_[timestamp - tracker_base_].second;
}

void Customer::AddResponse(int timestamp, int num) {
  std::lock_guard<std::mutex> lk(tracker_mu_);
  if (timestamp >= tracker_base_) tracker_[timestamp - tracker_base_].second += num;
  // forget completed requests beyond the window of recent ones
  while (tracker_.size() > kTrackerWindow && tracker_.front().first <= tracker_.front().second) {
    tracker_.pop_front();
    ++tracker_base_;
  }
  // Notified under the lock.  The caller may be a thread that the customer does not own (the
  // device plane's completion thread): the thread released from Wait may destroy the customer
  // at once, and then must not find this thread still inside the condition variable.
  tracker_cond_.notify_all();
}

void Customer::Receiving() {
  for (;;) {
    Message recv;
    recv_queue_.WaitAndPop(&recv);
    if (!recv.meta.control.empty() && recv.meta.control.cmd == Control::TERMINATE) break;
    // The handler runs first, so a completion callback fired by the last response has
    // finished by the time WaitRequest is released (reference: src/customer.cc:57-62).
    recv_handle_(recv);
    if (!recv.meta.request) AddResponse(recv.meta.timestamp, 1);
  }
}

}  // namespace ps
