#include "ps/internal/resender.h"

#include <vector>

#include "ps/internal/van.h"

namespace ps {

Resender::Resender(int timeout_ms, int max_retry, Van* van)
    : timeout_ms_(timeout_ms), max_retry_(max_retry), van_(van) {
  monitor_ = std::thread(&Resender::Monitoring, this);
}

Resender::~Resender() {
  exit_ = true;
  monitor_.join();
}

uint64_t Resender::Signature(const Message& msg) {
  const Meta& m = msg.meta;
  // [app 7 bits][sender 12][recver 12][timestamp 32][request 1]
  const uint64_t app = m.app_id == Meta::kEmpty ? 0x7f : (static_cast<uint64_t>(m.app_id) & 0x7f);
  return (app << 57) | ((static_cast<uint64_t>(m.sender) & 0xfff) << 45) |
         ((static_cast<uint64_t>(m.recver) & 0xfff) << 33) |
         ((static_cast<uint64_t>(static_cast<uint32_t>(m.timestamp))) << 1) |
         (m.request ? 1u : 0u);
}

// Registration traffic is outside the reliability layer: it flows before node ids exist
// (an ACK could not be addressed) and the scheduler de-duplicates it by address.
static bool Untracked(const Message& msg) {
  const Control::Command c = msg.meta.control.cmd;
  return c == Control::ADD_NODE || c == Control::TERMINATE ||
         msg.meta.sender == Meta::kEmpty || msg.meta.recver == Meta::kEmpty;
}

void Resender::AddOutgoing(const Message& msg) {
  if (msg.meta.control.cmd == Control::ACK || Untracked(msg)) return;
  CHECK_NE(msg.meta.timestamp, Meta::kEmpty) << msg.DebugString();
  const uint64_t sig = Signature(msg);
  std::lock_guard<std::mutex> lk(mu_);
  if (pending_.count(sig)) return;  // a retransmission of something already tracked
  Entry& e = pending_[sig];
  e.msg = msg;
  e.sent = Clock::now();
}

bool Resender::AddIncomming(const Message& msg) {
  if (msg.meta.control.cmd != Control::ACK && Untracked(msg)) return false;
  if (msg.meta.control.cmd == Control::ACK) {
    std::lock_guard<std::mutex> lk(mu_);
    pending_.erase(msg.meta.control.msg_sig);
    return true;
  }
  const uint64_t sig = Signature(msg);
  bool duplicate;
  {
    std::lock_guard<std::mutex> lk(mu_);
    duplicate = !seen_.insert(sig).second;
  }
  // acknowledge every copy: the earlier ACK may be the thing that was lost
  Message ack;
  ack.meta.recver = msg.meta.sender;
  ack.meta.sender = msg.meta.recver;
  ack.meta.control.cmd = Control::ACK;
  ack.meta.control.msg_sig = sig;
  van_->Send(ack);
  if (duplicate) LOG(WARNING) << "duplicated message: " << msg.DebugString();
  return duplicate;
}

bool Resender::WaitDrained(int max_ms) {
  const auto deadline = Clock::now() + std::chrono::milliseconds(max_ms);
  for (;;) {
    {
      std::lock_guard<std::mutex> lk(mu_);
      if (pending_.empty()) return true;
    }
    if (Clock::now() > deadline) return false;
    std::this_thread::sleep_for(std::chrono::milliseconds(5));
  }
}

void Resender::Monitoring() {
  while (!exit_.load()) {
    std::this_thread::sleep_for(std::chrono::milliseconds(std::max(1, timeout_ms_ / 4)));
    std::vector<Message> again;
    const auto now = Clock::now();
    {
      std::lock_guard<std::mutex> lk(mu_);
      for (auto& kv : pending_) {
        Entry& e = kv.second;
        const auto wait = std::chrono::milliseconds(
            static_cast<int64_t>(timeout_ms_) * (1 + e.retries));
        if (now - e.sent > wait) {
          if (e.retries >= max_retry_) {
            if (quiet_.load()) continue;
            LOG(FATAL) << "no acknowledgement after " << max_retry_
                       << " retries: " << e.msg.DebugString();
          }
          ++e.retries;
          e.sent = now;
          again.push_back(e.msg);
        }
      }
    }
    for (const Message& m : again) {
      LOG(WARNING) << "timeout waiting for an ACK, resend " << m.DebugString();
      ++resent_;
      van_->Send(m);
    }
  }
}

}  // namespace ps
