// Resender: at-least-once delivery with de-duplication on top of any van (PS_RESEND=1).
//
// Every outgoing message except ACKs is remembered under a 64-bit signature; the receiver
// answers each such message (duplicates too) with an ACK carrying the signature and hands
// only the first copy to the application; a monitor thread retransmits what has not been
// acknowledged after `timeout` ms, growing the wait with each retry, and gives up with a
// fatal error after `max_retry` attempts.  Reference: src/resender.h:24-131.  The signature
// here keeps all 32 bits of the timestamp and 12 bits of each node id (the reference
// truncates ids to 8 bits, src/resender.h:95-105).
#ifndef PS_INTERNAL_RESENDER_H_
#define PS_INTERNAL_RESENDER_H_
#include <atomic>
#include <chrono>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <unordered_set>

#include "ps/internal/message.h"

namespace ps {

class Van;

class Resender {
 public:
  Resender(int timeout_ms, int max_retry, Van* van);
  ~Resender();

  // Remember an outgoing message until it is acknowledged.
  void AddOutgoing(const Message& msg);
  // Inspect an incoming message.  Returns true if the caller must not process it
  // (it is an ACK, or a duplicate of something already delivered).
  bool AddIncomming(const Message& msg);

  // Signature of a message as seen from its sender.
  static uint64_t Signature(const Message& msg);
  // Waits until everything sent has been acknowledged, at most `max_ms`; returns whether it
  // drained.  Called before the van stops so that a lost final message can still be resent.
  bool WaitDrained(int max_ms);
  // After this, an exhausted retry budget is logged instead of raised (used at shutdown).
  void set_quiet(bool q) { quiet_ = q; }
  // Number of retransmissions so far (for tests and statistics).
  int64_t num_resent() const { return resent_.load(); }

 private:
  using Clock = std::chrono::steady_clock;
  struct Entry {
    Message msg;
    Clock::time_point sent;
    int retries = 0;
  };
  void Monitoring();

  const int timeout_ms_;
  const int max_retry_;
  Van* van_;
  std::mutex mu_;
  std::unordered_map<uint64_t, Entry> pending_;
  std::unordered_set<uint64_t> seen_;
  std::atomic<bool> exit_{false};
  std::atomic<bool> quiet_{false};
  std::atomic<int64_t> resent_{0};
  std::thread monitor_;
};

}  // namespace ps
#endif  // PS_INTERNAL_RESENDER_H_
