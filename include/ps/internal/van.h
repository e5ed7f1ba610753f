// Van: the transport of a node, plus the control-plane protocol that runs on top of it.
//
// Responsibilities (reference: include/ps/internal/van.h:51-107, src/van.cc:44-443):
//   * rendezvous with the scheduler (ADD_NODE), node-id assignment, recovery registration;
//   * barriers counted at the scheduler; heartbeats; TERMINATE;
//   * delivery of data messages to the addressed Customer;
//   * optional reliability (ACK / resend / de-duplication) and receive-side drop injection.
// Backends implement four hooks: Bind, Connect, SendMsg, RecvMsg.
//
// What is new here:
//   * a process may host several node ids (role JOINT = server id 8+2r and worker id 9+2r
//     in one process, one per GPU); messages carry explicit sender and receiver ids and a
//     message addressed to one of the process's own ids is delivered in-process;
//   * priority sending (the reference's P3Van, src/p3_van.h:12-57) is a mode of any backend;
//   * backends: "tcp" (epoll, TCP or Unix sockets; "zmq" is accepted as an alias),
//     "p3" (tcp + priority send queue) and "loop" (single process, no sockets).
#ifndef PS_INTERNAL_VAN_H_
#define PS_INTERNAL_VAN_H_
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <ctime>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "ps/base.h"
#include "ps/internal/message.h"
#include "ps/internal/threadsafe_pqueue.h"
#include "ps/internal/threadsafe_queue.h"

namespace ps {

class Resender;
class Customer;

class Van {
 public:
  // Backend factory; `type` is the value of DMLC_PS_VAN_TYPE.
  static Van* Create(const std::string& type);

  Van() = default;
  virtual ~Van();

  // Binds, registers with the scheduler and blocks until the node table is known.
  // Only the first call per process does the work; later customers reuse the van.
  virtual void Start(int customer_id);
  // Stops the service threads and releases the sockets.
  virtual void Stop();

  // Sends `msg` to node `msg.meta.recver` (never a group id).  Returns the number of
  // bytes handed to the transport, or -1 on failure.  Thread safe.
  int Send(const Message& msg);

  // The node this process registered as.  For a JOINT process `id` is the worker id.
  const Node& my_node() const {
    CHECK(ready_.load()) << "call Start() first";
    return my_node_;
  }
  // All node ids hosted by this process (two for a JOINT process).
  const std::vector<int>& my_ids() const { return my_ids_; }
  bool IsLocalId(int id) const;

  // Next timestamp for control messages sent by this node.
  int GetTimestamp() { return timestamp_++; }
  bool IsReady() const { return ready_.load(); }

  // Tells the receive loop that a customer registered, so that messages that arrived
  // before their application endpoint existed are delivered now.
  void Kick();

  // Traffic counters (payload + meta bytes), readable at any time.
  size_t send_bytes() const { return send_bytes_.load(); }
  size_t recv_bytes() const { return recv_bytes_.load(); }

  // Serialise / parse the PBMeta bytes of a message (wire contract of meta.proto).
  void PackMeta(const Meta& meta, char** meta_buf, int* buf_size);
  void UnpackMeta(const char* meta_buf, int buf_size, Meta* meta);

 protected:
  // ---- backend hooks ----
  // Opens a sending path to `node` (idempotent; a second call for the same id reconnects).
  virtual void Connect(const Node& node) = 0;
  // Starts receiving on `node`'s address.  Returns the bound port or -1; on failure the
  // backend may retry up to `max_retry` times on other ports.
  virtual int Bind(const Node& node, int max_retry) = 0;
  // Blocks for the next message; returns its size in bytes, or -1 when the van stopped.
  // The default takes the next message queued by Deliver().
  virtual int RecvMsg(Message* msg);
  // Transmits one message; returns bytes sent or -1.
  virtual int SendMsg(const Message& msg) = 0;
  // Backend-specific setup before Bind (e.g. creating the I/O thread).
  virtual void StartBackend() {}
  virtual void StopBackend() {}
  // True for a backend in which this single process is scheduler, server and worker.
  virtual bool IsStandalone() const { return false; }

  Node scheduler_;
  Node my_node_;
  std::vector<int> my_ids_;
  bool is_scheduler_ = false;
  std::mutex start_mu_;

 private:
  // service loops
  void Receiving();
  void Heartbeat();
  void PrioritySending();

  // control-plane handlers; `recovery_nodes` etc. are scheduler state held in members
  void ProcessTerminateCommand();
  void ProcessAddNodeCommand(Message* msg);
  void ProcessBarrierCommand(Message* msg);
  void ProcessHeartbeat(Message* msg);
  void ProcessDataMsg(Message* msg);
  Customer* FindCustomer(const Message& msg);
  void RetryParked();
  void SchedulerRegister(Message* msg);
  void SchedulerAssignAndBroadcast();
  void SchedulerAdmitRecovery(const Node& newcomer, int reuse_server_id, int reuse_worker_id);
  void AdoptNodeTable(const std::vector<Node>& nodes);
  int DeliverLocal(const Message& msg);
  int Transmit(const Message& msg);

  std::atomic<bool> ready_{false};
  std::atomic<bool> stopping_{false};
  // Send gate: Stop() closes it and waits for the sends that are inside, so that a response
  // still being sent by an application thread never meets a half-dismantled van.
  std::mutex send_gate_mu_;
  std::condition_variable send_gate_cv_;
  int sends_in_flight_ = 0;
  bool send_closed_ = false;
  std::atomic<size_t> send_bytes_{0};
  std::atomic<size_t> recv_bytes_{0};
  std::atomic<int> timestamp_{0};
  int init_stage_ = 0;
  int drop_rate_ = 0;
  int heartbeat_timeout_ = 0;

  std::unique_ptr<std::thread> receiver_thread_;
  std::unique_ptr<std::thread> heartbeat_thread_;
  std::unique_ptr<std::thread> sender_thread_;  // priority mode only
  bool priority_mode_ = false;
  ThreadsafePQueue send_queue_;
  ThreadsafeQueue<Message> inbox_;  // complete messages awaiting the receive loop

  Resender* resender_ = nullptr;

  // data messages whose customer does not exist yet (touched by the receive loop only)
  struct Parked {
    Message msg;
    std::chrono::steady_clock::time_point since;
  };
  std::vector<Parked> parked_;

  // scheduler state
  struct Registration {
    Node node;  // as announced (role may be JOINT); id assigned later
  };
  std::vector<Registration> pending_;             // registrations before assignment
  std::vector<Node> table_;                       // assigned node table (one entry per id)
  std::unordered_map<std::string, std::vector<int>> addr_to_ids_;  // "host:port" -> ids
  std::vector<int> barrier_count_ = std::vector<int>(8, 0);
  int num_servers_seen_ = 0, num_workers_seen_ = 0;

  friend class Resender;
  friend class Postoffice;
  DISALLOW_COPY_AND_ASSIGN(Van);

 protected:
  void set_priority_mode(bool on) { priority_mode_ = on; }
  // Queues a complete message for the receive loop.  Backends call it from their I/O
  // thread; the base class calls it for messages addressed to this process's own ids.
  void Deliver(Message&& msg) { inbox_.Push(std::move(msg)); }
  bool stopping() const { return stopping_.load(); }
};

}  // namespace ps
#endif  // PS_INTERNAL_VAN_H_
