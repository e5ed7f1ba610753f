// Postoffice: the per-process hub that knows the cluster shape and owns the van.
//
// Public surface of the reference's Postoffice (include/ps/internal/postoffice.h:24-164):
// Start/Finalize, customer registry, node-group table, uniform server key ranges, barriers,
// heartbeat bookkeeping, rank/id conversions.  New: the role "joint" (DMLC_ROLE=joint), in
// which a process is a worker and a server at once; is_worker() and is_server() are then
// both true and customers are registered per side.
#ifndef PS_INTERNAL_POSTOFFICE_H_
#define PS_INTERNAL_POSTOFFICE_H_
#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "ps/internal/customer.h"
#include "ps/internal/device_route.h"
#include "ps/internal/env.h"
#include "ps/internal/van.h"
#include "ps/range.h"

namespace ps {

class Postoffice {
 public:
  static Postoffice* Get() {
    static Postoffice inst;
    return &inst;
  }

  Van* van() { return van_; }

  // Reads the DMLC_* environment, creates and starts the van, optionally waits at a global
  // barrier.  `argv0` is only used for log lines.  Safe to call once per customer thread.
  void Start(int customer_id, const char* argv0, const bool do_barrier);
  // Optional global barrier, then (for customer 0) stops the van, resets the state and runs
  // the exit callback.
  void Finalize(const int customer_id, const bool do_barrier = true);

  void AddCustomer(Customer* customer);
  void RemoveCustomer(Customer* customer);
  // The lock under which the van delivers a message to a customer (see customer_gate_).
  std::mutex& customer_gate() { return customer_gate_; }
  // Looks up a registered customer; polls up to `timeout` seconds for it to appear.
  // `side` < 0 accepts either side (worker-side preferred).
  Customer* GetCustomer(int app_id, int customer_id, int timeout = 0, int side = -1) const;

  // Node ids denoted by `node_id`: the id itself, or the members of a group id (< 8).
  const std::vector<int>& GetNodeIDs(int node_id) const {
    const auto it = node_ids_.find(node_id);
    CHECK(it != node_ids_.cend()) << "node " << node_id << " doesn't exist";
    return it->second;
  }

  // The key range of every server: server i owns [kMaxKey/S*i, kMaxKey/S*(i+1)).
  const std::vector<Range>& GetServerKeyRanges();

  using Callback = std::function<void()>;
  void RegisterExitCallback(const Callback& cb) { exit_callback_ = cb; }

  static inline int WorkerRankToID(int rank) { return rank * 2 + 9; }
  static inline int ServerRankToID(int rank) { return rank * 2 + 8; }
  static inline int IDtoRank(int id) { return std::max((id - 8) / 2, 0); }
  static inline bool IsServerID(int id) { return id >= 8 && (id % 2) == 0; }
  static inline bool IsWorkerID(int id) { return id >= 9 && (id % 2) == 1; }

  int num_workers() const { return num_workers_; }
  int num_servers() const { return num_servers_; }
  int my_rank() const { return IDtoRank(van_->my_node().id); }
  int is_worker() const { return is_worker_; }
  int is_server() const { return is_server_; }
  int is_scheduler() const { return is_scheduler_; }
  int is_joint() const { return is_worker_ && is_server_; }
  int verbose() const { return verbose_; }
  bool is_recovery() const { return van_->my_node().is_recovery; }

  // The device plane, when one is attached (see ps/internal/device_route.h); KVWorker asks
  // it first whether it serves the keys of a request.
  DeviceRoute* device_route() const { return device_route_.load(std::memory_order_acquire); }
  void set_device_route(DeviceRoute* route) {
    device_route_.store(route, std::memory_order_release);
  }

  // Blocks until every node of `node_group` (which must include this node) entered.
  void Barrier(int customer_id, int node_group);
  // Called by the van for control responses that concern the Postoffice (barrier release).
  void Manage(const Message& recv);

  void UpdateHeartbeat(int node_id, time_t t) {
    std::lock_guard<std::mutex> lk(heartbeat_mu_);
    heartbeats_[node_id] = t;
  }
  // Ids whose last heartbeat is older than `t` seconds (empty while heartbeats are off or
  // the process is younger than `t`).
  std::vector<int> GetDeadNodes(int t = 60);

 private:
  Postoffice();
  // A process that ends without Finalize still has the van's service threads running.  Tearing
  // the van down under them blocks or aborts, so in that case it is left to the operating
  // system, and the process ends with the status its program chose.
  ~Postoffice() {
    if (van_ && !van_->IsReady()) delete van_;
  }
  void InitEnvironment();
  void BarrierImpl(int customer_id, int node_group, bool process_wide);

  Van* van_ = nullptr;
  std::atomic<DeviceRoute*> device_route_{nullptr};
  mutable std::mutex mu_;
  // Held by the van while it looks a customer up and hands it a message, and by
  // RemoveCustomer: once a customer has been removed, no delivery to it is under way.
  std::mutex customer_gate_;
  // (app_id, customer_id, side) -> customer
  std::map<std::tuple<int, int, int>, Customer*> customers_;
  std::unordered_map<int, std::vector<int>> node_ids_;
  std::mutex server_key_ranges_mu_;
  std::vector<Range> server_key_ranges_;
  bool is_worker_ = false, is_server_ = false, is_scheduler_ = false;
  int num_servers_ = 0, num_workers_ = 0;
  int verbose_ = 0;
  // One barrier round per node group: the first caller sends the requests, later callers
  // of the same round join it, and the round ends when every id of this process has been
  // released by the scheduler.
  struct Round {
    bool in_flight = false;
    bool process_wide = false;  // opened by Start/Finalize on behalf of every customer
    int pending = 0;
    uint64_t generation = 0;    // rounds released so far
    uint64_t floor = 0;         // rounds that count as passed by every customer
    std::unordered_map<int, uint64_t> passed;  // customer id -> rounds it has passed
  };
  std::unordered_map<int, Round> rounds_;
  int started_customers_ = 0;
  int finalizing_customers_ = 0;
  uint64_t finalize_generation_ = 0;
  bool start_barrier_begun_ = false, start_barrier_done_ = false;
  std::mutex barrier_mu_;
  std::condition_variable barrier_cond_;
  std::mutex heartbeat_mu_;
  std::mutex start_mu_;
  int init_stage_ = 0;
  std::unordered_map<int, time_t> heartbeats_;
  Callback exit_callback_;
  std::shared_ptr<Environment> env_ref_;
  time_t start_time_ = 0;
  DISALLOW_COPY_AND_ASSIGN(Postoffice);
};

// Verbose logging gated by PS_VERBOSE.
#define PS_VLOG(x) LOG_IF(INFO, x <= ::ps::Postoffice::Get()->verbose())

}  // namespace ps
#endif  // PS_INTERNAL_POSTOFFICE_H_
