// Postoffice: cluster shape, customer registry, barriers, key ranges, heartbeat table.
// Behavioural reference: src/postoffice.cc:16-215 of ps-lite.
#include "ps/internal/postoffice.h"

#include <unistd.h>

#include <chrono>
#include <thread>

#include "ps/base.h"

namespace ps {

Postoffice::Postoffice() { env_ref_ = Environment::_GetSharedRef(); }

void Postoffice::InitEnvironment() {
  const std::string van_type = GetEnv("DMLC_PS_VAN_TYPE", std::string("tcp"));
  van_ = Van::Create(van_type);
  verbose_ = GetEnv("PS_VERBOSE", 0);
  if (van_type == "loop") {
    // a single process that is scheduler, server 0 and worker 0
    num_workers_ = num_servers_ = 1;
    is_worker_ = is_server_ = is_scheduler_ = true;
    return;
  }
  const char* nw = Environment::Get()->find("DMLC_NUM_WORKER");
  const char* ns = Environment::Get()->find("DMLC_NUM_SERVER");
  const char* role = Environment::Get()->find("DMLC_ROLE");
  CHECK(nw) << "DMLC_NUM_WORKER is not set";
  CHECK(ns) << "DMLC_NUM_SERVER is not set";
  CHECK(role) << "DMLC_ROLE is not set";
  num_workers_ = atoi(nw);
  num_servers_ = atoi(ns);
  const std::string r(role);
  is_worker_ = (r == "worker" || r == "joint");
  is_server_ = (r == "server" || r == "joint");
  is_scheduler_ = (r == "scheduler");
  CHECK(is_worker_ || is_server_ || is_scheduler_)
      << "DMLC_ROLE must be worker, server, scheduler or joint, got '" << r << "'";
}

void Postoffice::Start(int customer_id, const char* argv0, const bool do_barrier) {
  bool first;
  {
    std::lock_guard<std::mutex> lk(start_mu_);
    first = (init_stage_ == 0);
    if (first) {
      InitEnvironment();
      // group tables: for every non-empty subset g of {scheduler, servers, workers} the
      // ids in it; and every concrete id names itself
      for (int g = 1; g < 8; ++g) {
        std::vector<int>& ids = node_ids_[g];
        if (g & kScheduler) ids.push_back(kScheduler);
        if (g & kServerGroup)
          for (int i = 0; i < num_servers_; ++i) ids.push_back(ServerRankToID(i));
        if (g & kWorkerGroup)
          for (int i = 0; i < num_workers_; ++i) ids.push_back(WorkerRankToID(i));
      }
      for (int i = 0; i < num_servers_; ++i) node_ids_[ServerRankToID(i)] = {ServerRankToID(i)};
      for (int i = 0; i < num_workers_; ++i) node_ids_[WorkerRankToID(i)] = {WorkerRankToID(i)};
      init_stage_ = 1;
    }
    ++started_customers_;
  }
  if (argv0 && verbose_ >= 1)
    LOG(INFO) << "starting " << argv0 << " (customer " << customer_id << ")";

  van_->Start(customer_id);

  {
    std::lock_guard<std::mutex> lk(start_mu_);
    if (init_stage_ == 1) {
      start_time_ = time(nullptr);
      init_stage_ = 2;
    }
  }
  // One global barrier per process, entered by whichever customer comes first; customers
  // that start later wait for that same barrier to be released.
  if (do_barrier) {
    bool leader = false;
    {
      std::unique_lock<std::mutex> lk(barrier_mu_);
      if (!start_barrier_begun_) {
        start_barrier_begun_ = true;
        leader = true;
      }
    }
    if (leader) {
      BarrierImpl(customer_id, kWorkerGroup + kServerGroup + kScheduler, true);
      std::lock_guard<std::mutex> lk(barrier_mu_);
      start_barrier_done_ = true;
      barrier_cond_.notify_all();
    } else {
      std::unique_lock<std::mutex> lk(barrier_mu_);
      barrier_cond_.wait(lk, [this] { return start_barrier_done_; });
    }
  }
}

void Postoffice::Finalize(const int customer_id, const bool do_barrier) {
  // The customers of one process leave together: the last one to arrive runs the global
  // barrier, and customer 0 tears the van down once that barrier has been released.
  bool last;
  uint64_t gen;
  {
    std::unique_lock<std::mutex> lk(barrier_mu_);
    gen = finalize_generation_;
    ++finalizing_customers_;
    last = (finalizing_customers_ >= started_customers_);
  }
  if (last) {
    if (do_barrier) BarrierImpl(customer_id, kWorkerGroup + kServerGroup + kScheduler, true);
    std::lock_guard<std::mutex> lk(barrier_mu_);
    ++finalize_generation_;
    barrier_cond_.notify_all();
  } else {
    std::unique_lock<std::mutex> lk(barrier_mu_);
    barrier_cond_.wait(lk, [this, gen] { return finalize_generation_ != gen; });
  }
  if (customer_id == 0) {
    // let the other customer threads get out of the wait above before the state goes away
    num_workers_ = num_servers_ = 0;
    van_->Stop();
    {
      std::lock_guard<std::mutex> lk(start_mu_);
      init_stage_ = 0;
      started_customers_ = 0;
    }
    {
      std::lock_guard<std::mutex> lk(barrier_mu_);
      finalizing_customers_ = 0;
      start_barrier_begun_ = start_barrier_done_ = false;
      rounds_.clear();
    }
    {
      std::lock_guard<std::mutex> lk(mu_);
      customers_.clear();
    }
    node_ids_.clear();
    {
      std::lock_guard<std::mutex> lk(server_key_ranges_mu_);
      server_key_ranges_.clear();
    }
    {
      std::lock_guard<std::mutex> lk(heartbeat_mu_);
      heartbeats_.clear();
    }
    is_worker_ = is_server_ = is_scheduler_ = false;
    delete van_;
    van_ = nullptr;
    if (exit_callback_) exit_callback_();
  }
}

void Postoffice::AddCustomer(Customer* customer) {
  std::lock_guard<std::mutex> lk(mu_);
  const auto key = std::make_tuple(customer->app_id(), customer->customer_id(),
                                   static_cast<int>(customer->side()));
  CHECK(customers_.find(key) == customers_.end())
      << "customer " << customer->customer_id() << " of app " << customer->app_id()
      << " already exists on this side";
  customers_[key] = customer;
  if (van_ && van_->IsReady()) van_->Kick();
}

void Postoffice::RemoveCustomer(Customer* customer) {
  std::lock_guard<std::mutex> gate(customer_gate_);
  std::lock_guard<std::mutex> lk(mu_);
  customers_.erase(std::make_tuple(customer->app_id(), customer->customer_id(),
                                   static_cast<int>(customer->side())));
}

Customer* Postoffice::GetCustomer(int app_id, int customer_id, int timeout, int side) const {
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(timeout);
  for (;;) {
    {
      std::lock_guard<std::mutex> lk(mu_);
      if (side >= 0) {
        auto it = customers_.find(std::make_tuple(app_id, customer_id, side));
        if (it != customers_.end()) return it->second;
      } else {
        for (int s = 0; s < 2; ++s) {
          auto it = customers_.find(std::make_tuple(app_id, customer_id, s));
          if (it != customers_.end()) return it->second;
        }
      }
    }
    if (std::chrono::steady_clock::now() >= deadline) return nullptr;
    std::this_thread::sleep_for(std::chrono::milliseconds(1));
  }
}

void Postoffice::Barrier(int customer_id, int node_group) {
  BarrierImpl(customer_id, node_group, /*process_wide=*/false);
}

void Postoffice::BarrierImpl(int customer_id, int node_group, bool process_wide) {
  const std::vector<int>& members = GetNodeIDs(node_group);
  if (members.size() <= 1) return;
  std::vector<int> mine;
  for (int id : van_->my_ids())
    if (std::find(members.begin(), members.end(), id) != members.end()) mine.push_back(id);
  CHECK(!mine.empty()) << "this node is not a member of group " << node_group;

  std::unique_lock<std::mutex> lk(barrier_mu_);
  Round& r = rounds_[node_group];
  if (!process_wide) {
    // Every customer's k-th call belongs to the k-th round of the group.  A round that a
    // sibling customer of this process opened may already have been released when this
    // customer calls: it then takes that round instead of opening another one, which would
    // leave a half-counted round at the scheduler.
    uint64_t& passed = r.passed[customer_id];
    if (passed < r.floor) passed = r.floor;
    if (passed < r.generation) {
      ++passed;
      return;
    }
  }
  const uint64_t gen = r.generation;
  if (!r.in_flight) {
    // first caller of this round: announce every id this process hosts in the group;
    // customers that call while the round is open simply join it
    r.in_flight = true;
    r.process_wide = process_wide;
    r.pending = static_cast<int>(mine.size());
    lk.unlock();
    for (int id : mine) {
      Message req;
      req.meta.recver = kScheduler;
      req.meta.sender = id;
      req.meta.request = true;
      req.meta.control.cmd = Control::BARRIER;
      req.meta.control.barrier_group = node_group;
      req.meta.app_id = 0;
      req.meta.customer_id = customer_id;
      req.meta.timestamp = van_->GetTimestamp();
      van_->Send(req);
    }
    lk.lock();
  } else if (process_wide) {
    r.process_wide = true;
  }
  barrier_cond_.wait(lk, [this, node_group, gen] { return rounds_[node_group].generation != gen; });
  if (!process_wide) {
    Round& rr = rounds_[node_group];
    uint64_t& passed = rr.passed[customer_id];
    if (passed < gen + 1) passed = gen + 1;
  }
}

void Postoffice::Manage(const Message& recv) {
  const Control& ctrl = recv.meta.control;
  if (ctrl.cmd == Control::BARRIER && !recv.meta.request) {
    std::lock_guard<std::mutex> lk(barrier_mu_);
    Round& r = rounds_[ctrl.barrier_group];
    if (r.in_flight && --r.pending <= 0) {
      r.in_flight = false;
      ++r.generation;
      // a round entered once for the whole process (Start, Finalize) counts for every customer
      if (r.process_wide) r.floor = r.generation;
      r.process_wide = false;
      barrier_cond_.notify_all();
    }
  }
}

const std::vector<Range>& Postoffice::GetServerKeyRanges() {
  std::lock_guard<std::mutex> lk(server_key_ranges_mu_);
  if (server_key_ranges_.empty()) {
    const uint64_t width = kMaxKey / static_cast<uint64_t>(num_servers_);
    for (int i = 0; i < num_servers_; ++i)
      server_key_ranges_.push_back(Range(width * i, width * (i + 1)));
  }
  return server_key_ranges_;
}

std::vector<int> Postoffice::GetDeadNodes(int t) {
  std::vector<int> dead;
  if (!van_ || !van_->IsReady() || t <= 0) return dead;
  const time_t now = time(nullptr);
  // the scheduler watches everyone; everyone else watches the scheduler
  const std::vector<int>& watched =
      is_scheduler_ ? GetNodeIDs(kWorkerGroup + kServerGroup) : GetNodeIDs(kScheduler);
  std::lock_guard<std::mutex> lk(heartbeat_mu_);
  for (int id : watched) {
    if (van_->IsLocalId(id)) continue;
    auto it = heartbeats_.find(id);
    const bool silent = (it == heartbeats_.end() || it->second + t < now);
    if (silent && start_time_ + t < now) dead.push_back(id);
  }
  return dead;
}

}  // namespace ps
