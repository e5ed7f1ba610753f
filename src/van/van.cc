// Transport-independent part of the van: start-up, the control protocol (registration, node
// ids, barriers, heartbeats, termination), message dispatch, priority sending, reliability
// hooks and drop injection.  Behavioural reference: src/van.cc:44-443 of ps-lite; the
// structure here is organised around a node table in which one process may own several ids.
#include "ps/internal/van.h"

#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <random>
#include <sstream>

#include "ps/internal/customer.h"
#include "ps/internal/pb_codec.h"
#include "ps/internal/postoffice.h"
#include "ps/internal/resender.h"
#include "van/network_utils.h"
#include "van/backends.h"

namespace ps {

namespace {
std::string AddrKey(const Node& n) { return n.hostname + ":" + std::to_string(n.port); }

size_t MessageBytes(const Message& m) {
  size_t b = 0;
  for (const auto& d : m.data) b += d.size();
  return b;
}
}  // namespace

Van* Van::Create(const std::string& type) {
  if (type == "tcp" || type == "zmq" || type == "0" || type.empty()) {
    return NewTcpVan(false);
  } else if (type == "p3") {
    return NewTcpVan(true);
  } else if (type == "loop") {
    return NewLoopVan();
  } else if (type == "ibverbs") {
    LOG(FATAL) << "van type 'ibverbs' is not built: this runtime has no RDMA NIC transport; "
                  "device-resident tensors travel over NVLink through the device data plane "
                  "(ps/device/psdev.h), host messages over 'tcp' or 'p3'";
  } else {
    LOG(FATAL) << "unknown DMLC_PS_VAN_TYPE: " << type;
  }
  return nullptr;
}

Van::~Van() {}

bool Van::IsLocalId(int id) const {
  for (int x : my_ids_) if (x == id) return true;
  return false;
}

int Van::RecvMsg(Message* msg) {
  if (parked_.empty()) {
    inbox_.WaitAndPop(msg);
  } else if (!inbox_.WaitAndPopFor(msg, 5)) {
    // nothing arrived: look at the parked messages again (their customer may exist or be
    // mature by now) -- same effect as Kick()
    *msg = Message();
    msg->meta.body = "__kick__";
    msg->meta.sender = msg->meta.recver = my_node_.id;
  }
  return static_cast<int>(MessageBytes(*msg)) + 64;
}

void Van::PackMeta(const Meta& meta, char** meta_buf, int* buf_size) {
  std::string s;
  pb::EncodeMeta(meta, &s);
  *buf_size = static_cast<int>(s.size());
  if (*meta_buf == nullptr) *meta_buf = new char[s.size() + 1];
  memcpy(*meta_buf, s.data(), s.size());
}

void Van::UnpackMeta(const char* meta_buf, int buf_size, Meta* meta) {
  CHECK(pb::DecodeMeta(meta_buf, static_cast<size_t>(buf_size), meta)) << "failed to parse meta";
}

// ---------------------------------------------------------------------------------------------
void Van::Start(int customer_id) {
  Postoffice* po = Postoffice::Get();
  const bool standalone = IsStandalone();
  {
    std::lock_guard<std::mutex> lk(start_mu_);
    if (init_stage_ == 0) {
      stopping_ = false;
      {
        std::lock_guard<std::mutex> gate(send_gate_mu_);
        send_closed_ = false;
      }
      scheduler_.hostname = GetEnv("DMLC_PS_ROOT_URI", std::string("127.0.0.1"));
      scheduler_.port = GetEnv("DMLC_PS_ROOT_PORT", 0);
      scheduler_.role = Node::SCHEDULER;
      scheduler_.id = kScheduler;
      is_scheduler_ = po->is_scheduler();
      heartbeat_timeout_ = GetEnv("PS_HEARTBEAT_TIMEOUT", 0);
      drop_rate_ = GetEnv("PS_DROP_MSG", 0);

      if (standalone) {
        // one process is scheduler, server 0 and worker 0; nothing to negotiate
        my_node_.role = Node::JOINT;
        my_node_.hostname = "local";
        my_node_.port = 0;
        my_node_.id = Postoffice::WorkerRankToID(0);
        my_node_.customer_id = customer_id;
        my_ids_ = {kScheduler, Postoffice::ServerRankToID(0), my_node_.id};
        StartBackend();
        ready_ = true;
      } else if (is_scheduler_) {
        CHECK(scheduler_.port > 0) << "DMLC_PS_ROOT_PORT must be set";
        my_node_ = scheduler_;
        my_ids_ = {kScheduler};
        StartBackend();
        my_node_.port = Bind(my_node_, 0);
        CHECK_NE(my_node_.port, -1) << "scheduler cannot bind to " << AddrKey(scheduler_);
      } else {
        CHECK(scheduler_.port > 0) << "DMLC_PS_ROOT_PORT must be set";
        my_node_.role = po->is_joint() ? Node::JOINT
                                       : (po->is_worker() ? Node::WORKER : Node::SERVER);
        std::string host = GetEnv("DMLC_NODE_HOST", std::string());
        if (host.empty()) {
          std::string itf = GetEnv("DMLC_INTERFACE", std::string());
          if (!itf.empty()) host = net::IpOfInterface(itf);
          if (host.empty()) host = net::FirstNonLoopbackIp();
          if (host.empty()) host = "127.0.0.1";
          // a scheduler on loopback can only be reached from loopback
          if (scheduler_.hostname == "127.0.0.1" || scheduler_.hostname == "localhost")
            host = "127.0.0.1";
        }
        int port = GetEnv("PORT", 0);
        if (port <= 0) port = net::FreePort();
        CHECK(port > 0) << "no free port";
        my_node_.hostname = host;
        my_node_.port = port;
        my_node_.id = Node::kEmpty;
        my_node_.customer_id = customer_id;
        StartBackend();
        my_node_.port = Bind(my_node_, 40);
        CHECK_NE(my_node_.port, -1) << "bind failed";
      }
      PS_VLOG(1) << "bound to " << my_node_.DebugString();
      if (!standalone) Connect(scheduler_);
      // The reliability layer exists before the first message can arrive, so that nothing
      // is delivered without being recorded for de-duplication.
      if (GetEnv("PS_RESEND", 0) != 0 && !standalone) {
        const int timeout_ms = GetEnv("PS_RESEND_TIMEOUT", 1000);
        resender_ = new Resender(timeout_ms, 10, this);
      }
      receiver_thread_.reset(new std::thread(&Van::Receiving, this));
      if (priority_mode_) sender_thread_.reset(new std::thread(&Van::PrioritySending, this));
      init_stage_ = 1;
    }
  }

  if (!is_scheduler_ && !standalone) {
    // every customer thread of this process announces itself: the scheduler gives each a
    // worker id and maps registrations from one address onto one connection
    Node me = my_node_;
    me.customer_id = customer_id;
    me.id = Node::kEmpty;
    Message msg;
    msg.meta.recver = kScheduler;
    msg.meta.control.cmd = Control::ADD_NODE;
    msg.meta.control.node.push_back(me);
    msg.meta.timestamp = timestamp_++;
    msg.meta.request = true;
    Send(msg);
  }

  // wait for the node table
  while (!ready_.load()) std::this_thread::sleep_for(std::chrono::milliseconds(2));

  {
    std::lock_guard<std::mutex> lk(start_mu_);
    if (init_stage_ == 1) {
      if (!is_scheduler_ && !standalone && GetEnv("PS_HEARTBEAT_INTERVAL", 0) > 0) {
        heartbeat_thread_.reset(new std::thread(&Van::Heartbeat, this));
      }
      init_stage_ = 2;
    }
  }
}

void Van::Stop() {
  if (resender_) {
    // Give lost final messages (for instance a barrier release) a chance to be resent: a peer
    // that never gets it would wait forever.  Retransmissions back off (after 1, 3, 6 and 10
    // timeouts), so ten timeouts cover four of them; with everything acknowledged this
    // returns at once.
    resender_->set_quiet(true);
    resender_->WaitDrained(10 * GetEnv("PS_RESEND_TIMEOUT", 1000));
  }
  // wake the receive loop with a TERMINATE addressed to ourselves
  Message exit;
  exit.meta.control.cmd = Control::TERMINATE;
  exit.meta.recver = my_node_.id;
  exit.meta.sender = my_node_.id;
  exit.meta.customer_id = 0;
  stopping_ = true;
  Deliver(std::move(exit));
  if (receiver_thread_) receiver_thread_->join();
  receiver_thread_.reset();
  if (sender_thread_) {
    Message wake;
    wake.meta.control.cmd = Control::TERMINATE;
    wake.meta.priority = INT_MIN;
    send_queue_.Push(wake);
    sender_thread_->join();
    sender_thread_.reset();
  }
  if (heartbeat_thread_) heartbeat_thread_->join();
  heartbeat_thread_.reset();
  {
    // no send may be inside the van while it is taken apart; later ones are refused
    std::unique_lock<std::mutex> lk(send_gate_mu_);
    send_closed_ = true;
    send_gate_cv_.wait(lk, [this] { return sends_in_flight_ == 0; });
  }
  delete resender_;
  resender_ = nullptr;
  StopBackend();
  ready_ = false;
  init_stage_ = 0;
  my_ids_.clear();
  pending_.clear();
  parked_.clear();
  table_.clear();
  addr_to_ids_.clear();
  std::fill(barrier_count_.begin(), barrier_count_.end(), 0);
  num_servers_seen_ = num_workers_seen_ = 0;
  timestamp_ = 0;
  my_node_ = Node();
  Message junk;
  while (inbox_.TryPop(&junk)) {}
}

// ---------------------------------------------------------------------------------------------
int Van::Send(const Message& msg) {
  Message m = msg;
  if (m.meta.sender == Meta::kEmpty) m.meta.sender = my_node_.id;
  if (priority_mode_ && m.meta.control.empty()) {
    // priority mode: data messages wait in the send queue; the sender thread always takes
    // the pending message of highest priority (reference: src/p3_van.h:35-50)
    send_queue_.Push(m);
    return static_cast<int>(MessageBytes(m));
  }
  return Transmit(m);
}

int Van::Transmit(const Message& m) {
  {
    std::lock_guard<std::mutex> lk(send_gate_mu_);
    if (send_closed_) return -1;
    ++sends_in_flight_;
  }
  struct Leave {
    Van* v;
    ~Leave() {
      std::lock_guard<std::mutex> lk(v->send_gate_mu_);
      if (--v->sends_in_flight_ == 0) v->send_gate_cv_.notify_all();
    }
  } leave{this};
  int bytes;
  if (ready_.load() && IsLocalId(m.meta.recver)) {
    bytes = DeliverLocal(m);
  } else {
    bytes = SendMsg(m);
    if (bytes >= 0 && resender_) resender_->AddOutgoing(m);
  }
  if (bytes < 0) {
    LOG(WARNING) << "failed to send: " << m.DebugString();
    return -1;
  }
  send_bytes_ += bytes;
  if (Postoffice::Get()->verbose() >= 2) PS_VLOG(2) << "send " << m.DebugString();
  return bytes;
}

int Van::DeliverLocal(const Message& m) {
  Message copy = m;
  Deliver(std::move(copy));
  return static_cast<int>(MessageBytes(m));
}

void Van::PrioritySending() {
  for (;;) {
    Message m;
    send_queue_.WaitAndPop(&m);
    if (!m.meta.control.empty() && m.meta.control.cmd == Control::TERMINATE) break;
    Transmit(m);
  }
}

// ---------------------------------------------------------------------------------------------
void Van::Receiving() {
  std::mt19937 rng(static_cast<unsigned>(time(nullptr)) + static_cast<unsigned>(getpid()));
  for (;;) {
    Message msg;
    const int bytes = RecvMsg(&msg);
    if (bytes < 0) break;
    const Control& ctrl = msg.meta.control;
    if (ctrl.empty() && msg.meta.app_id == Meta::kEmpty && msg.meta.body == "__kick__") {
      RetryParked();  // a customer registered
      continue;
    }
    const bool local = IsLocalId(msg.meta.sender) && ready_.load();
    // fault injection: lose a share of the received messages once the node is ready
    if (ready_.load() && drop_rate_ > 0 && !local &&
        !(ctrl.cmd == Control::TERMINATE) &&
        static_cast<int>(rng() % 100) < drop_rate_) {
      LOG(WARNING) << "drop message " << msg.DebugString();
      continue;
    }
    recv_bytes_ += bytes;
    if (Postoffice::Get()->verbose() >= 2) PS_VLOG(2) << "recv " << msg.DebugString();
    if (resender_ && !local && resender_->AddIncomming(msg)) continue;  // ACK or duplicate

    if (!ctrl.empty()) {
      if (ctrl.cmd == Control::TERMINATE) {
        ProcessTerminateCommand();
        break;
      } else if (ctrl.cmd == Control::ADD_NODE) {
        ProcessAddNodeCommand(&msg);
      } else if (ctrl.cmd == Control::BARRIER) {
        ProcessBarrierCommand(&msg);
      } else if (ctrl.cmd == Control::HEARTBEAT) {
        ProcessHeartbeat(&msg);
      } else if (ctrl.cmd == Control::ACK) {
        // an ACK that reached us without a resender: nothing to do
      } else {
        LOG(WARNING) << "drop unknown control message " << msg.DebugString();
      }
    } else {
      ProcessDataMsg(&msg);
    }
    RetryParked();
  }
}

void Van::ProcessTerminateCommand() {
  PS_VLOG(1) << my_node_.ShortDebugString() << " is stopped";
  ready_ = false;
}

Customer* Van::FindCustomer(const Message& msg) {
  const int app_id = msg.meta.app_id;
  Postoffice* po = Postoffice::Get();
  if (!msg.meta.simple_app) {
    // key-value traffic: requests go to the server-side endpoint of the app (registered
    // with customer id = app id), responses to the worker-side endpoint that asked
    if (msg.meta.request) return po->GetCustomer(app_id, app_id, 0, Customer::kServerSide);
    return po->GetCustomer(app_id, msg.meta.customer_id, 0, Customer::kWorkerSide);
  }
  Customer* c = nullptr;
  if (Postoffice::IsServerID(msg.meta.recver))
    c = po->GetCustomer(app_id, app_id, 0, Customer::kServerSide);
  if (!c) c = po->GetCustomer(app_id, msg.meta.customer_id, 0, -1);
  if (!c) c = po->GetCustomer(app_id, app_id, 0, -1);
  return c;
}

// A simple-app request for a customer that has only just been created waits a moment: its
// application object may not have been given its request handle yet (see Customer::Mature).
static bool Deliverable(const Message& msg, const Customer* c) {
  return !(msg.meta.simple_app && msg.meta.request) || c->Mature();
}

void Van::ProcessDataMsg(Message* msg) {
  CHECK_NE(msg->meta.sender, Meta::kEmpty);
  CHECK_NE(msg->meta.recver, Meta::kEmpty);
  CHECK_NE(msg->meta.app_id, Meta::kEmpty);
  {
    std::lock_guard<std::mutex> gate(Postoffice::Get()->customer_gate());
    Customer* c = FindCustomer(*msg);
    if (c && Deliverable(*msg, c)) {
      c->Accept(*msg);
      return;
    }
  }
  // The application endpoint does not exist yet (a peer was faster than this node's own
  // start-up).  The receive loop must not wait for it -- the barrier release that lets the
  // application get that far may be the next message -- so the message is parked and
  // retried whenever something else arrives or a customer registers.
  parked_.push_back(Parked{*msg, std::chrono::steady_clock::now()});
}

void Van::RetryParked() {
  if (parked_.empty()) return;
  const int limit_s = GetEnv("PS_CUSTOMER_TIMEOUT", 30);
  const auto now = std::chrono::steady_clock::now();
  for (auto it = parked_.begin(); it != parked_.end();) {
    bool delivered = false;
    {
      std::lock_guard<std::mutex> gate(Postoffice::Get()->customer_gate());
      Customer* c = FindCustomer(it->msg);
      if (c && Deliverable(it->msg, c)) {
        c->Accept(it->msg);
        delivered = true;
      }
    }
    if (delivered) {
      it = parked_.erase(it);
    } else if (now - it->since > std::chrono::seconds(limit_s)) {
      LOG(ERROR) << "dropping a message for which no customer appeared within " << limit_s
                 << " s at node " << my_node_.id << ": " << it->msg.DebugString();
      it = parked_.erase(it);
    } else {
      ++it;
    }
  }
}

void Van::Kick() {
  Message m;
  m.meta.body = "__kick__";
  m.meta.sender = m.meta.recver = my_node_.id;
  Deliver(std::move(m));
}

// ---- barriers -------------------------------------------------------------------------------
void Van::ProcessBarrierCommand(Message* msg) {
  const Control& ctrl = msg->meta.control;
  if (msg->meta.request) {
    CHECK(IsLocalId(kScheduler)) << "barrier request reached a non-scheduler node";
    const int group = ctrl.barrier_group;
    CHECK(group > 0 && group < 8) << "bad barrier group " << group;
    ++barrier_count_[group];
    const auto& members = Postoffice::Get()->GetNodeIDs(group);
    PS_VLOG(1) << "barrier count for group " << group << ": " << barrier_count_[group] << "/"
               << members.size();
    if (barrier_count_[group] == static_cast<int>(members.size())) {
      barrier_count_[group] = 0;
      Message res;
      res.meta.request = false;
      res.meta.app_id = msg->meta.app_id;
      res.meta.customer_id = msg->meta.customer_id;
      res.meta.control.cmd = Control::BARRIER;
      res.meta.control.barrier_group = group;
      res.meta.sender = kScheduler;
      for (int r : members) {
        res.meta.recver = r;
        res.meta.timestamp = timestamp_++;
        Send(res);
      }
    }
  } else {
    Postoffice::Get()->Manage(*msg);
  }
}

// ---- heartbeats -----------------------------------------------------------------------------
void Van::ProcessHeartbeat(Message* msg) {
  const time_t now = time(nullptr);
  for (const Node& n : msg->meta.control.node) {
    Postoffice::Get()->UpdateHeartbeat(n.id, now);
    if (IsLocalId(kScheduler) && msg->meta.request) {
      // echo so that the node can tell the scheduler is alive
      Message back;
      back.meta.control.cmd = Control::HEARTBEAT;
      back.meta.control.node.push_back(scheduler_);
      back.meta.request = false;
      back.meta.sender = kScheduler;
      back.meta.recver = n.id;
      back.meta.timestamp = timestamp_++;
      Send(back);
    }
  }
}

void Van::Heartbeat() {
  const int interval = GetEnv("PS_HEARTBEAT_INTERVAL", 0);
  const auto step = std::chrono::milliseconds(50);
  auto next = std::chrono::steady_clock::now();
  while (interval > 0 && !stopping_.load()) {
    if (std::chrono::steady_clock::now() < next || !ready_.load()) {
      std::this_thread::sleep_for(step);
      continue;
    }
    next = std::chrono::steady_clock::now() + std::chrono::seconds(interval);
    for (int id : my_ids_) {
      Message msg;
      msg.meta.recver = kScheduler;
      msg.meta.sender = id;
      msg.meta.request = true;
      msg.meta.control.cmd = Control::HEARTBEAT;
      Node me = my_node_;
      me.id = id;
      msg.meta.control.node.push_back(me);
      msg.meta.timestamp = timestamp_++;
      Send(msg);
    }
  }
}

// ---- registration ---------------------------------------------------------------------------
void Van::ProcessAddNodeCommand(Message* msg) {
  if (IsLocalId(kScheduler)) {
    SchedulerRegister(msg);
    return;
  }
  const auto& nodes = msg->meta.control.node;
  if (!ready_.load()) {
    AdoptNodeTable(nodes);
  } else {
    // a recovered node joined under an existing id: point that id at its new address
    for (const Node& n : nodes) {
      if (IsLocalId(n.id)) continue;
      Connect(n);
      PS_VLOG(1) << my_node_.ShortDebugString() << " reconnected to " << n.DebugString();
    }
  }
}

void Van::AdoptNodeTable(const std::vector<Node>& nodes) {
  const std::string mine = AddrKey(my_node_);
  std::vector<int> ids;
  bool recovered = false;
  for (const Node& n : nodes) {
    if (n.role != Node::SCHEDULER && AddrKey(n) == mine) {
      ids.push_back(n.id);
      recovered = recovered || n.is_recovery;
    }
  }
  CHECK(!ids.empty()) << "the node table does not list " << mine;
  std::sort(ids.begin(), ids.end());
  my_ids_ = ids;
  // primary id: the first worker id if this process has one, else the first server id
  int primary = ids[0];
  for (int id : ids) {
    if (Postoffice::IsWorkerID(id)) { primary = id; break; }
  }
  my_node_.id = primary;
  my_node_.is_recovery = recovered;
  const int rank = Postoffice::IDtoRank(primary);
  Environment::Get()->set("DMLC_RANK", std::to_string(rank));
  setenv("DMLC_RANK", std::to_string(rank).c_str(), 1);
  for (const Node& n : nodes) {
    if (IsLocalId(n.id)) continue;
    Connect(n);
  }
  PS_VLOG(1) << my_node_.ShortDebugString() << " joined; ids:" << [&] {
    std::ostringstream os;
    for (int id : my_ids_) os << " " << id;
    return os.str();
  }();
  ready_ = true;
}

void Van::SchedulerRegister(Message* msg) {
  Postoffice* po = Postoffice::Get();
  CHECK_EQ(msg->meta.control.node.size(), (size_t)1) << "ADD_NODE must carry one node";
  Node node = msg->meta.control.node[0];
  const time_t now = time(nullptr);

  if (table_.empty()) {
    // still collecting: ignore retransmissions of the same (address, customer)
    for (const auto& r : pending_) {
      if (AddrKey(r.node) == AddrKey(node) && r.node.customer_id == node.customer_id) return;
    }
    pending_.push_back(Registration{node});
    if (node.role == Node::SERVER || node.role == Node::JOINT) ++num_servers_seen_;
    if (node.role == Node::WORKER || node.role == Node::JOINT) ++num_workers_seen_;
    PS_VLOG(1) << "registration " << pending_.size() << ": " << node.DebugString();
    if (num_servers_seen_ >= po->num_servers() && num_workers_seen_ >= po->num_workers()) {
      CHECK_EQ(num_servers_seen_, po->num_servers()) << "more servers registered than expected";
      CHECK_EQ(num_workers_seen_, po->num_workers()) << "more workers registered than expected";
      SchedulerAssignAndBroadcast();
    }
    return;
  }

  // The table is complete: this is a replacement for a node that died.  It takes over the
  // ids of dead nodes of its role (reference: src/van.cc:136-153, :100-122).
  std::vector<int> dead = po->GetDeadNodes(heartbeat_timeout_);
  std::unordered_set<int> dead_set(dead.begin(), dead.end());
  // a retransmitted registration of an already admitted newcomer
  for (const Node& t : table_) {
    if (AddrKey(t) == AddrKey(node) && t.role != Node::SCHEDULER) return;
  }
  int reuse_server = -1, reuse_worker = -1;
  const bool want_server = node.role == Node::SERVER || node.role == Node::JOINT;
  const bool want_worker = node.role == Node::WORKER || node.role == Node::JOINT;
  for (const Node& t : table_) {
    if (!dead_set.count(t.id)) continue;
    if (want_server && reuse_server < 0 && t.role == Node::SERVER) {
      if (node.role == Node::JOINT) {
        // a joint replacement needs the matching worker id to be dead as well
        const int wid = Postoffice::WorkerRankToID(Postoffice::IDtoRank(t.id));
        if (!dead_set.count(wid)) continue;
        reuse_worker = wid;
      }
      reuse_server = t.id;
    } else if (want_worker && !want_server && reuse_worker < 0 && t.role == Node::WORKER) {
      reuse_worker = t.id;
    }
  }
  if ((want_server && reuse_server < 0) || (want_worker && reuse_worker < 0)) {
    LOG(WARNING) << "registration from " << node.DebugString()
                 << " rejected: the node table is full and no node of that role is dead";
    return;
  }
  (void)now;
  SchedulerAdmitRecovery(node, reuse_server, reuse_worker);
}

void Van::SchedulerAssignAndBroadcast() {
  // rank order = order of (hostname, port, customer id), which every run reproduces for the
  // same placement
  std::sort(pending_.begin(), pending_.end(), [](const Registration& a, const Registration& b) {
    if (a.node.hostname != b.node.hostname) return a.node.hostname < b.node.hostname;
    if (a.node.port != b.node.port) return a.node.port < b.node.port;
    return a.node.customer_id < b.node.customer_id;
  });
  const time_t now = time(nullptr);
  int next_server = 0, next_worker = 0;
  for (const auto& r : pending_) {
    auto add = [&](Node::Role role, int id) {
      Node n = r.node;
      n.role = role;
      n.id = id;
      table_.push_back(n);
      addr_to_ids_[AddrKey(n)].push_back(id);
      Connect(n);
      Postoffice::Get()->UpdateHeartbeat(id, now);
      PS_VLOG(1) << "assign id " << id << " to " << n.DebugString();
    };
    if (r.node.role == Node::SERVER || r.node.role == Node::JOINT)
      add(Node::SERVER, Postoffice::ServerRankToID(next_server++));
    if (r.node.role == Node::WORKER || r.node.role == Node::JOINT)
      add(Node::WORKER, Postoffice::WorkerRankToID(next_worker++));
  }
  table_.push_back(my_node_);  // the scheduler itself

  Message back;
  back.meta.control.cmd = Control::ADD_NODE;
  back.meta.control.node = table_;
  back.meta.sender = kScheduler;
  back.meta.request = false;
  for (const auto& kv : addr_to_ids_) {
    back.meta.recver = kv.second.front();  // one copy per process
    back.meta.timestamp = timestamp_++;
    Send(back);
  }
  PS_VLOG(1) << "the scheduler is connected to " << next_worker << " workers and "
             << next_server << " servers";
  ready_ = true;
}

void Van::SchedulerAdmitRecovery(const Node& newcomer, int reuse_server_id,
                                 int reuse_worker_id) {
  const time_t now = time(nullptr);
  std::vector<Node> fresh;
  for (Node& t : table_) {
    if (t.id == reuse_server_id || t.id == reuse_worker_id) {
      auto& old_ids = addr_to_ids_[AddrKey(t)];
      old_ids.erase(std::remove(old_ids.begin(), old_ids.end(), t.id), old_ids.end());
      if (old_ids.empty()) addr_to_ids_.erase(AddrKey(t));
      t.hostname = newcomer.hostname;
      t.port = newcomer.port;
      t.customer_id = newcomer.customer_id;
      t.is_recovery = true;
      addr_to_ids_[AddrKey(t)].push_back(t.id);
      Connect(t);
      Postoffice::Get()->UpdateHeartbeat(t.id, now);
      fresh.push_back(t);
      PS_VLOG(1) << "node " << t.id << " is replaced by " << t.DebugString();
    }
  }
  std::vector<int> dead = Postoffice::Get()->GetDeadNodes(heartbeat_timeout_);
  std::unordered_set<int> dead_set(dead.begin(), dead.end());
  // the newcomer gets the full table; every live process gets the newcomer's entries
  for (const auto& kv : addr_to_ids_) {
    const int rid = kv.second.front();
    const bool is_newcomer = (kv.first == AddrKey(newcomer));
    if (!is_newcomer && dead_set.count(rid)) continue;
    Message back;
    back.meta.control.cmd = Control::ADD_NODE;
    back.meta.control.node = is_newcomer ? table_ : fresh;
    back.meta.sender = kScheduler;
    back.meta.request = false;
    back.meta.recver = rid;
    back.meta.timestamp = timestamp_++;
    Send(back);
  }
}

}  // namespace ps
