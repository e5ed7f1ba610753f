// Key-value applications: KVWorker pushes and pulls sorted (key -> value[]) lists to the
// servers that own the key ranges; KVServer runs a user-defined request handle.
//
// Public surface of the reference's include/ps/kv_app.h (KVPairs :33-45, KVWorker :54-372,
// KVMeta :375-388, KVServer :393-434, KVServerDefaultHandle :440-463).  Internals are new:
// the slicer computes all cut points in one pass over the range boundaries, and pulled
// slices are kept per server rank, so reassembly is a walk in rank order with no sort.
#ifndef PS_KV_APP_H_
#define PS_KV_APP_H_
#include <algorithm>
#include <chrono>
#include <condition_variable>
#include <exception>
#include <functional>
#include <memory>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <utility>
#include <vector>

#include "ps/base.h"
#include "ps/simple_app.h"

namespace ps {

// A list of key-value pairs.  Keys are unique and increasing.  Without `lens` every value
// has the same length k = vals.size() / keys.size(); with `lens`, value i has lens[i]
// elements and values are concatenated in key order.
template <typename Val>
struct KVPairs {
  SArray<Key> keys;
  SArray<Val> vals;
  SArray<int> lens;
  int priority = 0;
};

template <typename Val>
class KVWorker : public SimpleApp {
 public:
  using SimpleApp::obj_;
  // Runs when a push or pull has completed (on the receive thread of this worker).
  using Callback = std::function<void()>;

  // `app_id` must equal the KVServer's app id; `customer_id` is unique per worker endpoint
  // within this process.
  explicit KVWorker(int app_id, int customer_id) : SimpleApp() {
    slicer_ = [this](const KVPairs<Val>& send, const std::vector<Range>& ranges,
                     SlicedKVs* sliced) { DefaultSlicer(send, ranges, sliced); };
    obj_ = new Customer(app_id, customer_id, [this](const Message& m) { Process(m); },
                        Customer::kWorkerSide, /*start=*/false);
    obj_->StartReceiving();  // only now: Process uses obj_
  }
  virtual ~KVWorker() {
    delete obj_;
    obj_ = nullptr;
  }

  // Pushes key-value pairs to the servers.  Returns at once with a timestamp; the data is
  // copied, so the arguments may be reused immediately.  `cmd` is passed to the server
  // handle; `cb` runs on completion; `priority` orders transmission when the van sends by
  // priority.
  int Push(const std::vector<Key>& keys, const std::vector<Val>& vals,
           const std::vector<int>& lens = {}, int cmd = 0, const Callback& cb = nullptr,
           int priority = 0) {
    return ZPush(SArray<Key>(keys), SArray<Val>(vals), SArray<int>(lens), cmd, cb, priority);
  }

  // Pulls the values of `keys` into `*vals` (and their lengths into `*lens` if given).
  // The output vectors must stay alive until Wait(ts) returns or `cb` has run.
  int Pull(const std::vector<Key>& keys, std::vector<Val>* vals,
           std::vector<int>* lens = nullptr, int cmd = 0, const Callback& cb = nullptr,
           int priority = 0) {
    SArray<Key> skeys(keys);
    if (DeviceRoute* route = DeviceRouteFor(skeys)) {
      CHECK_NOTNULL(vals);
      if (vals->empty()) vals->resize(route->PullBytes(obj_->app_id(), skeys) / sizeof(Val));
      if (lens && lens->empty()) lens->resize(keys.size());
      return SubmitToDevice(route, false, true, cmd, skeys, nullptr, 0, vals->data(),
                            vals->size() * sizeof(Val), SArray<int>(),
                            lens ? lens->data() : nullptr, lens ? lens->size() : 0, cb, priority);
    }
    const int ts = AddPullCB(skeys, vals, lens, cmd, cb);
    KVPairs<Val> kvs;
    kvs.keys = skeys;
    kvs.priority = priority;
    Send(ts, false, true, cmd, kvs);
    return ts;
  }

  // Pushes `vals` and pulls the updated values of the same keys into `*outs`.
  int PushPull(const std::vector<Key>& keys, const std::vector<Val>& vals,
               std::vector<Val>* outs, std::vector<int>* lens = nullptr, int cmd = 0,
               const Callback& cb = nullptr, int priority = 0) {
    CHECK_NOTNULL(outs);
    if (outs->empty()) {
      outs->resize(vals.size());
    } else {
      CHECK_EQ(vals.size(), outs->size());
    }
    SArray<Key> skeys(keys);
    SArray<Val> svals(vals);
    // zero-copy views of the caller's output storage
    auto* souts = new SArray<Val>(outs->data(), outs->size());
    SArray<int>* slens = lens ? new SArray<int>(lens->data(), lens->size()) : nullptr;
    return ZPushPull(skeys, svals, souts, slens, cmd,
                     [cb, souts, slens]() {
                       delete souts;
                       delete slens;
                       if (cb) cb();
                     },
                     priority);
  }

  // Blocks until request `timestamp` has completed on every server it went to.
  void Wait(int timestamp) { obj_->WaitRequest(timestamp); }

  // Zero-copy variants: the arrays are shared, not copied; the caller must leave their
  // contents unchanged until the request has completed.
  int ZPush(const SArray<Key>& keys, const SArray<Val>& vals, const SArray<int>& lens = {},
            int cmd = 0, const Callback& cb = nullptr, int priority = 0) {
    if (DeviceRoute* route = DeviceRouteFor(keys)) {
      // the arrays are captured by the completion routine: they stay alive until then
      return SubmitToDevice(route, true, false, cmd, keys, vals.data(),
                            vals.size() * sizeof(Val), nullptr, 0, lens, nullptr, 0,
                            [keys, vals, lens, cb]() { if (cb) cb(); }, priority);
    }
    const int ts = obj_->NewRequest(kServerGroup);
    AddCallback(ts, cb);
    KVPairs<Val> kvs;
    kvs.keys = keys;
    kvs.vals = vals;
    kvs.lens = lens;
    kvs.priority = priority;
    Send(ts, true, false, cmd, kvs);
    return ts;
  }

  int ZPull(const SArray<Key>& keys, SArray<Val>* vals, SArray<int>* lens = nullptr,
            int cmd = 0, const Callback& cb = nullptr, int priority = 0) {
    if (DeviceRoute* route = DeviceRouteFor(keys)) {
      CHECK_NOTNULL(vals);
      if (vals->empty()) vals->resize(route->PullBytes(obj_->app_id(), keys) / sizeof(Val));
      if (lens && lens->empty()) lens->resize(keys.size());
      return SubmitToDevice(route, false, true, cmd, keys, nullptr, 0, vals->data(),
                            vals->size() * sizeof(Val), SArray<int>(),
                            lens ? lens->data() : nullptr, lens ? lens->size() : 0,
                            [keys, cb]() { if (cb) cb(); }, priority);
    }
    const int ts = AddPullCB(keys, vals, lens, cmd, cb);
    KVPairs<Val> kvs;
    kvs.keys = keys;
    kvs.priority = priority;
    Send(ts, false, true, cmd, kvs);
    return ts;
  }

  int ZPushPull(const SArray<Key>& keys, const SArray<Val>& vals, SArray<Val>* outs,
                SArray<int>* lens = nullptr, int cmd = 0, const Callback& cb = nullptr,
                int priority = 0) {
    if (DeviceRoute* route = DeviceRouteFor(keys)) {
      CHECK_NOTNULL(outs);
      if (outs->empty()) outs->resize(vals.size());
      return SubmitToDevice(route, true, true, cmd, keys, vals.data(),
                            vals.size() * sizeof(Val), outs->data(), outs->size() * sizeof(Val),
                            lens ? *lens : SArray<int>(), nullptr, 0,
                            [keys, vals, cb]() { if (cb) cb(); }, priority);
    }
    const int ts = AddPullCB(keys, outs, lens, cmd, cb);
    KVPairs<Val> kvs;
    kvs.keys = keys;
    kvs.vals = vals;
    kvs.priority = priority;
    if (lens) kvs.lens = *lens;
    Send(ts, true, true, cmd, kvs);
    return ts;
  }

  // sliced[i] = (true, pairs for server i) or (false, -) when server i gets nothing.
  using SlicedKVs = std::vector<std::pair<bool, KVPairs<Val>>>;
  // Splits a request by the servers' key ranges.
  using Slicer = std::function<void(const KVPairs<Val>& send, const std::vector<Range>& ranges,
                                    SlicedKVs* sliced)>;
  void set_slicer(const Slicer& slicer) {
    CHECK(slicer);
    slicer_ = slicer;
  }

 private:
  // The device plane, if it is attached and serves `keys` (a tensor registered for this app).
  DeviceRoute* DeviceRouteFor(const SArray<Key>& keys) {
    DeviceRoute* route = Postoffice::Get()->device_route();
    if (route && keys.size() && route->Claims(obj_->app_id(), keys)) return route;
    return nullptr;
  }

  // Hands a request to the device plane.  The tracker entry is the usual one (one response
  // expected per server); the plane credits all of them when its kernels have completed,
  // after the callback has run, so Wait(ts) has the reference's meaning.
  int SubmitToDevice(DeviceRoute* route, bool push, bool pull, int cmd, const SArray<Key>& keys,
                     const void* vals, size_t vals_bytes, void* outs, size_t outs_bytes,
                     const SArray<int>& lens, int* lens_out, size_t lens_out_n,
                     const Callback& cb, int priority) {
    const int ts = obj_->NewRequest(kServerGroup);
    DeviceRequest req;
    req.app_id = obj_->app_id();
    req.timestamp = ts;
    req.push = push;
    req.pull = pull;
    req.cmd = cmd;
    req.priority = priority;
    req.keys = keys;
    req.lens = lens;
    req.vals = vals;
    req.vals_bytes = vals_bytes;
    req.outs = outs;
    req.outs_bytes = outs_bytes;
    req.lens_out = lens_out;
    req.lens_out_n = lens_out_n;
    req.val_size = sizeof(Val);
    req.customer = obj_;
    req.responses = Postoffice::Get()->num_servers();
    req.on_done = cb;
    route->Submit(req);
    return ts;
  }

  // One pulled slice, kept in the slot of the server that sent it.
  struct PullSlot {
    bool filled = false;
    KVPairs<Val> kvs;
  };

  // Registers the completion routine of a pull: validate the slices, size the outputs,
  // concatenate in server-rank order (which is key order), then run the user callback.
  template <typename C, typename D>
  int AddPullCB(const SArray<Key>& keys, C* vals, D* lens, int cmd, const Callback& cb) {
    const int ts = obj_->NewRequest(kServerGroup);
    AddCallback(ts, [this, ts, keys, vals, lens, cb]() mutable {
      std::vector<PullSlot> slots;
      {
        std::lock_guard<std::mutex> lk(mu_);
        slots = std::move(pulled_[ts]);
        pulled_.erase(ts);
      }
      size_t nkeys = 0, nvals = 0;
      Key prev_last = 0;
      bool have_prev = false;
      for (const PullSlot& s : slots) {
        if (!s.filled || s.kvs.keys.empty()) continue;
        // slices must tile the requested keys in order
        CHECK_EQ(s.kvs.keys.front(), keys[static_cast<int>(nkeys)])
            << "pulled slice does not start at the expected key";
        if (have_prev) { CHECK_GT(s.kvs.keys.front(), prev_last); }
        prev_last = s.kvs.keys.back();
        have_prev = true;
        nkeys += s.kvs.keys.size();
        nvals += s.kvs.vals.size();
        if (lens) { CHECK_EQ(s.kvs.lens.size(), s.kvs.keys.size()); }
      }
      CHECK_EQ(nkeys, keys.size()) << "lost some servers?";
      if (vals->empty()) {
        vals->resize(nvals);
      } else {
        CHECK_EQ(vals->size(), nvals);
      }
      if (lens) {
        if (lens->empty()) {
          lens->resize(nkeys);
        } else {
          CHECK_EQ(lens->size(), nkeys);
        }
      }
      Val* vdst = vals->data();
      int* ldst = lens ? lens->data() : nullptr;
      for (const PullSlot& s : slots) {
        if (!s.filled) continue;
        if (!s.kvs.vals.empty()) {
          memcpy(vdst, s.kvs.vals.data(), s.kvs.vals.size() * sizeof(Val));
          vdst += s.kvs.vals.size();
        }
        if (ldst && !s.kvs.lens.empty()) {
          memcpy(ldst, s.kvs.lens.data(), s.kvs.lens.size() * sizeof(int));
          ldst += s.kvs.lens.size();
        }
      }
      if (cb) cb();
    });
    return ts;
  }

  void AddCallback(int timestamp, const Callback& cb) {
    if (!cb) return;
    std::lock_guard<std::mutex> lk(mu_);
    callbacks_[timestamp] = cb;
  }

  void RunCallback(int timestamp) {
    Callback cb;
    {
      std::lock_guard<std::mutex> lk(mu_);
      auto it = callbacks_.find(timestamp);
      if (it == callbacks_.end()) return;
      cb = std::move(it->second);
      callbacks_.erase(it);
    }
    cb();
  }

  // requests whose slices add up to at least this many bytes are sent to their servers in
  // parallel
  static constexpr size_t kParallelSendBytes = 1 << 20;

  void Send(int timestamp, bool push, bool pull, int cmd, const KVPairs<Val>& kvs) {
    SlicedKVs sliced;
    slicer_(kvs, Postoffice::Get()->GetServerKeyRanges(), &sliced);
    // servers that get nothing count as having answered
    int skipped = 0;
    for (const auto& s : sliced) skipped += s.first ? 0 : 1;
    obj_->AddResponse(timestamp, skipped);
    if (static_cast<size_t>(skipped) == sliced.size()) RunCallback(timestamp);

    std::vector<Message> msgs;
    size_t payload = 0;
    for (size_t i = 0; i < sliced.size(); ++i) {
      if (!sliced[i].first) continue;
      const KVPairs<Val>& part = sliced[i].second;
      msgs.emplace_back();
      Message& msg = msgs.back();
      msg.meta.app_id = obj_->app_id();
      msg.meta.customer_id = obj_->customer_id();
      msg.meta.request = true;
      msg.meta.push = push;
      msg.meta.pull = pull;
      msg.meta.head = cmd;
      msg.meta.timestamp = timestamp;
      msg.meta.recver = Postoffice::ServerRankToID(static_cast<int>(i));
      msg.meta.priority = kvs.priority;
      if (part.keys.size()) {
        msg.AddData(part.keys);
        msg.AddData(part.vals);  // empty for a pure pull: the frame is still sent
        if (part.lens.size()) msg.AddData(part.lens);
      }
      for (const auto& d : msg.data) payload += d.size();
    }
    Van* van = Postoffice::Get()->van();
    if (msgs.size() < 2 || payload < kParallelSendBytes) {
      for (const Message& m : msgs) van->Send(m);
      return;
    }
    // Large slices for several servers leave at the same time, one thread per further server:
    // a blocking send to one server would otherwise keep the others idle until it has been
    // received.  (Messages to one server keep their order: a server gets one slice.)
    std::vector<std::thread> others;
    std::vector<std::exception_ptr> failed(msgs.size());
    for (size_t i = 1; i < msgs.size(); ++i) {
      others.emplace_back([van, &msgs, &failed, i]() {
        try {
          van->Send(msgs[i]);
        } catch (...) {
          failed[i] = std::current_exception();
        }
      });
    }
    try {
      van->Send(msgs[0]);
    } catch (...) {
      failed[0] = std::current_exception();
    }
    for (auto& t : others) t.join();
    for (auto& f : failed)
      if (f) std::rethrow_exception(f);
  }

  // Handles a response from a server (or a simple-app message).
  void Process(const Message& msg) {
    if (msg.meta.simple_app) {
      SimpleApp::Process(msg);
      return;
    }
    const int ts = msg.meta.timestamp;
    if (msg.meta.pull) {
      CHECK_GE(msg.data.size(), (size_t)2);
      PullSlot slot;
      slot.filled = true;
      slot.kvs.keys = msg.data[0];
      slot.kvs.vals = msg.data[1];
      if (msg.data.size() > 2) slot.kvs.lens = msg.data[2];
      const int rank = Postoffice::IDtoRank(msg.meta.sender);
      std::lock_guard<std::mutex> lk(mu_);
      std::vector<PullSlot>& slots = pulled_[ts];
      if (slots.empty()) slots.resize(Postoffice::Get()->num_servers());
      CHECK_LT(static_cast<size_t>(rank), slots.size());
      slots[rank] = std::move(slot);
    }
    // This is the last outstanding response: complete the request now.  The customer
    // thread credits the response after this function returns, so Wait() cannot return
    // before the callback has finished.
    if (obj_->NumResponse(ts) == Postoffice::Get()->num_servers() - 1) RunCallback(ts);
  }

  // Cuts `send` at the servers' range boundaries with one binary search per boundary.
  void DefaultSlicer(const KVPairs<Val>& send, const std::vector<Range>& ranges,
                     SlicedKVs* sliced) {
    const size_t S = ranges.size();
    sliced->assign(S, std::make_pair(false, KVPairs<Val>()));
    const size_t n = send.keys.size();
    if (n == 0) return;
    const Key* kb = send.keys.begin();
    const Key* ke = send.keys.end();
    std::vector<size_t> cut(S + 1);
    const Key* at = std::lower_bound(kb, ke, static_cast<Key>(ranges[0].begin()));
    cut[0] = static_cast<size_t>(at - kb);
    for (size_t i = 0; i < S; ++i) {
      at = std::lower_bound(at, ke, static_cast<Key>(ranges[i].end()));
      cut[i + 1] = static_cast<size_t>(at - kb);
    }
    CHECK_EQ(cut[0], (size_t)0) << "key below the first server range";
    CHECK_EQ(cut[S], n) << "key beyond the last server range";

    // value offsets of the cut points
    std::vector<size_t> voff(S + 1, 0);
    if (send.lens.empty()) {
      const size_t k = send.vals.size() / n;
      CHECK_EQ(k * n, send.vals.size()) << "values do not divide evenly among keys";
      for (size_t i = 0; i <= S; ++i) voff[i] = cut[i] * k;
    } else {
      CHECK_EQ(send.lens.size(), n);
      size_t acc = 0, c = 0;
      for (size_t i = 0; i <= S; ++i) {
        for (; c < cut[i]; ++c) acc += static_cast<size_t>(send.lens[static_cast<int>(c)]);
        voff[i] = acc;
      }
      if (!send.vals.empty()) { CHECK_EQ(acc, send.vals.size()); }
    }
    for (size_t i = 0; i < S; ++i) {
      if (cut[i + 1] == cut[i]) continue;
      auto& out = (*sliced)[i];
      out.first = true;
      out.second.keys = send.keys.segment(cut[i], cut[i + 1]);
      if (!send.vals.empty()) out.second.vals = send.vals.segment(voff[i], voff[i + 1]);
      if (!send.lens.empty()) out.second.lens = send.lens.segment(cut[i], cut[i + 1]);
      out.second.priority = send.priority;
    }
  }

  std::unordered_map<int, std::vector<PullSlot>> pulled_;
  std::unordered_map<int, Callback> callbacks_;
  std::mutex mu_;
  Slicer slicer_;
};

// What a server handle learns about a request besides its data.
struct KVMeta {
  int cmd;
  bool push;
  bool pull;
  int sender;
  int timestamp;
  int customer_id;
};

template <typename Val>
class KVServer : public SimpleApp {
 public:
  // The server-side endpoint of app `app_id`.
  explicit KVServer(int app_id) : SimpleApp() {
    obj_ = new Customer(app_id, app_id, [this](const Message& m) { Process(m); },
                        Customer::kServerSide, /*start=*/false);
    obj_->StartReceiving();  // only now: Process uses obj_
  }
  virtual ~KVServer() {
    delete obj_;
    obj_ = nullptr;
  }

  // The handle runs for every push or pull request.  It must call server->Response(req_meta,
  // ...) exactly once per request, now or later (for instance after all workers pushed).
  using ReqHandle = std::function<void(const KVMeta& req_meta, const KVPairs<Val>& req_data,
                                       KVServer* server)>;
  void set_request_handle(const ReqHandle& request_handle) {
    CHECK(request_handle) << "invalid request handle";
    {
      std::lock_guard<std::mutex> lk(handle_mu_);
      request_handle_ = std::make_shared<ReqHandle>(request_handle);
    }
    handle_cv_.notify_all();
  }

  // Answers request `req`; `res` carries the pulled pairs (empty for a push).
  void Response(const KVMeta& req, const KVPairs<Val>& res = KVPairs<Val>()) {
    Message msg;
    msg.meta.app_id = obj_->app_id();
    msg.meta.customer_id = req.customer_id;
    msg.meta.request = false;
    msg.meta.push = req.push;
    msg.meta.pull = req.pull;
    msg.meta.head = req.cmd;
    msg.meta.timestamp = req.timestamp;
    msg.meta.recver = req.sender;
    if (Postoffice::Get()->is_server())
      msg.meta.sender = Postoffice::ServerRankToID(Postoffice::Get()->my_rank());
    if (res.keys.size()) {
      msg.AddData(res.keys);
      msg.AddData(res.vals);
      if (res.lens.size()) msg.AddData(res.lens);
    }
    Postoffice::Get()->van()->Send(msg);
  }

 private:
  void Process(const Message& msg) {
    if (msg.meta.simple_app) {
      SimpleApp::Process(msg);
      return;
    }
    KVMeta meta;
    meta.cmd = msg.meta.head;
    meta.push = msg.meta.push;
    meta.pull = msg.meta.pull;
    meta.sender = msg.meta.sender;
    meta.timestamp = msg.meta.timestamp;
    meta.customer_id = msg.meta.customer_id;
    KVPairs<Val> data;
    const size_t n = msg.data.size();
    if (n) {
      CHECK_GE(n, (size_t)2);
      data.keys = msg.data[0];
      data.vals = msg.data[1];
      if (n > 2) {
        CHECK_EQ(n, (size_t)3);
        data.lens = msg.data[2];
        CHECK_EQ(data.lens.size(), data.keys.size());
      }
    }
    data.priority = msg.meta.priority;
    // A request can arrive between the construction of the server and set_request_handle
    // (the receive thread starts with the constructor): it waits for the handle instead of
    // failing.  One instance of the handle serves every request, so a handle with state of
    // its own (such as KVServerDefaultHandle's store) keeps it.
    std::shared_ptr<ReqHandle> handle;
    {
      std::unique_lock<std::mutex> lk(handle_mu_);
      handle_cv_.wait_for(lk, std::chrono::seconds(30),
                          [this] { return request_handle_ != nullptr; });
      handle = request_handle_;
    }
    CHECK(handle) << "no request handle set on the server";
    (*handle)(meta, data, this);
  }

  std::mutex handle_mu_;
  std::condition_variable handle_cv_;
  std::shared_ptr<ReqHandle> request_handle_;
};

// Example server handle: values are accumulated per key (push: store[key] += val; pull:
// returns store[key]).  Fixed-length values of any width are supported; with one value per
// key this is the reference's KVServerDefaultHandle (include/ps/kv_app.h:440-463).
template <typename Val>
struct KVServerDefaultHandle {
  void operator()(const KVMeta& req_meta, const KVPairs<Val>& req_data, KVServer<Val>* server) {
    const size_t n = req_data.keys.size();
    KVPairs<Val> res;
    size_t k = 1;
    if (req_meta.push) {
      CHECK(req_data.lens.empty()) << "the default handle takes fixed-length values";
      if (n) {
        k = req_data.vals.size() / n;
        CHECK_EQ(k * n, req_data.vals.size());
        if (width == 0) width = k;
        CHECK_EQ(k, width) << "value width changed";
      }
    } else {
      k = width ? width : 1;
    }
    if (req_meta.pull) {
      res.keys = req_data.keys;
      res.vals.resize(n * k);
    }
    for (size_t i = 0; i < n; ++i) {
      const Key key = req_data.keys[static_cast<int>(i)];
      if (k == 1) {
        Val& slot = store[key];
        if (req_meta.push) slot += req_data.vals[static_cast<int>(i)];
        if (req_meta.pull) res.vals[static_cast<int>(i)] = slot;
      } else {
        std::vector<Val>& slot = wide_store[key];
        if (slot.empty()) slot.assign(k, Val());
        if (req_meta.push)
          for (size_t j = 0; j < k; ++j) slot[j] += req_data.vals[static_cast<int>(i * k + j)];
        if (req_meta.pull)
          for (size_t j = 0; j < k; ++j) res.vals[static_cast<int>(i * k + j)] = slot[j];
      }
    }
    server->Response(req_meta, res);
  }
  std::unordered_map<Key, Val> store;
  std::unordered_map<Key, std::vector<Val>> wide_store;
  size_t width = 0;
};

}  // namespace ps
#endif  // PS_KV_APP_H_
