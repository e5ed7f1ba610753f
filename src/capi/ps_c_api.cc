#include "ps/internal/shm_pool.h"
#include "capi/ps_c_api.h"

#include <cstring>
#include <string>

#include "ps/internal/pb_codec.h"
#include "ps/ps.h"

using namespace ps;

namespace {
thread_local std::string g_err;

template <typename F>
int Guard(F&& f) {
  try {
    return f();
  } catch (const std::exception& e) {
    g_err = e.what();
    return -1;
  }
}

struct ServerBox {
  KVServer<float>* server = nullptr;
  ps_capi_handle_t handle = nullptr;
  void* user = nullptr;
};
struct SimpleBox {
  SimpleApp* app = nullptr;
};
}  // namespace

extern "C" {

const char* ps_capi_last_error(void) { return g_err.c_str(); }
// for the other translation units of the C ABI
void ps_capi_set_error(const char* text) { g_err = text ? text : ""; }

int ps_capi_setenv(const char* key, const char* value) {
  return Guard([&] {
    Environment::Get()->set(key, value);
    return 0;
  });
}

int ps_capi_start(int customer_id, int do_barrier) {
  return Guard([&] {
    Postoffice::Get()->Start(customer_id, nullptr, do_barrier != 0);
    return 0;
  });
}
int ps_capi_finalize(int customer_id, int do_barrier) {
  return Guard([&] {
    Postoffice::Get()->Finalize(customer_id, do_barrier != 0);
    return 0;
  });
}
int ps_capi_barrier(int customer_id, int node_group) {
  return Guard([&] {
    Postoffice::Get()->Barrier(customer_id, node_group);
    return 0;
  });
}
int ps_capi_num_workers(void) { return NumWorkers(); }
int ps_capi_num_servers(void) { return NumServers(); }
int ps_capi_my_rank(void) { return Guard([] { return MyRank(); }); }
int ps_capi_is_worker(void) { return IsWorker(); }
int ps_capi_is_server(void) { return IsServer(); }
int ps_capi_is_scheduler(void) { return IsScheduler(); }
int ps_capi_is_recovery(void) {
  return Guard([] { return Postoffice::Get()->is_recovery() ? 1 : 0; });
}
int ps_capi_dead_nodes(int timeout_s, int* ids, int cap) {
  return Guard([&] {
    std::vector<int> dead = Postoffice::Get()->GetDeadNodes(timeout_s);
    for (int i = 0; i < cap && i < static_cast<int>(dead.size()); ++i) ids[i] = dead[i];
    return static_cast<int>(dead.size());
  });
}
int ps_capi_server_key_range(int rank, uint64_t* begin, uint64_t* end) {
  return Guard([&] {
    const auto& r = Postoffice::Get()->GetServerKeyRanges();
    if (rank < 0 || rank >= static_cast<int>(r.size())) throw Error("rank out of range");
    *begin = r[rank].begin();
    *end = r[rank].end();
    return 0;
  });
}
int ps_capi_traffic(uint64_t* sent, uint64_t* received) {
  return Guard([&] {
    Van* v = Postoffice::Get()->van();
    if (!v) throw Error("van not started");
    *sent = v->send_bytes();
    *received = v->recv_bytes();
    return 0;
  });
}

int ps_capi_shm_stats(uint64_t out[6]) {
  const shm::Stats s = shm::GetStats();
  out[0] = s.segments_created;
  out[1] = s.segments_reused;
  out[2] = s.bytes_live;
  out[3] = s.bytes_pooled;
  out[4] = s.imports;
  out[5] = s.import_hits;
  return 0;
}

// ---- worker ----
void* ps_capi_worker_new(int app_id, int customer_id) {
  try {
    return new KVWorker<float>(app_id, customer_id);
  } catch (const std::exception& e) {
    g_err = e.what();
    return nullptr;
  }
}
int ps_capi_worker_delete(void* worker) {
  return Guard([&] {
    delete static_cast<KVWorker<float>*>(worker);
    return 0;
  });
}
int ps_capi_worker_push(void* worker, const uint64_t* keys, size_t nkeys, const float* vals,
                        size_t nvals, const int* lens, size_t nlens, int cmd, int priority) {
  return Guard([&] {
    SArray<Key> k;
    k.CopyFrom(keys, nkeys);
    SArray<float> v;
    v.CopyFrom(vals, nvals);
    SArray<int> l;
    if (lens && nlens) l.CopyFrom(lens, nlens);
    return static_cast<KVWorker<float>*>(worker)->ZPush(k, v, l, cmd, nullptr, priority);
  });
}
int ps_capi_worker_pull(void* worker, const uint64_t* keys, size_t nkeys, float* vals,
                        size_t nvals, int* lens, size_t nlens, int cmd, int priority) {
  return Guard([&] {
    SArray<Key> k;
    k.CopyFrom(keys, nkeys);
    auto* v = new SArray<float>(vals, nvals);
    SArray<int>* l = (lens && nlens) ? new SArray<int>(lens, nlens) : nullptr;
    return static_cast<KVWorker<float>*>(worker)->ZPull(
        k, v, l, cmd, [v, l]() { delete v; delete l; }, priority);
  });
}
int ps_capi_worker_push_pull(void* worker, const uint64_t* keys, size_t nkeys,
                             const float* vals, size_t nvals, float* outs, int* lens,
                             size_t nlens, int cmd, int priority) {
  return Guard([&] {
    SArray<Key> k;
    k.CopyFrom(keys, nkeys);
    SArray<float> v;
    v.CopyFrom(vals, nvals);
    auto* o = new SArray<float>(outs, nvals);
    SArray<int>* l = (lens && nlens) ? new SArray<int>(lens, nlens) : nullptr;
    return static_cast<KVWorker<float>*>(worker)->ZPushPull(
        k, v, o, l, cmd, [o, l]() { delete o; delete l; }, priority);
  });
}
int ps_capi_worker_wait(void* worker, int timestamp) {
  return Guard([&] {
    static_cast<KVWorker<float>*>(worker)->Wait(timestamp);
    return 0;
  });
}

// ---- server ----
void* ps_capi_server_new(int app_id, ps_capi_handle_t handle, void* user) {
  try {
    auto* box = new ServerBox;
    box->server = new KVServer<float>(app_id);
    box->handle = handle;
    box->user = user;
    if (!handle) {
      box->server->set_request_handle(KVServerDefaultHandle<float>());
    } else {
      box->server->set_request_handle(
          [box](const KVMeta& m, const KVPairs<float>& d, KVServer<float>*) {
            ps_capi_request_t r;
            r.cmd = m.cmd; r.push = m.push; r.pull = m.pull; r.sender = m.sender;
            r.timestamp = m.timestamp; r.customer_id = m.customer_id;
            r.keys = d.keys.data(); r.nkeys = d.keys.size();
            r.vals = d.vals.data(); r.nvals = d.vals.size();
            r.lens = d.lens.data(); r.nlens = d.lens.size();
            box->handle(box, &r, box->user);
          });
    }
    return box;
  } catch (const std::exception& e) {
    g_err = e.what();
    return nullptr;
  }
}
int ps_capi_server_delete(void* server) {
  return Guard([&] {
    auto* box = static_cast<ServerBox*>(server);
    delete box->server;
    delete box;
    return 0;
  });
}
int ps_capi_server_respond(void* server, const ps_capi_request_t* req, const uint64_t* keys,
                           size_t nkeys, const float* vals, size_t nvals, const int* lens,
                           size_t nlens) {
  return Guard([&] {
    auto* box = static_cast<ServerBox*>(server);
    KVMeta m;
    m.cmd = req->cmd; m.push = req->push != 0; m.pull = req->pull != 0; m.sender = req->sender;
    m.timestamp = req->timestamp; m.customer_id = req->customer_id;
    KVPairs<float> res;
    if (nkeys) {
      res.keys.CopyFrom(keys, nkeys);
      res.vals.CopyFrom(vals, nvals);
      if (lens && nlens) res.lens.CopyFrom(lens, nlens);
    }
    box->server->Response(m, res);
    return 0;
  });
}

// ---- simple app ----
void* ps_capi_simple_new(int app_id, int customer_id, ps_capi_simple_handle_t on_request,
                         void* user) {
  try {
    auto* box = new SimpleBox;
    box->app = new SimpleApp(app_id, customer_id);
    if (on_request) {
      box->app->set_request_handle([on_request, user](const SimpleData& d, SimpleApp* app) {
        on_request(d.head, d.body.data(), d.body.size(), d.sender, user);
        app->Response(d);
      });
    }
    return box;
  } catch (const std::exception& e) {
    g_err = e.what();
    return nullptr;
  }
}
int ps_capi_simple_delete(void* app) {
  return Guard([&] {
    auto* box = static_cast<SimpleBox*>(app);
    delete box->app;
    delete box;
    return 0;
  });
}
int ps_capi_simple_request(void* app, int head, const char* body, size_t body_len, int recver) {
  return Guard([&] {
    return static_cast<SimpleBox*>(app)->app->Request(head, std::string(body, body_len), recver);
  });
}
int ps_capi_simple_wait(void* app, int timestamp) {
  return Guard([&] {
    static_cast<SimpleBox*>(app)->app->Wait(timestamp);
    return 0;
  });
}

// ---- codec ----
long ps_capi_encode_meta(const ps_capi_meta_t* in, char* out, size_t cap) {
  try {
    Meta m;
    m.head = in->head; m.app_id = in->app_id; m.customer_id = in->customer_id;
    m.timestamp = in->timestamp; m.request = in->request; m.push = in->push;
    m.pull = in->pull; m.simple_app = in->simple_app; m.priority = in->priority;
    m.control.cmd = static_cast<Control::Command>(in->control_cmd);
    m.control.barrier_group = in->barrier_group;
    m.control.msg_sig = in->msg_sig;
    for (int i = 0; i < in->num_data_types && i < 8; ++i)
      m.data_type.push_back(static_cast<DataType>(in->data_types[i]));
    for (int i = 0; i < in->num_nodes && i < 8; ++i) {
      Node n;
      n.role = static_cast<Node::Role>(in->nodes[i].role);
      n.id = in->nodes[i].id; n.port = in->nodes[i].port;
      n.is_recovery = in->nodes[i].is_recovery; n.customer_id = in->nodes[i].customer_id;
      n.hostname = in->nodes[i].hostname;
      m.control.node.push_back(n);
    }
    m.body.assign(in->body, static_cast<size_t>(in->body_len));
    std::string s;
    pb::EncodeMeta(m, &s);
    if (s.size() <= cap) memcpy(out, s.data(), s.size());
    return static_cast<long>(s.size());
  } catch (const std::exception& e) {
    g_err = e.what();
    return -1;
  }
}
int ps_capi_decode_meta(const char* buf, size_t len, ps_capi_meta_t* out) {
  return Guard([&] {
    Meta m;
    if (!pb::DecodeMeta(buf, len, &m)) throw Error("malformed meta");
    memset(out, 0, sizeof(*out));
    out->head = m.head; out->app_id = m.app_id; out->customer_id = m.customer_id;
    out->timestamp = m.timestamp; out->request = m.request; out->push = m.push;
    out->pull = m.pull; out->simple_app = m.simple_app; out->priority = m.priority;
    out->control_cmd = m.control.cmd; out->barrier_group = m.control.barrier_group;
    out->msg_sig = m.control.msg_sig;
    out->num_data_types = static_cast<int>(std::min<size_t>(8, m.data_type.size()));
    for (int i = 0; i < out->num_data_types; ++i) out->data_types[i] = m.data_type[i];
    out->num_nodes = static_cast<int>(std::min<size_t>(8, m.control.node.size()));
    for (int i = 0; i < out->num_nodes; ++i) {
      const Node& n = m.control.node[i];
      out->nodes[i].role = n.role; out->nodes[i].id = n.id; out->nodes[i].port = n.port;
      out->nodes[i].is_recovery = n.is_recovery; out->nodes[i].customer_id = n.customer_id;
      strncpy(out->nodes[i].hostname, n.hostname.c_str(), 63);
    }
    out->body_len = static_cast<int>(std::min<size_t>(255, m.body.size()));
    memcpy(out->body, m.body.data(), static_cast<size_t>(out->body_len));
    return 0;
  });
}

}  // extern "C"
