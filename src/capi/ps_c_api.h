/*
 * C ABI of the host runtime, for language bindings (Python ctypes in ps_lite_b200.host).
 * It exposes the same operations as the C++ API of include/ps/ps.h for float values:
 * start/finalize, role queries, barriers, KVWorker push/pull/push-pull/wait, KVServer with
 * the built-in sum handle or a callback handle, SimpleApp requests, and the PBMeta codec.
 * The reference has no C or Python binding; its CMake build only generates Python protobuf
 * classes (CMakeLists.txt:44-57).
 */
#ifndef PS_CAPI_PS_C_API_H_
#define PS_CAPI_PS_C_API_H_
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* All functions return 0 (or a non-negative value) on success and -1 after an error whose
 * text ps_capi_last_error() returns (thread local). */
const char* ps_capi_last_error(void);

/* Overrides for the DMLC_* / PS_* environment, consulted before getenv. */
int ps_capi_setenv(const char* key, const char* value);

int ps_capi_start(int customer_id, int do_barrier);
int ps_capi_finalize(int customer_id, int do_barrier);
int ps_capi_barrier(int customer_id, int node_group);
int ps_capi_num_workers(void);
int ps_capi_num_servers(void);
int ps_capi_my_rank(void);
int ps_capi_is_worker(void);
int ps_capi_is_server(void);
int ps_capi_is_scheduler(void);
int ps_capi_is_recovery(void);
/* Writes up to `cap` dead node ids (no heartbeat for `timeout_s`); returns the count. */
int ps_capi_dead_nodes(int timeout_s, int* ids, int cap);
/* Begin/end of server `rank`'s key range. */
int ps_capi_server_key_range(int rank, uint64_t* begin, uint64_t* end);
/* Bytes sent / received by the van so far. */
int ps_capi_traffic(uint64_t* sent, uint64_t* received);
/* Counters of the shared-memory array pool (ps/internal/shm_pool.h), in this order: segments
 * created, segments recycled, bytes backing live arrays, bytes idle in the pool, segments
 * received from peers, of which already mapped.  Works before Start. */
int ps_capi_shm_stats(uint64_t out[6]);

/* ---- KVWorker<float> ---- */
void* ps_capi_worker_new(int app_id, int customer_id);
int ps_capi_worker_delete(void* worker);
/* keys/vals/lens are copied; returns the timestamp. lens may be NULL (nlens = 0). */
int ps_capi_worker_push(void* worker, const uint64_t* keys, size_t nkeys, const float* vals,
                        size_t nvals, const int* lens, size_t nlens, int cmd, int priority);
/* vals (and lens if not NULL) are filled in place when the request completes; they must
 * stay valid until ps_capi_worker_wait(ts) has returned.  nvals must be the exact total. */
int ps_capi_worker_pull(void* worker, const uint64_t* keys, size_t nkeys, float* vals,
                        size_t nvals, int* lens, size_t nlens, int cmd, int priority);
int ps_capi_worker_push_pull(void* worker, const uint64_t* keys, size_t nkeys,
                             const float* vals, size_t nvals, float* outs, int* lens,
                             size_t nlens, int cmd, int priority);
int ps_capi_worker_wait(void* worker, int timestamp);

/* ---- KVServer<float> ---- */
/* Request seen by a callback handle.  Pointers are valid only during the call. */
typedef struct {
  int cmd, push, pull, sender, timestamp, customer_id;
  const uint64_t* keys;
  size_t nkeys;
  const float* vals;
  size_t nvals;
  const int* lens;
  size_t nlens;
} ps_capi_request_t;
/* The handle must call ps_capi_server_respond exactly once per request (now or later). */
typedef void (*ps_capi_handle_t)(void* server, const ps_capi_request_t* req, void* user);

/* handle == NULL installs the built-in accumulate handle (KVServerDefaultHandle). */
void* ps_capi_server_new(int app_id, ps_capi_handle_t handle, void* user);
int ps_capi_server_delete(void* server);
int ps_capi_server_respond(void* server, const ps_capi_request_t* req, const uint64_t* keys,
                           size_t nkeys, const float* vals, size_t nvals, const int* lens,
                           size_t nlens);

/* ---- SimpleApp ---- */
typedef void (*ps_capi_simple_handle_t)(int head, const char* body, size_t body_len,
                                        int sender, void* user);
void* ps_capi_simple_new(int app_id, int customer_id, ps_capi_simple_handle_t on_request,
                         void* user);
int ps_capi_simple_delete(void* app);
int ps_capi_simple_request(void* app, int head, const char* body, size_t body_len, int recver);
int ps_capi_simple_wait(void* app, int timestamp);

/* ---- PBMeta codec (flat form, for tests and tools) ---- */
typedef struct {
  int head, app_id, customer_id, timestamp, request, push, pull, simple_app, priority;
  int control_cmd, barrier_group;
  uint64_t msg_sig;
  int num_data_types;
  int data_types[8];
  int num_nodes;
  struct {
    int role, id, port, is_recovery, customer_id;
    char hostname[64];
  } nodes[8];
  char body[256];
  int body_len;
} ps_capi_meta_t;
/* Returns the encoded size (may exceed cap, in which case nothing is written), or -1. */
long ps_capi_encode_meta(const ps_capi_meta_t* meta, char* out, size_t cap);
int ps_capi_decode_meta(const char* buf, size_t len, ps_capi_meta_t* meta);

#ifdef __cplusplus
}
#endif
#endif /* PS_CAPI_PS_C_API_H_ */
