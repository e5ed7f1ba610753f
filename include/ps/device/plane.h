// The device plane under ps::Start: GPU-resident key-value traffic of a parameter-server job.
//
// A job is started exactly like a CPU job (DMLC_* environment, scheduler, ps::Start).  Every
// worker process then calls Plane::Get()->Start(): it creates its arena of the symmetric heap,
// exchanges the arena handles with the other workers THROUGH THE CONTROL PLANE (simple-app
// messages over the van that ps::Start brought up), maps every peer's arena, optionally binds
// all arenas to one NVSwitch multicast object, and attaches itself to the Postoffice.  From
// then on KVWorker<Val>::Push/Pull/PushPull/ZPush/ZPull/ZPushPull on keys that name a
// registered tensor run as kernels over NVLink instead of messages, and complete the same
// Customer tracker, so timestamps, callbacks and Wait() keep the reference's meaning
// (include/ps/kv_app.h:54-372 of ps-lite).
//
// Correspondence with the reference: this is what its RDMA van does for host memory --
// register memory once, exchange addresses through the rendezvous, then move payloads
// one-sidedly (src/ibverbs_van.h:86-214, :632-957) -- redone for HBM over NVLink, with the
// server handle fused into the transfer.  Barriers are Postoffice::Barrier; no collective
// library is involved.
//
// Key layout of a dense tensor (`tensor_id`, n values): one key per device shard,
//     key_j = KeyRanges()[j].begin() + tensor_id,   value length of key j = its share of n,
// i.e. the tensor is cut into W contiguous pieces and piece j lives on worker j's GPU, which
// also runs the server handle for it.  A request may name any subset of these keys; every
// worker must issue the same sequence of requests per tensor (the kernels rendezvous).
//
// This header has no CUDA dependency: streams are passed as void*.
#ifndef PS_DEVICE_PLANE_H_
#define PS_DEVICE_PLANE_H_
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "ps/base.h"
#include "ps/device/psdev.h"
#include "ps/internal/device_route.h"
#include "ps/range.h"

namespace ps {
namespace device {

// `cmd` of a push that should also leave the new values of the owned blocks in the owner's own
// weight buffer (for a later pull fused into a GEMM, psdev_pull_gemm_bf16).
static const int kCmdPublish = 0x5055424c;  // "PUBL"

struct PlaneOptions {
  size_t heap_bytes = size_t(1) << 30;
  // CUDA device of this process; -1 runs the CPU stand-in (arenas in shared memory, the
  // kernels' work done by host loops), which exists so that the rendezvous, routing and
  // completion logic can be tested on machines without a GPU.
  int device = 0;
  // "ipc": cudaMalloc + CUDA IPC handles (byte strings through the control plane);
  // "vmm": cuMemCreate arenas exported as file descriptors (Unix sockets whose names travel
  //        through the control plane); needed for the multicast alias;
  // "auto": vmm when every rank supports it, else ipc.
  std::string backend = "auto";
  int multicast = -1;           // 1 / 0: bind the arenas to an NVSwitch multicast object or
                                // not; -1: yes when the backend is vmm and all ranks can
  std::string device_lib;       // libpsb200_device.so; empty: PSB200_DEVICE_LIB, else the
                                // directory of this library
  size_t slice_bytes = 16u << 20;  // staging granularity for host-resident values
  uint64_t timeout_ns = 20000000000ull;  // bound of every device-side wait
};

// A registered dense tensor, as seen by this rank.
struct DenseInfo {
  int app_id = 0;
  uint64_t tensor_id = 0;
  int64_t n = 0;            // values (padded to a multiple of 8)
  int64_t n_user = 0;       // values the user asked for
  int64_t share = 0;        // values named by one key (the last key's share may be shorter)
  int channel = 0;
  bool nvls = false;        // reduce/broadcast through the multicast alias
  int num_ctas = 0;
  psdev_table_t table;      // offsets in the arena, owner state pointers, dtypes
  psdev_opt_t opt;          // server handle and its hyper-parameters
  void* grad = nullptr;     // this rank's gradient buffer (arena)
  void* weight = nullptr;   // this rank's pulled-weight buffer (arena)
  int64_t step = 0;         // pushes seen (Adam bias correction)
  bool owns_state = false;  // master/state allocated by the plane
};

// A registered keyed (sparse) table of an app, as seen by this rank.
struct SparseInfo {
  int app_id = 0;
  uint64_t key_space = 0;   // keys are below this; server s owns [s*range, (s+1)*range)
  int64_t max_keys = 0;     // keys per request at most
  int width = 1;            // fp32 elements per value
  psdev_sparse_t table;     // offsets of the request buffers, owner state, handle
  void* keys = nullptr;     // this rank's request buffers in the arena
  void* vals = nullptr;
  void* out = nullptr;
  bool var_len = false;     // values have per-key lengths of at most `width` elements
  void* lens = nullptr;     // i32[max_keys] lengths of the current request (var_len)
  void* offs = nullptr;     // i64[max_keys+1] their running sum
};

class Plane : public DeviceRoute {
 public:
  static Plane* Get();

  // Collective over the worker group; call after ps::Start on every worker (or joint) process.
  void Start(const PlaneOptions& options);
  // Collective: waits for outstanding requests, barrier, unbinds and unmaps, detaches.
  void Stop();
  bool started() const;

  int rank() const;
  int world() const;
  const psdev_world_t& world_struct() const;
  const PlaneOptions& options() const;
  const std::string& backend() const;  // "ipc", "vmm" or "sim"

  // ---- collectives over the control plane (simple-app messages among the workers) ----------
  std::vector<std::string> AllGather(const std::string& mine);
  void Barrier();

  // ---- symmetric heap ------------------------------------------------------------------------
  // Deterministic first-fit: the same sequence of calls gives the same offsets on every rank.
  int64_t Alloc(size_t bytes, size_t align = 256);  // offset, or -1
  void Free(int64_t offset);
  void* Local(int64_t offset) const;                // address in this rank's arena
  size_t heap_in_use() const;

  // ---- dense tensors -------------------------------------------------------------------------
  // Uniform key ranges of the W device shards (equal to Postoffice::GetServerKeyRanges() when
  // the job has as many servers as workers, as with DMLC_ROLE=joint).
  std::vector<Range> KeyRanges() const;
  std::vector<Key> DenseKeys(uint64_t tensor_id) const;
  // Declares a tensor (same order and arguments on every rank): allocates gradient and weight
  // buffers in the arena and the owner's fp32 master weights and handle state.  dtypes are
  // PSDEV_F32 / PSDEV_BF16 (gradients also PSDEV_I8).  `opt` selects the server handle.
  const DenseInfo& DeclareDense(int app_id, uint64_t tensor_id, int64_t n, int grad_dtype,
                                int out_dtype, const psdev_opt_t& opt);
  // Registers a tensor whose buffers the caller has laid out itself (language bindings).
  const DenseInfo& RegisterDense(int app_id, uint64_t tensor_id, int64_t n_user,
                                 const psdev_table_t& table, const psdev_opt_t& opt, int channel,
                                 bool nvls, int num_ctas);
  void UnregisterDense(int app_id, uint64_t tensor_id);
  const DenseInfo* FindDense(int app_id, uint64_t tensor_id) const;
  void SetOptimizer(int app_id, uint64_t tensor_id, const psdev_opt_t& opt);
  // After a failed request (Wait threw because a peer did not arrive): puts the tensor back
  // into service.  Collective: every worker calls it, also those that saw no error.
  void ClearStatus(int app_id, uint64_t tensor_id);
  int NewChannel();

  // ---- keyed (sparse) tables ---------------------------------------------------------------
  // One keyed table per app: sorted unique uint64 keys below `key_space`, `width` fp32 elements
  // per key, owner state in a direct-index store; handle `kind` 0 = sum, 1 = SGD (lr),
  // 2 = FTRL-proximal (alpha, beta, l1, l2).  Same call on every rank.  Afterwards a KVWorker
  // request of that app whose key array lives in DEVICE memory (SArray::FromDevice) is served by
  // the keyed kernels (src/kernels/sparse.cu): values and outputs are device arrays too.
  // `var_len`: the value of key i has lens[i] <= width elements, packed back to back (the
  // reference's `lens`, include/ps/kv_app.h:24-45).  A push (ZPush, ZPushPull) names the lengths
  // in a device array; a pull (ZPull) sizes its output for `width` per key, and receives the
  // packed values and, in its `lens` array (device memory), the lengths that the owners hold.
  // On such a table every worker issues the same kind of request at the same position of its
  // sequence of requests (the pull has two device barriers that the push has not).
  const SparseInfo& DeclareSparse(int app_id, uint64_t key_space, int64_t max_keys, int width,
                                  int kind, float lr, float alpha, float beta, float l1,
                                  float l2, bool var_len = false);
  const SparseInfo* FindSparse(int app_id) const;
  // Synchronous copy between host and device memory in either direction (set-up and tests of
  // programs that are not compiled with the CUDA headers).
  void Memcpy(void* dst, const void* src, size_t bytes);

  // Stream on which requests of the calling thread are ordered: a request with device-resident
  // values runs on it; a staged request starts after what the stream holds and the stream
  // waits for its end.  A null handle names the legacy default stream.  Without a call (or
  // after ClearStream) requests run on the plane's own streams.  Thread local.
  void SetStream(void* stream);
  void ClearStream();
  // Staging granularity for host-resident values of later requests (multiple of 64 bytes).
  void SetSliceBytes(size_t bytes);

  // ---- DeviceRoute ---------------------------------------------------------------------------
  bool Claims(int app_id, const SArray<Key>& keys) override;
  size_t PullBytes(int app_id, const SArray<Key>& keys) override;
  void Submit(const DeviceRequest& req) override;

  // Kernels launched through the plane (for reports).
  uint64_t launches() const;
  // Returns when every request handed to the plane so far has completed (its callback has run
  // and its customer has been credited).  Call before destroying a KVWorker whose requests were
  // not all waited for.
  void Drain();

  struct Impl;

 private:
  void SubmitSparse(const DeviceRequest& req);
  Plane();
  ~Plane();
  std::unique_ptr<Impl> impl_;
};

}  // namespace device
}  // namespace ps
#endif  // PS_DEVICE_PLANE_H_
