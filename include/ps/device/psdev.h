/*
 * psdev: the device data plane of the parameter server (C ABI).
 *
 * Every process drives one GPU and plays both roles of a parameter server:
 * it is a worker (it owns a gradient buffer and a pulled-weight buffer) and a
 * server shard (it owns fp32 master weights and optimizer state for the key
 * blocks whose index is congruent to its rank).  All worker-side buffers live
 * in a "symmetric heap": an arena of identical layout on every rank, mapped
 * into every process, so a kernel on one GPU reaches the same tensor on a peer
 * at `peer_base[p] + offset`.
 *
 * The reference library moves these bytes as ZMQ/RDMA messages between
 * processes (src/zmq_van.h:131-227, src/ibverbs_van.h:632-957) and applies the
 * server handle on a CPU thread (include/ps/kv_app.h:440-463).  Here the
 * transfer, the reduction over workers and the server-side update are a single
 * kernel that loads and stores peer HBM over NVLink.
 *
 * All functions return 0 on success or a negative psdev error / positive
 * cudaError_t value.  None of them synchronises the stream unless stated.
 */
#ifndef PS_DEVICE_PSDEV_H_
#define PS_DEVICE_PSDEV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PSDEV_MAX_RANKS 8
#define PSDEV_NUM_CHANNELS 64
/* bytes reserved at the start of every heap for flags, epochs and status */
#define PSDEV_CTRL_BYTES 65536
#define PSDEV_IPC_HANDLE_BYTES 64

/* element types of gradients (wire) and of pulled weights */
/* PSDEV_I8 (gradients only): int8 values with one fp32 scale per 256 values, as written by
 * psdev_filter_int8_pack; the push kernel applies the scales while it reduces */
enum { PSDEV_F32 = 0, PSDEV_BF16 = 1, PSDEV_I8 = 2 };

/* built-in server handles (the "request handle" of a KVServer, run on device) */
enum {
  PSDEV_OPT_SUM = 0,      /* store += scale * sum_w g          (KVServerDefaultHandle) */
  PSDEV_OPT_SGD = 1,      /* w -= lr * (g + wd*w)                                       */
  PSDEV_OPT_MOMENTUM = 2, /* m = mu*m + g + wd*w ; w -= lr*m                            */
  PSDEV_OPT_ADAM = 3,     /* Adam / AdamW with host-computed bias corrections           */
  PSDEV_OPT_ASSIGN = 4,   /* w = scale * sum_w g   (initialisation push)                */
  /* kinds from here on belong to handles that applications compile and register themselves
   * (include/ps/device/user_handle.cuh) */
  PSDEV_OPT_USER = 100
};

/* which halves of the round trip a launch performs */
enum { PSDEV_OP_PUSH = 1, PSDEV_OP_PULL = 2, PSDEV_OP_PUSHPULL = 3,
       /* PUSH | PUBLISH: push, and write the owned blocks' new values into the owner's own
        * weight buffer only, for a later pull fused with a GEMM */
       PSDEV_OP_PUBLISH = 4 };

/* error codes (negative); also stored in the per-channel device status word */
enum {
  PSDEV_OK = 0,
  PSDEV_ERR_ARG = -1,
  PSDEV_ERR_TIMEOUT_ENTRY = -2, /* a peer never announced its gradients   */
  PSDEV_ERR_TIMEOUT_EXIT = -3,  /* a peer never finished reading/writing  */
  PSDEV_ERR_UNSUPPORTED = -4,
  PSDEV_ERR_NOMEM = -5,
  PSDEV_ERR_TIMEOUT_PIPE = -6,  /* an mbarrier wait inside a GEMM pipeline ran out */
  /* -7: PSDEV_ERR_TOO_LARGE of the no-alloc GEMM (src/kernels/pull_gemm_noalloc.h) */
  PSDEV_ERR_BOUNDS = -8         /* a buffer does not fit into the heap (host check), or, in the
                                   checks build, a kernel computed an index outside it */
};

/* The ranks of one job as seen from this process. */
typedef struct {
  int32_t rank;
  int32_t world;
  void* peer_base[PSDEV_MAX_RANKS]; /* heap base of every rank in this address space */
  void* mc_base;                    /* NVLS multicast alias of the heap, or NULL       */
  uint64_t heap_bytes;              /* size of every rank's arena; 0 = unknown (no extent
                                       checks)                                          */
} psdev_world_t;

/* Hyper-parameters of the server handle; unused fields are ignored. */
typedef struct {
  int32_t kind;      /* PSDEV_OPT_* */
  float scale;       /* applied to the summed gradient (1/W for averaging)        */
  float lr;
  float momentum;    /* MOMENTUM: mu                                               */
  float weight_decay;
  float beta1, beta2, eps; /* ADAM                                                 */
  float bias1, bias2;      /* ADAM: 1-beta1^t and sqrt(1-beta2^t), from the host   */
  int32_t decoupled_wd;    /* ADAM: 1 = AdamW                                      */
  float user[4];           /* free for user-defined handles                         */
} psdev_opt_t;

/*
 * One dense table: `n` elements, cut into blocks of `blk` elements; block j is
 * owned by server rank j % world (blk = ceil(n/world) gives the reference's
 * contiguous ranges, include/ps/../src/postoffice.cc:169-180; a small blk gives
 * a block-cyclic layout that balances any sub-range).  Element i of block j is
 * stored by its owner at state index (j / world) * blk + (i - j*blk).
 */
typedef struct {
  uint64_t grad_off;   /* heap offset of the worker's gradient buffer           */
  uint64_t weight_off; /* heap offset of the worker's pulled-weight buffer      */
  int64_t n;
  int64_t blk;         /* multiple of 8                                          */
  float* master;       /* owner state, local memory: fp32 weights                */
  float* state1;       /* momentum / Adam m, or NULL                             */
  float* state2;       /* Adam v, or NULL                                        */
  int32_t grad_dtype;  /* PSDEV_F32 | PSDEV_BF16                                 */
  int32_t out_dtype;   /* dtype of the pulled-weight buffer                      */
  uint64_t gscale_off; /* PSDEV_I8 gradients: heap offset of the fp32 scales     */
  /* Optional low-latency region (0 / 0: none): psdev_ll_bytes(world, ll_cap) zero-filled bytes
   * at heap offset ll_off.  A fused push+pull of at most ll_cap values then runs without flag
   * rendezvous: values travel next to a sequence number (include/ps/device/push_pull_ll.cuh). */
  uint64_t ll_off;
  int64_t ll_cap;
} psdev_table_t;

/* ---- symmetric heap ------------------------------------------------------ */
int psdev_heap_create(size_t bytes, void** base, unsigned char* ipc_handle /*64 B*/);
int psdev_heap_open(const unsigned char* ipc_handle, void** peer_base);
int psdev_heap_close(void* peer_base);
int psdev_heap_destroy(void* base);
/* Enable direct access from the current device to `peer_device` (same process). */
int psdev_enable_peer(int peer_device);

/* Arena from the virtual-memory-management API (src/device/vmm_heap.cu): physical memory
 * exported as a POSIX file descriptor and mapped by every rank.  psdev_vmm_supported: 1 when
 * the current device offers it.  psdev_vmm_create: arena of at least `bytes` on the current
 * device; *mapped_bytes is the rounded size that peers pass to psdev_vmm_import, *fd belongs
 * to the caller (send it to the peers over a Unix socket, then close it); the control region
 * is cleared.  psdev_vmm_import maps a peer's arena from its descriptor (which stays the
 * caller's).  psdev_vmm_release unmaps either kind. */
int psdev_vmm_supported(void);
int psdev_vmm_create(size_t bytes, void** base, int* fd, size_t* mapped_bytes);
int psdev_vmm_create_aligned(size_t bytes, size_t align, void** base, int* fd,
                             size_t* mapped_bytes);
int psdev_vmm_import(int fd, size_t mapped_bytes, void** base);
int psdev_vmm_release(void* base);

/* NVSwitch multicast object over the arenas of all ranks (NVLS): loads through the alias can
 * reduce over, and stores replicate into, every rank's arena (multimem.* instructions).  The
 * ranks go through these steps together, with a host barrier between them:
 *   rank 0: psdev_mc_create (exports a descriptor), others: psdev_mc_import;
 *   all: psdev_mc_add_device; barrier; all: psdev_mc_bind(arena); barrier;
 *   all: psdev_mc_map -> alias for psdev_world_t.mc_base.
 * Arenas must come from psdev_vmm_create_aligned with align = psdev_mc_granularity and have
 * the object's size.  psdev_mc_release (after a barrier that follows the last kernel using
 * the alias) unmaps, unbinds and drops the object. */
int psdev_mc_supported(void);
int psdev_mc_granularity(int num_devices, size_t bytes, size_t* gran);
int psdev_mc_create(size_t bytes, int num_devices, int* fd, void** mc);
int psdev_mc_import(int fd, size_t bytes, void** mc);
int psdev_mc_add_device(void* mc);
int psdev_mc_bind(void* mc, void* arena_base);
int psdev_mc_map(void* mc, void** mc_base);
int psdev_mc_release(void* mc);

/* first-fit sub-allocator over [PSDEV_CTRL_BYTES, bytes): pure host bookkeeping,
 * deterministic, so every rank that issues the same calls gets the same offsets */
void* psdev_suballoc_new(size_t heap_bytes);
void psdev_suballoc_delete(void* sa);
int64_t psdev_suballoc_alloc(void* sa, size_t bytes, size_t align); /* <0: no room */
int psdev_suballoc_free(void* sa, int64_t offset);
size_t psdev_suballoc_in_use(void* sa);

/* ---- channel state ------------------------------------------------------- */
/* Reads (synchronously) the status word and epoch of a channel of the local heap. */
int psdev_channel_status(void* local_base, int channel, int32_t* status, uint64_t* epoch);
/* Same, with the copies issued on `stream` (then synchronised) instead of the default stream. */
int psdev_channel_status_on(void* local_base, int channel, void* stream, int32_t* status,
                            uint64_t* epoch);
/* Clears status (not the epoch) of a channel after an error was handled. */
int psdev_channel_clear(void* local_base, int channel);

/* ---- dense push / pull --------------------------------------------------- */
/*
 * Runs `op` on elements [begin, end) of table `t` (both multiples of 8).
 *   PUSH     : each owner sums the workers' gradients of its blocks over NVLink,
 *              applies the handle to master/state.
 *   PULL     : each owner casts its master blocks and stores them into every
 *              worker's weight buffer.
 *   PUSHPULL : both in one pass; the summed gradient never touches memory.
 * `sync` is a bit set.  Bit 1 (value 2): reduce and broadcast through the NVSwitch multicast
 * alias `w->mc_base` (multimem.ld_reduce / multimem.st) instead of per-peer loads and stores;
 * ignored when mc_base is NULL.  Bit 0 (value 1) set: ranks rendezvous through epoch flags in
 * the heap on `channel`
 * (every rank must issue the same sequence of calls per channel).  Bit 0 clear:
 * no flags are touched (used when the caller has already ordered the ranks, and
 * to run all ranks' roles back to back on one GPU).
 * `timeout_ns` bounds every flag wait; on expiry the kernel records an error in
 * the channel status and returns without touching the data.
 */
int psdev_dense_op(const psdev_world_t* w, const psdev_table_t* t, int op,
                   int64_t begin, int64_t end, const psdev_opt_t* opt,
                   int channel, int num_ctas, uint64_t timeout_ns, int sync,
                   void* stream);

/* Several slices of one table in one launch and one rendezvous.  `segs`: device memory with
 * `nseg` (<= 1024) triples (begin, end, priority) of int64; a small kernel orders them by
 * priority (highest first, ties in submission order) and numbers the tiles across slices, so
 * the CTAs work on the most urgent slice first.  `sched`: device scratch of
 * psdev_sched_bytes(nseg) bytes. */
int psdev_dense_op_multi(const psdev_world_t* w, const psdev_table_t* t, int op,
                         const int64_t* segs, int nseg, void* sched, const psdev_opt_t* opt,
                         int channel, int num_ctas, uint64_t timeout_ns, int sync, void* stream);
size_t psdev_sched_bytes(int nseg);

/* Bytes of the low-latency region of a table for requests of up to ll_cap values. */
size_t psdev_ll_bytes(int world, int64_t ll_cap);

/* Number of kernels this library has launched in this process (for reporting). */
uint64_t psdev_launch_count(void);
void psdev_count_launch(void);
/* State arrays (0, 1 or 2) that the handle of `kind` needs, or -1 for an unknown kind. */
int psdev_handle_states(int kind);

/* Flag-only rendezvous of all ranks on a channel (device barrier). */
/* 1 when a dense request of `bytes` gradient bytes among `world` ranks is faster on the NVSwitch
 * multicast path than on plain peer accesses (measured limits; PSB200_NVLS_MAX_BYTES overrides). */
int psdev_multicast_pays(int world, uint64_t bytes);
int psdev_device_barrier(const psdev_world_t* w, int channel, uint64_t timeout_ns,
                         void* stream);

/* ---- sparse (keyed) push / pull --------------------------------------------------------- */
/*
 * One keyed table.  Server s owns keys [s*range, (s+1)*range); a value has `width` fp32
 * elements, or, when lens_off != 0, lens[i] <= width elements packed back to back in the request
 * (dynamic-length values).  Request buffers live in every rank's arena at the same offsets; the
 * owner's state arrays (`slots` x `width` elements) are local memory.
 */
typedef struct {
  uint64_t range;      /* keys per shard                                                  */
  uint64_t keys_off;   /* u64[max_n]   request keys, sorted and unique                    */
  uint64_t grads_off;  /* f32[max_vals] pushed values                                     */
  uint64_t out_off;    /* f32[max_vals] pulled values                                     */
  uint64_t pos_off;    /* i64[world+2] cut points of the key list, [world+1] = n          */
  uint64_t acc_off;    /* f32[slots*width] the server's gradient accumulator              */
  float* w;            /* values                                                          */
  float* z;            /* FTRL z, or NULL                                                 */
  float* n;            /* FTRL n, or NULL                                                 */
  int32_t kind;        /* 0 sum, 1 SGD, 2 FTRL-proximal                                   */
  float lr, alpha, beta, l1, l2;
  uint64_t hkeys_off;  /* hash store: u64[capacity] key table (filled with 0xff)          */
  uint64_t capacity;   /* hash store: slots per server, power of two; 0 = direct index    */
  int32_t* overflow;   /* hash store: device int set to 1 when a table is full            */
  int32_t width;       /* elements per value (maximum, with lengths)                      */
  int32_t channel;     /* rendezvous channel of the table                                 */
  int64_t max_n;       /* keys per request at most                                        */
  int64_t max_vals;    /* values per request at most                                      */
  int64_t slots;       /* slots of the store: keys of the range, or capacity              */
  uint64_t lens_off;   /* i32[max_n] per-key lengths of the request, or 0                 */
  uint64_t offs_off;   /* i64[max_n+1] value offsets (computed by the scatter call)       */
  int32_t* klen;       /* owner state: stored length per slot (with lengths), or NULL     */
  uint64_t timeout_ns; /* bound of the rendezvous waits; 0 = 20 s                         */
  int32_t state_stride; /* floats between consecutive values in w, z and n: 0 or 1 = three
                           arrays; 4 = one array of {w, z, n, -} per value (w, z, n point at
                           its first three floats), so that an update touches one 16-byte
                           group instead of three sectors                                  */
} psdev_sparse_t;

/* Cut points of a sorted key list at the W+1 shard boundaries (device pointers; pos[world+1]
 * receives n). */
int psdev_key_shard_lookup(const uint64_t* keys, int64_t n, uint64_t range, int world,
                           int64_t* pos, void* stream);
/* offs[i] = lens[0] + ... + lens[i-1] for i = 0..n (device pointers). */
int psdev_lens_to_offsets(const int32_t* lens, int64_t n, int64_t* offs, void* stream);
/* Worker role: cut points (and value offsets), then every element of the n staged pairs is
 * added into its owner's accumulator over NVLink. */
int psdev_sparse_scatter(const psdev_world_t* w, const psdev_sparse_t* t, int64_t n, int num_ctas,
                         void* stream);
/* Server role: applies the handle to every key that any worker pushed.  sync != 0: first waits
 * until every rank has entered this kernel (i.e. finished its scatter). */
int psdev_sparse_apply(const psdev_world_t* w, const psdev_sparse_t* t, int num_ctas, int sync,
                       void* stream);
/* Server role: stores the value of every requested key into the requester's output buffer.
 * sync != 0: ends by waiting until every rank has done so. */
int psdev_sparse_respond(const psdev_world_t* w, const psdev_sparse_t* t, int num_ctas, int sync,
                         void* stream);

/* Server role, tables with lengths: stores the length of the value of every key that a worker
 * staged (keys in its arena, cut points computed with psdev_key_shard_lookup) into that worker's
 * array of lengths; 0 for a key that was never pushed.  Used by a pull that does not know the
 * lengths: barrier, this call, barrier, psdev_lens_to_offsets, then apply and respond. */
int psdev_sparse_lens(const psdev_world_t* w, const psdev_sparse_t* t, int num_ctas,
                      void* stream);

/* ---- bf16 GEMM on tcgen05, alone or fused with the pull of its weights ----------------- */
/* c[M,N] = x[M,K] * w[N,K]^T; all row-major bf16, 16-byte aligned, N and K multiples of 8. */
int psdev_gemm_bf16(const void* x, const void* w, void* c, int64_t M, int64_t N, int64_t K,
                    int num_ctas, uint64_t timeout_ns, void* stream);
/* Same product where w = elements [w_elem_off, w_elem_off + N*K) of table `t`'s bf16 weight
 * buffer: copy CTAs fetch the blocks owned by other ranks over NVLink panel by panel while
 * the tensor cores work on the panels that have landed.  Must follow, on `stream`, a
 * PUSH|PUBLISH of that range by every rank.  Uses a small per-device scratch block that the
 * library allocates on first use.  num_copy_ctas > 0 sets that many CTAs aside for the copy;
 * num_copy_ctas <= 0 selects ring mode: one thread of every GEMM CTA moves its share of the
 * remote blocks with bulk copies through a ring in shared memory (a cooperative launch, so
 * that all CTAs are resident; if that is not granted, 16 copy CTAs are used instead).
 * All GEMM launches on one device share the scratch block (panel counters, error word): order
 * them on one stream or with events; two of them running at the same time would mix counters. */
int psdev_pull_gemm_bf16(const psdev_world_t* w, const psdev_table_t* t, int64_t w_elem_off,
                         const void* x, void* c, int64_t M, int64_t N, int64_t K,
                         int num_copy_ctas, int num_ctas, uint64_t timeout_ns, void* stream);
/* Ring mode of psdev_pull_gemm_bf16 for later launches: mode 1 (default) moves W with bulk
 * (TMA) loads and stores issued by two threads per CTA, mode 0 with 16-byte asynchronous
 * copies by two warps per CTA; chunk_bytes is 4096, 8192, 16384 or 0 for the default (8192). */
int psdev_pull_ring_config(int mode, int chunk_bytes);
/* Host-side view of the pull plan of psdev_pull_gemm_bf16 in ring mode, for tests: returns the
 * number of chunk slots for W = elements [w_elem_off, w_elem_off + nk) and, for 0 <= i < that,
 * the owner and element range of slot i (empty when *begin >= *end). */
int64_t psdev_pull_plan_chunk(int64_t w_elem_off, int64_t nk, int blk, int world, int rank,
                              int64_t i, int* owner, int64_t* begin, int64_t* end);
/* Reads and clears the error word of the GEMM kernels on the current device (synchronous). */
int psdev_gemm_status(int32_t* status);

/* Copy kernel of the link-bandwidth benchmark (benchmarks/link_bandwidth.py): `bytes` from
 * `src` to `dst` with 16-byte loads and stores; either side may be a peer's arena. */
int psdev_link_copy(void* dst, const void* src, size_t bytes, int num_ctas, void* stream);

/* CUDA-runtime shims for the host runtime's device plane (src/device/runtime.cu). */
int psdev_rt_device_count(int* n);
int psdev_rt_set_device(int device);
int psdev_rt_get_device(int* device);
int psdev_rt_malloc(void** p, size_t bytes); /* zero-filled */
int psdev_rt_free(void* p);
int psdev_rt_memset_async(void* p, int value, size_t bytes, void* stream);
int psdev_rt_stream_create(void** stream, int priority);
int psdev_rt_stream_destroy(void* stream);
int psdev_rt_stream_sync(void* stream);
int psdev_rt_event_create(void** event);
int psdev_rt_event_destroy(void* event);
int psdev_rt_event_record(void* event, void* stream);
int psdev_rt_event_sync(void* event);
int psdev_rt_stream_wait_event(void* stream, void* event);
int psdev_rt_memcpy_async(void* dst, const void* src, size_t bytes, void* stream);
int psdev_rt_is_device_pointer(const void* p);
int psdev_rt_is_pinned_host(const void* p);
int psdev_rt_host_alloc(void** p, size_t bytes);
int psdev_rt_host_free(void* p);

#ifdef __cplusplus
}
#endif
#endif /* PS_DEVICE_PSDEV_H_ */
