/*
 * C ABI of the device plane (include/ps/device/plane.h) and of a byte-typed KVWorker whose
 * requests can name device-resident tensors, for language bindings (ps_lite_b200.kvstore).
 * Conventions as in ps_c_api.h: 0 / non-negative on success, -1 after an error whose text
 * ps_capi_last_error() returns.  The reference has no counterpart (it has no device path).
 */
#ifndef PS_CAPI_PS_NVL_C_API_H_
#define PS_CAPI_PS_NVL_C_API_H_
#include <stddef.h>
#include <stdint.h>

#include "ps/device/psdev.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Plane::Start after ps_capi_start.  device < 0 selects the CPU stand-in.  backend: "auto",
 * "ipc", "vmm".  multicast: -1 auto, 0 off, 1 on.  device_lib: path of libpsb200_device.so or
 * NULL.  slice_bytes, timeout_ns: 0 for the defaults. */
int psnvl_start(uint64_t heap_bytes, int device, const char* backend, int multicast,
                const char* device_lib, uint64_t slice_bytes, uint64_t timeout_ns);
int psnvl_stop(void);
int psnvl_started(void);
int psnvl_rank(void);
int psnvl_world(void);
int psnvl_world_struct(psdev_world_t* out);
/* "ipc", "vmm" or "sim" */
const char* psnvl_backend(void);
int psnvl_barrier(void);
/* All-gather of byte strings among the workers over the control plane.  `out` receives the
 * contributions back to back in rank order, sizes[r] their lengths; returns the total size
 * (which may exceed cap, in which case nothing is written). */
long psnvl_allgather(const void* mine, size_t n, void* out, size_t cap, size_t* sizes);
/* Symmetric-heap allocation: offset into every rank's arena, or -1. */
int64_t psnvl_alloc(uint64_t bytes, uint64_t align);
int psnvl_free(int64_t offset);
uint64_t psnvl_heap_in_use(void);
int psnvl_new_channel(void);
/* Registers a tensor laid out by the caller under (app_id, tensor_id). */
int psnvl_register_dense(int app_id, uint64_t tensor_id, int64_t n_user, const psdev_table_t* t,
                         const psdev_opt_t* opt, int channel, int nvls, int num_ctas);
int psnvl_unregister_dense(int app_id, uint64_t tensor_id);
int psnvl_set_optimizer(int app_id, uint64_t tensor_id, const psdev_opt_t* opt);
/* The W keys of a tensor (one per device shard), written to keys[0..world). */
int psnvl_dense_keys(uint64_t tensor_id, uint64_t* keys);
/* Stream that orders the calling thread's requests (NULL names the legacy default stream). */
int psnvl_set_stream(void* stream);
/* Staging granularity for host-resident values of later requests. */
int psnvl_set_slice_bytes(uint64_t bytes);
/* After a failed request on a tensor: clears the error word of its channel. */
int psnvl_clear_status(int app_id, uint64_t tensor_id);
uint64_t psnvl_launches(void);
/* Returns when every request handed to the plane so far has completed. */
int psnvl_drain(void);

/* ---- KVWorker over raw bytes ---- */
void* ps_capi_bworker_new(int app_id, int customer_id);
int ps_capi_bworker_delete(void* worker);
/* One request; returns its timestamp.  Nothing is copied: keys, vals and outs must stay valid
 * and unchanged until ps_capi_bworker_wait(ts) has returned.  vals == NULL: pull only;
 * outs == NULL with pull != 0 on a device tensor: the values land in the tensor's own weight
 * buffer.  Values may live in host or device memory. */
int ps_capi_bworker_request(void* worker, int push, int pull, const uint64_t* keys, size_t nkeys,
                            const void* vals, size_t vals_bytes, void* outs, size_t outs_bytes,
                            int cmd, int priority);
int ps_capi_bworker_wait(void* worker, int timestamp);

/* ---- keyed (sparse) tables ---- */
/* Plane::DeclareSparse: one keyed table for `app_id` (collective).  kind 0 sum, 1 SGD,
 * 2 FTRL-proximal; var_len != 0: values have per-key lengths of at most `width`. */
int psnvl_declare_sparse(int app_id, uint64_t key_space, int64_t max_keys, int width, int kind,
                         float lr, float alpha, float beta, float l1, float l2, int var_len);
/* One keyed request of a worker created for that app; every array is DEVICE memory and stays
 * valid until the wait returns.  keys: sorted unique uint64.  Push: vals (fp32) and, on a table
 * with lengths, lens (int32 per key).  Pull: outs, and on a table with lengths lens_out receives
 * the stored length of every key.  Returns the timestamp. */
int ps_capi_bworker_keyed_request(void* worker, int push, int pull, const uint64_t* keys_dev,
                                  size_t nkeys, const void* vals_dev, size_t vals_bytes,
                                  void* outs_dev, size_t outs_bytes, const int* lens_dev,
                                  int* lens_out_dev, int cmd);

#ifdef __cplusplus
}
#endif
#endif /* PS_CAPI_PS_NVL_C_API_H_ */
