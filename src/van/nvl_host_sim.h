// CPU stand-in for the kernels of the device plane.
//
// The device plane (src/van/nvl_van.cc) normally drives CUDA kernels.  On a machine without a
// GPU the same plane can run with arenas in shared host memory; the functions here then do a
// kernel's work with host loops and the same flag protocol in the arenas' control regions, so
// several processes rendezvous exactly as several GPUs would.  They exist for tests of the
// host-side logic (handle exchange, routing, completion); they are not a performance path.
#ifndef PS_VAN_NVL_HOST_SIM_H_
#define PS_VAN_NVL_HOST_SIM_H_
#include <cstdint>

#include "ps/device/psdev.h"

namespace ps {
namespace device {
namespace sim {

// Same contract as psdev_dense_op (include/ps/device/psdev.h); runs synchronously.
int DenseOp(const psdev_world_t* w, const psdev_table_t* t, int op, int64_t begin, int64_t end,
            const psdev_opt_t* opt, int channel, uint64_t timeout_ns, int sync);
// Keyed tables: same contracts as psdev_key_shard_lookup, psdev_lens_to_offsets,
// psdev_sparse_scatter / _apply / _respond / _lens and psdev_device_barrier (direct-index store
// only; the hash store needs a GPU).
int KeyShardLookup(const uint64_t* keys, int64_t n, uint64_t range, int world, int64_t* pos);
int LensToOffsets(const int32_t* lens, int64_t n, int64_t* offs);
int SparseScatter(const psdev_world_t* w, const psdev_sparse_t* t, int64_t n);
int SparseApply(const psdev_world_t* w, const psdev_sparse_t* t, int sync);
int SparseRespond(const psdev_world_t* w, const psdev_sparse_t* t, int sync);
int SparseLens(const psdev_world_t* w, const psdev_sparse_t* t);
int DeviceBarrier(const psdev_world_t* w, int channel, uint64_t timeout_ns);
// Same contract as psdev_channel_status / psdev_channel_clear.
int ChannelStatus(void* local_base, int channel, int32_t* status, uint64_t* epoch);
int ChannelClear(void* local_base, int channel);

}  // namespace sim
}  // namespace device
}  // namespace ps
#endif  // PS_VAN_NVL_HOST_SIM_H_
