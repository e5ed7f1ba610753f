// Shared-memory backing for large host arrays.
//
// With Unix-domain sockets between processes of one host (DMLC_LOCAL=1) a large payload does
// not have to travel through the socket at all: when the array lives in a memfd segment, the
// van passes the segment's file descriptor (SCM_RIGHTS) with an (offset, length) pair, and the
// receiver maps the same pages.  This header is the allocator and the registry behind that:
//
//   * ArrayAlloc / ArrayFree: what SArray uses for its own allocations.  Requests of at least
//     MinBytes() come from memfd segments (recycled through a free list, so a steady-state
//     training loop neither page-faults nor zero-fills), smaller ones from the heap.
//   * Share: does [p, p + len) lie inside a registered segment (own or imported)?  The van asks
//     this for every data frame it is about to send.
//   * Import / Release: map a segment received from a peer.  Mappings are cached by inode, so a
//     peer that keeps sending from the same recycled segment is mapped once.
//
// An imported array aliases the sender's pages (MAP_SHARED), exactly like a message that
// stays inside one process with the loop van: treat received arrays as read-only.  The
// reference has no counterpart; its closest relative is the registered memory pool of the RDMA
// van (src/ibverbs_van.h:86-214), which serves the same purpose for a NIC.
#ifndef PS_INTERNAL_SHM_POOL_H_
#define PS_INTERNAL_SHM_POOL_H_
#include <cstddef>
#include <cstdint>

namespace ps {
namespace shm {

// PS_SHM=0 switches shared-memory arrays off, PS_SHM=1 on; the default is on when DMLC_LOCAL is
// set to a non-zero value.  Read once.
bool Enabled();
// Arrays of at least this many bytes are placed in shared memory (PS_SHM_MIN_BYTES, 256 KiB).
size_t MinBytes();

// Storage for `bytes` bytes (never null; at least 1 byte).  Contents are unspecified.
char* ArrayAlloc(size_t bytes);
void ArrayFree(char* p);

// Sender side.  True when [p, p + len) lies inside one registered segment (own or imported);
// then *fd is a descriptor of it (owned by the registry: do not close), *offset the position
// of p inside the segment and *seg_size the segment's length, and the segment's count of views
// in flight has been raised by one on behalf of the receiver.  Unshare takes that back when the
// message could not be sent.
bool Share(const void* p, size_t len, int* fd, uint64_t* offset, uint64_t* seg_size);
void Unshare(const void* p);

// Receiver side.  Maps the segment behind `fd` (length seg_size) and returns its base address,
// or nullptr on failure.  Takes ownership of `fd` in every case.  Each successful Import needs
// one Release, which also lowers the segment's count of views in flight.  A segment is recycled
// by its owner only while that count is zero, so a view that a receiver keeps stays intact.
char* Import(int fd, uint64_t seg_size);
void Release(char* base);

// Counters for tests and statistics.
struct Stats {
  uint64_t segments_created, segments_reused, bytes_live, bytes_pooled, imports, import_hits;
};
Stats GetStats();
// Drops pooled segments and cached imports that are not in use.
void Trim();

}  // namespace shm
}  // namespace ps
#endif  // PS_INTERNAL_SHM_POOL_H_
