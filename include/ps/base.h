// Fundamental types and node-group identifiers.  The numeric values are those of the
// reference (include/ps/base.h:10-30) because they travel on the wire and appear in user
// programs: scheduler = 1, server group = 2, worker group = 4, and any sum of them.
#ifndef PS_BASE_H_
#define PS_BASE_H_
#include <cstdint>
#include <limits>

#include "ps/internal/utils.h"

namespace ps {

// Key type: 64-bit unless the library is built with USE_KEY32.
#ifdef USE_KEY32
typedef uint32_t Key;
#else
typedef uint64_t Key;
#endif

// Largest key; server ranges are cut from [0, kMaxKey).
constexpr Key kMaxKey = std::numeric_limits<Key>::max();

// Group identifiers are bit flags below 8; concrete node ids start at 8.
enum : int {
  kScheduler = 1 << 0,
  kServerGroup = 1 << 1,
  kWorkerGroup = 1 << 2,
};

// True for an id that names a group (or a union of groups) rather than a node.
constexpr bool IsGroupId(int id) { return id > 0 && id < 8; }
// The union of all nodes.
constexpr int kAllNodes = kScheduler | kServerGroup | kWorkerGroup;

}  // namespace ps
#endif  // PS_BASE_H_
