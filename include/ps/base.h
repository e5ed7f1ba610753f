// Fundamental types and node-group identifiers (same values as the reference,
// include/ps/base.h:10-30, because they appear on the wire and in user programs).
#ifndef PS_BASE_H_
#define PS_BASE_H_
#include <cstdint>
#include <limits>

#include "ps/internal/utils.h"

namespace ps {

#ifdef USE_KEY32
using Key = uint32_t;
#else
using Key = uint64_t;
#endif
// largest key value
static const Key kMaxKey = std::numeric_limits<Key>::max();

// Node ids below 8 name groups: bit 0 = scheduler, bit 1 = all servers, bit 2 = all
// workers; any OR of them is a valid group (e.g. 6 = servers + workers, 7 = everyone).
static const int kScheduler = 1;
static const int kServerGroup = 2;
static const int kWorkerGroup = 4;

}  // namespace ps
#endif  // PS_BASE_H_
