// Half-open interval [begin, end) of keys or positions (reference: include/ps/range.h:12-23).
#ifndef PS_RANGE_H_
#define PS_RANGE_H_
#include <cstdint>

namespace ps {

class Range {
 public:
  Range() = default;
  Range(uint64_t begin, uint64_t end) : lo_(begin), hi_(end) {}
  uint64_t begin() const { return lo_; }
  uint64_t end() const { return hi_; }
  uint64_t size() const { return hi_ - lo_; }
  bool contains(uint64_t x) const { return x >= lo_ && x < hi_; }

 private:
  uint64_t lo_ = 0;
  uint64_t hi_ = 0;
};

}  // namespace ps
#endif  // PS_RANGE_H_
