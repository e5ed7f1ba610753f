// Ordered match of two sorted unique key lists: for every key present in both,
// dst_val op= src_val, with `k` values per key (reference:
// include/ps/internal/parallel_kv_match.h:29-120, a recursive thread-splitting merge-join).
// Here the source keys are cut into one contiguous chunk per thread; each thread narrows the
// destination range with two binary searches and merges its chunk sequentially.
#ifndef PS_INTERNAL_PARALLEL_KV_MATCH_H_
#define PS_INTERNAL_PARALLEL_KV_MATCH_H_
#include <algorithm>
#include <atomic>
#include <thread>
#include <vector>

#include "ps/internal/assign_op.h"
#include "ps/sarray.h"

namespace ps {

// Returns the number of matched keys.  dst_val must hold dst_key.size()*k elements (it is
// resized and zero-filled if empty).
template <typename K, typename V>
size_t ParallelOrderedMatch(const SArray<K>& src_key, const SArray<V>& src_val,
                            const SArray<K>& dst_key, SArray<V>* dst_val, int k = 1,
                            AssignOp op = ASSIGN, int num_threads = 2) {
  CHECK_GT(k, 0);
  CHECK_EQ(src_key.size() * k, src_val.size());
  CHECK_NOTNULL(dst_val);
  if (dst_val->empty()) dst_val->resize(dst_key.size() * k);
  CHECK_EQ(dst_val->size(), dst_key.size() * k);
  if (src_key.empty() || dst_key.empty()) return 0;
  const size_t parts =
      std::max<size_t>(1, std::min<size_t>(num_threads, src_key.size() / 1024 + 1));
  std::atomic<size_t> matched{0};
  auto work = [&](size_t lo, size_t hi) {
    const K* sk = src_key.data();
    const K* db = std::lower_bound(dst_key.begin(), dst_key.end(), sk[lo]);
    const K* de = std::upper_bound(db, dst_key.end(), sk[hi - 1]);
    size_t n = 0, i = lo;
    const K* d = db;
    while (i < hi && d < de) {
      if (sk[i] < *d) {
        ++i;
      } else if (*d < sk[i]) {
        ++d;
      } else {
        const size_t j = static_cast<size_t>(d - dst_key.begin());
        for (int c = 0; c < k; ++c)
          AssignFunc(src_val.data()[i * k + c], op, dst_val->data() + j * k + c);
        ++n; ++i; ++d;
      }
    }
    matched += n;
  };
  std::vector<std::thread> pool;
  for (size_t p = 0; p < parts; ++p) {
    const size_t lo = src_key.size() * p / parts, hi = src_key.size() * (p + 1) / parts;
    if (lo < hi) pool.emplace_back(work, lo, hi);
  }
  for (auto& t : pool) t.join();
  return matched.load();
}

}  // namespace ps
#endif  // PS_INTERNAL_PARALLEL_KV_MATCH_H_
