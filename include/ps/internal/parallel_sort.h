// Multi-threaded sort of an array (reference: include/ps/internal/parallel_sort.h:23-55,
// recursive thread split with inplace_merge).  Here the array is cut into one chunk per
// thread, chunks are sorted concurrently and then merged pairwise, level by level.
#ifndef PS_INTERNAL_PARALLEL_SORT_H_
#define PS_INTERNAL_PARALLEL_SORT_H_
#include <algorithm>
#include <functional>
#include <thread>
#include <vector>

#include "ps/sarray.h"

namespace ps {

template <typename T, class Cmp = std::less<T>>
void ParallelSort(T* data, size_t len, size_t num_threads = 2, Cmp cmp = Cmp()) {
  if (num_threads <= 1 || len < 4096) {
    std::sort(data, data + len, cmp);
    return;
  }
  const size_t parts = std::min(num_threads, len / 1024 + 1);
  std::vector<size_t> cut(parts + 1);
  for (size_t i = 0; i <= parts; ++i) cut[i] = len * i / parts;
  std::vector<std::thread> pool;
  for (size_t i = 0; i < parts; ++i)
    pool.emplace_back([=] { std::sort(data + cut[i], data + cut[i + 1], cmp); });
  for (auto& t : pool) t.join();
  for (size_t width = 1; width < parts; width *= 2) {
    pool.clear();
    for (size_t i = 0; i + width < parts; i += 2 * width) {
      const size_t lo = cut[i], mid = cut[i + width], hi = cut[std::min(i + 2 * width, parts)];
      pool.emplace_back([=] { std::inplace_merge(data + lo, data + mid, data + hi, cmp); });
    }
    for (auto& t : pool) t.join();
  }
}

template <typename T, class Cmp = std::less<T>>
void ParallelSort(SArray<T>* arr, size_t num_threads = 2, Cmp cmp = Cmp()) {
  CHECK_NOTNULL(arr);
  ParallelSort(arr->data(), arr->size(), num_threads, cmp);
}

}  // namespace ps
#endif  // PS_INTERNAL_PARALLEL_SORT_H_
