// SArray<V>: a reference-counted array view used for zero-copy message payloads.
//
// Same public surface as the reference's SArray (include/ps/sarray.h:40-261): cheap copies
// that share storage, reinterpreting construction from an SArray of another POD type,
// adoption of caller memory with or without ownership, segment() slices that keep the
// owner alive, and the vector-like mutators.  The representation differs: the storage is
// an untyped `std::shared_ptr<void>` owner plus a typed pointer, so one owner can back
// views of any element type (message frames are `SArray<char>`), and each array records
// whether its bytes live in host or device memory so that the device data plane can carry
// HBM-resident payloads through the same Message structure.
#ifndef PS_SARRAY_H_
#define PS_SARRAY_H_
#include <algorithm>
#include <cstring>
#include <initializer_list>
#include <iterator>
#include <memory>
#include <sstream>
#include <string>
#include <type_traits>
#include <vector>

#include "ps/internal/logging.h"
#include "ps/internal/shm_pool.h"
#include "ps/range.h"

namespace ps {

// Where the bytes of an SArray live.
enum class MemKind : int { kHost = 0, kDevice = 1 };

template <typename V>
class SArray {
 public:
  SArray() = default;
  ~SArray() = default;

  // `size` elements, each set to `val`.
  explicit SArray(size_t size, V val = 0) { resize(size, val); }

  // Share storage with an array of another element type; sizes are rescaled by the ratio of
  // element sizes (the byte length must divide evenly).
  template <typename W>
  explicit SArray(const SArray<W>& other) { *this = other; }

  template <typename W>
  void operator=(const SArray<W>& other) {
    const size_t bytes = other.size() * sizeof(W);
    CHECK_EQ(bytes % sizeof(V), (size_t)0) << "cannot view " << bytes << " bytes as elements of "
                                           << sizeof(V) << " bytes";
    owner_ = other.owner();
    data_ = reinterpret_cast<V*>(other.data());
    size_ = bytes / sizeof(V);
    capacity_ = other.capacity() * sizeof(W) / sizeof(V);
    kind_ = other.mem_kind();
  }

  // Adopt `data[0..size)`.  With deletable the array frees it with delete[] when the last
  // view goes away; otherwise the caller keeps ownership and must outlive every view.
  SArray(V* data, size_t size, bool deletable = false) {
    if (deletable) {
      reset(data, size, [](V* p) { delete[] p; });
    } else {
      reset(data, size, [](V*) {});
    }
  }

  // Fresh storage for n elements.  Large arrays of plain data come from the shared-memory pool
  // (ps/internal/shm_pool.h), so that a van between processes of one host can pass them by
  // reference; everything else comes from the heap.
  static V* NewStorage(size_t n, bool* pooled) {
    const size_t bytes = (n ? n : 1) * sizeof(V);
    *pooled = std::is_trivially_copyable<V>::value && bytes >= (size_t(64) << 10);
    if (*pooled) return reinterpret_cast<V*>(shm::ArrayAlloc(bytes));
    return new V[n ? n : 1];
  }
  void ResetOwned(V* p, size_t size, bool pooled) {
    if (pooled) {
      reset(p, size, [](V* q) { shm::ArrayFree(reinterpret_cast<char*>(q)); });
    } else {
      reset(p, size, [](V* q) { delete[] q; });
    }
  }

  // Deep copies.
  void CopyFrom(const V* src, size_t size) {
    bool pooled = false;
    V* fresh = NewStorage(size, &pooled);
    if (size) memcpy(fresh, src, size * sizeof(V));
    ResetOwned(fresh, size, pooled);
  }
  void CopyFrom(const SArray<V>& other) {
    if (this == &other) return;
    CHECK(other.mem_kind() == MemKind::kHost) << "CopyFrom needs host memory";
    CopyFrom(other.data(), other.size());
  }
  template <typename ForwardIt>
  void CopyFrom(const ForwardIt& first, const ForwardIt& last) {
    const size_t n = static_cast<size_t>(std::distance(first, last));
    bool pooled = false;
    V* fresh = NewStorage(n, &pooled);
    std::copy(first, last, fresh);
    ResetOwned(fresh, n, pooled);
  }

  explicit SArray(const std::vector<V>& vec) { CopyFrom(vec.data(), vec.size()); }

  // Share a vector held by a shared_ptr (no copy; the vector stays alive with the array).
  explicit SArray(const std::shared_ptr<std::vector<V>>& vec) {
    owner_ = vec;
    data_ = vec->data();
    size_ = capacity_ = vec->size();
  }

  template <typename W>
  SArray(const std::initializer_list<W>& list) { CopyFrom(list.begin(), list.end()); }
  template <typename W>
  void operator=(const std::initializer_list<W>& list) { CopyFrom(list.begin(), list.end()); }

  // Point at `data` and run `del(data)` when the last view is destroyed.
  template <typename Deleter>
  void reset(V* data, size_t size, Deleter del) {
    owner_ = std::shared_ptr<void>(static_cast<void*>(data),
                                   [del](void* p) mutable { del(static_cast<V*>(p)); });
    data_ = data;
    size_ = capacity_ = size;
    kind_ = MemKind::kHost;
  }

  // Device flavour: a view of `size` elements of device memory kept alive by `owner`.
  static SArray<V> FromDevice(V* dev_ptr, size_t size, std::shared_ptr<void> owner = nullptr) {
    SArray<V> a;
    a.owner_ = std::move(owner);
    a.data_ = dev_ptr;
    a.size_ = a.capacity_ = size;
    a.kind_ = MemKind::kDevice;
    return a;
  }

  // Grow or shrink to `size`; new elements take `val`.  Storage is reallocated only when the
  // capacity is exceeded (with a little slack, so repeated push_back stays amortised).
  void resize(size_t size, V val = 0) {
    CHECK(kind_ == MemKind::kHost) << "resize needs host memory";
    const size_t old = size_;
    if (size > capacity_) {
      // an empty array grows to exactly what was asked for; a filled one gets slack
      const size_t cap = old ? size + size / 2 + 4 : size;
      bool pooled = false;
      V* fresh = NewStorage(cap, &pooled);
      if (old) memcpy(fresh, data_, old * sizeof(V));
      ResetOwned(fresh, size, pooled);
      capacity_ = cap;
    } else {
      size_ = size;
    }
    if (size > old) {
      if (val == 0 && std::is_trivially_copyable<V>::value) {
        memset(static_cast<void*>(data_ + old), 0, (size - old) * sizeof(V));
      } else {
        std::fill(data_ + old, data_ + size, val);
      }
    }
  }

  // Ensure capacity for `size` elements without changing size().
  void reserve(size_t size) {
    if (size <= capacity_) return;
    const size_t keep = size_;
    resize(size);
    size_ = keep;
  }

  void clear() {
    owner_.reset();
    data_ = nullptr;
    size_ = capacity_ = 0;
    kind_ = MemKind::kHost;
  }

  bool empty() const { return size_ == 0; }
  size_t size() const { return size_; }
  size_t capacity() const { return capacity_; }
  MemKind mem_kind() const { return kind_; }

  V* begin() { return data_; }
  const V* begin() const { return data_; }
  V* end() { return data_ + size_; }
  const V* end() const { return data_ + size_; }
  V* data() const { return data_; }
  const std::shared_ptr<void>& owner() const { return owner_; }

  V back() const { CHECK(!empty()); return data_[size_ - 1]; }
  V front() const { CHECK(!empty()); return data_[0]; }
  V& operator[](int i) { return data_[i]; }
  const V& operator[](int i) const { return data_[i]; }

  void push_back(const V& val) {
    if (size_ == capacity_) reserve(size_ * 2 + 5);
    data_[size_++] = val;
  }
  void pop_back() { if (size_) --size_; }

  void append(const SArray<V>& tail) {
    if (tail.empty()) return;
    const size_t old = size_;
    resize(old + tail.size());
    memcpy(data_ + old, tail.data(), tail.size() * sizeof(V));
  }

  // Zero-copy slice [begin, end) sharing ownership with this array.
  SArray<V> segment(size_t begin, size_t end) const {
    CHECK_GE(end, begin);
    CHECK_LE(end, size_);
    SArray<V> s;
    s.owner_ = owner_;
    s.data_ = data_ + begin;
    s.size_ = s.capacity_ = end - begin;
    s.kind_ = kind_;
    return s;
  }

 private:
  template <typename W> friend class SArray;
  std::shared_ptr<void> owner_;
  V* data_ = nullptr;
  size_t size_ = 0;
  size_t capacity_ = 0;
  MemKind kind_ = MemKind::kHost;
};

// Positions [first, last) of the elements of sorted `arr` that lie in [lower, upper).
template <typename V>
Range FindRange(const SArray<V>& arr, V lower, V upper) {
  if (upper < lower) return Range(0, 0);
  const V* lo = std::lower_bound(arr.begin(), arr.end(), lower);
  const V* hi = std::lower_bound(lo, arr.end(), upper);
  return Range(static_cast<uint64_t>(lo - arr.begin()), static_cast<uint64_t>(hi - arr.begin()));
}

// "[n]: a b c ... y z" with at most m leading and trailing elements.
template <typename V>
inline std::string DebugStr(const V* data, int n, int m = 5) {
  std::ostringstream os;
  os << "[" << n << "]: ";
  if (n <= 2 * m) {
    for (int i = 0; i < n; ++i) os << data[i] << " ";
  } else {
    for (int i = 0; i < m; ++i) os << data[i] << " ";
    os << "... ";
    for (int i = n - m; i < n; ++i) os << data[i] << " ";
  }
  return os.str();
}

template <typename V>
std::ostream& operator<<(std::ostream& os, const SArray<V>& obj) {
  if (obj.mem_kind() == MemKind::kDevice) {
    os << "[" << obj.size() << "]: <device memory>";
  } else {
    os << DebugStr(obj.data(), static_cast<int>(obj.size()));
  }
  return os;
}

}  // namespace ps
#endif  // PS_SARRAY_H_
