// Shared-memory array pool: see ps/internal/shm_pool.h.
#include "ps/internal/shm_pool.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <utility>

namespace ps {
namespace shm {
namespace {

constexpr size_t kPage = 4096;
constexpr uint32_t kMagic = 0x4d485350u;  // "PSHM"

// First page of every segment; the data starts at kPage.
struct Header {
  uint32_t magic;
  std::atomic<uint32_t> inflight;  // views handed to (or held by) other mappers
};

struct Seg {
  char* base = nullptr;
  size_t size = 0;  // whole segment, header page included
  int fd = -1;
  bool imported = false;
  bool in_use = false;   // own: backs a live array
  int refs = 0;          // imported (or own, echoed back): live local views
  uint64_t stamp = 0;    // last time it became idle
  std::pair<uint64_t, uint64_t> inode{0, 0};
};

struct Registry {
  std::mutex mu;
  std::map<uintptr_t, Seg> segs;                               // by base address
  std::map<std::pair<uint64_t, uint64_t>, uintptr_t> by_inode;  // (dev, ino) -> base
  size_t pooled = 0, cached = 0, live = 0;
  uint64_t clock = 0;
  Stats st{};
};

Registry& R() {
  static Registry* r = new Registry();  // never destroyed: arrays may be freed at exit
  return *r;
}

size_t EnvSize(const char* name, size_t dflt) {
  const char* e = getenv(name);
  if (!e || !*e) return dflt;
  return static_cast<size_t>(strtoull(e, nullptr, 10));
}

size_t PoolCap() {
  static const size_t v = EnvSize("PS_SHM_POOL_MB", 512) << 20;
  return v;
}
size_t ImportCap() {
  static const size_t v = EnvSize("PS_SHM_IMPORT_CACHE_MB", 512) << 20;
  return v;
}

Header* Head(char* base) { return reinterpret_cast<Header*>(base); }

void Unmap(Registry& r, std::map<uintptr_t, Seg>::iterator it) {
  Seg& s = it->second;
  auto bi = r.by_inode.find(s.inode);
  if (bi != r.by_inode.end() && bi->second == it->first) r.by_inode.erase(bi);
  munmap(s.base, s.size);
  if (s.fd >= 0) ::close(s.fd);
  r.segs.erase(it);
}

// Drops idle segments of one kind (pooled own ones or cached imports), oldest first, until
// `need` more bytes fit under `cap`.  `keep` (a base address, or 0) is never dropped.
void Evict(Registry& r, bool imported, size_t need, size_t cap, uintptr_t keep = 0) {
  size_t& total = imported ? r.cached : r.pooled;
  while (total + need > cap) {
    auto victim = r.segs.end();
    for (auto it = r.segs.begin(); it != r.segs.end(); ++it) {
      const Seg& s = it->second;
      if (s.imported != imported || s.in_use || s.refs > 0 || it->first == keep) continue;
      if (victim == r.segs.end() || s.stamp < victim->second.stamp) victim = it;
    }
    if (victim == r.segs.end()) return;
    total -= victim->second.size;
    Unmap(r, victim);
  }
}

// The segment that contains p, or end().
std::map<uintptr_t, Seg>::iterator Find(Registry& r, const void* p) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  auto it = r.segs.upper_bound(a);
  if (it == r.segs.begin()) return r.segs.end();
  --it;
  if (a >= it->first + it->second.size) return r.segs.end();
  return it;
}

// An own segment has just lost its array, or a mapping its last local view.
void BecameIdle(Registry& r, std::map<uintptr_t, Seg>::iterator it) {
  Seg& s = it->second;
  s.stamp = ++r.clock;
  if (s.imported) {
    if (s.size > ImportCap()) {
      Unmap(r, it);
      return;
    }
    Evict(r, true, s.size, ImportCap(), it->first);
    r.cached += s.size;
    return;
  }
  // Own segment: recycle it only when no other process holds a view of its contents.
  if (Head(s.base)->inflight.load(std::memory_order_acquire) != 0 || s.size > PoolCap()) {
    Unmap(r, it);
    return;
  }
  Evict(r, false, s.size, PoolCap(), it->first);
  r.pooled += s.size;
}

}  // namespace

bool Enabled() {
  static const bool on = [] {
    const char* e = getenv("PS_SHM");
    if (e && *e) return atoi(e) != 0;
    const char* l = getenv("DMLC_LOCAL");
    return l && *l && atoi(l) != 0;
  }();
  return on;
}

size_t MinBytes() {
  static const size_t v = EnvSize("PS_SHM_MIN_BYTES", 256 << 10);
  return v < kPage ? kPage : v;
}

char* ArrayAlloc(size_t bytes) {
  if (!Enabled() || bytes < MinBytes()) return new char[bytes ? bytes : 1];
  const size_t need = kPage + ((bytes + kPage - 1) / kPage) * kPage;
  Registry& r = R();
  {
    std::lock_guard<std::mutex> lk(r.mu);
    // smallest idle own segment that fits without wasting more than a quarter
    auto best = r.segs.end();
    for (auto it = r.segs.begin(); it != r.segs.end(); ++it) {
      const Seg& s = it->second;
      if (s.imported || s.in_use || s.refs > 0) continue;
      if (s.size < need || s.size > need + need / 4) continue;
      if (Head(s.base)->inflight.load(std::memory_order_acquire) != 0) continue;
      if (best == r.segs.end() || s.size < best->second.size) best = it;
    }
    if (best != r.segs.end()) {
      best->second.in_use = true;
      r.pooled -= best->second.size;
      r.live += best->second.size;
      ++r.st.segments_reused;
      return best->second.base + kPage;
    }
  }
  int fd = static_cast<int>(syscall(SYS_memfd_create, "psb200_array", 1u /* MFD_CLOEXEC */));
  if (fd < 0) return new char[bytes];
  if (ftruncate(fd, static_cast<off_t>(need)) != 0) {
    ::close(fd);
    return new char[bytes];
  }
  void* m = mmap(nullptr, need, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (m == MAP_FAILED) {
    ::close(fd);
    return new char[bytes];
  }
  struct stat sb {};
  fstat(fd, &sb);
  Seg s;
  s.base = static_cast<char*>(m);
  s.size = need;
  s.fd = fd;
  s.in_use = true;
  s.inode = {static_cast<uint64_t>(sb.st_dev), static_cast<uint64_t>(sb.st_ino)};
  Head(s.base)->magic = kMagic;
  Head(s.base)->inflight.store(0, std::memory_order_release);
  std::lock_guard<std::mutex> lk(r.mu);
  r.segs[reinterpret_cast<uintptr_t>(s.base)] = s;
  r.by_inode[s.inode] = reinterpret_cast<uintptr_t>(s.base);
  r.live += need;
  ++r.st.segments_created;
  return s.base + kPage;
}

void ArrayFree(char* p) {
  if (!p) return;
  Registry& r = R();
  {
    std::lock_guard<std::mutex> lk(r.mu);
    auto it = r.segs.find(reinterpret_cast<uintptr_t>(p) - kPage);
    if (it != r.segs.end() && !it->second.imported && it->second.in_use) {
      it->second.in_use = false;
      r.live -= it->second.size;
      if (it->second.refs == 0) BecameIdle(r, it);
      return;
    }
  }
  delete[] p;
}

bool Share(const void* p, size_t len, int* fd, uint64_t* offset, uint64_t* seg_size) {
  if (!Enabled() || len < MinBytes()) return false;
  Registry& r = R();
  std::lock_guard<std::mutex> lk(r.mu);
  auto it = Find(r, p);
  if (it == r.segs.end()) return false;
  const Seg& s = it->second;
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  if (a < it->first + kPage || a + len > it->first + s.size) return false;
  Head(s.base)->inflight.fetch_add(1, std::memory_order_acq_rel);
  *fd = s.fd;
  *offset = a - it->first;
  *seg_size = s.size;
  return true;
}

void Unshare(const void* p) {
  Registry& r = R();
  std::lock_guard<std::mutex> lk(r.mu);
  auto it = Find(r, p);
  if (it != r.segs.end()) Head(it->second.base)->inflight.fetch_sub(1, std::memory_order_acq_rel);
}

char* Import(int fd, uint64_t seg_size) {
  struct stat sb {};
  if (fd < 0) return nullptr;
  if (fstat(fd, &sb) != 0 || static_cast<uint64_t>(sb.st_size) < seg_size || seg_size <= kPage) {
    ::close(fd);
    return nullptr;
  }
  const std::pair<uint64_t, uint64_t> inode{static_cast<uint64_t>(sb.st_dev),
                                            static_cast<uint64_t>(sb.st_ino)};
  Registry& r = R();
  std::lock_guard<std::mutex> lk(r.mu);
  ++r.st.imports;
  auto known = r.by_inode.find(inode);
  if (known != r.by_inode.end()) {
    auto it = r.segs.find(known->second);
    if (it != r.segs.end() && it->second.size == seg_size) {
      Seg& s = it->second;
      if (s.imported && s.refs == 0) r.cached -= s.size;                 // leaves the idle cache
      if (!s.imported && !s.in_use && s.refs == 0) r.pooled -= s.size;   // own, echoed back late
      ++s.refs;
      ++r.st.import_hits;
      ::close(fd);
      return s.base;
    }
  }
  void* m = mmap(nullptr, seg_size, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (m == MAP_FAILED || Head(static_cast<char*>(m))->magic != kMagic) {
    if (m != MAP_FAILED) munmap(m, seg_size);
    ::close(fd);
    return nullptr;
  }
  Seg s;
  s.base = static_cast<char*>(m);
  s.size = seg_size;
  s.fd = fd;
  s.imported = true;
  s.refs = 1;
  s.inode = inode;
  r.segs[reinterpret_cast<uintptr_t>(s.base)] = s;
  r.by_inode[inode] = reinterpret_cast<uintptr_t>(s.base);
  return s.base;
}

void Release(char* base) {
  if (!base) return;
  Registry& r = R();
  std::lock_guard<std::mutex> lk(r.mu);
  auto it = r.segs.find(reinterpret_cast<uintptr_t>(base));
  if (it == r.segs.end()) return;
  Seg& s = it->second;
  Head(s.base)->inflight.fetch_sub(1, std::memory_order_acq_rel);
  if (s.refs > 0) --s.refs;
  if (s.refs == 0 && !s.in_use) BecameIdle(r, it);
}

Stats GetStats() {
  Registry& r = R();
  std::lock_guard<std::mutex> lk(r.mu);
  Stats s = r.st;
  s.bytes_live = r.live;
  s.bytes_pooled = r.pooled;
  return s;
}

void Trim() {
  Registry& r = R();
  std::lock_guard<std::mutex> lk(r.mu);
  Evict(r, false, PoolCap(), PoolCap());
  Evict(r, true, ImportCap(), ImportCap());
}

}  // namespace shm
}  // namespace ps
