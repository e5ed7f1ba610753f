// nvl_van: the device plane of the host runtime (declaration and overview: ps/device/plane.h).
//
// What happens here, in the order of a job's life:
//   * Start: bind the CUDA library at run time, create this rank's arena, exchange arena
//     handles with the other workers over the control plane, map the peers, optionally build
//     the multicast alias, attach to the Postoffice as its DeviceRoute.
//   * Submit: a KVWorker request on a registered tensor becomes copies and kernel launches on
//     CUDA streams (a slice pipeline when values live in host memory), followed by an event.
//   * Completing: a thread waits for those events in submission order, reads the channel's
//     status word, runs the request's callback and credits the Customer tracker -- the role
//     the Customer's receive thread plays for responses that arrive as messages
//     (reference: src/customer.cc:49-64, include/ps/kv_app.h:616-640).
//   * Stop: drain, barrier, unbind, unmap.
#include <dlfcn.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <random>
#include <sstream>
#include <thread>

#include "ps/device/ctrl_layout.h"
#include "ps/device/plane.h"
#include "ps/internal/postoffice.h"
#include "ps/simple_app.h"
#include "van/nvl_host_sim.h"

namespace ps {
namespace device {
namespace {

constexpr int kPlaneApp = 0x6e766c;  // app id of the plane's own simple-app endpoint ("nvl")
constexpr int kHeadGather = 1;

// ---- run-time binding of the CUDA library -----------------------------------------------------
struct Rt {
  int (*set_device)(int) = nullptr;
  int (*malloc_)(void**, size_t) = nullptr;
  int (*free_)(void*) = nullptr;
  int (*stream_create)(void**, int) = nullptr;
  int (*stream_destroy)(void*) = nullptr;
  int (*stream_sync)(void*) = nullptr;
  int (*event_create)(void**) = nullptr;
  int (*event_destroy)(void*) = nullptr;
  int (*event_record)(void*, void*) = nullptr;
  int (*event_sync)(void*) = nullptr;
  int (*stream_wait_event)(void*, void*) = nullptr;
  int (*memcpy_async)(void*, const void*, size_t, void*) = nullptr;
  int (*memset_async)(void*, int, size_t, void*) = nullptr;
  size_t (*ll_bytes)(int, int64_t) = nullptr;
  int (*handle_states)(int) = nullptr;
  int (*sparse_scatter)(const psdev_world_t*, const psdev_sparse_t*, int64_t, int, void*) = nullptr;
  int (*sparse_apply)(const psdev_world_t*, const psdev_sparse_t*, int, int, void*) = nullptr;
  int (*sparse_respond)(const psdev_world_t*, const psdev_sparse_t*, int, int, void*) = nullptr;
  int (*sparse_lens)(const psdev_world_t*, const psdev_sparse_t*, int, void*) = nullptr;
  int (*key_shard_lookup)(const uint64_t*, int64_t, uint64_t, int, int64_t*, void*) = nullptr;
  int (*lens_to_offsets)(const int32_t*, int64_t, int64_t*, void*) = nullptr;
  int (*device_barrier)(const psdev_world_t*, int, uint64_t, void*) = nullptr;
  int (*multicast_pays)(int, uint64_t) = nullptr;
  int (*is_device_pointer)(const void*) = nullptr;
  int (*heap_create)(size_t, void**, unsigned char*) = nullptr;
  int (*heap_open)(const unsigned char*, void**) = nullptr;
  int (*heap_close)(void*) = nullptr;
  int (*heap_destroy)(void*) = nullptr;
  int (*vmm_supported)() = nullptr;
  int (*vmm_create_aligned)(size_t, size_t, void**, int*, size_t*) = nullptr;
  int (*vmm_import)(int, size_t, void**) = nullptr;
  int (*vmm_release)(void*) = nullptr;
  int (*mc_supported)() = nullptr;
  int (*mc_granularity)(int, size_t, size_t*) = nullptr;
  int (*mc_create)(size_t, int, int*, void**) = nullptr;
  int (*mc_import)(int, size_t, void**) = nullptr;
  int (*mc_add_device)(void*) = nullptr;
  int (*mc_bind)(void*, void*) = nullptr;
  int (*mc_map)(void*, void**) = nullptr;
  int (*mc_release)(void*) = nullptr;
  int (*channel_status_on)(void*, int, void*, int32_t*, uint64_t*) = nullptr;
  int (*channel_clear)(void*, int) = nullptr;
  int (*dense_op)(const psdev_world_t*, const psdev_table_t*, int, int64_t, int64_t,
                  const psdev_opt_t*, int, int, uint64_t, int, void*) = nullptr;
  uint64_t (*launch_count)() = nullptr;
};

template <typename Fn>
void Bind(void* lib, const char* name, Fn* out) {
  void* p = dlsym(lib, name);
  CHECK(p) << "the device library lacks " << name;
  *out = reinterpret_cast<Fn>(p);
}

std::string DirOfThisLibrary() {
  Dl_info info;
  if (dladdr(reinterpret_cast<void*>(&DirOfThisLibrary), &info) && info.dli_fname) {
    std::string path(info.dli_fname);
    const size_t cut = path.rfind('/');
    if (cut != std::string::npos) return path.substr(0, cut);
  }
  return ".";
}

void* LoadRt(const std::string& configured, Rt* rt) {
  std::string path = configured;
  if (path.empty()) {
    const char* env = getenv("PSB200_DEVICE_LIB");
    path = env ? env : DirOfThisLibrary() + "/libpsb200_device.so";
  }
  void* lib = dlopen(path.c_str(), RTLD_NOW | RTLD_GLOBAL);
  CHECK(lib) << "cannot load the device library " << path << ": " << dlerror();
  Bind(lib, "psdev_rt_set_device", &rt->set_device);
  Bind(lib, "psdev_rt_malloc", &rt->malloc_);
  Bind(lib, "psdev_rt_free", &rt->free_);
  Bind(lib, "psdev_rt_stream_create", &rt->stream_create);
  Bind(lib, "psdev_rt_stream_destroy", &rt->stream_destroy);
  Bind(lib, "psdev_rt_stream_sync", &rt->stream_sync);
  Bind(lib, "psdev_rt_event_create", &rt->event_create);
  Bind(lib, "psdev_rt_event_destroy", &rt->event_destroy);
  Bind(lib, "psdev_rt_event_record", &rt->event_record);
  Bind(lib, "psdev_rt_event_sync", &rt->event_sync);
  Bind(lib, "psdev_rt_stream_wait_event", &rt->stream_wait_event);
  Bind(lib, "psdev_rt_memcpy_async", &rt->memcpy_async);
  Bind(lib, "psdev_rt_memset_async", &rt->memset_async);
  Bind(lib, "psdev_ll_bytes", &rt->ll_bytes);
  Bind(lib, "psdev_handle_states", &rt->handle_states);
  Bind(lib, "psdev_sparse_scatter", &rt->sparse_scatter);
  Bind(lib, "psdev_sparse_apply", &rt->sparse_apply);
  Bind(lib, "psdev_sparse_respond", &rt->sparse_respond);
  Bind(lib, "psdev_sparse_lens", &rt->sparse_lens);
  Bind(lib, "psdev_key_shard_lookup", &rt->key_shard_lookup);
  Bind(lib, "psdev_lens_to_offsets", &rt->lens_to_offsets);
  Bind(lib, "psdev_device_barrier", &rt->device_barrier);
  Bind(lib, "psdev_multicast_pays", &rt->multicast_pays);
  Bind(lib, "psdev_rt_is_device_pointer", &rt->is_device_pointer);
  Bind(lib, "psdev_heap_create", &rt->heap_create);
  Bind(lib, "psdev_heap_open", &rt->heap_open);
  Bind(lib, "psdev_heap_close", &rt->heap_close);
  Bind(lib, "psdev_heap_destroy", &rt->heap_destroy);
  Bind(lib, "psdev_vmm_supported", &rt->vmm_supported);
  Bind(lib, "psdev_vmm_create_aligned", &rt->vmm_create_aligned);
  Bind(lib, "psdev_vmm_import", &rt->vmm_import);
  Bind(lib, "psdev_vmm_release", &rt->vmm_release);
  Bind(lib, "psdev_mc_supported", &rt->mc_supported);
  Bind(lib, "psdev_mc_granularity", &rt->mc_granularity);
  Bind(lib, "psdev_mc_create", &rt->mc_create);
  Bind(lib, "psdev_mc_import", &rt->mc_import);
  Bind(lib, "psdev_mc_add_device", &rt->mc_add_device);
  Bind(lib, "psdev_mc_bind", &rt->mc_bind);
  Bind(lib, "psdev_mc_map", &rt->mc_map);
  Bind(lib, "psdev_mc_release", &rt->mc_release);
  Bind(lib, "psdev_channel_status_on", &rt->channel_status_on);
  Bind(lib, "psdev_channel_clear", &rt->channel_clear);
  Bind(lib, "psdev_dense_op", &rt->dense_op);
  Bind(lib, "psdev_launch_count", &rt->launch_count);
  return lib;
}

// ---- CPU stand-in of the same table: arenas are shared memory, work is done at once ---------
std::atomic<uint64_t> g_sim_launches{0};
int SimOk1(void*) { return 0; }
int SimSetDevice(int) { return 0; }
int SimMalloc(void** p, size_t bytes) {
  *p = calloc(1, bytes ? bytes : 1);
  return *p ? 0 : PSDEV_ERR_NOMEM;
}
int SimFree(void* p) {
  free(p);
  return 0;
}
int SimStreamCreate(void** s, int) {
  *s = nullptr;
  return 0;
}
int SimEventCreate(void** e) {
  *e = nullptr;
  return 0;
}
int SimEventRecord(void*, void*) { return 0; }
int SimMemcpy(void* dst, const void* src, size_t bytes, void*) {
  memmove(dst, src, bytes);
  return 0;
}
int SimChannelStatusOn(void* base, int channel, void*, int32_t* st, uint64_t* ep) {
  return sim::ChannelStatus(base, channel, st, ep);
}
int SimDenseOp(const psdev_world_t* w, const psdev_table_t* t, int op, int64_t b, int64_t e,
               const psdev_opt_t* o, int channel, int, uint64_t tmo, int sync, void*) {
  g_sim_launches.fetch_add(1, std::memory_order_relaxed);
  return sim::DenseOp(w, t, op, b, e, o, channel, tmo, sync);
}
int SimMemset(void* dst, int value, size_t bytes, void*) {
  memset(dst, value, bytes);
  return 0;
}
int SimSparseScatter(const psdev_world_t* w, const psdev_sparse_t* t, int64_t n, int, void*) {
  g_sim_launches.fetch_add(1, std::memory_order_relaxed);
  return sim::SparseScatter(w, t, n);
}
int SimSparseApply(const psdev_world_t* w, const psdev_sparse_t* t, int, int sync, void*) {
  g_sim_launches.fetch_add(1, std::memory_order_relaxed);
  return sim::SparseApply(w, t, sync);
}
int SimSparseRespond(const psdev_world_t* w, const psdev_sparse_t* t, int, int sync, void*) {
  g_sim_launches.fetch_add(1, std::memory_order_relaxed);
  return sim::SparseRespond(w, t, sync);
}
int SimSparseLens(const psdev_world_t* w, const psdev_sparse_t* t, int, void*) {
  g_sim_launches.fetch_add(1, std::memory_order_relaxed);
  return sim::SparseLens(w, t);
}
int SimKeyShardLookup(const uint64_t* keys, int64_t n, uint64_t range, int world, int64_t* pos,
                      void*) {
  return sim::KeyShardLookup(keys, n, range, world, pos);
}
int SimLensToOffsets(const int32_t* lens, int64_t n, int64_t* offs, void*) {
  return sim::LensToOffsets(lens, n, offs);
}
int SimDeviceBarrier(const psdev_world_t* w, int channel, uint64_t tmo, void*) {
  return sim::DeviceBarrier(w, channel, tmo);
}
uint64_t SimLaunchCount() { return g_sim_launches.load(std::memory_order_relaxed); }

void FillSimRt(Rt* rt) {
  rt->set_device = SimSetDevice;
  rt->malloc_ = SimMalloc;
  rt->free_ = SimFree;
  rt->stream_create = SimStreamCreate;
  rt->stream_destroy = SimOk1;
  rt->stream_sync = SimOk1;
  rt->event_create = SimEventCreate;
  rt->event_destroy = SimOk1;
  rt->event_record = SimEventRecord;
  rt->event_sync = SimOk1;
  rt->stream_wait_event = SimEventRecord;
  rt->memcpy_async = SimMemcpy;
  rt->memset_async = SimMemset;
  rt->sparse_scatter = SimSparseScatter;
  rt->sparse_apply = SimSparseApply;
  rt->sparse_respond = SimSparseRespond;
  rt->sparse_lens = SimSparseLens;
  rt->key_shard_lookup = SimKeyShardLookup;
  rt->lens_to_offsets = SimLensToOffsets;
  rt->device_barrier = SimDeviceBarrier;
  rt->channel_status_on = SimChannelStatusOn;
  rt->channel_clear = sim::ChannelClear;
  rt->dense_op = SimDenseOp;
  rt->launch_count = SimLaunchCount;
}

// ---- first-fit sub-allocator of the arena (host bookkeeping only) ---------------------------
class SubAlloc {
 public:
  explicit SubAlloc(size_t bytes) : bytes_(bytes) {
    free_[PSDEV_CTRL_BYTES] = bytes - PSDEV_CTRL_BYTES;
  }
  int64_t Alloc(size_t bytes, size_t align) {
    if (align < 16) align = 16;
    bytes = (bytes + 255) & ~size_t(255);
    if (bytes == 0) bytes = 256;
    for (auto it = free_.begin(); it != free_.end(); ++it) {
      const size_t lo = it->first, len = it->second;
      const size_t at = (lo + align - 1) / align * align;
      if (at + bytes > lo + len) continue;
      free_.erase(it);
      if (at > lo) free_[lo] = at - lo;
      if (at + bytes < lo + len) free_[at + bytes] = lo + len - (at + bytes);
      used_[at] = bytes;
      in_use_ += bytes;
      return static_cast<int64_t>(at);
    }
    return -1;
  }
  bool Free(int64_t off) {
    auto it = used_.find(static_cast<size_t>(off));
    if (it == used_.end()) return false;
    size_t lo = it->first, len = it->second;
    in_use_ -= len;
    used_.erase(it);
    auto next = free_.lower_bound(lo);
    if (next != free_.end() && lo + len == next->first) {
      len += next->second;
      next = free_.erase(next);
    }
    if (next != free_.begin()) {
      auto prev = std::prev(next);
      if (prev->first + prev->second == lo) {
        lo = prev->first;
        len += prev->second;
        free_.erase(prev);
      }
    }
    free_[lo] = len;
    return true;
  }
  size_t in_use() const { return in_use_; }

 private:
  size_t bytes_;
  std::map<size_t, size_t> free_, used_;
  size_t in_use_ = 0;
};

// ---- descriptors between the processes of one host -------------------------------------------
// Each rank binds a datagram socket in the abstract namespace; the names go round through
// `gather` (the control plane); every rank then sends its descriptors to every peer as
// SCM_RIGHTS data.  Returns, for every rank, the descriptors it sent (own entry: duplicates).
std::vector<std::vector<int>> ExchangeFds(int rank, int world, const std::vector<int>& mine,
                                          const std::function<std::vector<std::string>(
                                              const std::string&)>& gather) {
  std::vector<std::vector<int>> got(world);
  for (int fd : mine) got[rank].push_back(dup(fd));
  if (world == 1) return got;
  std::random_device rd;
  std::ostringstream name;
  name << "psb200-nvl-" << getpid() << "-" << rd() << "-" << rank;
  const std::string mine_name = name.str();
  const int srv = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  CHECK_GE(srv, 0) << "socket: " << strerror(errno);
  auto addr_of = [](const std::string& n, sockaddr_un* a) {
    memset(a, 0, sizeof(*a));
    a->sun_family = AF_UNIX;
    CHECK_LT(n.size() + 1, sizeof(a->sun_path));
    memcpy(a->sun_path + 1, n.data(), n.size());  // leading NUL: abstract namespace
    return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n.size());
  };
  sockaddr_un me;
  const socklen_t me_len = addr_of(mine_name, &me);
  CHECK_EQ(bind(srv, reinterpret_cast<sockaddr*>(&me), me_len), 0) << strerror(errno);
  timeval tv{60, 0};
  setsockopt(srv, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  const std::vector<std::string> names = gather(mine_name);  // everyone is bound after this
  CHECK_EQ(names.size(), static_cast<size_t>(world));
  const int out = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  CHECK_GE(out, 0);
  const size_t nfd = mine.size();
  CHECK(nfd >= 1 && nfd <= 8);
  for (int p = 0; p < world; ++p) {
    if (p == rank) continue;
    sockaddr_un to;
    const socklen_t to_len = addr_of(names[p], &to);
    int32_t hdr[2] = {rank, static_cast<int32_t>(nfd)};
    iovec iov{hdr, sizeof(hdr)};
    alignas(cmsghdr) char ctl[CMSG_SPACE(sizeof(int) * 8)];
    memset(ctl, 0, sizeof(ctl));
    msghdr msg{};
    msg.msg_name = &to;
    msg.msg_namelen = to_len;
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = ctl;
    msg.msg_controllen = CMSG_SPACE(sizeof(int) * nfd);
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int) * nfd);
    memcpy(CMSG_DATA(c), mine.data(), sizeof(int) * nfd);
    CHECK_GE(sendmsg(out, &msg, 0), 0) << "sendmsg to rank " << p << ": " << strerror(errno);
  }
  close(out);
  for (int k = 0; k < world - 1; ++k) {
    int32_t hdr[2] = {-1, 0};
    iovec iov{hdr, sizeof(hdr)};
    alignas(cmsghdr) char ctl[CMSG_SPACE(sizeof(int) * 8)];
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = ctl;
    msg.msg_controllen = sizeof(ctl);
    const ssize_t n = recvmsg(srv, &msg, MSG_CMSG_CLOEXEC);
    CHECK_EQ(n, static_cast<ssize_t>(sizeof(hdr))) << "descriptor exchange: " << strerror(errno);
    const int src = hdr[0];
    CHECK(src >= 0 && src < world && src != rank && got[src].empty())
        << "unexpected descriptor message from rank " << src;
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    CHECK(c && c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS);
    const size_t cnt = (c->cmsg_len - CMSG_LEN(0)) / sizeof(int);
    CHECK_EQ(cnt, static_cast<size_t>(hdr[1]));
    got[src].resize(cnt);
    memcpy(got[src].data(), CMSG_DATA(c), cnt * sizeof(int));
  }
  close(srv);
  return got;
}

// ---- all-gather among the workers over simple-app messages ---------------------------------
class Exchange : public SimpleApp {
 public:
  Exchange() : SimpleApp(kPlaneApp, kPlaneApp) {
    set_request_handle([this](const SimpleData& req, SimpleApp* app) {
      if (req.head == kHeadGather && req.body.size() >= 4) {
        uint32_t round;
        memcpy(&round, req.body.data(), 4);
        const int from = Postoffice::IDtoRank(req.sender);
        {
          std::lock_guard<std::mutex> lk(mu_);
          rounds_[round][from] = req.body.substr(4);
        }
        cv_.notify_all();
      }
      app->Response(req);
    });
  }

  std::vector<std::string> AllGather(const std::string& mine, int world) {
    uint32_t round;
    {
      std::lock_guard<std::mutex> lk(mu_);
      round = next_round_++;
    }
    std::string body(4, '\0');
    memcpy(&body[0], &round, 4);
    body += mine;
    Wait(Request(kHeadGather, body, kWorkerGroup));
    std::unique_lock<std::mutex> lk(mu_);
    const bool ok = cv_.wait_for(lk, std::chrono::seconds(120), [&] {
      return rounds_[round].size() == static_cast<size_t>(world);
    });
    CHECK(ok) << "all-gather round " << round << " got " << rounds_[round].size() << " of "
              << world << " contributions";
    std::vector<std::string> out(world);
    for (auto& kv : rounds_[round]) {
      CHECK(kv.first >= 0 && kv.first < world);
      out[kv.first] = std::move(kv.second);
    }
    rounds_.erase(round);
    return out;
  }

 private:
  std::mutex mu_;
  std::condition_variable cv_;
  uint32_t next_round_ = 0;
  std::map<uint32_t, std::map<int, std::string>> rounds_;
};

size_t DtypeSize(int dt) { return dt == PSDEV_F32 ? 4 : (dt == PSDEV_BF16 ? 2 : 1); }

// Ends of the slices of [begin, end): sizes small, 2*small, 4*small ... below `step`, then
// slices of `step`, then the same ramp mirrored.  All cuts but the last are multiples of 8
// away from `begin`.
std::vector<int64_t> SliceEnds(int64_t begin, int64_t end, int64_t small, int64_t step) {
  // the plan is made for the length rounded up to a multiple of 8, then the last cut is
  // pulled back to `end`
  const int64_t len = (end - begin + 7) & ~int64_t(7);
  std::vector<int64_t> ramp;
  int64_t used = 0;
  for (int64_t sz = small; sz < step && used + 2 * sz + step <= len; sz *= 2) {
    ramp.push_back(sz);
    used += 2 * sz;
  }
  std::vector<int64_t> cuts;
  int64_t at = 0;
  for (int64_t sz : ramp) cuts.push_back(at += sz);
  const int64_t mid_end = len - used / 2;
  while (at + step < mid_end) cuts.push_back(at += step);
  if (mid_end > at) cuts.push_back(at = mid_end);
  for (auto it = ramp.rbegin(); it != ramp.rend(); ++it) cuts.push_back(at += *it);
  for (int64_t& c : cuts) c = std::min(begin + c, end);
  if (cuts.empty() || cuts.back() != end) cuts.push_back(end);
  return cuts;
}

thread_local void* tls_stream = nullptr;
thread_local bool tls_has_stream = false;

}  // namespace

// ================================================================================================
struct Plane::Impl {
  PlaneOptions opts;
  bool copy_out_lag = true;  // PSB200_COPY_OUT_LAG=0: copy out as soon as the kernel is done
  bool started = false;
  bool sim = false;
  std::string backend_name;
  Rt rt;
  void* lib = nullptr;
  int rank = 0, world = 1;
  psdev_world_t ws{};
  size_t arena_bytes = 0;
  void* mc = nullptr;
  std::unique_ptr<Exchange> exchange;
  std::unique_ptr<SubAlloc> sub;
  mutable std::mutex mu;  // tables, allocator, channel counter
  std::map<std::pair<int, uint64_t>, std::unique_ptr<DenseInfo>> dense;
  std::map<int, std::unique_ptr<SparseInfo>> sparse;
  int next_channel = 0;

  void* s_h2d = nullptr;
  void* s_compute = nullptr;
  void* s_d2h = nullptr;
  void* s_status = nullptr;
  std::vector<void*> event_pool;
  std::mutex ev_mu;
  // requests on one tensor are serialised against each other: the last event of the previous
  // one (keyed by DenseInfo*)
  std::map<const void*, void*> last_done;

  struct Pending {
    void* event = nullptr;
    std::vector<void*> events_to_recycle;
    int channel = 0;
    int timestamp = 0;
    int responses = 1;
    Customer* customer = nullptr;
    std::function<void()> on_done;
    int* lens_out = nullptr;
    std::vector<int> lens;
    const void* tensor = nullptr;  // DenseInfo* or SparseInfo*: key of the ordering entry
  };
  std::mutex q_mu;
  std::condition_variable q_cv, idle_cv;
  std::deque<Pending> queue;
  bool stop = false;
  int in_flight = 0;
  std::thread completer;

  void* NewEvent() {
    {
      std::lock_guard<std::mutex> lk(ev_mu);
      if (!event_pool.empty()) {
        void* e = event_pool.back();
        event_pool.pop_back();
        return e;
      }
    }
    void* e = nullptr;
    CHECK_EQ(rt.event_create(&e), 0);
    return e;
  }
  void RecycleEvent(void* e) {
    if (sim) return;
    std::lock_guard<std::mutex> lk(ev_mu);
    event_pool.push_back(e);
  }

  void Completing() {
    rt.set_device(opts.device);
    for (;;) {
      Pending p;
      {
        std::unique_lock<std::mutex> lk(q_mu);
        q_cv.wait(lk, [&] { return stop || !queue.empty(); });
        if (queue.empty()) return;
        p = std::move(queue.front());
        queue.pop_front();
      }
      int rc = rt.event_sync(p.event);
      int32_t status = 0;
      if (rc == 0)
        rc = rt.channel_status_on(ws.peer_base[rank], p.channel, s_status, &status, nullptr);
      if (p.lens_out)
        for (size_t i = 0; i < p.lens.size(); ++i) p.lens_out[i] = p.lens[i];
      if (p.on_done) p.on_done();  // before the request counts as complete, like the reference
      if (p.customer) {
        if (rc != 0 || status != 0) {
          std::ostringstream why;
          why << "device plane: ";
          if (rc != 0) why << "CUDA error " << rc;
          else why << "status " << status << " on channel " << p.channel
                   << (status == PSDEV_ERR_TIMEOUT_ENTRY || status == PSDEV_ERR_TIMEOUT_EXIT
                           ? " (a peer did not arrive within the deadline)"
                           : "");
          p.customer->FailRequest(p.timestamp, why.str());
        } else {
          p.customer->AddResponse(p.timestamp, p.responses);
        }
      }
      {
        // the event stops being the ordering point of its tensor before it is reused
        std::lock_guard<std::mutex> lk(mu);
        auto it = last_done.find(p.tensor);
        if (it != last_done.end() && it->second == p.event) last_done.erase(it);
      }
      RecycleEvent(p.event);
      for (void* e : p.events_to_recycle) RecycleEvent(e);
      {
        std::lock_guard<std::mutex> lk(q_mu);
        --in_flight;
      }
      idle_cv.notify_all();
    }
  }

  void Drain() {
    std::unique_lock<std::mutex> lk(q_mu);
    idle_cv.wait(lk, [&] { return in_flight == 0; });
  }
};

Plane::Plane() : impl_(new Impl) {}
Plane::~Plane() {}

Plane* Plane::Get() {
  static Plane* p = new Plane;  // outlives static destruction, like the Postoffice
  return p;
}

bool Plane::started() const { return impl_->started; }
int Plane::rank() const { return impl_->rank; }
int Plane::world() const { return impl_->world; }
const psdev_world_t& Plane::world_struct() const { return impl_->ws; }
const PlaneOptions& Plane::options() const { return impl_->opts; }
const std::string& Plane::backend() const { return impl_->backend_name; }
uint64_t Plane::launches() const { return impl_->rt.launch_count ? impl_->rt.launch_count() : 0; }
void Plane::Drain() {
  if (impl_->started) impl_->Drain();
}
void Plane::SetStream(void* stream) {
  tls_stream = stream;
  tls_has_stream = true;  // a null handle is a stream too: the legacy default stream
}
void Plane::ClearStream() {
  tls_stream = nullptr;
  tls_has_stream = false;
}
void Plane::SetSliceBytes(size_t bytes) {
  CHECK_GE(bytes, size_t(64));
  std::lock_guard<std::mutex> lk(impl_->mu);
  impl_->opts.slice_bytes = bytes & ~size_t(63);
}

std::vector<std::string> Plane::AllGather(const std::string& mine) {
  Impl& m = *impl_;
  CHECK(m.exchange) << "the device plane is not started";
  if (m.world == 1) return {mine};
  return m.exchange->AllGather(mine, m.world);
}

void Plane::Barrier() {
  if (impl_->world > 1) Postoffice::Get()->Barrier(kPlaneApp, kWorkerGroup);
}

void Plane::Start(const PlaneOptions& options) {
  Impl& m = *impl_;
  CHECK(!m.started) << "the device plane is already started";
  Postoffice* po = Postoffice::Get();
  CHECK(po->van() && po->is_worker())
      << "start the device plane after ps::Start, on a worker or joint process";
  m.opts = options;
  m.sim = options.device < 0;
  m.rank = po->my_rank();
  m.world = po->num_workers();
  CHECK(m.world >= 1 && m.world <= PSDEV_MAX_RANKS)
      << "the device plane serves up to " << PSDEV_MAX_RANKS << " workers of one machine";
  if (m.sim) {
    FillSimRt(&m.rt);
  } else {
    m.lib = LoadRt(options.device_lib, &m.rt);
    CHECK_EQ(m.rt.set_device(options.device), 0) << "cannot select CUDA device " << options.device;
  }
  m.exchange.reset(new Exchange);
  // nobody sends before every endpoint exists
  Barrier();

  const int R = m.rank, W = m.world;
  auto gather = [this](const std::string& s) { return AllGather(s); };
  if (const char* env = getenv("PSB200_COPY_OUT_LAG")) m.copy_out_lag = atoi(env) != 0;
  std::string backend = m.sim ? "sim" : options.backend;
  if (backend == "auto") {
    const char* env = getenv("PSB200_HEAP");
    backend = env ? env : "auto";
  }
  if (backend == "auto") {
    const std::string mine = m.rt.vmm_supported() ? "1" : "0";
    bool all = true;
    for (const auto& s : AllGather(mine)) all = all && s == "1";
    backend = all ? "vmm" : "ipc";
  }
  CHECK(backend == "sim" || backend == "ipc" || backend == "vmm")
      << "unknown heap backend " << backend;
  m.backend_name = backend;
  m.ws = psdev_world_t{};
  m.ws.rank = R;
  m.ws.world = W;
  size_t bytes = (options.heap_bytes + 255) & ~size_t(255);
  CHECK_GE(bytes, size_t(2) * PSDEV_CTRL_BYTES);

  if (backend == "sim") {
    // shared memory, handed round as descriptors like the vmm arenas
    const int fd = memfd_create("psb200-arena", MFD_CLOEXEC);
    CHECK_GE(fd, 0) << strerror(errno);
    CHECK_EQ(ftruncate(fd, static_cast<off_t>(bytes)), 0);
    auto fds = ExchangeFds(R, W, {fd}, gather);
    close(fd);
    for (int p = 0; p < W; ++p) {
      void* at = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fds[p][0], 0);
      CHECK(at != MAP_FAILED) << strerror(errno);
      m.ws.peer_base[p] = at;
      close(fds[p][0]);
    }
  } else if (backend == "ipc") {
    void* base = nullptr;
    unsigned char handle[PSDEV_IPC_HANDLE_BYTES];
    CHECK_EQ(m.rt.heap_create(bytes, &base, handle), 0) << "arena of " << bytes << " bytes";
    m.ws.peer_base[R] = base;
    const auto handles = AllGather(std::string(reinterpret_cast<char*>(handle), sizeof(handle)));
    for (int p = 0; p < W; ++p) {
      if (p == R) continue;
      CHECK_EQ(handles[p].size(), sizeof(handle));
      void* at = nullptr;
      const int rc = m.rt.heap_open(reinterpret_cast<const unsigned char*>(handles[p].data()), &at);
      CHECK_EQ(rc, 0) << "cannot map the arena of rank " << p;
      m.ws.peer_base[p] = at;
    }
  } else {
    // multicast wanted?  every rank must be able, and the arena size must suit the object
    bool want_mc = W > 1 && options.multicast != 0;
    if (const char* env = getenv("PSB200_MULTICAST")) want_mc = want_mc && atoi(env) != 0;
    size_t gran = 0;
    if (want_mc) {
      std::string mine = "0";
      if (m.rt.mc_supported() && m.rt.mc_granularity(W, bytes, &gran) == 0 && gran)
        mine = std::to_string(gran);
      for (const auto& s : AllGather(mine)) want_mc = want_mc && s == mine && s != "0";
      if (!want_mc && options.multicast == 1)
        LOG(WARNING) << "NVSwitch multicast was requested but is not available on every rank";
    }
    void* base = nullptr;
    int fd = -1;
    size_t mapped = 0;
    CHECK_EQ(m.rt.vmm_create_aligned(bytes, want_mc ? gran : 0, &base, &fd, &mapped), 0)
        << "arena of " << bytes << " bytes";
    m.ws.peer_base[R] = base;
    const auto sizes = AllGather(std::to_string(mapped));
    auto fds = ExchangeFds(R, W, {fd}, gather);
    close(fd);
    for (int p = 0; p < W; ++p) {
      if (p != R) {
        CHECK_EQ(sizes[p], std::to_string(mapped)) << "ranks disagree on the arena size";
        void* at = nullptr;
        CHECK_EQ(m.rt.vmm_import(fds[p][0], mapped, &at), 0)
            << "cannot map the arena of rank " << p;
        m.ws.peer_base[p] = at;
      }
      close(fds[p][0]);
    }
    bytes = mapped;
    if (want_mc) {
      // every step is agreed on by all ranks before the next one; any failure drops the
      // alias everywhere and the job continues with plain peer accesses
      auto agree = [&](bool ok) {
        bool all = true;
        for (const auto& s : AllGather(ok ? "1" : "0")) all = all && s == "1";
        return all;
      };
      int mfd = -1;
      bool ok = true;
      if (R == 0) ok = m.rt.mc_create(mapped, W, &mfd, &m.mc) == 0;
      ok = agree(ok);  // everyone learns whether rank 0 has an object to hand out
      if (ok) {
        // rank 0's descriptor goes to everyone (the others contribute a placeholder)
        const int mine_fd = R == 0 ? mfd : open("/dev/null", O_RDONLY | O_CLOEXEC);
        auto mfds = ExchangeFds(R, W, {mine_fd}, gather);
        if (R != 0) ok = m.rt.mc_import(mfds[0][0], mapped, &m.mc) == 0;
        for (auto& v : mfds)
          for (int f : v) close(f);
        close(mine_fd);
      }
      ok = agree(ok);
      if (ok) ok = agree(m.rt.mc_add_device(m.mc) == 0);
      if (ok) ok = agree(m.rt.mc_bind(m.mc, base) == 0);
      void* alias = nullptr;
      if (ok) ok = agree(m.rt.mc_map(m.mc, &alias) == 0);
      if (ok) {
        m.ws.mc_base = alias;
      } else {
        LOG(WARNING) << "NVSwitch multicast alias not available; using peer loads and stores";
        if (m.mc) m.rt.mc_release(m.mc);
        m.mc = nullptr;
      }
    }
  }
  m.arena_bytes = bytes;
  m.ws.heap_bytes = bytes;
  m.sub.reset(new SubAlloc(bytes));
  m.next_channel = 0;
  CHECK_EQ(m.rt.stream_create(&m.s_h2d, 0), 0);
  CHECK_EQ(m.rt.stream_create(&m.s_compute, 1), 0);
  CHECK_EQ(m.rt.stream_create(&m.s_d2h, 0), 0);
  CHECK_EQ(m.rt.stream_create(&m.s_status, 0), 0);
  m.stop = false;
  m.in_flight = 0;
  m.completer = std::thread(&Impl::Completing, &m);
  m.started = true;
  po->set_device_route(this);
  // every rank has mapped every arena before anybody's kernel touches one
  Barrier();
  PS_VLOG(1) << "device plane up: rank " << R << "/" << W << ", backend " << backend
             << (m.ws.mc_base ? " + multicast" : "") << ", arena " << bytes << " bytes";
}

void Plane::Stop() {
  Impl& m = *impl_;
  if (!m.started) return;
  m.Drain();
  if (!m.sim) {
    m.rt.stream_sync(m.s_h2d);
    m.rt.stream_sync(m.s_compute);
    m.rt.stream_sync(m.s_d2h);
  }
  // nobody unmaps while a peer may still run a kernel that touches this arena
  Barrier();
  Postoffice::Get()->set_device_route(nullptr);
  {
    std::lock_guard<std::mutex> lk(m.q_mu);
    m.stop = true;
  }
  m.q_cv.notify_all();
  if (m.completer.joinable()) m.completer.join();
  {
    std::lock_guard<std::mutex> lk(m.mu);
    for (auto& kv : m.dense) {
      DenseInfo& d = *kv.second;
      if (d.owns_state) {
        m.rt.free_(d.table.master);
        if (d.table.state1) m.rt.free_(d.table.state1);
        if (d.table.state2) m.rt.free_(d.table.state2);
      }
    }
    m.dense.clear();
    for (auto& kv : m.sparse) {
      psdev_sparse_t& t = kv.second->table;
      m.rt.free_(t.w);
      if (t.state_stride <= 1) {  // (interleaved: z and n are inside the block that w begins)
        if (t.z) m.rt.free_(t.z);
        if (t.n) m.rt.free_(t.n);
      }
      if (t.overflow) m.rt.free_(t.overflow);
      if (t.klen) m.rt.free_(t.klen);
    }
    m.sparse.clear();
    m.last_done.clear();
  }
  if (m.mc) {
    m.rt.mc_release(m.mc);
    m.mc = nullptr;
    Barrier();  // every rank has unbound before the arenas go away
  }
  for (int p = 0; p < m.world; ++p) {
    void* at = m.ws.peer_base[p];
    if (!at) continue;
    if (m.backend_name == "sim") munmap(at, m.arena_bytes);
    else if (m.backend_name == "vmm") m.rt.vmm_release(at);
    else if (p != m.rank) m.rt.heap_close(at);
  }
  if (m.backend_name == "ipc") {
    Barrier();  // peers have closed their mappings of this arena
    m.rt.heap_destroy(m.ws.peer_base[m.rank]);
  }
  if (!m.sim) {
    for (void* e : m.event_pool) m.rt.event_destroy(e);
    m.rt.stream_destroy(m.s_h2d);
    m.rt.stream_destroy(m.s_compute);
    m.rt.stream_destroy(m.s_d2h);
    m.rt.stream_destroy(m.s_status);
  }
  m.event_pool.clear();
  m.exchange.reset();
  m.sub.reset();
  m.ws = psdev_world_t{};
  m.started = false;
}

// ---- heap ---------------------------------------------------------------------------------------
int64_t Plane::Alloc(size_t bytes, size_t align) {
  std::lock_guard<std::mutex> lk(impl_->mu);
  CHECK(impl_->sub) << "the device plane is not started";
  return impl_->sub->Alloc(bytes, align);
}
void Plane::Free(int64_t offset) {
  std::lock_guard<std::mutex> lk(impl_->mu);
  if (impl_->sub) {
    CHECK(impl_->sub->Free(offset)) << "not an allocation: offset " << offset;
  }
}
void* Plane::Local(int64_t offset) const {
  return static_cast<char*>(impl_->ws.peer_base[impl_->rank]) + offset;
}
size_t Plane::heap_in_use() const {
  std::lock_guard<std::mutex> lk(impl_->mu);
  return impl_->sub ? impl_->sub->in_use() : 0;
}
int Plane::NewChannel() {
  std::lock_guard<std::mutex> lk(impl_->mu);
  // the last channel is kept for device barriers
  CHECK_LT(impl_->next_channel, PSDEV_NUM_CHANNELS - 1)
      << "out of rendezvous channels: at most " << PSDEV_NUM_CHANNELS - 1 << " tensors";
  return impl_->next_channel++;
}

// ---- dense tensors ------------------------------------------------------------------------------
std::vector<Range> Plane::KeyRanges() const {
  const uint64_t W = static_cast<uint64_t>(impl_->world);
  const uint64_t width = kMaxKey / W;
  std::vector<Range> r;
  for (uint64_t i = 0; i < W; ++i) r.push_back(Range(width * i, width * (i + 1)));
  return r;
}

std::vector<Key> Plane::DenseKeys(uint64_t tensor_id) const {
  std::vector<Key> keys;
  for (const Range& r : KeyRanges()) keys.push_back(static_cast<Key>(r.begin() + tensor_id));
  return keys;
}

static int BuiltinStates(int kind) {
  return kind == PSDEV_OPT_MOMENTUM ? 1 : (kind == PSDEV_OPT_ADAM ? 2 : 0);
}

const DenseInfo& Plane::DeclareDense(int app_id, uint64_t tensor_id, int64_t n, int grad_dtype,
                                     int out_dtype, const psdev_opt_t& opt) {
  Impl& m = *impl_;
  CHECK(m.started);
  CHECK_GT(n, 0);
  const int W = m.world;
  const int64_t align = grad_dtype == PSDEV_I8 ? 256 : 8;
  psdev_table_t t{};
  t.n = (n + align - 1) / align * align;
  t.blk = ((t.n + W - 1) / W + align - 1) / align * align;  // contiguous ranges, one per shard
  const int64_t local_len = t.blk;  // one block per rank
  t.grad_dtype = grad_dtype;
  t.out_dtype = out_dtype;
  const int64_t goff = Alloc(static_cast<size_t>(t.n) * DtypeSize(grad_dtype));
  const int64_t woff = Alloc(static_cast<size_t>(t.n) * DtypeSize(out_dtype));
  CHECK(goff >= 0 && woff >= 0) << "symmetric heap exhausted (tensor of " << n << " values)";
  t.grad_off = static_cast<uint64_t>(goff);
  t.weight_off = static_cast<uint64_t>(woff);
  if (grad_dtype == PSDEV_I8) {
    const int64_t soff = Alloc(static_cast<size_t>(t.n / 256) * 4);
    CHECK_GE(soff, 0);
    t.gscale_off = static_cast<uint64_t>(soff);
  }
  if (!m.sim && W > 1 && grad_dtype != PSDEV_I8) {
    // low-latency region for small fused requests; cleared before any peer may write into it
    int64_t cap = 128 << 10;
    if (const char* env = getenv("PSB200_LL_CAP")) cap = atoll(env);
    cap = std::min<int64_t>(cap, t.n);
    if (cap > 0) {
      const size_t nb = m.rt.ll_bytes(W, cap);
      const int64_t loff = Alloc(nb);
      CHECK_GE(loff, 0) << "symmetric heap exhausted";
      m.rt.set_device(m.opts.device);
      CHECK_EQ(m.rt.memset_async(Local(loff), 0, nb, m.s_compute), 0);
      CHECK_EQ(m.rt.stream_sync(m.s_compute), 0);
      t.ll_off = static_cast<uint64_t>(loff);
      t.ll_cap = cap;
      Barrier();
    }
  }
  void* p = nullptr;
  CHECK_EQ(m.rt.malloc_(&p, static_cast<size_t>(local_len) * 4), 0);
  t.master = static_cast<float*>(p);
  // (a handle that the application registered says itself how much state it keeps)
  const int num_states =
      m.rt.handle_states ? m.rt.handle_states(opt.kind) : BuiltinStates(opt.kind);
  CHECK_GE(num_states, 0) << "no server handle is registered as kind " << opt.kind;
  if (num_states >= 1) {
    CHECK_EQ(m.rt.malloc_(&p, static_cast<size_t>(local_len) * 4), 0);
    t.state1 = static_cast<float*>(p);
  }
  if (num_states >= 2) {
    CHECK_EQ(m.rt.malloc_(&p, static_cast<size_t>(local_len) * 4), 0);
    t.state2 = static_cast<float*>(p);
  }
  bool nvls = W >= 4;
  if (const char* env = getenv("PSB200_NVLS")) nvls = atoi(env) != 0;
  const DenseInfo& d = RegisterDense(app_id, tensor_id, n, t, opt, NewChannel(), nvls, 0);
  const_cast<DenseInfo&>(d).owns_state = true;
  return d;
}

const DenseInfo& Plane::RegisterDense(int app_id, uint64_t tensor_id, int64_t n_user,
                                      const psdev_table_t& table, const psdev_opt_t& opt,
                                      int channel, bool nvls, int num_ctas) {
  Impl& m = *impl_;
  CHECK(m.started);
  std::unique_ptr<DenseInfo> d(new DenseInfo);
  d->app_id = app_id;
  d->tensor_id = tensor_id;
  d->n = table.n;
  d->n_user = n_user;
  {
    // key j names the j-th of W contiguous pieces of the tensor, whoever owns its blocks
    const int64_t align = table.grad_dtype == PSDEV_I8 ? 256 : 8;
    d->share = ((table.n + m.world - 1) / m.world + align - 1) / align * align;
  }
  d->channel = channel;
  d->nvls = nvls && m.ws.mc_base != nullptr && m.world > 1;
  d->num_ctas = num_ctas;
  d->table = table;
  d->opt = opt;
  d->grad = Local(static_cast<int64_t>(table.grad_off));
  d->weight = Local(static_cast<int64_t>(table.weight_off));
  std::lock_guard<std::mutex> lk(m.mu);
  auto key = std::make_pair(app_id, tensor_id);
  CHECK(m.dense.find(key) == m.dense.end())
      << "tensor " << tensor_id << " of app " << app_id << " is already registered";
  DenseInfo* raw = d.get();
  m.dense[key] = std::move(d);
  return *raw;
}

void Plane::UnregisterDense(int app_id, uint64_t tensor_id) {
  Impl& m = *impl_;
  m.Drain();
  std::lock_guard<std::mutex> lk(m.mu);
  auto it = m.dense.find(std::make_pair(app_id, tensor_id));
  if (it == m.dense.end()) return;
  m.last_done.erase(it->second.get());
  m.dense.erase(it);
}

const DenseInfo* Plane::FindDense(int app_id, uint64_t tensor_id) const {
  std::lock_guard<std::mutex> lk(impl_->mu);
  auto it = impl_->dense.find(std::make_pair(app_id, tensor_id));
  return it == impl_->dense.end() ? nullptr : it->second.get();
}

void Plane::ClearStatus(int app_id, uint64_t tensor_id) {
  const DenseInfo* d = FindDense(app_id, tensor_id);
  CHECK(d) << "unknown tensor " << tensor_id;
  Impl& m = *impl_;
  m.Drain();
  m.rt.set_device(m.opts.device);
  Barrier();  // nobody is inside a kernel on this tensor any more
  CHECK_EQ(m.rt.channel_clear(m.ws.peer_base[m.rank], d->channel), 0);
  if (d->table.ll_cap > 0 && !m.sim) {
    // words of the abandoned round must not be mistaken for those of a later one
    const size_t nb = m.rt.ll_bytes(m.world, d->table.ll_cap);
    void* region = Local(static_cast<int64_t>(d->table.ll_off));
    CHECK_EQ(m.rt.memset_async(region, 0, nb, m.s_compute), 0);
    CHECK_EQ(m.rt.stream_sync(m.s_compute), 0);
  }
  Barrier();
}

void Plane::SetOptimizer(int app_id, uint64_t tensor_id, const psdev_opt_t& opt) {
  std::lock_guard<std::mutex> lk(impl_->mu);
  auto it = impl_->dense.find(std::make_pair(app_id, tensor_id));
  CHECK(it != impl_->dense.end()) << "unknown tensor " << tensor_id;
  it->second->opt = opt;
}

// ---- routing ------------------------------------------------------------------------------------
namespace {
// shard and tensor id named by a key
inline void SplitKey(Key key, int world, int* shard, uint64_t* tensor_id) {
  const uint64_t width = kMaxKey / static_cast<uint64_t>(world);
  uint64_t s = static_cast<uint64_t>(key) / width;
  if (s >= static_cast<uint64_t>(world)) s = world - 1;
  *shard = static_cast<int>(s);
  *tensor_id = static_cast<uint64_t>(key) - width * s;
}
}  // namespace

bool Plane::Claims(int app_id, const SArray<Key>& keys) {
  Impl& m = *impl_;
  if (!m.started || keys.empty()) return false;
  // a key array in device memory addresses the app's keyed table
  if (keys.mem_kind() == MemKind::kDevice) return FindSparse(app_id) != nullptr;
  int shard;
  uint64_t id;
  SplitKey(keys[0], m.world, &shard, &id);
  return FindDense(app_id, id) != nullptr;
}

size_t Plane::PullBytes(int app_id, const SArray<Key>& keys) {
  Impl& m = *impl_;
  if (!m.started || keys.empty()) return 0;
  if (keys.mem_kind() == MemKind::kDevice) {
    const SparseInfo* sp = FindSparse(app_id);
    return sp ? keys.size() * static_cast<size_t>(sp->width) * 4 : 0;
  }
  int shard;
  uint64_t id;
  SplitKey(keys[0], m.world, &shard, &id);
  const DenseInfo* d = FindDense(app_id, id);
  if (!d) return 0;
  size_t elems = 0;
  for (size_t i = 0; i < keys.size(); ++i) {
    uint64_t id_i;
    SplitKey(keys[static_cast<int>(i)], m.world, &shard, &id_i);
    const int64_t lo = std::min<int64_t>(shard * d->share, d->n_user);
    const int64_t hi = std::min<int64_t>((shard + 1) * d->share, d->n_user);
    elems += static_cast<size_t>(hi - lo);
  }
  return elems * DtypeSize(d->table.out_dtype);
}

// ---- keyed tables -----------------------------------------------------------------------------
const SparseInfo& Plane::DeclareSparse(int app_id, uint64_t key_space, int64_t max_keys, int width,
                                       int kind, float lr, float alpha, float beta, float l1,
                                       float l2, bool var_len) {
  Impl& m = *impl_;
  CHECK(m.started);
  CHECK(key_space > 0 && max_keys > 0 && width >= 1 && kind >= 0 && kind <= 2);
  CHECK(!FindSparse(app_id)) << "app " << app_id << " already has a keyed table";
  const int W = m.world;
  std::unique_ptr<SparseInfo> sp(new SparseInfo);
  sp->app_id = app_id;
  sp->key_space = key_space;
  sp->max_keys = max_keys;
  sp->width = width;
  sp->var_len = var_len;
  psdev_sparse_t& t = sp->table;
  t = psdev_sparse_t{};
  t.range = (key_space + W - 1) / W;
  t.width = width;
  t.max_n = max_keys;
  t.max_vals = max_keys * width;
  t.slots = static_cast<int64_t>(t.range);
  t.kind = kind;
  t.lr = lr; t.alpha = alpha; t.beta = beta; t.l1 = l1; t.l2 = l2;
  t.channel = NewChannel();
  t.timeout_ns = m.opts.timeout_ns;
  auto alloc = [&](size_t bytes) {
    const int64_t off = Alloc(bytes);
    CHECK_GE(off, 0) << "symmetric heap exhausted (keyed table)";
    return static_cast<uint64_t>(off);
  };
  t.keys_off = alloc(8 * static_cast<size_t>(max_keys));
  t.grads_off = alloc(4 * static_cast<size_t>(t.max_vals));
  t.out_off = alloc(4 * static_cast<size_t>(t.max_vals));
  t.pos_off = alloc(8 * static_cast<size_t>(W + 2));
  const size_t acc_bytes = 4 * static_cast<size_t>(t.slots) * width;
  t.acc_off = alloc(acc_bytes);
  if (var_len) {
    t.lens_off = alloc(4 * static_cast<size_t>(max_keys));
    t.offs_off = alloc(8 * static_cast<size_t>(max_keys + 1));
  }
  m.rt.set_device(m.opts.device);
  void* acc = Local(static_cast<int64_t>(t.acc_off));
  void* pos = Local(static_cast<int64_t>(t.pos_off));
  CHECK_EQ(m.rt.memset_async(acc, 0, acc_bytes, m.s_compute), 0);
  CHECK_EQ(m.rt.memset_async(pos, 0, 8 * static_cast<size_t>(W + 2), m.s_compute), 0);
  CHECK_EQ(m.rt.stream_sync(m.s_compute), 0);
  void* p = nullptr;
  if (kind == 2) {
    // FTRL keeps three numbers per value; they sit side by side ({w, z, n, -}), so that an
    // update reads and writes one 16-byte group instead of three sectors of three arrays
    CHECK_EQ(m.rt.malloc_(&p, 4 * acc_bytes), 0);
    t.w = static_cast<float*>(p);
    t.z = t.w + 1;
    t.n = t.w + 2;
    t.state_stride = 4;
  } else {
    CHECK_EQ(m.rt.malloc_(&p, acc_bytes), 0);
    t.w = static_cast<float*>(p);
  }
  sp->keys = Local(static_cast<int64_t>(t.keys_off));
  sp->vals = Local(static_cast<int64_t>(t.grads_off));
  sp->out = Local(static_cast<int64_t>(t.out_off));
  if (var_len) {
    const size_t klen_bytes = 4 * static_cast<size_t>(t.slots);
    CHECK_EQ(m.rt.malloc_(&p, klen_bytes), 0);
    t.klen = static_cast<int32_t*>(p);
    sp->lens = Local(static_cast<int64_t>(t.lens_off));
    sp->offs = Local(static_cast<int64_t>(t.offs_off));
    CHECK_EQ(m.rt.memset_async(t.klen, 0, klen_bytes, m.s_compute), 0);
    CHECK_EQ(m.rt.memset_async(sp->lens, 0, 4 * static_cast<size_t>(max_keys), m.s_compute), 0);
    CHECK_EQ(m.rt.stream_sync(m.s_compute), 0);
  }
  SparseInfo* raw = sp.get();
  {
    std::lock_guard<std::mutex> lk(m.mu);
    m.sparse[app_id] = std::move(sp);
  }
  Barrier();  // every rank's accumulator is clear before anybody scatters into it
  return *raw;
}

const SparseInfo* Plane::FindSparse(int app_id) const {
  std::lock_guard<std::mutex> lk(impl_->mu);
  auto it = impl_->sparse.find(app_id);
  return it == impl_->sparse.end() ? nullptr : it->second.get();
}

void Plane::Memcpy(void* dst, const void* src, size_t bytes) {
  Impl& m = *impl_;
  CHECK(m.started);
  m.rt.set_device(m.opts.device);
  CHECK_EQ(m.rt.memcpy_async(dst, src, bytes, m.s_status), 0);
  CHECK_EQ(m.rt.stream_sync(m.s_status), 0);
}

void Plane::Submit(const DeviceRequest& req) {
  Impl& m = *impl_;
  CHECK(m.started);
  m.rt.set_device(m.opts.device);
  if (req.keys.mem_kind() == MemKind::kDevice) {
    SubmitSparse(req);
    return;
  }
  const int W = m.world;
  int shard;
  uint64_t id;
  SplitKey(req.keys[0], W, &shard, &id);
  DenseInfo* d = const_cast<DenseInfo*>(FindDense(req.app_id, id));
  CHECK(d) << "no tensor registered under key " << req.keys[0];
  const psdev_table_t& t = d->table;
  const size_t gsz = DtypeSize(t.grad_dtype), osz = DtypeSize(t.out_dtype);

  // keys -> runs of consecutive shards -> element ranges (in user elements: the last shard's
  // share may be short)
  struct Run { int64_t begin, end; };
  std::vector<Run> runs;
  std::vector<int> lens(req.keys.size());
  int prev = -2;
  for (size_t i = 0; i < req.keys.size(); ++i) {
    uint64_t id_i;
    SplitKey(req.keys[static_cast<int>(i)], W, &shard, &id_i);
    CHECK_EQ(id_i, id) << "one request addresses one tensor (keys of tensors " << id << " and "
                       << id_i << " were mixed)";
    CHECK_GT(shard, prev == -2 ? -1 : prev) << "keys must be increasing";
    const int64_t lo = std::min<int64_t>(shard * d->share, d->n_user);
    const int64_t hi = std::min<int64_t>((shard + 1) * d->share, d->n_user);
    lens[i] = static_cast<int>(hi - lo);
    if (!req.lens.empty()) {
      CHECK_EQ(req.lens[static_cast<int>(i)], lens[i])
          << "length of key " << req.keys[static_cast<int>(i)] << " differs from its share";
    }
    if (shard == prev + 1 && !runs.empty()) runs.back().end = hi;
    else runs.push_back(Run{lo, hi});
    prev = shard;
  }
  size_t total = 0;
  for (const Run& r : runs) total += static_cast<size_t>(r.end - r.begin);
  if (req.push) {
    CHECK(req.vals) << "push without values";
    CHECK_EQ(req.vals_bytes, total * gsz)
        << "pushed bytes do not match the keys' shares of tensor " << id << " ("
        << total << " values of " << gsz << " bytes)";
  }
  if (req.pull && req.outs) {
    CHECK_EQ(req.outs_bytes, total * osz) << "output size does not match the pulled values";
  }
  if (req.lens_out) { CHECK_EQ(req.lens_out_n, lens.size()); }

  // (the CPU stand-in calls "device memory" what lies in an arena)
  auto on_device = [&](const void* p) {
    if (!m.sim) return m.rt.is_device_pointer(p) != 0;
    const char* c = static_cast<const char*>(p);
    const char* lo = static_cast<const char*>(m.ws.peer_base[m.rank]);
    return c >= lo && c < lo + m.arena_bytes;
  };
  const bool in_dev = req.push && on_device(req.vals);
  const bool out_dev = req.pull && req.outs && on_device(req.outs);
  const bool host_in = req.push && !in_dev;
  const bool host_out = req.pull && req.outs && !out_dev;
  const bool staged = host_in || host_out;
  int op = (req.push ? PSDEV_OP_PUSH : 0) | (req.pull ? PSDEV_OP_PULL : 0);
  if (req.push && !req.pull && req.cmd == kCmdPublish) op |= PSDEV_OP_PUBLISH;

  psdev_opt_t opt;
  {
    std::lock_guard<std::mutex> lk(m.mu);
    if (req.push) ++d->step;
    opt = d->opt;
    if (opt.kind == PSDEV_OPT_ADAM) {
      const double s = static_cast<double>(std::max<int64_t>(d->step, 1));
      opt.bias1 = static_cast<float>(1.0 - std::pow(static_cast<double>(opt.beta1), s));
      opt.bias2 = static_cast<float>(std::sqrt(1.0 - std::pow(static_cast<double>(opt.beta2), s)));
    }
  }
  // bit 0: rendezvous with the other ranks; bit 1: NVSwitch multicast path, chosen per launch
  // by the size of what that launch moves
  auto sync_for = [&](int64_t elems) {
    const bool mc = d->nvls && m.rt.multicast_pays &&
                    m.rt.multicast_pays(m.world, static_cast<uint64_t>(elems) * gsz);
    return 1 | (mc ? 2 : 0);
  };
  // the kernel works on multiples of 8 values; the padding of the last shard belongs to it
  auto pad8 = [&](int64_t e) { return e >= d->n_user ? t.n : e; };

  Impl::Pending pend;
  pend.channel = d->channel;
  pend.timestamp = req.timestamp;
  pend.responses = req.responses;
  pend.customer = req.customer;
  pend.on_done = req.on_done;
  pend.lens_out = req.lens_out;
  pend.tensor = d;
  if (req.lens_out) pend.lens = lens;

  void* prev_done = nullptr;
  {
    std::lock_guard<std::mutex> lk(m.mu);
    auto it = m.last_done.find(d);
    if (it != m.last_done.end()) prev_done = it->second;
  }
  void* done = m.NewEvent();
  const char* vals = static_cast<const char*>(req.vals);
  char* outs = static_cast<char*>(req.outs);
  char* grad = static_cast<char*>(d->grad);
  char* weight = static_cast<char*>(d->weight);

  if (!staged) {
    // values already on the device: everything in order on one stream
    void* s = tls_has_stream ? tls_stream : m.s_compute;
    if (prev_done && !m.sim) m.rt.stream_wait_event(s, prev_done);
    size_t eoff = 0;  // position in the request's value list, in elements
    for (const Run& r : runs) {
      const size_t cnt = static_cast<size_t>(r.end - r.begin);
      if (req.push && vals + eoff * gsz != grad + r.begin * gsz) {
        CHECK_EQ(m.rt.memcpy_async(grad + r.begin * gsz, vals + eoff * gsz, cnt * gsz, s), 0);
      }
      const int rc = m.rt.dense_op(&m.ws, &t, op, r.begin, pad8(r.end), &opt, d->channel,
                                   d->num_ctas, m.opts.timeout_ns,
                                   sync_for(pad8(r.end) - r.begin), s);
      CHECK_EQ(rc, 0) << "psdev_dense_op failed";
      if (req.pull && outs && outs + eoff * osz != weight + r.begin * osz) {
        CHECK_EQ(m.rt.memcpy_async(outs + eoff * osz, weight + r.begin * osz, cnt * osz, s), 0);
      }
      eoff += cnt;
    }
    m.rt.event_record(done, s);
  } else {
    // host-resident values: slices flow host -> device -> kernel -> host on three streams,
    // so the copy of slice k+1 in, the kernel of slice k and the copy of slice k-1 out overlap
    void* origin = tls_stream;  // work the caller has queued on its stream comes first
    void* start = nullptr;
    if (tls_has_stream) {
      start = m.NewEvent();
      m.rt.event_record(start, origin);
      pend.events_to_recycle.push_back(start);
    }
    for (void* s : {m.s_h2d, m.s_compute, m.s_d2h}) {
      if (prev_done) m.rt.stream_wait_event(s, prev_done);
      if (start) m.rt.stream_wait_event(s, start);
    }
    const int64_t step_g =
        std::max<int64_t>(8, static_cast<int64_t>(m.opts.slice_bytes / gsz) & ~int64_t(7));
    // The first slice's copy in and the last slice's copy out overlap with nothing, so the
    // slices grow from 1/16 of the configured size (at least 256 KiB), doubling up to it, and
    // shrink again the same way towards the end of a run.
    const int64_t small_g = std::max<int64_t>(
        8, std::min<int64_t>(step_g, std::max<int64_t>(step_g / 16, (256 << 10) / gsz)) &
               ~int64_t(7));
    // A slice's copy out needs its copy in and its kernel, and the next slice's copy in ends
    // at about the moment the previous copy out does: issued as soon as possible, every copy
    // out would start one kernel and one event hand-over late, with the link idle in that
    // direction meanwhile.  So the copy out of slice k is held until the copy in of slice k+1
    // has finished as well: from then on its own dependencies are met long before its turn.
    const bool lagged = m.copy_out_lag && host_in && host_out && req.push && req.pull && outs;
    struct Held {
      char* dst; const char* src; size_t bytes; void* after_kernel;
    } held{nullptr, nullptr, 0, nullptr};
    bool holding = false;
    auto copy_out = [&](const Held& h, void* also_after) {
      m.rt.stream_wait_event(m.s_d2h, h.after_kernel);
      if (also_after) m.rt.stream_wait_event(m.s_d2h, also_after);
      CHECK_EQ(m.rt.memcpy_async(h.dst, h.src, h.bytes, m.s_d2h), 0);
    };
    size_t elem_off = 0;  // position in the request's value list
    for (const Run& r : runs) {
      const std::vector<int64_t> cuts = SliceEnds(r.begin, r.end, small_g, step_g);
      int64_t b = r.begin;
      for (const int64_t e : cuts) {
        if (e <= b) continue;
        const size_t at = elem_off + static_cast<size_t>(b - r.begin);
        const size_t cnt = static_cast<size_t>(e - b);
        if (req.push) {
          void* in_stream = host_in ? m.s_h2d : m.s_compute;
          if (host_in || vals + at * gsz != grad + b * gsz) {
            CHECK_EQ(m.rt.memcpy_async(grad + b * gsz, vals + at * gsz, cnt * gsz, in_stream), 0);
          }
          if (host_in) {
            void* ev = m.NewEvent();
            m.rt.event_record(ev, m.s_h2d);
            m.rt.stream_wait_event(m.s_compute, ev);
            pend.events_to_recycle.push_back(ev);
            if (holding) {
              copy_out(held, ev);
              holding = false;
            }
          }
        }
        const int rc = m.rt.dense_op(&m.ws, &t, op, b, pad8(e), &opt, d->channel, d->num_ctas,
                                     m.opts.timeout_ns, sync_for(pad8(e) - b), m.s_compute);
        CHECK_EQ(rc, 0) << "psdev_dense_op failed";
        if (req.pull && outs) {
          if (host_out) {
            void* ev = m.NewEvent();
            m.rt.event_record(ev, m.s_compute);
            pend.events_to_recycle.push_back(ev);
            const Held h{outs + at * osz, weight + b * osz, cnt * osz, ev};
            if (lagged) {
              held = h;
              holding = true;
            } else {
              copy_out(h, nullptr);
            }
          } else if (outs + at * osz != weight + b * osz) {
            CHECK_EQ(
                m.rt.memcpy_async(outs + at * osz, weight + b * osz, cnt * osz, m.s_compute), 0);
          }
        }
        b = e;
      }
      elem_off += static_cast<size_t>(r.end - r.begin);
    }
    if (holding) copy_out(held, nullptr);
    // the request is complete when the last kernel and the last copy out are
    void* tail = m.NewEvent();
    m.rt.event_record(tail, m.s_d2h);
    m.rt.stream_wait_event(m.s_compute, tail);
    pend.events_to_recycle.push_back(tail);
    m.rt.event_record(done, m.s_compute);
    if (tls_has_stream) m.rt.stream_wait_event(origin, done);
  }
  pend.event = done;
  {
    std::lock_guard<std::mutex> lk(m.mu);
    // `done` doubles as the ordering point for the next request on this tensor
    m.last_done[d] = done;
  }
  {
    std::lock_guard<std::mutex> lk(m.q_mu);
    ++m.in_flight;
    m.queue.push_back(std::move(pend));
  }
  m.q_cv.notify_one();
}

// A keyed request: keys, values and outputs are device arrays.  The request is staged into the
// table's buffers in the arena (device-to-device, unless it already lives there), then scatter,
// apply and respond run on the caller's stream; the rendezvous of the ranks is inside the last
// two kernels.  A push without pull still runs the respond kernel (it closes the round); a pull
// without push scatters zeros, which changes nothing on the owners.
void Plane::SubmitSparse(const DeviceRequest& req) {
  Impl& m = *impl_;
  SparseInfo* sp = const_cast<SparseInfo*>(FindSparse(req.app_id));
  CHECK(sp) << "app " << req.app_id << " has no keyed table";
  const psdev_sparse_t& t = sp->table;
  const int64_t n = static_cast<int64_t>(req.keys.size());
  CHECK_LE(n, sp->max_keys) << "more keys than the table was declared for";
  // Tables with lengths: a push names the length of every value (a device array, like the keys);
  // a pull asks the owners for the stored lengths first and returns them beside the values.
  const bool ask_lens = sp->var_len && !req.push;
  if (sp->var_len) {
    if (req.push) { CHECK_EQ(static_cast<int64_t>(req.lens.size()), n) << "one length per key"; }
  } else {
    CHECK(req.lens.empty()) << "app " << req.app_id << " holds fixed-width values";
  }
  const size_t cap_bytes = static_cast<size_t>(t.max_vals) * 4;
  const size_t vbytes = sp->var_len ? req.vals_bytes : static_cast<size_t>(n) * sp->width * 4;
  if (req.push) {
    CHECK(req.vals && req.vals_bytes == vbytes && vbytes <= cap_bytes && vbytes % 4 == 0)
        << "expected " << (sp->var_len ? "at most " : "") << sp->width << " fp32 per key";
  }
  const size_t obytes = sp->var_len ? req.outs_bytes : vbytes;
  if (req.pull && req.outs) {
    CHECK(req.outs_bytes == obytes && obytes <= cap_bytes) << "output of " << req.outs_bytes
                                                           << " bytes does not fit the request";
  }
  void* s = tls_has_stream ? tls_stream : m.s_compute;
  void* prev_done = nullptr;
  {
    std::lock_guard<std::mutex> lk(m.mu);
    auto it = m.last_done.find(sp);
    if (it != m.last_done.end()) prev_done = it->second;
  }
  if (prev_done) m.rt.stream_wait_event(s, prev_done);
  const void* kptr = req.keys.data();
  if (kptr != sp->keys) {
    CHECK_EQ(m.rt.memcpy_async(sp->keys, kptr, static_cast<size_t>(n) * 8, s), 0);
  }
  if (req.push) {
    if (req.vals != sp->vals) {
      CHECK_EQ(m.rt.memcpy_async(sp->vals, req.vals, vbytes, s), 0);
    }
  } else if (!sp->var_len) {
    CHECK_EQ(m.rt.memset_async(sp->vals, 0, vbytes, s), 0);
  }
  const int sync = m.world > 1 ? 1 : 0;
  const uint64_t tmo = t.timeout_ns ? t.timeout_ns : 20000000000ull;
  if (sp->var_len && !ask_lens && req.lens.data() != sp->lens) {
    CHECK_EQ(m.rt.memcpy_async(sp->lens, req.lens.data(), static_cast<size_t>(n) * 4, s), 0);
  }
  if (ask_lens) {
    // cut points of my keys; then every owner stores the lengths it holds into the requesters'
    // arrays (a device barrier on either side), and the offsets follow from them
    CHECK_EQ(m.rt.memset_async(sp->lens, 0, static_cast<size_t>(n) * 4, s), 0);
    CHECK_EQ(m.rt.key_shard_lookup(static_cast<const uint64_t*>(sp->keys), n, t.range, m.world,
                                   static_cast<int64_t*>(Local(static_cast<int64_t>(t.pos_off))),
                                   s), 0);
    if (sync) { CHECK_EQ(m.rt.device_barrier(&m.ws, t.channel, tmo, s), 0); }
    CHECK_EQ(m.rt.sparse_lens(&m.ws, &t, 0, s), 0) << "psdev_sparse_lens failed";
    if (sync) { CHECK_EQ(m.rt.device_barrier(&m.ws, t.channel, tmo, s), 0); }
    CHECK_EQ(m.rt.lens_to_offsets(static_cast<const int32_t*>(sp->lens), n,
                                  static_cast<int64_t*>(sp->offs), s), 0);
  } else {
    CHECK_EQ(m.rt.sparse_scatter(&m.ws, &t, n, 0, s), 0) << "psdev_sparse_scatter failed";
  }
  CHECK_EQ(m.rt.sparse_apply(&m.ws, &t, 0, sync, s), 0) << "psdev_sparse_apply failed";
  CHECK_EQ(m.rt.sparse_respond(&m.ws, &t, 0, sync, s), 0) << "psdev_sparse_respond failed";
  if (req.pull && req.outs && req.outs != sp->out) {
    CHECK_EQ(m.rt.memcpy_async(req.outs, sp->out, obytes, s), 0);
  }
  if (sp->var_len && req.pull && req.lens_out && req.lens_out != sp->lens) {
    // the lengths of the answer, beside it (device memory, like the keys)
    CHECK_EQ(req.lens_out_n, static_cast<size_t>(n));
    CHECK_EQ(m.rt.memcpy_async(req.lens_out, sp->lens, static_cast<size_t>(n) * 4, s), 0);
  }
  void* done = m.NewEvent();
  m.rt.event_record(done, s);
  Impl::Pending pend;
  pend.event = done;
  pend.channel = t.channel;
  pend.timestamp = req.timestamp;
  pend.responses = req.responses;
  pend.customer = req.customer;
  pend.on_done = req.on_done;
  pend.tensor = sp;
  {
    std::lock_guard<std::mutex> lk(m.mu);
    m.last_done[sp] = done;
  }
  {
    std::lock_guard<std::mutex> lk(m.q_mu);
    ++m.in_flight;
    m.queue.push_back(std::move(pend));
  }
  m.q_cv.notify_one();
}

}  // namespace device
}  // namespace ps
