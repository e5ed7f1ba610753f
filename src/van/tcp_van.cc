// Socket van: length-prefixed frames over TCP (or Unix-domain sockets with DMLC_LOCAL=1),
// one epoll thread for all receives, one lazily opened sending connection per peer process.
//
// It takes the place of the reference's ZMQVan (src/zmq_van.h:37-248) without libzmq.  What is
// kept: one listening endpoint per process, sends serialised per destination, zero-copy
// hand-over of received frames to SArray (each data frame is read straight into the buffer
// that the SArray then owns), DMLC_LOCAL for same-host IPC, DMLC_USE_KUBERNETES to bind the
// wildcard address, random-port retries on bind.  What differs: the frame header carries the
// sender and receiver node ids explicitly (ZMQ derived the sender from the socket identity,
// src/zmq_van.h:234-248), which is what lets one process host several ids.
//
// Frame: [FrameHeader][n_data x u64 lengths][meta bytes (PBMeta)][data 0]...[data n-1]
#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/epoll.h>
#include <sys/eventfd.h>
#include <sys/file.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <limits.h>
#include <sys/uio.h>
#include <sys/un.h>
#include <unistd.h>

#include <chrono>
#include <cstring>
#include <deque>
#include <map>
#include <new>
#include <random>

#include "ps/internal/pb_codec.h"
#include "ps/internal/postoffice.h"
#include "ps/internal/shm_pool.h"
#include "van/backends.h"

namespace ps {
namespace {

constexpr uint32_t kMagic = 0x32425350u;  // "PSB2"
constexpr uint32_t kMaxFrames = 64;
constexpr uint32_t kMaxMetaBytes = 64u << 20;      // a meta block is a few hundred bytes
constexpr uint64_t kMaxFrameBytes = 1ull << 40;    // no single array is a terabyte

struct FrameHeader {
  uint32_t magic;
  int32_t sender;
  int32_t recver;
  uint32_t meta_len;
  uint32_t n_data;
};
static_assert(sizeof(FrameHeader) == 20, "frame header layout");

std::string UnixPath(int port) { return "/tmp/psb200_" + std::to_string(port) + ".sock"; }

// A data frame whose length word has this bit set does not carry its bytes: the array lives in
// a shared-memory segment (ps/internal/shm_pool.h), the frame body is a ShmRef and the segment's
// file descriptor rides on the message as SCM_RIGHTS ancillary data (Unix sockets only), in
// frame order.
constexpr uint64_t kShmFrame = 1ull << 63;
struct ShmRef {
  uint64_t seg_size;
  uint64_t offset;
};

// Writes all of iov.  `fds` (may be empty) are attached to the first byte.
bool WriteAll(int fd, struct iovec* iov, int iovcnt, const std::vector<int>& fds) {
  bool first = true;
  alignas(struct cmsghdr) char ctrl[CMSG_SPACE(sizeof(int) * kMaxFrames)];
  while (iovcnt > 0) {
    struct msghdr mh {};
    mh.msg_iov = iov;
    mh.msg_iovlen = static_cast<size_t>(iovcnt > IOV_MAX ? IOV_MAX : iovcnt);
    if (first && !fds.empty()) {
      memset(ctrl, 0, sizeof(ctrl));
      mh.msg_control = ctrl;
      mh.msg_controllen = CMSG_SPACE(sizeof(int) * fds.size());
      struct cmsghdr* cm = CMSG_FIRSTHDR(&mh);
      cm->cmsg_level = SOL_SOCKET;
      cm->cmsg_type = SCM_RIGHTS;
      cm->cmsg_len = CMSG_LEN(sizeof(int) * fds.size());
      memcpy(CMSG_DATA(cm), fds.data(), sizeof(int) * fds.size());
    }
    // MSG_NOSIGNAL: a peer that has gone away yields EPIPE here, not a SIGPIPE
    ssize_t n = ::sendmsg(fd, &mh, MSG_NOSIGNAL);
    if (n < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    if (n > 0) first = false;
    size_t left = static_cast<size_t>(n);
    while (iovcnt > 0 && left >= iov->iov_len) {
      left -= iov->iov_len;
      ++iov;
      --iovcnt;
    }
    if (iovcnt > 0 && left > 0) {
      iov->iov_base = static_cast<char*>(iov->iov_base) + left;
      iov->iov_len -= left;
    }
  }
  return true;
}

// Recycles large receive buffers.  A fresh allocation of tens of megabytes costs about as much
// in page faults and zero-filling as copying the bytes into it, so buffers of at least 1 MiB go
// back to a free list (bounded by PS_RECV_POOL_MB, default 256) when their array is released.
class RecvPool {
 public:
  RecvPool() : limit_(static_cast<size_t>(GetEnv("PS_RECV_POOL_MB", 256)) << 20) {}
  ~RecvPool() {
    for (auto& kv : free_) delete[] kv.second;
  }
  static constexpr size_t kMin = size_t(1) << 20;
  // A buffer of at least `len` bytes; *cap is what to hand back to Put.
  char* Get(size_t len, size_t* cap) {
    if (len < kMin) {
      *cap = 0;
      return new char[len ? len : 1];
    }
    const size_t want = (len + kMin - 1) / kMin * kMin;
    {
      std::lock_guard<std::mutex> lk(mu_);
      auto it = free_.lower_bound(want);
      if (it != free_.end() && it->first <= want + want / 4) {
        char* p = it->second;
        *cap = it->first;
        held_ -= it->first;
        free_.erase(it);
        return p;
      }
    }
    *cap = want;
    return new char[want];
  }
  void Put(char* p, size_t cap) {
    if (cap >= kMin) {
      std::lock_guard<std::mutex> lk(mu_);
      if (held_ + cap <= limit_) {
        free_.emplace(cap, p);
        held_ += cap;
        return;
      }
    }
    delete[] p;
  }

 private:
  std::mutex mu_;
  std::multimap<size_t, char*> free_;
  size_t held_ = 0;
  const size_t limit_;
};

// Receive-side state of one accepted connection.
struct InConn {
  int fd = -1;
  enum Phase { kHeader, kLens, kMeta, kData } phase = kHeader;
  FrameHeader hdr{};
  std::vector<uint64_t> lens;
  std::string meta;
  Message msg;
  size_t frame = 0;       // index of the data frame being read
  char* dst = nullptr;    // where the current phase reads into
  size_t need = 0, got = 0;
  char* frame_buf = nullptr;  // buffer of the data frame being read (not yet owned by msg)
  size_t frame_cap = 0;       // what RecvPool::Put wants back with it
  ShmRef shm_ref{};           // body of a shared-memory frame
  bool frame_is_shm = false;
  std::deque<int> fds;        // descriptors received and not yet claimed by a frame
  bool bad = false;           // a frame was refused (absurd length): close the connection
};

struct OutConn {
  std::mutex mu;
  int fd = -1;
  bool was_connected = false;  // a connection to this address has existed before
  std::string host;
  int port = 0;
};

class TcpVan : public Van {
 public:
  explicit TcpVan(bool priority) { set_priority_mode(priority); }
  ~TcpVan() override {}

 protected:
  void StartBackend() override {
    local_ = GetEnv("DMLC_LOCAL", 0) != 0;
    epfd_ = epoll_create1(EPOLL_CLOEXEC);
    CHECK_GE(epfd_, 0) << "epoll_create1: " << strerror(errno);
    wakefd_ = eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
    CHECK_GE(wakefd_, 0);
    struct epoll_event ev {};
    ev.events = EPOLLIN;
    ev.data.fd = wakefd_;
    epoll_ctl(epfd_, EPOLL_CTL_ADD, wakefd_, &ev);
    io_stop_ = false;
    io_thread_.reset(new std::thread(&TcpVan::IoLoop, this));
  }

  void StopBackend() override {
    io_stop_ = true;
    uint64_t one = 1;
    ssize_t r = ::write(wakefd_, &one, sizeof(one));
    (void)r;
    if (io_thread_) io_thread_->join();
    io_thread_.reset();
    for (auto& kv : in_) {
      ::close(kv.first);
      delete[] kv.second.frame_buf;
      for (int f : kv.second.fds) ::close(f);
    }
    in_.clear();
    {
      std::lock_guard<std::mutex> lk(out_mu_);
      for (auto& kv : out_) {
        std::lock_guard<std::mutex> l2(kv.second->mu);
        if (kv.second->fd >= 0) ::close(kv.second->fd);
        kv.second->fd = -1;
      }
      out_.clear();
      id_addr_.clear();
    }
    if (listen_fd_ >= 0) ::close(listen_fd_);
    listen_fd_ = -1;
    if (!unix_path_.empty()) {
      ::unlink(unix_path_.c_str());
      if (unix_lock_fd_ >= 0) ::unlink((unix_path_ + ".lock").c_str());
    }
    unix_path_.clear();
    if (unix_lock_fd_ >= 0) ::close(unix_lock_fd_);  // gives the name back
    unix_lock_fd_ = -1;
    ::close(wakefd_);
    ::close(epfd_);
    wakefd_ = epfd_ = -1;
  }

  int Bind(const Node& node, int max_retry) override {
    std::mt19937 rng(static_cast<unsigned>(getpid()) * 2654435761u +
                     static_cast<unsigned>(time(nullptr)));
    int port = node.port;
    for (int attempt = 0; attempt <= max_retry; ++attempt) {
      int fd = TryListen(port);
      if (fd >= 0) {
        listen_fd_ = fd;
        struct epoll_event ev {};
        ev.events = EPOLLIN;
        ev.data.fd = fd;
        epoll_ctl(epfd_, EPOLL_CTL_ADD, fd, &ev);
        return port;
      }
      port = 10000 + static_cast<int>(rng() % 40000);
    }
    return -1;
  }

  void Connect(const Node& node) override {
    CHECK_NE(node.id, Node::kEmpty);
    CHECK_NE(node.port, Node::kEmpty);
    std::lock_guard<std::mutex> lk(out_mu_);
    const std::string key = node.hostname + ":" + std::to_string(node.port);
    auto it = id_addr_.find(node.id);
    if (it != id_addr_.end() && it->second != key) {
      // the id moved to a new address (a recovered node): drop the old path if unused
      const std::string old = it->second;
      bool still_used = false;
      for (auto& kv : id_addr_) still_used |= (kv.first != node.id && kv.second == old);
      if (!still_used) {
        auto oc = out_.find(old);
        if (oc != out_.end()) {
          // keep the connection object alive until its lock has been released
          std::shared_ptr<OutConn> gone = oc->second;
          out_.erase(oc);
          std::lock_guard<std::mutex> l2(gone->mu);
          if (gone->fd >= 0) ::close(gone->fd);
          gone->fd = -1;
        }
      }
    }
    id_addr_[node.id] = key;
    if (!out_.count(key)) {
      auto c = std::make_shared<OutConn>();
      c->host = node.hostname;
      c->port = node.port;
      out_[key] = c;
    }
  }

  int SendMsg(const Message& msg) override {
    const int id = msg.meta.recver;
    CHECK_NE(id, Meta::kEmpty);
    std::shared_ptr<OutConn> c;
    {
      std::lock_guard<std::mutex> lk(out_mu_);
      auto it = id_addr_.find(id);
      if (it == id_addr_.end()) {
        LOG(WARNING) << "there is no path to node " << id;
        return -1;
      }
      c = out_[it->second];
    }
    std::string meta;
    pb::EncodeMeta(msg.meta, &meta);
    const size_t n = msg.data.size();
    CHECK_LE(n, (size_t)kMaxFrames);
    FrameHeader h{kMagic, msg.meta.sender, msg.meta.recver, static_cast<uint32_t>(meta.size()),
                  static_cast<uint32_t>(n)};
    std::vector<uint64_t> lens(n);
    std::vector<ShmRef> refs(n);
    std::vector<int> fds;
    std::vector<struct iovec> iov;
    iov.reserve(3 + n);
    iov.push_back({&h, sizeof(h)});
    size_t total = sizeof(h) + meta.size();
    for (size_t i = 0; i < n; ++i) {
      CHECK(msg.data[i].mem_kind() == MemKind::kHost)
          << "device-resident payloads travel through the device data plane, not the socket van";
      lens[i] = msg.data[i].size();
      total += lens[i] + 8;
      int fd = -1;
      if (local_ && lens[i] &&
          shm::Share(msg.data[i].data(), lens[i], &fd, &refs[i].offset, &refs[i].seg_size)) {
        // the peer maps the segment instead of receiving the bytes
        lens[i] |= kShmFrame;
        fds.push_back(fd);
      }
    }
    if (n) iov.push_back({lens.data(), n * sizeof(uint64_t)});
    iov.push_back({const_cast<char*>(meta.data()), meta.size()});
    for (size_t i = 0; i < n; ++i) {
      if (lens[i] & kShmFrame) {
        iov.push_back({&refs[i], sizeof(ShmRef)});
      } else if (lens[i]) {
        iov.push_back({msg.data[i].data(), static_cast<size_t>(lens[i])});
      }
    }

    std::lock_guard<std::mutex> lk(c->mu);
    for (int attempt = 0; attempt < 2; ++attempt) {
      if (c->fd < 0) c->fd = Dial(c->host, c->port, c->was_connected);
      if (c->fd < 0) break;
      c->was_connected = true;
      std::vector<struct iovec> tmp = iov;
      if (WriteAll(c->fd, tmp.data(), static_cast<int>(tmp.size()), fds))
        return static_cast<int>(total);
      // the peer went away (for instance it was replaced): reconnect once
      ::close(c->fd);
      c->fd = -1;
    }
    // nobody will map the shared frames of this message
    for (size_t i = 0; i < n; ++i)
      if (lens[i] & kShmFrame) shm::Unshare(msg.data[i].data());
    return -1;
  }

 private:
  int TryListen(int port) {
    int fd;
    if (local_) {
      fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
      if (fd < 0) return -1;
      struct sockaddr_un addr {};
      addr.sun_family = AF_UNIX;
      const std::string path = UnixPath(port);
      strncpy(addr.sun_path, path.c_str(), sizeof(addr.sun_path) - 1);
      // A port number is only a name here, and two processes can be handed the same one.  The
      // owner of a name holds a lock on "<path>.lock" for as long as it lives (the kernel drops
      // it when the process dies, so a stale socket file of a crashed run is not in the way);
      // whoever cannot get the lock tries another number instead of unlinking a live socket.
      const std::string lock_path = path + ".lock";
      const int lock_fd = ::open(lock_path.c_str(), O_CREAT | O_RDWR | O_CLOEXEC, 0600);
      struct stat held {}, named {};
      // the lock file is removed by its owner at Stop: a lock on a file that is no longer the
      // one behind the name does not count
      if (lock_fd < 0 || flock(lock_fd, LOCK_EX | LOCK_NB) != 0 || fstat(lock_fd, &held) != 0 ||
          stat(lock_path.c_str(), &named) != 0 || held.st_ino != named.st_ino) {
        if (lock_fd >= 0) ::close(lock_fd);
        ::close(fd);
        return -1;
      }
      ::unlink(path.c_str());
      if (bind(fd, reinterpret_cast<struct sockaddr*>(&addr), sizeof(addr)) != 0) {
        ::close(lock_fd);
        ::close(fd);
        return -1;
      }
      unix_path_ = path;
      unix_lock_fd_ = lock_fd;
    } else {
      fd = socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
      if (fd < 0) return -1;
      int one = 1;
      setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
      struct sockaddr_in addr {};
      addr.sin_family = AF_INET;
      addr.sin_addr.s_addr = htonl(INADDR_ANY);  // also what DMLC_USE_KUBERNETES asks for
      addr.sin_port = htons(static_cast<uint16_t>(port));
      if (bind(fd, reinterpret_cast<struct sockaddr*>(&addr), sizeof(addr)) != 0) {
        ::close(fd);
        return -1;
      }
    }
    if (listen(fd, 256) != 0) {
      ::close(fd);
      return -1;
    }
    fcntl(fd, F_SETFL, fcntl(fd, F_GETFL, 0) | O_NONBLOCK);
    return fd;
  }

  // Blocking connect with retries: peers may still be starting.
  // Connects to host:port.  A peer that has never been reached may still be starting up, so
  // the first connection keeps trying for PS_CONNECT_TIMEOUT seconds.  A peer that was
  // connected before and no longer accepts has gone away: `redial` gives it a quarter of a
  // second, so that a caller with more to send (the resender, above all) is not held up.
  int Dial(const std::string& host, int port, bool redial) {
    const int water = GetEnv("DMLC_PS_WATER_MARK", 0);
    const auto deadline =
        std::chrono::steady_clock::now() +
        (redial ? std::chrono::milliseconds(250)
                : std::chrono::milliseconds(1000LL * GetEnv("PS_CONNECT_TIMEOUT", 60)));
    while (!stopping()) {
      int fd = -1;
      bool ok = false;
      if (local_) {
        fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
        struct sockaddr_un addr {};
        addr.sun_family = AF_UNIX;
        strncpy(addr.sun_path, UnixPath(port).c_str(), sizeof(addr.sun_path) - 1);
        ok = fd >= 0 && connect(fd, reinterpret_cast<struct sockaddr*>(&addr), sizeof(addr)) == 0;
      } else {
        struct addrinfo hints {}, *res = nullptr;
        hints.ai_family = AF_INET;
        hints.ai_socktype = SOCK_STREAM;
        if (getaddrinfo(host.c_str(), std::to_string(port).c_str(), &hints, &res) == 0 && res) {
          fd = socket(res->ai_family, res->ai_socktype | SOCK_CLOEXEC, res->ai_protocol);
          ok = fd >= 0 && connect(fd, res->ai_addr, res->ai_addrlen) == 0;
          freeaddrinfo(res);
        }
      }
      if (ok) {
        int one = 1;
        if (!local_) setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        int buf = water > 0 ? water : (4 << 20);
        setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf, sizeof(buf));
        return fd;
      }
      if (fd >= 0) ::close(fd);
      if (std::chrono::steady_clock::now() > deadline) break;
      std::this_thread::sleep_for(std::chrono::milliseconds(20));
    }
    LOG(WARNING) << "cannot connect to " << host << ":" << port;
    return -1;
  }

  void Arm(InConn* c, InConn::Phase phase, char* dst, size_t need) {
    c->phase = phase;
    c->dst = dst;
    c->need = need;
    c->got = 0;
  }

  // Moves the connection to its next phase once the current one has all its bytes.
  // Returns false on a protocol error.
  bool Advance(InConn* c) {
    for (;;) {
      if (c->bad) return false;
      switch (c->phase) {
        case InConn::kHeader:
          // a peer that is not one of ours (or a corrupted stream) must not make this process
          // allocate without bound
          if (c->hdr.magic != kMagic || c->hdr.n_data > kMaxFrames ||
              c->hdr.meta_len > kMaxMetaBytes)
            return false;
          c->lens.assign(c->hdr.n_data, 0);
          c->msg = Message();
          c->frame = 0;
          if (c->hdr.n_data) {
            Arm(c, InConn::kLens, reinterpret_cast<char*>(c->lens.data()),
                c->hdr.n_data * sizeof(uint64_t));
            return true;
          }
          // fall through to meta
          c->phase = InConn::kLens;
          continue;
        case InConn::kLens:
          c->meta.resize(c->hdr.meta_len);
          Arm(c, InConn::kMeta, &c->meta[0], c->hdr.meta_len);
          if (c->need) return true;
          continue;
        case InConn::kMeta: {
          c->msg.meta.sender = c->hdr.sender;
          c->msg.meta.recver = c->hdr.recver;
          if (!pb::DecodeMeta(c->meta.data(), c->meta.size(), &c->msg.meta)) return false;
          c->msg.meta.sender = c->hdr.sender;
          c->msg.meta.recver = c->hdr.recver;
          c->frame = 0;
          c->phase = InConn::kData;
          if (!NextFrame(c)) return true;  // message complete (delivered)
          if (c->need) return true;
          continue;
        }
        case InConn::kData: {
          // frame `c->frame` is complete: hand its buffer to the message
          SArray<char> arr;
          if (c->frame_is_shm) {
            // the bytes stay where the sender has them: map its segment
            const uint64_t len = c->lens[c->frame] & ~kShmFrame;
            if (c->fds.empty()) return false;
            const int fd = c->fds.front();
            c->fds.pop_front();
            if (c->shm_ref.offset > c->shm_ref.seg_size ||
                len > c->shm_ref.seg_size - c->shm_ref.offset) {
              ::close(fd);
              return false;
            }
            char* base = shm::Import(fd, c->shm_ref.seg_size);
            if (!base) return false;
            arr.reset(base + c->shm_ref.offset, len, [base](char*) { shm::Release(base); });
          } else {
            std::shared_ptr<RecvPool> pool = recv_pool_;
            const size_t cap = c->frame_cap;
            arr.reset(c->frame_buf, c->lens[c->frame], [pool, cap](char* p) { pool->Put(p, cap); });
            c->frame_buf = nullptr;
          }
          c->msg.data.push_back(arr);
          ++c->frame;
          if (!NextFrame(c)) return true;
          if (c->need) return true;
          continue;
        }
      }
    }
  }

  // Arms the read of data frame c->frame, or delivers the message when none is left.
  // Returns false when the message was delivered and the connection re-armed for a header.
  bool NextFrame(InConn* c) {
    if (c->frame >= c->lens.size()) {
      size_t bytes = c->meta.size();
      for (uint64_t l : c->lens) bytes += (l & ~kShmFrame);
      c->msg.meta.data_size = static_cast<int>(bytes - c->meta.size());
      Deliver(std::move(c->msg));
      Arm(c, InConn::kHeader, reinterpret_cast<char*>(&c->hdr), sizeof(FrameHeader));
      return false;
    }
    if (c->lens[c->frame] & kShmFrame) {
      c->frame_is_shm = true;
      Arm(c, InConn::kData, reinterpret_cast<char*>(&c->shm_ref), sizeof(ShmRef));
      return true;
    }
    c->frame_is_shm = false;
    const size_t len = c->lens[c->frame];
    c->frame_buf = nullptr;
    if (len <= kMaxFrameBytes) {
      try {
        c->frame_buf = recv_pool_->Get(len, &c->frame_cap);
      } catch (const std::bad_alloc&) {
      }
    }
    if (!c->frame_buf) {
      // refuse the stream: Advance returns a protocol error on its next turn
      c->bad = true;
      Arm(c, InConn::kData, reinterpret_cast<char*>(&c->shm_ref), 0);
      return true;
    }
    Arm(c, InConn::kData, c->frame_buf, len);
    return true;
  }

  void CloseIn(int fd) {
    epoll_ctl(epfd_, EPOLL_CTL_DEL, fd, nullptr);
    ::close(fd);
    auto it = in_.find(fd);
    if (it != in_.end()) {
      delete[] it->second.frame_buf;
      for (int f : it->second.fds) ::close(f);
      in_.erase(it);
    }
  }

  // read() for a Unix socket: descriptors that ride on the bytes are queued on the connection.
  ssize_t ReadWithFds(int fd, InConn* c) {
    alignas(struct cmsghdr) char ctrl[CMSG_SPACE(sizeof(int) * kMaxFrames)];
    struct iovec iov {c->dst + c->got, c->need - c->got};
    struct msghdr mh {};
    mh.msg_iov = &iov;
    mh.msg_iovlen = 1;
    mh.msg_control = ctrl;
    mh.msg_controllen = sizeof(ctrl);
    ssize_t n = ::recvmsg(fd, &mh, MSG_CMSG_CLOEXEC);
    if (n < 0) return n;
    for (struct cmsghdr* cm = CMSG_FIRSTHDR(&mh); cm; cm = CMSG_NXTHDR(&mh, cm)) {
      if (cm->cmsg_level != SOL_SOCKET || cm->cmsg_type != SCM_RIGHTS) continue;
      const size_t cnt = (cm->cmsg_len - CMSG_LEN(0)) / sizeof(int);
      for (size_t i = 0; i < cnt; ++i) {
        int f;
        memcpy(&f, CMSG_DATA(cm) + i * sizeof(int), sizeof(int));
        c->fds.push_back(f);
      }
    }
    return n;
  }

  void OnReadable(int fd) {
    auto it = in_.find(fd);
    if (it == in_.end()) return;
    InConn* c = &it->second;
    for (;;) {
      if (c->need == c->got) {
        if (!Advance(c)) {
          LOG(WARNING) << "protocol error on an incoming connection; closing it";
          CloseIn(fd);
          return;
        }
      }
      ssize_t n = local_ ? ReadWithFds(fd, c) : ::read(fd, c->dst + c->got, c->need - c->got);
      if (n > 0) {
        c->got += static_cast<size_t>(n);
        continue;
      }
      if (n == 0) {
        CloseIn(fd);
        return;
      }
      if (errno == EINTR) continue;
      if (errno == EAGAIN || errno == EWOULDBLOCK) return;
      CloseIn(fd);
      return;
    }
  }

  void IoLoop() {
    struct epoll_event evs[64];
    while (!io_stop_.load()) {
      int n = epoll_wait(epfd_, evs, 64, 200);
      if (n < 0) {
        if (errno == EINTR) continue;
        break;
      }
      for (int i = 0; i < n; ++i) {
        const int fd = evs[i].data.fd;
        if (fd == wakefd_) {
          uint64_t v;
          ssize_t r = ::read(wakefd_, &v, sizeof(v));
          (void)r;
        } else if (fd == listen_fd_) {
          for (;;) {
            int cfd = accept4(listen_fd_, nullptr, nullptr, SOCK_NONBLOCK | SOCK_CLOEXEC);
            if (cfd < 0) break;
            int buf = 4 << 20;
            setsockopt(cfd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof(buf));
            InConn& c = in_[cfd];
            c.fd = cfd;
            Arm(&c, InConn::kHeader, reinterpret_cast<char*>(&c.hdr), sizeof(FrameHeader));
            struct epoll_event ev {};
            ev.events = EPOLLIN;
            ev.data.fd = cfd;
            epoll_ctl(epfd_, EPOLL_CTL_ADD, cfd, &ev);
          }
        } else {
          OnReadable(fd);
        }
      }
    }
  }

  bool local_ = false;
  int unix_lock_fd_ = -1;  // lock that marks this process as the owner of its Unix socket name
  std::shared_ptr<RecvPool> recv_pool_ = std::make_shared<RecvPool>();
  int epfd_ = -1, wakefd_ = -1, listen_fd_ = -1;
  std::string unix_path_;
  std::atomic<bool> io_stop_{false};
  std::unique_ptr<std::thread> io_thread_;
  std::map<int, InConn> in_;  // touched only by the I/O thread (and StopBackend after join)

  std::mutex out_mu_;
  std::unordered_map<int, std::string> id_addr_;               // node id -> "host:port"
  std::unordered_map<std::string, std::shared_ptr<OutConn>> out_;  // one path per process
};

}  // namespace

Van* NewTcpVan(bool priority) { return new TcpVan(priority); }

}  // namespace ps
