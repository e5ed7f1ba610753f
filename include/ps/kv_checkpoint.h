// Checkpoint and restore of a server's key-value store on the host plane.
//
// The reference keeps the store inside the user's request handle and offers no way to save it
// (its example handle: include/ps/kv_app.h:440-463); applications build "save model" commands
// from the `cmd` field or from SimpleApp messages.  This header supplies that piece:
//
//   * CheckpointableHandle<Val>: the summing handle of KVServerDefaultHandle with its store
//     behind a shared pointer, so that the copy that the server keeps and the object the
//     application holds are the same store; Save(path) / Load(path) write and read it.
//   * EnableCheckpointCommands(server, handle): a worker (or the scheduler) can then make every
//     server save or load with one group request,
//         kv.Wait(kv.Request(kCheckpointSave, "/some/dir", kServerGroup));
//     each server writes <dir>/server-<rank>.kv.  The command runs on the server's handler
//     thread, between two requests, so the file is a consistent cut of that server's shard.
//
// File format (little endian): magic "PSKV", u32 version 1, u32 sizeof(Val), u64 value width,
// u64 number of keys, then per key: u64 key, `width` values.
//
// The device plane has its own shard files (DenseTable.save/load, SparseTable.save/load).
#ifndef PS_KV_CHECKPOINT_H_
#define PS_KV_CHECKPOINT_H_
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "ps/kv_app.h"

namespace ps {

// Heads of the simple-app requests understood after EnableCheckpointCommands.
static const int kCheckpointSave = 0x50534b53;  // "PSKS"
static const int kCheckpointLoad = 0x50534b4c;  // "PSKL"

template <typename Val>
class CheckpointableHandle {
 public:
  struct State {
    std::unordered_map<Key, std::vector<Val>> store;
    size_t width = 0;  // values per key, fixed by the first push
  };

  CheckpointableHandle() : state_(std::make_shared<State>()) {}

  // Same contract as KVServerDefaultHandle: push adds to the stored values, pull returns them.
  void operator()(const KVMeta& req_meta, const KVPairs<Val>& req_data, KVServer<Val>* server) {
    State& st = *state_;
    const size_t n = req_data.keys.size();
    KVPairs<Val> res;
    size_t k = st.width ? st.width : 1;
    if (req_meta.push && n) {
      CHECK(req_data.lens.empty()) << "this handle takes fixed-length values";
      k = req_data.vals.size() / n;
      CHECK_EQ(k * n, req_data.vals.size());
      if (st.width == 0) st.width = k;
      CHECK_EQ(k, st.width) << "value width changed";
    }
    if (req_meta.pull) {
      res.keys = req_data.keys;
      res.vals.resize(n * k);
    }
    // A pull that comes before the first push finds no width yet: it is answered with one
    // zero per key and stores nothing, so that the first push is free to fix the width.  A
    // slot whose length differs from the width (a file written by an older layout) is
    // brought to the width before it is touched.
    const bool may_insert = req_meta.push || st.width != 0;
    for (size_t i = 0; i < n; ++i) {
      const Key key = req_data.keys[static_cast<int>(i)];
      if (!may_insert) {
        auto it = st.store.find(key);
        if (it == st.store.end()) continue;  // res.vals is zero-filled already
      }
      std::vector<Val>& slot = st.store[key];
      if (slot.size() != k) slot.resize(k, Val());
      if (req_meta.push)
        for (size_t j = 0; j < k; ++j) slot[j] += req_data.vals[static_cast<int>(i * k + j)];
      if (req_meta.pull)
        for (size_t j = 0; j < k; ++j) res.vals[static_cast<int>(i * k + j)] = slot[j];
    }
    server->Response(req_meta, res);
  }

  // Writes the store to `path` (through a temporary file, renamed when complete).
  bool Save(const std::string& path) const {
    const State& st = *state_;
    const std::string tmp = path + ".tmp";
    FILE* f = fopen(tmp.c_str(), "wb");
    if (!f) return false;
    const uint32_t version = 1, vsize = sizeof(Val);
    const uint64_t width = st.width, count = st.store.size();
    bool ok = fwrite("PSKV", 1, 4, f) == 4 && fwrite(&version, 4, 1, f) == 1 &&
              fwrite(&vsize, 4, 1, f) == 1 && fwrite(&width, 8, 1, f) == 1 &&
              fwrite(&count, 8, 1, f) == 1;
    // sorted by key: two saves of the same store give the same bytes
    std::map<Key, const std::vector<Val>*> sorted;
    for (const auto& kv : st.store) sorted[kv.first] = &kv.second;
    for (const auto& kv : sorted) {
      const uint64_t key = kv.first;
      ok = ok && fwrite(&key, 8, 1, f) == 1 && kv.second->size() == width &&
           (width == 0 || fwrite(kv.second->data(), sizeof(Val), width, f) == width);
    }
    ok = (fclose(f) == 0) && ok;
    if (!ok) {
      remove(tmp.c_str());
      return false;
    }
    return rename(tmp.c_str(), path.c_str()) == 0;
  }

  // Replaces the store by the contents of `path`; the store is untouched when the file is
  // missing, truncated or of another value type.
  bool Load(const std::string& path) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return false;
    char magic[4];
    uint32_t version = 0, vsize = 0;
    uint64_t width = 0, count = 0;
    bool ok = fread(magic, 1, 4, f) == 4 && memcmp(magic, "PSKV", 4) == 0 &&
              fread(&version, 4, 1, f) == 1 && version == 1 && fread(&vsize, 4, 1, f) == 1 &&
              vsize == sizeof(Val) && fread(&width, 8, 1, f) == 1 && fread(&count, 8, 1, f) == 1 &&
              width < (uint64_t(1) << 32);
    std::unordered_map<Key, std::vector<Val>> fresh;
    for (uint64_t i = 0; ok && i < count; ++i) {
      uint64_t key = 0;
      std::vector<Val> vals(width);
      ok = fread(&key, 8, 1, f) == 1 &&
           (width == 0 || fread(vals.data(), sizeof(Val), width, f) == width);
      if (ok) fresh[static_cast<Key>(key)] = std::move(vals);
    }
    fclose(f);
    if (!ok) return false;
    state_->store.swap(fresh);
    state_->width = width;
    return true;
  }

  size_t size() const { return state_->store.size(); }
  const State& state() const { return *state_; }

 private:
  std::shared_ptr<State> state_;
};

// File of server `rank` inside checkpoint directory `dir`.
inline std::string CheckpointFile(const std::string& dir, int rank) {
  return dir + "/server-" + std::to_string(rank) + ".kv";
}

// Makes `server` obey kCheckpointSave / kCheckpointLoad requests (body = directory).  The
// response body is "ok" or "failed".  Other simple-app requests are answered empty, as before.
template <typename Val>
void EnableCheckpointCommands(KVServer<Val>* server, CheckpointableHandle<Val> handle) {
  server->SimpleApp::set_request_handle(
      [handle](const SimpleData& req, SimpleApp* app) mutable {
        if (req.head == kCheckpointSave || req.head == kCheckpointLoad) {
          const std::string file = CheckpointFile(req.body, Postoffice::Get()->my_rank());
          const bool ok = req.head == kCheckpointSave ? handle.Save(file) : handle.Load(file);
          app->Response(req, ok ? "ok" : "failed");
        } else {
          app->Response(req);
        }
      });
}

}  // namespace ps
#endif  // PS_KV_CHECKPOINT_H_
