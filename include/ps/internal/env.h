// Process-wide configuration lookup: an optional override map consulted before getenv.
// Reference: include/ps/internal/env.h:20-49 (Environment::Get/Init/find).
#ifndef PS_INTERNAL_ENV_H_
#define PS_INTERNAL_ENV_H_
#include <cstdlib>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>

namespace ps {

class Environment {
 public:
  // The singleton.  The first call may install an override map (see Init).
  static Environment* Get() { return Holder(nullptr).get(); }
  // Shared reference (keeps the singleton alive for objects that outlive main).
  static std::shared_ptr<Environment> _GetSharedRef() { return Holder(nullptr); }
  // Installs `envs` as overrides.  Only the first Init/Get in a process takes effect for
  // creation; later Init calls merge into the existing map.
  static Environment* Init(const std::unordered_map<std::string, std::string>& envs) {
    Environment* e = Holder(&envs).get();
    std::lock_guard<std::mutex> lk(e->mu_);
    for (const auto& kv : envs) e->kvs_[kv.first] = kv.second;
    return e;
  }
  // Override value if present, else getenv, else nullptr.
  const char* find(const char* k) {
    {
      std::lock_guard<std::mutex> lk(mu_);
      auto it = kvs_.find(k);
      if (it != kvs_.end()) return it->second.c_str();
    }
    return getenv(k);
  }
  // Set or replace one override (used by the van to export DMLC_RANK).
  void set(const std::string& k, const std::string& v) {
    std::lock_guard<std::mutex> lk(mu_);
    kvs_[k] = v;
  }

 private:
  Environment() = default;
  static std::shared_ptr<Environment>& Holder(
      const std::unordered_map<std::string, std::string>* envs) {
    static std::shared_ptr<Environment> inst(new Environment());
    (void)envs;
    return inst;
  }
  std::mutex mu_;
  std::unordered_map<std::string, std::string> kvs_;
};

}  // namespace ps
#endif  // PS_INTERNAL_ENV_H_
