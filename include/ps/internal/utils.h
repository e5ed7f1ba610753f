// Small helpers: environment lookups with defaults (reference: include/ps/internal/utils.h:
// 29-57) and the LL shorthand used by the reference's test programs.
#ifndef PS_INTERNAL_UTILS_H_
#define PS_INTERNAL_UTILS_H_
#include <cstdlib>
#include <string>

#include "ps/internal/env.h"
#include "ps/internal/logging.h"

namespace ps {

// Integer value of environment variable `name` (override map first), or `dflt`.
inline int GetEnv(const char* name, int dflt) {
  const char* v = Environment::Get()->find(name);
  return (v && *v) ? atoi(v) : dflt;
}
// String value, or `dflt`.
inline std::string GetEnv(const char* name, const std::string& dflt) {
  const char* v = Environment::Get()->find(name);
  return v ? std::string(v) : dflt;
}
inline double GetEnvDouble(const char* name, double dflt) {
  const char* v = Environment::Get()->find(name);
  return (v && *v) ? atof(v) : dflt;
}

}  // namespace ps

#ifndef LL
#define LL LOG(ERROR)
#endif
#ifndef LN
#define LN LOG(ERROR) << "  "
#endif

#endif  // PS_INTERNAL_UTILS_H_
