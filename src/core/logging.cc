#include "ps/internal/logging.h"

#include <execinfo.h>
#include <time.h>
#include <unistd.h>

#include <cstdlib>
#include <cstring>

namespace ps {
namespace log {

void Emit(Severity sev, const char* file, int line, const std::string& text) {
  (void)sev;
  time_t now = time(nullptr);
  struct tm tmv;
  localtime_r(&now, &tmv);
  char head[64];
  snprintf(head, sizeof(head), "[%02d:%02d:%02d] ", tmv.tm_hour, tmv.tm_min, tmv.tm_sec);
  std::string out;
  out.reserve(text.size() + 96);
  out.append(head).append(file).append(":").append(std::to_string(line)).append(": ");
  out.append(text).append("\n");
  ssize_t r = ::write(STDERR_FILENO, out.data(), out.size());
  (void)r;
}

std::string StackTrace(int skip) {
  void* frames[32];
  int n = backtrace(frames, 32);
  if (n <= skip) return std::string();
  char** names = backtrace_symbols(frames, n);
  if (!names) return std::string();
  std::string s = "Stack trace:\n";
  for (int i = skip; i < n; ++i) {
    s += "  ";
    s += names[i];
    s += "\n";
  }
  free(names);
  return s;
}

}  // namespace log
}  // namespace ps
