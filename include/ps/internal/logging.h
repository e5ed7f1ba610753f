// Minimal logging and checking macros of the host runtime.
//
// Same surface as the glog-style subset the reference ships (include/dmlc/logging.h:76-142):
// LOG(severity), LOG_IF, CHECK, CHECK_{EQ,NE,LT,LE,GT,GE}, CHECK_NOTNULL, DCHECK*.  A failed
// CHECK or LOG(FATAL) throws ps::Error (aliased as dmlc::Error) carrying the message, like
// the reference built with DMLC_LOG_FATAL_THROW=1 (include/dmlc/base.h:20-22).
#ifndef PS_INTERNAL_LOGGING_H_
#define PS_INTERNAL_LOGGING_H_

#include <cstdio>
#include <sstream>
#include <stdexcept>
#include <string>

namespace ps {

struct Error : public std::runtime_error {
  explicit Error(const std::string& s) : std::runtime_error(s) {}
};

namespace log {

enum Severity { kInfo = 0, kWarning = 1, kError = 2, kFatal = 3 };

// Writes "[HH:MM:SS] file:line: text" to stderr in one write() so that lines of
// concurrently logging processes do not interleave.
void Emit(Severity sev, const char* file, int line, const std::string& text);
// Text of the current call stack (best effort; empty if unavailable).
std::string StackTrace(int skip);

class Line {
 public:
  Line(Severity sev, const char* file, int line) : sev_(sev), file_(file), line_(line) {}
  ~Line() noexcept(false) {
    if (sev_ == kFatal) {
      std::string what = os_.str();
      Emit(sev_, file_, line_, what);
      throw Error(std::string(file_) + ":" + std::to_string(line_) + ": " + what + "\n" +
                  StackTrace(2));
    }
    Emit(sev_, file_, line_, os_.str());
  }
  std::ostringstream& stream() { return os_; }

 private:
  Severity sev_;
  const char* file_;
  int line_;
  std::ostringstream os_;
};

// Turns "cond ? (void)0 : Voidify() & stream" into a statement of type void.
struct Voidify {
  void operator&(std::ostream&) {}
};

template <typename A, typename B>
inline std::string* CheckFailText(const A& a, const B& b, const char* expr) {
  std::ostringstream os;
  os << "Check failed: " << expr << " (" << a << " vs. " << b << ") ";
  return new std::string(os.str());
}

// Holder that is "true" when the check passed (so the macro can use if/else with a
// declaration as the condition, which C++11 has).
struct CheckResult {
  std::string* text;
  explicit CheckResult(std::string* t) : text(t) {}
  CheckResult(CheckResult&& o) : text(o.text) { o.text = nullptr; }
  CheckResult(const CheckResult&) = delete;
  CheckResult& operator=(const CheckResult&) = delete;
  ~CheckResult() { delete text; }
  explicit operator bool() const { return text == nullptr; }
};

#define PS_DEFINE_CHECK_OP(name, op)                                            \
  template <typename A, typename B>                                             \
  inline CheckResult Check##name(const A& a, const B& b, const char* expr) {    \
    if (a op b) return CheckResult(nullptr);                                    \
    return CheckResult(CheckFailText(a, b, expr));                              \
  }                                                                             \
  inline CheckResult Check##name(int a, int b, const char* expr) {              \
    return Check##name<int, int>(a, b, expr);                                   \
  }
PS_DEFINE_CHECK_OP(EQ, ==)
PS_DEFINE_CHECK_OP(NE, !=)
PS_DEFINE_CHECK_OP(LT, <)
PS_DEFINE_CHECK_OP(LE, <=)
PS_DEFINE_CHECK_OP(GT, >)
PS_DEFINE_CHECK_OP(GE, >=)
#undef PS_DEFINE_CHECK_OP

}  // namespace log
}  // namespace ps

namespace dmlc {
using Error = ::ps::Error;
}

#define PS_LOG_INFO ::ps::log::Line(::ps::log::kInfo, __FILE__, __LINE__)
#define PS_LOG_WARNING ::ps::log::Line(::ps::log::kWarning, __FILE__, __LINE__)
#define PS_LOG_ERROR ::ps::log::Line(::ps::log::kError, __FILE__, __LINE__)
#define PS_LOG_FATAL ::ps::log::Line(::ps::log::kFatal, __FILE__, __LINE__)

#define PS_LOG_QFATAL PS_LOG_FATAL
#ifdef NDEBUG
#define PS_LOG_DFATAL PS_LOG_ERROR
#else
#define PS_LOG_DFATAL PS_LOG_FATAL
#endif

#ifndef LOG
#define LOG(severity) PS_LOG_##severity.stream()
#define LOG_IF(severity, cond) \
  !(cond) ? (void)0 : ::ps::log::Voidify() & LOG(severity)
// the other logging macros that programs written for the reference may use
#define LG LOG(INFO)
#define VLOG(level) LOG(INFO)
#define LOG_EVERY_N(severity, n) LOG(severity)
#ifdef NDEBUG
#define DLOG(severity) LOG_IF(severity, false)
#define DLOG_IF(severity, cond) LOG_IF(severity, false)
#else
#define DLOG(severity) LOG(severity)
#define DLOG_IF(severity, cond) LOG_IF(severity, cond)
#endif
#define CHECK(x) \
  if (x) {    \
  } else      \
    PS_LOG_FATAL.stream() << "Check failed: " #x << ' '
#define PS_CHECK_OP(name, op, a, b)                                                   \
  if (::ps::log::CheckResult _ps_cr =                                                 \
          ::ps::log::Check##name((a), (b), #a " " #op " " #b)) {                      \
  } else                                                                              \
    PS_LOG_FATAL.stream() << *_ps_cr.text
#define CHECK_EQ(a, b) PS_CHECK_OP(EQ, ==, a, b)
#define CHECK_NE(a, b) PS_CHECK_OP(NE, !=, a, b)
#define CHECK_LT(a, b) PS_CHECK_OP(LT, <, a, b)
#define CHECK_LE(a, b) PS_CHECK_OP(LE, <=, a, b)
#define CHECK_GT(a, b) PS_CHECK_OP(GT, >, a, b)
#define CHECK_GE(a, b) PS_CHECK_OP(GE, >=, a, b)
#define CHECK_NOTNULL(x) \
  ((x) == nullptr ? (PS_LOG_FATAL.stream() << "Check notnull: " #x << ' ', (x)) : (x))
#ifdef NDEBUG
#define DCHECK(x) while (false) CHECK(x)
#define DCHECK_EQ(a, b) while (false) CHECK_EQ(a, b)
#define DCHECK_NE(a, b) while (false) CHECK_NE(a, b)
#define DCHECK_LT(a, b) while (false) CHECK_LT(a, b)
#define DCHECK_LE(a, b) while (false) CHECK_LE(a, b)
#define DCHECK_GT(a, b) while (false) CHECK_GT(a, b)
#define DCHECK_GE(a, b) while (false) CHECK_GE(a, b)
#else
#define DCHECK(x) CHECK(x)
#define DCHECK_EQ(a, b) CHECK_EQ(a, b)
#define DCHECK_NE(a, b) CHECK_NE(a, b)
#define DCHECK_LT(a, b) CHECK_LT(a, b)
#define DCHECK_LE(a, b) CHECK_LE(a, b)
#define DCHECK_GT(a, b) CHECK_GT(a, b)
#define DCHECK_GE(a, b) CHECK_GE(a, b)
#endif
#endif  // LOG

#ifndef DISALLOW_COPY_AND_ASSIGN
#define DISALLOW_COPY_AND_ASSIGN(T) \
  T(const T&) = delete;             \
  void operator=(const T&) = delete
#endif

#endif  // PS_INTERNAL_LOGGING_H_
