// Syntax check of the helper headers that no test program includes otherwise: the assignment
// operators, the parallel sort and the ordered match (reference: include/ps/internal/
// assign_op.h, parallel_sort.h, parallel_kv_match.h) must build with the same language
// standard as the rest of the public headers.
#include "ps/internal/assign_op.h"
#include "ps/internal/message.h"
#include "ps/internal/parallel_kv_match.h"
#include "ps/internal/parallel_sort.h"

int main() {
  float a = 1.f, b = 2.f;
  ps::AssignFunc(a, ps::PLUS, &b);
  int x = 1, y = 3;
  ps::AssignFunc(x, ps::XOR, &y);
  ps::SArray<int> keys({3, 1, 2});
  ps::ParallelSort(&keys, 2);
  // the logging macros and small helpers that programs written for the reference may use
  LG << "plain";
  VLOG(2) << "verbose";
  DLOG(INFO) << "debug";
  DLOG_IF(INFO, x == 1) << "debug if";
  LOG_EVERY_N(INFO, 10) << "every n";
  LOG_IF(WARNING, false) << "never";
  DCHECK_EQ(x, 1);
  const bool same = ps::SameType<const float, float>() && !ps::SameType<int, float>();
  return (b == 3.f && y == 2 && same) ? 0 : 1;
}
