// Assignment operators `dst op= src` selectable at run time.  The reference declares the same
// set (include/ps/internal/assign_op.h:12-21) but its AssignFunc does not compile; this one
// does, and the device kernels in src/kernels/sort_match.cu use the same numbering.
#ifndef PS_INTERNAL_ASSIGN_OP_H_
#define PS_INTERNAL_ASSIGN_OP_H_
#include <type_traits>

#include "ps/internal/logging.h"

namespace ps {

enum AssignOp { ASSIGN, PLUS, MINUS, TIMES, DIVIDE, AND, OR, XOR };

namespace detail {
// Bitwise operators exist for integral types only; the choice is made by overload on a tag so
// that the header needs nothing newer than C++11.
template <typename T>
inline void BitwiseAssign(const T& src, AssignOp op, T* dst, std::true_type) {
  if (op == AND) *dst &= src;
  else if (op == OR) *dst |= src;
  else *dst ^= src;
}
template <typename T>
inline void BitwiseAssign(const T&, AssignOp, T*, std::false_type) {
  LOG(FATAL) << "bitwise assignment on a non-integral type";
}
}  // namespace detail

// Applies `op` to one element.  Bitwise operators are defined for integral types only.
template <typename T>
inline void AssignFunc(const T& src, AssignOp op, T* dst) {
  switch (op) {
    case ASSIGN: *dst = src; break;
    case PLUS: *dst += src; break;
    case MINUS: *dst -= src; break;
    case TIMES: *dst *= src; break;
    case DIVIDE: *dst /= src; break;
    case AND:
    case OR:
    case XOR:
      detail::BitwiseAssign(src, op, dst, typename std::is_integral<T>::type());
      break;
  }
}

}  // namespace ps
#endif  // PS_INTERNAL_ASSIGN_OP_H_
