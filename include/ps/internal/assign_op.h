// Assignment operators `dst op= src` selectable at run time.  The reference declares the same
// set (include/ps/internal/assign_op.h:12-21) but its AssignFunc does not compile; this one
// does, and the device kernels in src/kernels/sort_match.cu use the same numbering.
#ifndef PS_INTERNAL_ASSIGN_OP_H_
#define PS_INTERNAL_ASSIGN_OP_H_
#include <type_traits>

#include "ps/internal/logging.h"

namespace ps {

enum AssignOp { ASSIGN, PLUS, MINUS, TIMES, DIVIDE, AND, OR, XOR };

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
      if constexpr (std::is_integral<T>::value) {
        if (op == AND) *dst &= src;
        else if (op == OR) *dst |= src;
        else *dst ^= src;
      } else {
        LOG(FATAL) << "bitwise assignment on a non-integral type";
      }
      break;
  }
}

}  // namespace ps
#endif  // PS_INTERNAL_ASSIGN_OP_H_
