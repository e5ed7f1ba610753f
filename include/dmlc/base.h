// Source compatibility: programs written against the reference include "dmlc/base.h".
#ifndef DMLC_BASE_H_
#define DMLC_BASE_H_
#include "ps/internal/logging.h"
#endif
