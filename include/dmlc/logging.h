// Source compatibility: programs written against the reference include "dmlc/logging.h".
#ifndef DMLC_LOGGING_H_
#define DMLC_LOGGING_H_
#include "ps/internal/logging.h"
#endif
