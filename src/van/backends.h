// Constructors of the van backends (defined in tcp_van.cc and loop_van.cc).
#ifndef PS_VAN_BACKENDS_H_
#define PS_VAN_BACKENDS_H_
#include "ps/internal/van.h"

namespace ps {
// TCP (or Unix-domain, with DMLC_LOCAL=1) sockets driven by one epoll thread.
// `priority` enables the priority send queue (van type "p3").
Van* NewTcpVan(bool priority);
// Single-process van: the process is scheduler, server 0 and worker 0; no sockets.
Van* NewLoopVan();
}  // namespace ps
#endif  // PS_VAN_BACKENDS_H_
