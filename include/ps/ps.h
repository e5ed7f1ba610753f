// Entry points of the library: start and stop the node, ask who it is.
//
// The names and meanings are those of the reference (include/ps/ps.h:16-75), so a program
// written for it compiles unchanged; everything here forwards to the process-wide Postoffice.
// Additions: DMLC_ROLE=joint makes a process worker and server at once (both role queries are
// true then), and a process may call Start again after Finalize.
#ifndef PS_PS_H_
#define PS_PS_H_
#include <functional>

#include "ps/base.h"
#include "ps/kv_app.h"
#include "ps/simple_app.h"

namespace ps {
namespace detail {
inline Postoffice& Office() { return *Postoffice::Get(); }
}  // namespace detail

// ---- life cycle --------------------------------------------------------------------------
// Start: reads the DMLC_* environment, binds, registers with the scheduler and returns once
// every node of the job has done the same.  StartAsync returns without that last barrier.
// `argv0` only labels the log lines.
inline void Start(int customer_id, const char* argv0 = nullptr) {
  detail::Office().Start(customer_id, argv0, /*do_barrier=*/true);
}
inline void StartAsync(int customer_id, const char* argv0 = nullptr) {
  detail::Office().Start(customer_id, argv0, /*do_barrier=*/false);
}
// Finalize: with `do_barrier`, first waits until every node is ready to stop; customer 0
// then shuts the van down and the exit callback runs.
inline void Finalize(int customer_id, const bool do_barrier = true) {
  detail::Office().Finalize(customer_id, do_barrier);
}
// `cb` runs at the very end of Finalize, after the van has stopped -- the place to delete a
// server application that must outlive the last request.
inline void RegisterExitCallback(const std::function<void()>& cb) {
  detail::Office().RegisterExitCallback(cb);
}

// ---- who am I ----------------------------------------------------------------------------
inline bool IsScheduler() { return detail::Office().is_scheduler(); }
inline bool IsServer() { return detail::Office().is_server(); }
inline bool IsWorker() { return detail::Office().is_worker(); }
// Position inside the own group: [0, NumServers()) for a server, [0, NumWorkers()) for a worker.
inline int MyRank() { return detail::Office().my_rank(); }

// ---- size of the job ---------------------------------------------------------------------
inline int NumServers() { return detail::Office().num_servers(); }
inline int NumWorkers() { return detail::Office().num_workers(); }

}  // namespace ps
#endif  // PS_PS_H_
