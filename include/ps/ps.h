// The primary interface of the parameter server (same free functions as the reference's
// include/ps/ps.h:16-75).
#ifndef PS_PS_H_
#define PS_PS_H_
#include "ps/base.h"
#include "ps/kv_app.h"
#include "ps/simple_app.h"

namespace ps {

// Number of worker / server nodes in the job.
inline int NumWorkers() { return Postoffice::Get()->num_workers(); }
inline int NumServers() { return Postoffice::Get()->num_servers(); }
// Role of this process.  A process started with DMLC_ROLE=joint is a worker and a server.
inline bool IsWorker() { return Postoffice::Get()->is_worker(); }
inline bool IsServer() { return Postoffice::Get()->is_server(); }
inline bool IsScheduler() { return Postoffice::Get()->is_scheduler(); }
// Rank of this node within its group, in [0, NumWorkers()) or [0, NumServers()).
inline int MyRank() { return Postoffice::Get()->my_rank(); }

// Starts the system and blocks until every node has started.
inline void Start(int customer_id, const char* argv0 = nullptr) {
  Postoffice::Get()->Start(customer_id, argv0, true);
}
// Starts the system without waiting for the other nodes.
inline void StartAsync(int customer_id, const char* argv0 = nullptr) {
  Postoffice::Get()->Start(customer_id, argv0, false);
}
// Stops the system; with do_barrier it first waits until every node is ready to stop.
inline void Finalize(int customer_id, const bool do_barrier = true) {
  Postoffice::Get()->Finalize(customer_id, do_barrier);
}
// Registers a function that runs at the end of Finalize (typically: delete the server app).
inline void RegisterExitCallback(const std::function<void()>& cb) {
  Postoffice::Get()->RegisterExitCallback(cb);
}

}  // namespace ps
#endif  // PS_PS_H_
