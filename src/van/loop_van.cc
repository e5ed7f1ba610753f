// In-process van: one process plays scheduler, server 0 and worker 0.  Every message is
// addressed to one of the process's own ids and is handed straight to the receive loop, so
// the full runtime (Postoffice, Customer, KVWorker/KVServer, SimpleApp) can be exercised
// without sockets or a launcher.  The reference has no such backend: its tests always start
// one OS process per role (tests/local.sh:8-37).
#include "van/backends.h"

namespace ps {
namespace {

class LoopVan : public Van {
 protected:
  bool IsStandalone() const override { return true; }
  void Connect(const Node&) override {}
  int Bind(const Node& node, int) override { return node.port; }
  int SendMsg(const Message& msg) override {
    LOG(WARNING) << "the loop van has no remote nodes; cannot reach node " << msg.meta.recver;
    return -1;
  }
};

}  // namespace

Van* NewLoopVan() { return new LoopVan(); }

}  // namespace ps
