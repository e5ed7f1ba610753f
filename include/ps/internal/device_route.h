// Hook through which key-value requests on device-resident tensors leave the message path.
//
// In the reference every byte of a push or pull goes KVWorker::Send -> slicer -> Van::Send
// (include/ps/kv_app.h:574-613).  Here a request whose keys name a tensor that was registered
// with the device plane is handed to that plane instead: the transfer, the reduction over
// workers and the server handle run as kernels over NVLink (src/van/nvl_van.cc), and the
// plane's completion thread credits the request in the Customer's tracker, so that
// timestamps, callbacks and Wait() behave exactly as for message traffic.
//
// This header belongs to the host library and knows nothing about CUDA.
#ifndef PS_INTERNAL_DEVICE_ROUTE_H_
#define PS_INTERNAL_DEVICE_ROUTE_H_
#include <functional>

#include "ps/base.h"
#include "ps/sarray.h"

namespace ps {

class Customer;

// One key-value request as the device plane sees it.  `vals` / `outs` are raw bytes of the
// worker's value type; either may live in host or device memory (the plane finds out).
struct DeviceRequest {
  int app_id = 0;
  int timestamp = 0;
  bool push = false;
  bool pull = false;
  int cmd = 0;
  int priority = 0;
  SArray<Key> keys;        // sorted, unique; host memory, or device memory for keyed tables
  SArray<int> lens;        // optional: values per key (host memory)
  const void* vals = nullptr;  // pushed values (push)
  size_t vals_bytes = 0;
  void* outs = nullptr;        // where pulled values go (pull); nullptr: the table's own buffer
  size_t outs_bytes = 0;
  int* lens_out = nullptr;     // pull: per-key value counts are written here when not null
  size_t lens_out_n = 0;
  size_t val_size = 4;         // sizeof(Val) of the KVWorker
  Customer* customer = nullptr;
  int responses = 1;           // what the tracker expects for this timestamp
  std::function<void()> on_done;  // runs before the request is credited (user callback)
};

class DeviceRoute {
 public:
  virtual ~DeviceRoute() {}
  // True when the plane serves these keys (a tensor registered under keys[0] for this app,
  // or a keyed table of this app when the keys are device-resident).
  virtual bool Claims(int app_id, const SArray<Key>& keys) = 0;
  // Bytes that a pull of `keys` returns (0 when unknown): lets a worker size an empty output.
  virtual size_t PullBytes(int app_id, const SArray<Key>& keys) = 0;
  // Takes the request; completion is reported through req.customer (AddResponse, or
  // FailRequest when a device-side wait ran out).
  virtual void Submit(const DeviceRequest& req) = 0;
};

}  // namespace ps
#endif  // PS_INTERNAL_DEVICE_ROUTE_H_
