// SimpleApp: request/response of an (int head, string body) pair between nodes or node
// groups.  Public surface of the reference's include/ps/simple_app.h:32-182.
#ifndef PS_SIMPLE_APP_H_
#define PS_SIMPLE_APP_H_
#include <functional>
#include <memory>
#include <mutex>
#include <string>

#include "ps/internal/message.h"
#include "ps/internal/postoffice.h"

namespace ps {

// What a handler sees of a received request or response.
struct SimpleData {
  int head;
  std::string body;
  int sender;
  int timestamp;
  int customer_id;
};

class SimpleApp {
 public:
  // `app_id` must match on every node that talks to this app; `customer_id` distinguishes
  // several endpoints of the app inside one process.
  explicit SimpleApp(int app_id, int customer_id) : SimpleApp() {
    obj_ = new Customer(app_id, customer_id, [this](const Message& msg) { this->Process(msg); },
                        Customer::kWorkerSide, /*start=*/false);
    obj_->StartReceiving();  // only now: Process and Response use obj_
  }
  virtual ~SimpleApp() {
    delete obj_;
    obj_ = nullptr;
  }

  // Sends (req_head, req_body) to node or group `recv_id`; returns the request timestamp.
  virtual inline int Request(int req_head, const std::string& req_body, int recv_id) {
    Message msg;
    msg.meta.head = req_head;
    msg.meta.body = req_body;
    msg.meta.request = true;
    msg.meta.simple_app = true;
    msg.meta.app_id = obj_->app_id();
    msg.meta.customer_id = obj_->customer_id();
    const int ts = obj_->NewRequest(recv_id);
    msg.meta.timestamp = ts;
    for (int r : Postoffice::Get()->GetNodeIDs(recv_id)) {
      msg.meta.recver = r;
      Postoffice::Get()->van()->Send(msg);
    }
    return ts;
  }
  // Blocks until every recipient of request `timestamp` has responded.
  virtual inline void Wait(int timestamp) { obj_->WaitRequest(timestamp); }
  // Answers a received request.
  virtual inline void Response(const SimpleData& recv_req, const std::string& res_body = "") {
    Message msg;
    msg.meta.head = recv_req.head;
    msg.meta.body = res_body;
    msg.meta.timestamp = recv_req.timestamp;
    msg.meta.request = false;
    msg.meta.simple_app = true;
    msg.meta.app_id = obj_->app_id();
    msg.meta.customer_id = recv_req.customer_id;
    msg.meta.recver = recv_req.sender;
    msg.meta.sender = reply_from_;
    Postoffice::Get()->van()->Send(msg);
  }

  using Handle = std::function<void(const SimpleData& recved, SimpleApp* app)>;
  // Handles may be replaced while messages are already arriving (the receive thread starts
  // with the constructor): a message is served by the handle installed when it is processed.
  virtual inline void set_request_handle(const Handle& request_handle) {
    CHECK(request_handle) << "invalid request handle";
    std::lock_guard<std::mutex> lk(handle_mu_);
    request_handle_ = std::make_shared<Handle>(request_handle);
  }
  virtual inline void set_response_handle(const Handle& response_handle) {
    CHECK(response_handle) << "invalid response handle";
    std::lock_guard<std::mutex> lk(handle_mu_);
    response_handle_ = std::make_shared<Handle>(response_handle);
  }
  virtual inline Customer* get_customer() { return obj_; }

 protected:
  // For subclasses that create their own Customer.
  inline SimpleApp() : obj_(nullptr) {
    request_handle_ = std::make_shared<Handle>(
        [](const SimpleData& recved, SimpleApp* app) { app->Response(recved); });
    response_handle_ = std::make_shared<Handle>([](const SimpleData&, SimpleApp*) {});
  }
  // Dispatches a received simple-app message to the request or response handler.
  virtual inline void Process(const Message& msg) {
    SimpleData recv;
    recv.sender = msg.meta.sender;
    recv.head = msg.meta.head;
    recv.body = msg.meta.body;
    recv.timestamp = msg.meta.timestamp;
    recv.customer_id = msg.meta.customer_id;
    std::shared_ptr<Handle> handle;
    {
      std::lock_guard<std::mutex> lk(handle_mu_);
      handle = msg.meta.request ? request_handle_ : response_handle_;
    }
    CHECK(handle && *handle);
    if (msg.meta.request) {
      // a process with several node ids answers from the id that was addressed
      reply_from_ = msg.meta.recver;
      (*handle)(recv, this);
      reply_from_ = Meta::kEmpty;
    } else {
      (*handle)(recv, this);
    }
  }

  Customer* obj_;
  // id to answer from while a request handler runs (kEmpty: the van's primary id)
  int reply_from_ = Meta::kEmpty;

 private:
  std::mutex handle_mu_;
  std::shared_ptr<Handle> request_handle_;
  std::shared_ptr<Handle> response_handle_;
};

}  // namespace ps
#endif  // PS_SIMPLE_APP_H_
