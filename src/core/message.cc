#include "ps/internal/message.h"

#include <sstream>

namespace ps {

const int Node::kEmpty = kEmptyField;
const int Meta::kEmpty = kEmptyField;

static const char* RoleName(Node::Role r) {
  switch (r) {
    case Node::SERVER: return "server";
    case Node::WORKER: return "worker";
    case Node::SCHEDULER: return "scheduler";
    case Node::JOINT: return "joint";
  }
  return "?";
}

std::string Node::DebugString() const {
  std::ostringstream os;
  os << "role=" << RoleName(role);
  if (id != kEmpty) os << ", id=" << id;
  os << ", ip=" << hostname << ", port=" << port << ", is_recovery=" << is_recovery;
  return os.str();
}

std::string Node::ShortDebugString() const {
  std::ostringstream os;
  os << "SWHJ"[static_cast<int>(role)];
  if (id != kEmpty) os << "[" << id << "]";
  return os.str();
}

std::string Control::DebugString() const {
  if (empty()) return "";
  static const char* names[] = {"EMPTY", "TERMINATE", "ADD_NODE", "BARRIER", "ACK", "HEARTBEAT"};
  std::ostringstream os;
  os << "cmd=" << names[cmd];
  if (!node.empty()) {
    os << ", node={";
    for (const Node& n : node) os << " " << n.DebugString();
    os << " }";
  }
  if (cmd == BARRIER) os << ", barrier_group=" << barrier_group;
  if (cmd == ACK) os << ", msg_sig=" << msg_sig;
  return os.str();
}

std::string Meta::DebugString() const {
  std::ostringstream os;
  if (sender == kEmpty) os << "?"; else os << sender;
  os << " => " << recver << ". Meta: request=" << request;
  if (timestamp != kEmpty) os << ", timestamp=" << timestamp;
  if (!control.empty()) {
    os << ", control={ " << control.DebugString() << " }";
  } else {
    os << ", app_id=" << app_id << ", customer_id=" << customer_id
       << ", simple_app=" << simple_app << ", push=" << push << ", pull=" << pull;
  }
  if (head != kEmpty) os << ", head=" << head;
  if (!body.empty()) os << ", body=" << body;
  if (!data_type.empty()) {
    os << ", data_type={";
    for (DataType d : data_type) os << " " << DataTypeName[static_cast<int>(d)];
    os << " }";
  }
  if (priority) os << ", priority=" << priority;
  return os.str();
}

std::string Message::DebugString() const {
  std::ostringstream os;
  os << meta.DebugString();
  if (!data.empty()) {
    os << " Body: data_size=";
    for (const auto& d : data) os << " " << d.size();
  }
  return os.str();
}

}  // namespace ps
