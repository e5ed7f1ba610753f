// Address helpers for the socket van (role of the reference's src/network_utils.h:28-255).
#ifndef PS_VAN_NETWORK_UTILS_H_
#define PS_VAN_NETWORK_UTILS_H_
#include <string>

namespace ps {
namespace net {
// IPv4 address of interface `name`, or "" if it has none.
std::string IpOfInterface(const std::string& name);
// IPv4 address of the first interface that is up and not loopback, or "".
std::string FirstNonLoopbackIp();
// A TCP port that was free a moment ago (bind to port 0, read it back), or 0.
int FreePort();
}  // namespace net
}  // namespace ps
#endif  // PS_VAN_NETWORK_UTILS_H_
