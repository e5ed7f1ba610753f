#include "van/network_utils.h"

#include <arpa/inet.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netinet/in.h>
#include <sys/socket.h>
#include <unistd.h>

namespace ps {
namespace net {

static std::string Scan(const std::string* want_name) {
  struct ifaddrs* list = nullptr;
  if (getifaddrs(&list) != 0) return std::string();
  std::string found;
  for (struct ifaddrs* it = list; it; it = it->ifa_next) {
    if (!it->ifa_addr || it->ifa_addr->sa_family != AF_INET) continue;
    if (want_name) {
      if (*want_name != it->ifa_name) continue;
    } else {
      if ((it->ifa_flags & IFF_LOOPBACK) || !(it->ifa_flags & IFF_UP)) continue;
    }
    char buf[INET_ADDRSTRLEN];
    auto* sin = reinterpret_cast<struct sockaddr_in*>(it->ifa_addr);
    if (inet_ntop(AF_INET, &sin->sin_addr, buf, sizeof(buf))) {
      found = buf;
      break;
    }
  }
  freeifaddrs(list);
  return found;
}

std::string IpOfInterface(const std::string& name) { return Scan(&name); }
std::string FirstNonLoopbackIp() { return Scan(nullptr); }

int FreePort() {
  int fd = socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return 0;
  struct sockaddr_in addr {};
  addr.sin_family = AF_INET;
  addr.sin_addr.s_addr = htonl(INADDR_ANY);
  addr.sin_port = 0;
  int port = 0;
  if (bind(fd, reinterpret_cast<struct sockaddr*>(&addr), sizeof(addr)) == 0) {
    socklen_t len = sizeof(addr);
    if (getsockname(fd, reinterpret_cast<struct sockaddr*>(&addr), &len) == 0)
      port = ntohs(addr.sin_port);
  }
  close(fd);
  return port;
}

}  // namespace net
}  // namespace ps
