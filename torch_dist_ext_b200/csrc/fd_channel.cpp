// Descriptor passing between the processes of one node; see tdx/fd_channel.h.
#include "tdx/fd_channel.h"
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>
#include <chrono>
#include <cstddef>
#include <cstdio>
#include <cstring>

namespace tdx {
namespace {

socklen_t abstract_addr(sockaddr_un* addr, const char* name) {
  std::memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  size_t n = std::strlen(name);
  if (n > sizeof(addr->sun_path) - 2) n = sizeof(addr->sun_path) - 2;
  std::memcpy(addr->sun_path + 1, name, n);  // sun_path[0] == 0: abstract namespace, no file to clean up
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

bool send_fd(int sock, int fd) {
  char byte = 'f';
  iovec iov{&byte, 1};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))] = {};
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
  return sendmsg(sock, &msg, MSG_NOSIGNAL) == 1;
}

int recv_fd(int sock) {
  char byte = 0;
  iovec iov{&byte, 1};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))] = {};
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  if (recvmsg(sock, &msg, 0) != 1) return -1;
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  if (c == nullptr || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) return -1;
  int fd = -1;
  std::memcpy(&fd, CMSG_DATA(c), sizeof(int));
  return fd;
}

}  // namespace

FdServer::FdServer() : listen_fd_(-1), stop_(false) {
  name_[0] = 0;
  for (auto& f : fds_) f.store(-1);
}

FdServer::~FdServer() { stop(); }

void FdServer::offer(char key, int fd) { fds_[(unsigned char)key].store(fd); }

bool FdServer::start(const char* tag) {
  if (listen_fd_ >= 0) return true;
  std::snprintf(name_, sizeof(name_), "tdx-b200-%d-%.16s-%llx", (int)getpid(), tag,
                (unsigned long long)std::chrono::steady_clock::now().time_since_epoch().count());
  listen_fd_ = socket(AF_UNIX, SOCK_STREAM, 0);
  sockaddr_un addr;
  const socklen_t len = abstract_addr(&addr, name_);
  if (listen_fd_ < 0 || bind(listen_fd_, reinterpret_cast<sockaddr*>(&addr), len) != 0 || listen(listen_fd_, 32) != 0) {
    if (listen_fd_ >= 0) close(listen_fd_);
    listen_fd_ = -1;
    name_[0] = 0;
    return false;
  }
  stop_.store(false);
  thread_ = std::thread([this] { serve(); });
  return true;
}

void FdServer::stop() {
  stop_.store(true);
  if (thread_.joinable()) thread_.join();
  if (listen_fd_ >= 0) close(listen_fd_);
  listen_fd_ = -1;
}

void FdServer::serve() {
  while (!stop_.load()) {
    pollfd p{listen_fd_, POLLIN, 0};
    if (poll(&p, 1, 100) <= 0) continue;
    const int c = accept(listen_fd_, nullptr, nullptr);
    if (c < 0) continue;
    // a client that connects and then says nothing must not stall the others
    pollfd q{c, POLLIN, 0};
    char key = 0;
    if (poll(&q, 1, 1000) > 0 && read(c, &key, 1) == 1) {
      const int fd = fds_[(unsigned char)key].load();
      if (fd >= 0) send_fd(c, fd);
    }
    close(c);
  }
}

int request_fd(const char* name, char key, int attempts, int retry_ms) {
  sockaddr_un addr;
  const socklen_t len = abstract_addr(&addr, name);
  for (int attempt = 0; attempt < attempts; ++attempt) {
    const int s = socket(AF_UNIX, SOCK_STREAM, 0);
    if (s < 0) return -1;
    if (connect(s, reinterpret_cast<sockaddr*>(&addr), len) == 0) {
      int fd = -1;
      if (write(s, &key, 1) == 1) fd = recv_fd(s);
      close(s);
      return fd;
    }
    close(s);
    std::this_thread::sleep_for(std::chrono::milliseconds(retry_ms));
  }
  return -1;
}

}  // namespace tdx
