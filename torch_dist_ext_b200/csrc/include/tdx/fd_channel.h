// File descriptors handed from one process to another over an abstract Unix-domain socket
// (SCM_RIGHTS). The workspace manager uses it to share the POSIX-fd handles of cuMemCreate
// allocations and of the multicast object between the ranks of one node; nothing here depends on
// CUDA, so the channel is tested on its own (tests/cpp/fd_channel_test.cpp).
//
// The reference shares memory through cudaIpc handles only (src/ops/all_reduce_fusion.cpp:75-141),
// which are plain bytes; fd-based handles need a channel like this one.
#pragma once
#include <atomic>
#include <thread>

namespace tdx {

// Serves descriptors, looked up by a one-character key, to every process that connects.
class FdServer {
 public:
  FdServer();
  ~FdServer();   // stops the thread and closes the socket; the offered descriptors stay open
  FdServer(const FdServer&) = delete;
  FdServer& operator=(const FdServer&) = delete;

  // Descriptor handed out for `key` (-1 withdraws it). May be called before or after start().
  void offer(char key, int fd);
  // Binds a socket with a fresh name that contains `tag` and starts the serving thread.
  bool start(const char* tag);
  void stop();
  // Name to pass to request_fd (empty before start()); at most 63 characters.
  const char* name() const { return name_; }

 private:
  void serve();
  char name_[64];
  int listen_fd_;
  std::thread thread_;
  std::atomic<bool> stop_;
  std::atomic<int> fds_[256];
};

// Connects to the server called `name` and returns its descriptor for `key` as a new descriptor
// of the calling process, or -1 (no such server after `attempts` tries `retry_ms` apart, or no
// descriptor offered under that key).
int request_fd(const char* name, char key, int attempts = 200, int retry_ms = 25);

}  // namespace tdx
