// Cross-process test of the descriptor channel (no GPU, no CUDA): a child process asks the
// parent's FdServer for the read end of a pipe and must receive, through the descriptor it was
// handed, the bytes that the parent writes into the pipe. Exit code 0 = pass.
//
// Build: g++ -std=c++17 -pthread -I torch_dist_ext_b200/csrc/include tests/cpp/fd_channel_test.cpp
//        torch_dist_ext_b200/csrc/fd_channel.cpp -o fd_channel_test   (the CPU test suite does this)
#include <sys/wait.h>
#include <unistd.h>
#include <cstdio>
#include <cstring>
#include "tdx/fd_channel.h"

static int fail(const char* what) {
  std::fprintf(stderr, "fd_channel_test: %s\n", what);
  return 1;
}

int main() {
  int data[2], name_pipe[2];
  if (pipe(data) != 0 || pipe(name_pipe) != 0) return fail("pipe");
  const pid_t child = fork();   // before any thread exists in this process
  if (child < 0) return fail("fork");
  if (child == 0) {
    close(data[0]);
    close(data[1]);            // the child keeps NO inherited end of the data pipe
    close(name_pipe[1]);
    char name[64] = {};
    if (read(name_pipe[0], name, sizeof(name) - 1) <= 0) _exit(10);
    if (tdx::request_fd(name, 'z', 2, 10) != -1) _exit(11);        // nothing offered under this key
    const int fd = tdx::request_fd(name, 'p');
    if (fd < 0) _exit(12);
    char buf[16] = {};
    if (read(fd, buf, 5) != 5 || std::memcmp(buf, "hello", 5) != 0) _exit(13);
    _exit(0);
  }
  close(name_pipe[0]);
  if (tdx::request_fd("tdx-b200-no-such-server", 'p', 2, 10) != -1) return fail("request to a missing server succeeded");
  tdx::FdServer server;
  if (server.name()[0] != 0) return fail("name before start");
  server.offer('p', data[0]);
  if (!server.start("test")) return fail("start");
  if (std::strlen(server.name()) == 0 || std::strlen(server.name()) > 63) return fail("name length");
  if (write(name_pipe[1], server.name(), std::strlen(server.name())) <= 0) return fail("send name");
  close(name_pipe[1]);
  if (write(data[1], "hello", 5) != 5) return fail("write");
  int status = 0;
  if (waitpid(child, &status, 0) != child) return fail("waitpid");
  server.stop();
  server.stop();   // idempotent
  if (!WIFEXITED(status) || WEXITSTATUS(status) != 0) {
    std::fprintf(stderr, "fd_channel_test: child exit status %d\n", WIFEXITED(status) ? WEXITSTATUS(status) : -1);
    return 1;
  }
  std::printf("fd_channel_test: ok\n");
  return 0;
}
