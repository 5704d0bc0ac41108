// Unix-domain socket helpers for the control channel: SOCK_SEQPACKET connections
// (message boundaries kept, peer death seen as EOF), peer credentials, and file
// descriptor passing with SCM_RIGHTS. The reference does the same jobs over datagram
// sockets (src/ipc/core/src/unix.rs:41-257).
#pragma once
#include <stddef.h>
#include <sys/types.h>

#include <string>
#include <vector>

namespace mccs {
namespace ipc {

constexpr int kMaxFdsPerMessage = 4;

struct PeerCred { pid_t pid; uid_t uid; gid_t gid; };

// All functions return >= 0 on success and -errno on failure unless stated otherwise.
int uds_listen(const std::string& path, int backlog = 64);     // returns listening fd
int uds_connect(const std::string& path);                      // returns connected fd
int uds_accept(int listen_fd);                                 // non-blocking accept; -EAGAIN when none
int uds_peer_cred(int fd, PeerCred* out);
int set_nonblocking(int fd, bool on);

// Sends one message with optional fds. Returns bytes sent.
ssize_t uds_send(int fd, const void* data, size_t len, const int* fds = nullptr, int nfds = 0);
// Receives one message. `fds_out` receives any passed descriptors (caller closes them).
// Returns bytes received, 0 on orderly shutdown, -EAGAIN when non-blocking and empty.
ssize_t uds_recv(int fd, void* data, size_t cap, std::vector<int>* fds_out = nullptr);
// Waits until readable. timeout_ms < 0 blocks. Returns 1 readable, 0 timeout, -errno.
int wait_readable(int fd, int timeout_ms);

// Anonymous shared memory (memfd) of `bytes`, returns fd.
int memfd_make(const char* name, size_t bytes);
void* map_shared(int fd, size_t bytes);   // nullptr on failure
void unmap_shared(void* p, size_t bytes);

std::string dirname_of(const std::string& path);
int make_dirs(const std::string& path, int mode = 0700);

}  // namespace ipc
}  // namespace mccs
