#include "uds.h"

#include <errno.h>
#include <fcntl.h>
#include <poll.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <sys/un.h>
#include <unistd.h>

namespace mccs {
namespace ipc {

static int fill_addr(const std::string& path, sockaddr_un* addr, socklen_t* len) {
  if (path.size() + 1 > sizeof(addr->sun_path)) return -ENAMETOOLONG;
  memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  memcpy(addr->sun_path, path.c_str(), path.size() + 1);
  *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + path.size() + 1);
  return 0;
}

int uds_listen(const std::string& path, int backlog) {
  sockaddr_un addr;
  socklen_t len;
  int rc = fill_addr(path, &addr, &len);
  if (rc < 0) return rc;
  int fd = socket(AF_UNIX, SOCK_SEQPACKET | SOCK_CLOEXEC, 0);
  if (fd < 0) return -errno;
  unlink(path.c_str());
  if (bind(fd, (sockaddr*)&addr, len) < 0) { rc = -errno; close(fd); return rc; }
  if (listen(fd, backlog) < 0) { rc = -errno; close(fd); return rc; }
  set_nonblocking(fd, true);
  return fd;
}

int uds_connect(const std::string& path) {
  sockaddr_un addr;
  socklen_t len;
  int rc = fill_addr(path, &addr, &len);
  if (rc < 0) return rc;
  int fd = socket(AF_UNIX, SOCK_SEQPACKET | SOCK_CLOEXEC, 0);
  if (fd < 0) return -errno;
  if (connect(fd, (sockaddr*)&addr, len) < 0) { rc = -errno; close(fd); return rc; }
  return fd;
}

int uds_accept(int listen_fd) {
  int fd = accept4(listen_fd, nullptr, nullptr, SOCK_CLOEXEC);
  if (fd < 0) return (errno == EWOULDBLOCK) ? -EAGAIN : -errno;
  return fd;
}

int uds_peer_cred(int fd, PeerCred* out) {
  struct ucred cred;
  socklen_t len = sizeof cred;
  if (getsockopt(fd, SOL_SOCKET, SO_PEERCRED, &cred, &len) < 0) return -errno;
  out->pid = cred.pid; out->uid = cred.uid; out->gid = cred.gid;
  return 0;
}

int set_nonblocking(int fd, bool on) {
  int fl = fcntl(fd, F_GETFL, 0);
  if (fl < 0) return -errno;
  fl = on ? (fl | O_NONBLOCK) : (fl & ~O_NONBLOCK);
  return fcntl(fd, F_SETFL, fl) < 0 ? -errno : 0;
}

ssize_t uds_send(int fd, const void* data, size_t len, const int* fds, int nfds) {
  if (nfds > kMaxFdsPerMessage) return -EINVAL;
  struct iovec iov;
  iov.iov_base = const_cast<void*>(data);
  iov.iov_len = len;
  struct msghdr msg;
  memset(&msg, 0, sizeof msg);
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(struct cmsghdr) char ctrl[CMSG_SPACE(sizeof(int) * kMaxFdsPerMessage)];
  if (nfds > 0) {
    memset(ctrl, 0, sizeof ctrl);
    msg.msg_control = ctrl;
    msg.msg_controllen = CMSG_SPACE(sizeof(int) * nfds);
    struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int) * nfds);
    memcpy(CMSG_DATA(c), fds, sizeof(int) * nfds);
  }
  for (;;) {
    ssize_t n = sendmsg(fd, &msg, MSG_NOSIGNAL);
    if (n >= 0) return n;
    if (errno == EINTR) continue;
    return -errno;
  }
}

ssize_t uds_recv(int fd, void* data, size_t cap, std::vector<int>* fds_out) {
  struct iovec iov;
  iov.iov_base = data;
  iov.iov_len = cap;
  struct msghdr msg;
  memset(&msg, 0, sizeof msg);
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(struct cmsghdr) char ctrl[CMSG_SPACE(sizeof(int) * kMaxFdsPerMessage)];
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof ctrl;
  ssize_t n;
  for (;;) {
    n = recvmsg(fd, &msg, MSG_CMSG_CLOEXEC);
    if (n >= 0) break;
    if (errno == EINTR) continue;
    if (errno == EWOULDBLOCK) return -EAGAIN;
    return -errno;
  }
  for (struct cmsghdr* c = CMSG_FIRSTHDR(&msg); c; c = CMSG_NXTHDR(&msg, c)) {
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) {
      int count = (int)((c->cmsg_len - CMSG_LEN(0)) / sizeof(int));
      for (int i = 0; i < count; i++) {
        int f;
        memcpy(&f, CMSG_DATA(c) + sizeof(int) * i, sizeof(int));
        if (fds_out) fds_out->push_back(f);
        else close(f);
      }
    }
  }
  return n;
}

int wait_readable(int fd, int timeout_ms) {
  struct pollfd p;
  p.fd = fd;
  p.events = POLLIN;
  p.revents = 0;
  for (;;) {
    int rc = poll(&p, 1, timeout_ms);
    if (rc > 0) return 1;
    if (rc == 0) return 0;
    if (errno == EINTR) continue;
    return -errno;
  }
}

int memfd_make(const char* name, size_t bytes) {
  int fd = (int)syscall(SYS_memfd_create, name, 1u /* MFD_CLOEXEC */);
  if (fd < 0) return -errno;
  if (ftruncate(fd, (off_t)bytes) < 0) { int rc = -errno; close(fd); return rc; }
  return fd;
}

void* map_shared(int fd, size_t bytes) {
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  return p == MAP_FAILED ? nullptr : p;
}

void unmap_shared(void* p, size_t bytes) { if (p) munmap(p, bytes); }

std::string dirname_of(const std::string& path) {
  size_t pos = path.find_last_of('/');
  if (pos == std::string::npos) return ".";
  if (pos == 0) return "/";
  return path.substr(0, pos);
}

int make_dirs(const std::string& path, int mode) {
  if (path.empty() || path == "/" || path == ".") return 0;
  struct stat st;
  if (stat(path.c_str(), &st) == 0) return S_ISDIR(st.st_mode) ? 0 : -ENOTDIR;
  int rc = make_dirs(dirname_of(path), mode);
  if (rc < 0) return rc;
  if (mkdir(path.c_str(), (mode_t)mode) < 0 && errno != EEXIST) return -errno;
  return 0;
}

}  // namespace ipc
}  // namespace mccs
