// File-descriptor broker between the ranks of one node: a rank publishes a descriptor (the shareable handle of
// its device-memory arena) on a unix-domain socket and its peers fetch a duplicate of it with SCM_RIGHTS.
// Both sides are bounded: the server thread stops after `clients` deliveries or `timeout_ms`, a fetch gives up
// after `timeout_ms`.  Counterpart of the reference's vendored process broker
// (third_party/ThunderKittens/include/pyutils/broker.cuh:38-140), which pairs a POSIX shm barrier with the
// same descriptor passing; here the barrier is left to the process group that already exists.
#include <atomic>
#include <cerrno>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

namespace {

struct Server {
  std::thread thread;
  std::atomic<int> delivered{0};
  std::atomic<int> error{0};
  int listen_fd = -1;
  char path[108] = {0};
};

std::mutex g_mu;
std::vector<Server*> g_servers;

int64_t now_ms() {
  using namespace std::chrono;
  return duration_cast<milliseconds>(steady_clock::now().time_since_epoch()).count();
}

bool fill_addr(const char* path, sockaddr_un* addr) {
  std::memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  if (std::strlen(path) >= sizeof(addr->sun_path)) return false;
  std::strcpy(addr->sun_path, path);
  return true;
}

int send_fd(int sock, int fd) {
  char payload = 'F';
  iovec iov{&payload, 1};
  alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
  std::memset(control, 0, sizeof(control));
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = control;
  msg.msg_controllen = sizeof(control);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
  return sendmsg(sock, &msg, 0) == 1 ? 0 : -errno;
}

int recv_fd(int sock) {
  char payload = 0;
  iovec iov{&payload, 1};
  alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = control;
  msg.msg_controllen = sizeof(control);
  if (recvmsg(sock, &msg, 0) != 1) return -EIO;
  for (cmsghdr* c = CMSG_FIRSTHDR(&msg); c; c = CMSG_NXTHDR(&msg, c)) {
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) {
      int fd = -1;
      std::memcpy(&fd, CMSG_DATA(c), sizeof(int));
      return fd;
    }
  }
  return -ENOMSG;
}

void serve(Server* s, int fd, int clients, int timeout_ms) {
  const int64_t deadline = now_ms() + timeout_ms;
  while (s->delivered.load() < clients) {
    const int64_t left = deadline - now_ms();
    if (left <= 0) {
      s->error.store(ETIMEDOUT);
      break;
    }
    pollfd p{s->listen_fd, POLLIN, 0};
    const int r = poll(&p, 1, static_cast<int>(left < 200 ? left : 200));
    if (r < 0 && errno != EINTR) {
      s->error.store(errno);
      break;
    }
    if (r <= 0) continue;
    const int c = accept(s->listen_fd, nullptr, nullptr);
    if (c < 0) continue;
    if (send_fd(c, fd) == 0) s->delivered.fetch_add(1);
    close(c);
  }
  close(s->listen_fd);
  unlink(s->path);
}

}  // namespace

extern "C" {

// Starts a thread that hands a duplicate of `fd` to `clients` connections on the unix socket `path`.
// Returns a handle >= 0, or -errno.
int b200h_fd_serve(const char* path, int fd, int clients, int timeout_ms) {
  sockaddr_un addr;
  if (!fill_addr(path, &addr)) return -ENAMETOOLONG;
  const int s = socket(AF_UNIX, SOCK_STREAM, 0);
  if (s < 0) return -errno;
  unlink(path);
  if (bind(s, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || listen(s, 64) != 0) {
    const int e = errno;
    close(s);
    return -e;
  }
  Server* srv = new Server();
  srv->listen_fd = s;
  std::strcpy(srv->path, path);
  srv->thread = std::thread(serve, srv, fd, clients, timeout_ms);
  std::lock_guard<std::mutex> lock(g_mu);
  g_servers.push_back(srv);
  return static_cast<int>(g_servers.size()) - 1;
}

// Waits for the server thread; returns the number of descriptors it delivered, or -errno.
int b200h_fd_serve_join(int handle) {
  Server* srv = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    if (handle < 0 || handle >= static_cast<int>(g_servers.size()) || !g_servers[handle]) return -EINVAL;
    srv = g_servers[handle];
    g_servers[handle] = nullptr;
  }
  if (srv->thread.joinable()) srv->thread.join();
  const int err = srv->error.load(), n = srv->delivered.load();
  delete srv;
  return err ? -err : n;
}

// Connects to `path` (retrying until `timeout_ms`) and returns the received descriptor, or -errno.
int b200h_fd_fetch(const char* path, int timeout_ms) {
  sockaddr_un addr;
  if (!fill_addr(path, &addr)) return -ENAMETOOLONG;
  const int64_t deadline = now_ms() + timeout_ms;
  while (true) {
    const int s = socket(AF_UNIX, SOCK_STREAM, 0);
    if (s < 0) return -errno;
    if (connect(s, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) == 0) {
      pollfd p{s, POLLIN, 0};
      const int64_t left = deadline - now_ms();
      int fd = -ETIMEDOUT;
      if (left > 0 && poll(&p, 1, static_cast<int>(left)) > 0) fd = recv_fd(s);
      close(s);
      return fd;
    }
    close(s);
    if (now_ms() >= deadline) return -ETIMEDOUT;
    std::this_thread::sleep_for(std::chrono::milliseconds(5));
  }
}

}  // extern "C"
