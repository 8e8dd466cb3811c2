#include "unix_mesh.h"

#include <fcntl.h>
#include <poll.h>
#include <signal.h>
#include <sys/socket.h>
#include <sys/types.h>
#include <sys/un.h>
#include <sys/wait.h>
#include <time.h>
#include <unistd.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <sstream>
#include <thread>

#include "../common/check.h"

namespace b200ipc {
namespace {

using Clock = std::chrono::steady_clock;

int64_t ms_left(Clock::time_point deadline) {
  auto d = std::chrono::duration_cast<std::chrono::milliseconds>(deadline - Clock::now()).count();
  return d < 0 ? 0 : d;
}

socklen_t fill_abstract_addr(sockaddr_un& addr, const std::string& name) {
  std::memset(&addr, 0, sizeof(addr));
  addr.sun_family = AF_UNIX;
  B200_REQUIRE(name.size() + 1 < sizeof(addr.sun_path), "socket name too long: " << name);
  addr.sun_path[0] = '\0';  // abstract namespace: no file to clean up, dies with the process
  std::memcpy(addr.sun_path + 1, name.data(), name.size());
  return socklen_t(offsetof(sockaddr_un, sun_path) + 1 + name.size());
}

void wait_io(int fd, short events, Clock::time_point deadline, const char* what) {
  for (;;) {
    pollfd p{fd, events, 0};
    int64_t left = ms_left(deadline);
    B200_REQUIRE(left > 0, "bootstrap deadline passed while waiting to " << what);
    int rc = ::poll(&p, 1, int(left > 1000 ? 1000 : left));
    if (rc < 0 && errno == EINTR) continue;
    B200_SYS_CHECK(rc);
    if (rc > 0) {
      B200_REQUIRE((p.revents & (POLLERR | POLLNVAL)) == 0, "socket error while waiting to " << what);
      return;
    }
  }
}

// Abstract-namespace sockets carry no file permissions, so anyone on the machine could dial or
// squat a name.  The kernel tells who is at the other end: only a process of the same user may
// take part in the exchange of memory descriptors.
bool peer_is_same_user(int fd) {
  ucred cred{};
  socklen_t len = sizeof(cred);
  if (::getsockopt(fd, SOL_SOCKET, SO_PEERCRED, &cred, &len) != 0) return false;
  return cred.uid == ::getuid();
}

const char* env_or_null(const char* k) {
  const char* v = std::getenv(k);
  return (v && *v) ? v : nullptr;
}

}  // namespace

std::string UnixMesh::socket_name(const MeshOptions& opt, int rank) {
  std::ostringstream os;
  os << "b200ipc/" << ::getuid() << "/" << opt.job_id << "/i" << opt.instance << "/r" << rank;
  return os.str();
}

UnixMesh::UnixMesh(int rank, int world, const MeshOptions& opt)
    : rank_(rank), world_(world), opt_(opt), conn_(size_t(world), -1) {
  B200_REQUIRE(world >= 1 && rank >= 0 && rank < world, "bad rank/world " << rank << "/" << world);
  if (world == 1) return;
  const auto deadline = Clock::now() + std::chrono::milliseconds(opt.timeout_ms);

  listen_fd_ = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  B200_SYS_CHECK(listen_fd_);
  sockaddr_un addr;
  socklen_t len = fill_abstract_addr(addr, socket_name(opt, rank));
  B200_SYS_CHECK(::bind(listen_fd_, reinterpret_cast<sockaddr*>(&addr), len));
  B200_SYS_CHECK(::listen(listen_fd_, world));

  // Dial every lower rank; the server may not be listening yet, so retry until
  // the deadline (never forever).
  for (int peer = 0; peer < rank; ++peer) {
    sockaddr_un paddr;
    socklen_t plen = fill_abstract_addr(paddr, socket_name(opt, peer));
    for (;;) {
      int fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
      B200_SYS_CHECK(fd);
      if (::connect(fd, reinterpret_cast<sockaddr*>(&paddr), plen) == 0) {
        if (!peer_is_same_user(fd)) {
          ::close(fd);
          B200_REQUIRE(false, "the bootstrap socket of rank " << peer << " belongs to another user; refusing to exchange "
                                                                 "memory handles with it");
        }
        int32_t me = rank;
        conn_[size_t(peer)] = fd;
        send_all(peer, &me, sizeof(me));
        break;
      }
      int e = errno;
      ::close(fd);
      B200_REQUIRE(e == ECONNREFUSED || e == ENOENT || e == EAGAIN || e == EINTR,
                   "connect to rank " << peer << " failed: " << std::strerror(e));
      B200_REQUIRE(ms_left(deadline) > 0, "rank " << rank << ": rank " << peer
                                                  << " never opened its bootstrap socket (job '"
                                                  << opt.job_id << "', instance " << opt.instance << ")");
      std::this_thread::sleep_for(std::chrono::milliseconds(2));
    }
  }
  // Accept every higher rank.
  for (int n = rank + 1; n < world; ++n) {
    wait_io(listen_fd_, POLLIN, deadline, "accept a peer");
    int fd = ::accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
    B200_SYS_CHECK(fd);
    if (!peer_is_same_user(fd)) {  // not one of this job's ranks: drop it and keep waiting
      ::close(fd);
      --n;
      continue;
    }
    int32_t who = -1;
    size_t got = 0;
    while (got < sizeof(who)) {
      wait_io(fd, POLLIN, deadline, "read a peer's rank");
      ssize_t k = ::read(fd, reinterpret_cast<char*>(&who) + got, sizeof(who) - got);
      B200_REQUIRE(k > 0, "peer closed the bootstrap connection during hello");
      got += size_t(k);
    }
    B200_REQUIRE(who > rank && who < world && conn_[size_t(who)] == -1, "unexpected hello from rank " << who);
    conn_[size_t(who)] = fd;
  }
}

UnixMesh::~UnixMesh() {
  for (int fd : conn_)
    if (fd >= 0) ::close(fd);
  if (listen_fd_ >= 0) ::close(listen_fd_);
}

void UnixMesh::send_all(int peer, const void* p, size_t n) {
  const auto deadline = Clock::now() + std::chrono::milliseconds(opt_.timeout_ms);
  const char* c = static_cast<const char*>(p);
  int fd = conn_[size_t(peer)];
  while (n > 0) {
    wait_io(fd, POLLOUT, deadline, "send to a peer");
    ssize_t k = ::send(fd, c, n, MSG_NOSIGNAL);
    if (k < 0 && (errno == EINTR || errno == EAGAIN)) continue;
    B200_REQUIRE(k > 0, "send to rank " << peer << " failed: " << std::strerror(errno));
    c += k;
    n -= size_t(k);
  }
}

void UnixMesh::recv_all(int peer, void* p, size_t n) {
  const auto deadline = Clock::now() + std::chrono::milliseconds(opt_.timeout_ms);
  char* c = static_cast<char*>(p);
  int fd = conn_[size_t(peer)];
  while (n > 0) {
    wait_io(fd, POLLIN, deadline, "receive from a peer");
    ssize_t k = ::recv(fd, c, n, 0);
    if (k < 0 && (errno == EINTR || errno == EAGAIN)) continue;
    B200_REQUIRE(k > 0, "rank " << peer << " closed the bootstrap connection (it may have exited)");
    c += k;
    n -= size_t(k);
  }
}

void UnixMesh::send_fd(int peer, int fd) {
  const auto deadline = Clock::now() + std::chrono::milliseconds(opt_.timeout_ms);
  char tag = 'F';
  iovec iov{&tag, 1};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  std::memset(ctrl, 0, sizeof(ctrl));
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  cmsghdr* cm = CMSG_FIRSTHDR(&msg);
  cm->cmsg_level = SOL_SOCKET;
  cm->cmsg_type = SCM_RIGHTS;
  cm->cmsg_len = CMSG_LEN(sizeof(int));
  std::memcpy(CMSG_DATA(cm), &fd, sizeof(int));
  for (;;) {
    wait_io(conn_[size_t(peer)], POLLOUT, deadline, "pass a descriptor");
    ssize_t k = ::sendmsg(conn_[size_t(peer)], &msg, MSG_NOSIGNAL);
    if (k < 0 && (errno == EINTR || errno == EAGAIN)) continue;
    B200_REQUIRE(k == 1, "sendmsg(SCM_RIGHTS) to rank " << peer << " failed: " << std::strerror(errno));
    return;
  }
}

int UnixMesh::recv_fd(int peer) {
  const auto deadline = Clock::now() + std::chrono::milliseconds(opt_.timeout_ms);
  char tag = 0;
  iovec iov{&tag, 1};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  for (;;) {
    wait_io(conn_[size_t(peer)], POLLIN, deadline, "receive a descriptor");
    ssize_t k = ::recvmsg(conn_[size_t(peer)], &msg, MSG_CMSG_CLOEXEC);
    if (k < 0 && (errno == EINTR || errno == EAGAIN)) continue;
    B200_REQUIRE(k == 1 && tag == 'F', "rank " << peer << " closed the connection while passing a descriptor");
    break;
  }
  cmsghdr* cm = CMSG_FIRSTHDR(&msg);
  B200_REQUIRE(cm && cm->cmsg_level == SOL_SOCKET && cm->cmsg_type == SCM_RIGHTS,
               "no descriptor in the message from rank " << peer);
  int fd = -1;
  std::memcpy(&fd, CMSG_DATA(cm), sizeof(int));
  return fd;
}

void UnixMesh::allgather(const void* send, size_t nbytes, void* recv) {
  char* out = static_cast<char*>(recv);
  std::memcpy(out + size_t(rank_) * nbytes, send, nbytes);
  // Pairwise exchange in a fixed order (lower rank sends first) so that blobs
  // larger than a socket buffer cannot deadlock.
  for (int peer = 0; peer < world_; ++peer) {
    if (peer == rank_) continue;
    if (rank_ < peer) {
      send_all(peer, send, nbytes);
      recv_all(peer, out + size_t(peer) * nbytes, nbytes);
    } else {
      recv_all(peer, out + size_t(peer) * nbytes, nbytes);
      send_all(peer, send, nbytes);
    }
  }
}

std::vector<int> UnixMesh::allgather_fds(int fd) {
  std::vector<int> fds(static_cast<size_t>(world_), -1);
  fds[size_t(rank_)] = ::dup(fd);
  B200_SYS_CHECK(fds[size_t(rank_)]);
  for (int peer = 0; peer < world_; ++peer) {
    if (peer == rank_) continue;
    if (rank_ < peer) {
      send_fd(peer, fd);
      fds[size_t(peer)] = recv_fd(peer);
    } else {
      fds[size_t(peer)] = recv_fd(peer);
      send_fd(peer, fd);
    }
  }
  return fds;
}

int UnixMesh::broadcast_fd(int root, int fd) {
  if (rank_ == root) {
    for (int peer = 0; peer < world_; ++peer)
      if (peer != root) send_fd(peer, fd);
    int d = ::dup(fd);
    B200_SYS_CHECK(d);
    return d;
  }
  return recv_fd(root);
}

void UnixMesh::barrier() {
  if (world_ == 1) return;
  char token = 'B';
  std::vector<char> all(static_cast<size_t>(world_), 0);
  allgather(&token, 1, all.data());
}

int64_t UnixMesh::allreduce_max(int64_t v) {
  std::vector<int64_t> all(static_cast<size_t>(world_), 0);
  allgather(&v, sizeof(v), all.data());
  int64_t m = v;
  for (int64_t x : all) m = x > m ? x : m;
  return m;
}

RankEnv rank_env_from_environment() {
  RankEnv e;
  struct Triple { const char* rank; const char* world; const char* local; };
  static const Triple kSources[] = {
      {"B200IPC_RANK", "B200IPC_WORLD", "B200IPC_LOCAL_RANK"},
      {"RANK", "WORLD_SIZE", "LOCAL_RANK"},
      {"OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE", "OMPI_COMM_WORLD_LOCAL_RANK"},
      {"PMI_RANK", "PMI_SIZE", "MPI_LOCALRANKID"},
      {"PMIX_RANK", "PMIX_SIZE", "PMIX_LOCAL_RANK"},
      {"SLURM_PROCID", "SLURM_NTASKS", "SLURM_LOCALID"},
  };
  for (const Triple& t : kSources) {
    const char* r = env_or_null(t.rank);
    const char* w = env_or_null(t.world);
    if (!r || !w) continue;
    e.rank = std::atoi(r);
    e.world = std::atoi(w);
    const char* l = env_or_null(t.local);
    e.local_rank = l ? std::atoi(l) : e.rank;
    e.found = true;
    break;
  }
  if (const char* j = env_or_null("B200IPC_JOB_ID")) {
    e.job_id = j;
  } else if (const char* p = env_or_null("MASTER_PORT")) {
    e.job_id = std::string("port") + p;
  } else if (const char* s = env_or_null("SLURM_JOB_ID")) {
    e.job_id = std::string("slurm") + s;
  } else {
    e.job_id = "default";
  }
  return e;
}

int fork_ranks(int world, int (*child_main)(int, int, void*), void* arg) {
  std::vector<pid_t> pids(static_cast<size_t>(world), -1);
  std::ostringstream job;
  job << "fork" << ::getpid();
  ::setenv("B200IPC_JOB_ID", job.str().c_str(), 0);
  for (int r = 0; r < world; ++r) {
    pid_t pid = ::fork();
    B200_SYS_CHECK(pid);
    if (pid == 0) {
      ::setenv("B200IPC_RANK", std::to_string(r).c_str(), 1);
      ::setenv("B200IPC_WORLD", std::to_string(world).c_str(), 1);
      ::setenv("B200IPC_LOCAL_RANK", std::to_string(r).c_str(), 1);
      int rc = 1;
      try {
        rc = child_main(r, world, arg);
      } catch (const std::exception& ex) {
        std::fprintf(stderr, "[rank %d] %s\n", r, ex.what());
        rc = 1;
      }
      std::fflush(stdout);
      std::fflush(stderr);
      ::_exit(rc);
    }
    pids[size_t(r)] = pid;
  }
  // Reap the children.  After the first failure the others get a grace period to
  // notice on their own (their bounded waits and socket reads end with an error)
  // before the exact pids started here are signalled; nothing is killed by name.
  int worst = 0;
  int alive = world;
  Clock::time_point grace_end{};
  bool failing = false;
  bool signalled = false;
  while (alive > 0) {
    int st = 0;
    pid_t pid = ::waitpid(-1, &st, failing ? WNOHANG : 0);
    if (pid < 0) {
      if (errno == EINTR) continue;
      break;
    }
    if (pid == 0) {
      if (!signalled && Clock::now() > grace_end) {
        for (pid_t other : pids)
          if (other > 0) ::kill(other, SIGTERM);
        signalled = true;
      }
      std::this_thread::sleep_for(std::chrono::milliseconds(20));
      continue;
    }
    int rc = WIFEXITED(st) ? WEXITSTATUS(st) : 128 + (WIFSIGNALED(st) ? WTERMSIG(st) : 0);
    for (int r = 0; r < world; ++r) {
      if (pids[size_t(r)] == pid) {
        pids[size_t(r)] = -1;
        --alive;
        if (rc != 0 && worst == 0) {
          worst = rc;
          failing = true;
          grace_end = Clock::now() + std::chrono::seconds(20);
        }
      }
    }
  }
  return worst;
}

}  // namespace b200ipc
