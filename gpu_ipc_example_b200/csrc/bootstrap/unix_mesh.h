// Host-side bootstrap between the ranks of one node: a full mesh of Unix-domain
// stream sockets over which ranks all-gather small byte blobs, pass file
// descriptors (SCM_RIGHTS) and run host barriers.
//
// File descriptors of exported GPU allocations cannot travel as bytes, which is
// why this exists next to torch.distributed / MPI: those give rank and world,
// this moves the handles.
//
// Differences from the reference's socket all-gather (ipc_exchange.cpp:43-265):
// connections are kept for the life of the mesh (one per pair, the higher rank
// dials), socket names live in the abstract namespace and carry job id, instance
// and rank with separators (the reference concatenates rank and instance digits
// in a file path in the working directory, ipc_exchange.cpp:164,178), and every
// connect/accept/read has a deadline instead of spinning forever
// (ipc_exchange.cpp:144-150).
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace b200ipc {

struct MeshOptions {
  std::string job_id;    // namespaces concurrent jobs of one node
  int instance = 0;      // second namespace level (the CLI's -i)
  int timeout_ms = 60000;
};

class UnixMesh {
 public:
  UnixMesh(int rank, int world, const MeshOptions& opt);
  ~UnixMesh();
  UnixMesh(const UnixMesh&) = delete;
  UnixMesh& operator=(const UnixMesh&) = delete;

  int rank() const { return rank_; }
  int world() const { return world_; }

  // recv must hold world * nbytes; slot r receives rank r's blob.
  void allgather(const void* send, size_t nbytes, void* recv);
  // Returns world descriptors; entry [rank] is a dup of `fd`.  The caller owns
  // (closes) all of them.
  std::vector<int> allgather_fds(int fd);
  // Root sends one descriptor to everyone; returns the local copy (a dup on root).
  int broadcast_fd(int root, int fd);
  void barrier();
  // Largest value over ranks (used to agree on error state).
  int64_t allreduce_max(int64_t v);

  // Name of the listening socket of `rank` (without the leading NUL byte).
  static std::string socket_name(const MeshOptions& opt, int rank);

 private:
  void send_all(int peer, const void* p, size_t n);
  void recv_all(int peer, void* p, size_t n);
  void send_fd(int peer, int fd);
  int recv_fd(int peer);

  int rank_;
  int world_;
  MeshOptions opt_;
  int listen_fd_ = -1;
  std::vector<int> conn_;  // conn_[peer], -1 for self
};

// Rank / world / local rank from the environment of whichever launcher started
// the process: torchrun (RANK, WORLD_SIZE, LOCAL_RANK), Open MPI, Intel MPI / PMI,
// Slurm, or this library's own launcher (B200IPC_RANK, ...).  Capability parity:
// script/gpu_inference_test.py:9-19 maps the same MPI variables.
struct RankEnv {
  int rank = 0;
  int world = 1;
  int local_rank = 0;
  std::string job_id;
  bool found = false;
};
RankEnv rank_env_from_environment();

// Forks `world` copies of the current program (after fork, `child_main(rank)` is
// run and its return value becomes the exit code).  Returns the worst exit code.
// A child that dies takes the others down (SIGTERM) so no rank waits forever.
int fork_ranks(int world, int (*child_main)(int rank, int world, void* arg), void* arg);

}  // namespace b200ipc
