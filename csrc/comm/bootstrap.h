// Control plane between the ranks of one node: allgather / broadcast / barrier of
// small byte blobs, plus passing of file descriptors (the shareable handles of
// cuMem allocations and multicast objects).
//
// Parity: the reference's control plane is MPI only (src/comm/comm.cu:86-122:
// MPI_Init_thread, MPI_Comm_split_type, MPI_Bcast; src/comm/ipc.cu:103,261:
// MPI_Allgather of IPC handles; comm.cu:189: MPI_Barrier).  Here the same
// operations sit behind one interface with three implementations: in-process
// (threads or a single driver thread), Unix-domain sockets with an environment
// rendezvous (RANK / WORLD_SIZE / LOCAL_RANK / MASTER_PORT, i.e. what torchrun
// and the bundled launcher export), and MPI when built with YALI_MPI_SUPPORT.
#pragma once

#include <cstddef>
#include <memory>
#include <string>
#include <vector>

#include "../core/status.h"

namespace yali {

class Bootstrap {
   public:
    virtual ~Bootstrap() = default;
    virtual int rank() const = 0;
    virtual int world() const = 0;
    virtual int local_rank() const { return rank(); }
    // out has world()*bytes_each bytes; slot r holds rank r's contribution.
    virtual Result allgather(const void* in, void* out, size_t bytes_each) = 0;
    virtual Result broadcast(void* buf, size_t bytes, int root) = 0;
    virtual Result barrier() = 0;
    // Every rank contributes one open descriptor and receives one descriptor per
    // rank (its own slot holds a duplicate).  The caller closes what it receives.
    virtual Result allgather_fd(int my_fd, std::vector<int>* fds_out) = 0;
    // Root's descriptor is delivered to every rank (a duplicate on the root).
    virtual Result broadcast_fd(int* fd_inout, int root) = 0;
    // Last error text for diagnostics.
    const std::string& last_error() const { return err_; }

   protected:
    std::string err_;
};

// World of one: every operation is a local copy.
std::unique_ptr<Bootstrap> MakeSelfBootstrap();

// Rank 0 listens on an abstract Unix socket named after `job_id`; the others
// connect (retrying until `timeout_ms`).  All ranks must live on one node.
std::unique_ptr<Bootstrap> MakeSocketBootstrap(int rank, int world, int local_rank, const std::string& job_id,
                                               int timeout_ms, Result* res, std::string* err);

// Reads RANK / WORLD_SIZE / LOCAL_RANK (or the OMPI_* / SLURM_* / PMI_* spellings)
// and MASTER_PORT / YALI_JOB_ID.  Without RANK the result is a world of one.
// Each call in a process appends a counter to the job id so that several
// communicators can be created one after another, in the same order on all ranks.
std::unique_ptr<Bootstrap> MakeEnvBootstrap(Result* res, std::string* err);

#ifdef YALI_MPI_SUPPORT
std::unique_ptr<Bootstrap> MakeMpiBootstrap(int* argc, char*** argv, Result* res, std::string* err);
#endif

// Local rank from launcher environments, -1 when none is set.  Same lookup order
// as the reference's yaliGetLocalRankFromEnv (src/comm/comm.cu:28-65) plus LOCAL_RANK.
int LocalRankFromEnv();

}  // namespace yali
