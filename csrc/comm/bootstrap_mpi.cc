// MPI implementation of the bootstrap, compiled only with -DYALI_MPI_SUPPORT (needs
// <mpi.h> and an MPI library at link time; neither is required by the default build,
// whose control plane is the socket bootstrap).  File descriptors cannot travel over
// MPI, so descriptor passing falls back to a Unix-socket side channel created from the
// MPI rank / size with the job id broadcast by rank 0.
//
// Parity: yaliMPCommCreate's MPI_Init_thread / MPI_Comm_split_type / MPI_Bcast
// (src/comm/comm.cu:86-122), MPI_Allgather of handles (src/comm/ipc.cu:103,261),
// MPI_Barrier (comm.cu:189).
#ifdef YALI_MPI_SUPPORT
#include <mpi.h>
#include <unistd.h>

#include <climits>
#include <cstdlib>

#include "bootstrap.h"

namespace yali {
namespace {

class MpiBootstrap final : public Bootstrap {
   public:
    MpiBootstrap(bool owns_init) : owns_init_(owns_init) {
        MPI_Comm_rank(MPI_COMM_WORLD, &rank_);
        MPI_Comm_size(MPI_COMM_WORLD, &world_);
        MPI_Comm local;
        MPI_Comm_split_type(MPI_COMM_WORLD, MPI_COMM_TYPE_SHARED, rank_, MPI_INFO_NULL, &local);
        MPI_Comm_rank(local, &local_rank_);
        MPI_Comm_free(&local);
        const int env_local = LocalRankFromEnv();
        if (env_local >= 0) local_rank_ = env_local;
    }
    ~MpiBootstrap() override {
        side_.reset();
        if (owns_init_) MPI_Finalize();
    }
    int rank() const override { return rank_; }
    int world() const override { return world_; }
    int local_rank() const override { return local_rank_; }
    Result allgather(const void* in, void* out, size_t n) override {
        if (n > static_cast<size_t>(INT_MAX)) return Result::InvalidArg;
        return MPI_Allgather(in, static_cast<int>(n), MPI_BYTE, out, static_cast<int>(n), MPI_BYTE, MPI_COMM_WORLD) ==
                       MPI_SUCCESS
                   ? Result::Success
                   : Result::BootstrapError;
    }
    Result broadcast(void* buf, size_t n, int root) override {
        char* p = static_cast<char*>(buf);
        while (n) {  // chunks of at most INT_MAX bytes
            const int k = n > static_cast<size_t>(INT_MAX) ? INT_MAX : static_cast<int>(n);
            if (MPI_Bcast(p, k, MPI_BYTE, root, MPI_COMM_WORLD) != MPI_SUCCESS) return Result::BootstrapError;
            p += k;
            n -= static_cast<size_t>(k);
        }
        return Result::Success;
    }
    Result barrier() override { return MPI_Barrier(MPI_COMM_WORLD) == MPI_SUCCESS ? Result::Success : Result::BootstrapError; }
    Result allgather_fd(int my_fd, std::vector<int>* fds) override {
        Result r = EnsureSide();
        return r == Result::Success ? side_->allgather_fd(my_fd, fds) : r;
    }
    Result broadcast_fd(int* fd, int root) override {
        Result r = EnsureSide();
        return r == Result::Success ? side_->broadcast_fd(fd, root) : r;
    }

   private:
    Result EnsureSide() {
        if (side_ || world_ == 1) {
            if (!side_) side_ = MakeSelfBootstrap();
            return Result::Success;
        }
        long long id = 0;
        if (rank_ == 0) id = (static_cast<long long>(getpid()) << 20) ^ (++counter_);
        MPI_Bcast(&id, 1, MPI_LONG_LONG, 0, MPI_COMM_WORLD);
        Result r;
        side_ = MakeSocketBootstrap(rank_, world_, local_rank_, "mpi" + std::to_string(id), 60000, &r, &err_);
        return side_ ? Result::Success : r;
    }
    int rank_ = 0, world_ = 1, local_rank_ = 0;
    bool owns_init_;
    std::unique_ptr<Bootstrap> side_;
    static long long counter_;
};
long long MpiBootstrap::counter_ = 0;

}  // namespace

std::unique_ptr<Bootstrap> MakeMpiBootstrap(int* argc, char*** argv, Result* res, std::string* err) {
    int inited = 0;
    MPI_Initialized(&inited);
    bool owns = false;
    if (!inited) {
        int provided = 0;
        if (MPI_Init_thread(argc, argv, MPI_THREAD_MULTIPLE, &provided) != MPI_SUCCESS) {
            if (res) *res = Result::BootstrapError;
            if (err) *err = "MPI_Init_thread failed";
            return nullptr;
        }
        owns = true;
    }
    if (res) *res = Result::Success;
    return std::unique_ptr<Bootstrap>(new MpiBootstrap(owns));
}

}  // namespace yali
#endif  // YALI_MPI_SUPPORT
