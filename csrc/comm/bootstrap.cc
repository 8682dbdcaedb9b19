// Bootstrap implementations: self (world of one) and Unix-domain sockets.
// See bootstrap.h for the interface and its relation to the reference's MPI calls.
#include "bootstrap.h"

#include <errno.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <thread>

#include "../core/env.h"

namespace yali {

namespace {

constexpr uint32_t kMagic = 0x59414c49u;  // "YALI"

enum Op : uint32_t { kHello = 1, kAllgather = 2, kBroadcast = 3, kBarrier = 4, kFdGather = 5, kFdBcast = 6 };

struct Frame {
    uint32_t magic;
    uint32_t op;
    uint64_t bytes;
    uint32_t rank;
    uint32_t world;
};

class SelfBootstrap final : public Bootstrap {
   public:
    int rank() const override { return 0; }
    int world() const override { return 1; }
    Result allgather(const void* in, void* out, size_t n) override {
        if (n) std::memcpy(out, in, n);
        return Result::Success;
    }
    Result broadcast(void*, size_t, int root) override { return root == 0 ? Result::Success : Result::InvalidArg; }
    Result barrier() override { return Result::Success; }
    Result allgather_fd(int my_fd, std::vector<int>* out) override {
        out->assign(1, dup(my_fd));
        return (*out)[0] >= 0 ? Result::Success : Result::BootstrapError;
    }
    Result broadcast_fd(int* fd, int root) override {
        if (root != 0) return Result::InvalidArg;
        *fd = dup(*fd);
        return *fd >= 0 ? Result::Success : Result::BootstrapError;
    }
};

bool SendAll(int fd, const void* buf, size_t n) {
    const char* p = static_cast<const char*>(buf);
    while (n) {
        ssize_t k = ::send(fd, p, n, MSG_NOSIGNAL);
        if (k < 0) {
            if (errno == EINTR) continue;
            return false;
        }
        p += k;
        n -= static_cast<size_t>(k);
    }
    return true;
}

bool RecvAll(int fd, void* buf, size_t n) {
    char* p = static_cast<char*>(buf);
    while (n) {
        ssize_t k = ::recv(fd, p, n, 0);
        if (k == 0) return false;  // peer closed
        if (k < 0) {
            if (errno == EINTR) continue;
            return false;  // includes EAGAIN from SO_RCVTIMEO
        }
        p += k;
        n -= static_cast<size_t>(k);
    }
    return true;
}

bool SendFds(int sock, const int* fds, int count) {
    char payload = 'F';
    struct iovec iov = {&payload, 1};
    alignas(struct cmsghdr) char ctrl[CMSG_SPACE(sizeof(int) * kMaxRanks)];
    std::memset(ctrl, 0, sizeof(ctrl));
    struct msghdr msg = {};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = ctrl;
    msg.msg_controllen = CMSG_SPACE(sizeof(int) * count);
    struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int) * count);
    std::memcpy(CMSG_DATA(c), fds, sizeof(int) * count);
    for (;;) {
        ssize_t k = ::sendmsg(sock, &msg, MSG_NOSIGNAL);
        if (k < 0 && errno == EINTR) continue;
        return k == 1;
    }
}

bool RecvFds(int sock, int* fds, int count) {
    char payload = 0;
    struct iovec iov = {&payload, 1};
    alignas(struct cmsghdr) char ctrl[CMSG_SPACE(sizeof(int) * kMaxRanks)];
    struct msghdr msg = {};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    ssize_t k;
    do {
        k = ::recvmsg(sock, &msg, MSG_CMSG_CLOEXEC);
    } while (k < 0 && errno == EINTR);
    if (k != 1 || payload != 'F') return false;
    struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
    if (!c || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) return false;
    if (c->cmsg_len != CMSG_LEN(sizeof(int) * count)) return false;
    std::memcpy(fds, CMSG_DATA(c), sizeof(int) * count);
    return true;
}

void SetTimeouts(int fd, int timeout_ms) {
    struct timeval tv;
    tv.tv_sec = timeout_ms / 1000;
    tv.tv_usec = (timeout_ms % 1000) * 1000;
    setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
}

socklen_t AbstractAddr(const std::string& name, sockaddr_un* addr) {
    std::memset(addr, 0, sizeof(*addr));
    addr->sun_family = AF_UNIX;
    std::string n = name.substr(0, sizeof(addr->sun_path) - 2);
    std::memcpy(addr->sun_path + 1, n.data(), n.size());  // leading NUL: abstract namespace
    return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n.size());
}

// Star topology: rank 0 holds one connection per other rank; every collective is
// "gather at the root, then scatter from the root".  Messages carry a frame with
// the operation and byte count so that ranks that disagree fail instead of
// desynchronising.
class SocketBootstrap final : public Bootstrap {
   public:
    SocketBootstrap(int rank, int world, int local_rank) : rank_(rank), world_(world), local_rank_(local_rank) {}
    ~SocketBootstrap() override {
        for (int fd : conns_)
            if (fd >= 0) ::close(fd);
        if (listen_fd_ >= 0) ::close(listen_fd_);
    }

    Result connect_all(const std::string& job_id, int timeout_ms) {
        sockaddr_un addr;
        socklen_t len = AbstractAddr("yali-b200-" + job_id, &addr);
        auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
        if (rank_ == 0) {
            conns_.assign(world_, -1);
            listen_fd_ = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
            if (listen_fd_ < 0) return fail("socket() failed");
            if (::bind(listen_fd_, reinterpret_cast<sockaddr*>(&addr), len) != 0)
                return fail(std::string("bind failed (job id in use?): ") + std::strerror(errno));
            if (::listen(listen_fd_, world_) != 0) return fail("listen failed");
            for (int joined = 1; joined < world_;) {
                auto left = std::chrono::duration_cast<std::chrono::milliseconds>(deadline -
                                                                                  std::chrono::steady_clock::now())
                                .count();
                if (left <= 0) return fail("timed out waiting for ranks to join");
                struct pollfd p = {listen_fd_, POLLIN, 0};
                int pr = ::poll(&p, 1, static_cast<int>(left));
                if (pr < 0 && errno == EINTR) continue;
                if (pr <= 0) return fail("timed out waiting for ranks to join");
                int c = ::accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
                if (c < 0) continue;
                SetTimeouts(c, timeout_ms);
                Frame f;
                if (!RecvAll(c, &f, sizeof(f)) || f.magic != kMagic || f.op != kHello) {
                    ::close(c);
                    return fail("bad hello from a joining rank");
                }
                if (static_cast<int>(f.world) != world_ || f.rank == 0 || static_cast<int>(f.rank) >= world_ ||
                    conns_[f.rank] >= 0) {
                    ::close(c);
                    return fail("joining rank disagrees on world size or duplicates a rank");
                }
                conns_[f.rank] = c;
                ++joined;
            }
            // Tell everyone the world is complete.
            Frame ok = {kMagic, kHello, 0, 0, static_cast<uint32_t>(world_)};
            for (int r = 1; r < world_; ++r)
                if (!SendAll(conns_[r], &ok, sizeof(ok))) return fail("hello reply failed");
        } else {
            conns_.assign(1, -1);
            for (;;) {
                int s = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
                if (s < 0) return fail("socket() failed");
                if (::connect(s, reinterpret_cast<sockaddr*>(&addr), len) == 0) {
                    conns_[0] = s;
                    break;
                }
                ::close(s);
                if (std::chrono::steady_clock::now() > deadline) return fail("timed out connecting to rank 0");
                std::this_thread::sleep_for(std::chrono::milliseconds(10));
            }
            SetTimeouts(conns_[0], timeout_ms);
            Frame hello = {kMagic, kHello, 0, static_cast<uint32_t>(rank_), static_cast<uint32_t>(world_)};
            if (!SendAll(conns_[0], &hello, sizeof(hello))) return fail("hello failed");
            Frame ok;
            if (!RecvAll(conns_[0], &ok, sizeof(ok)) || ok.magic != kMagic || ok.op != kHello)
                return fail("rank 0 rejected the hello (world size mismatch or a rank never joined)");
        }
        return Result::Success;
    }

    int rank() const override { return rank_; }
    int world() const override { return world_; }
    int local_rank() const override { return local_rank_; }

    Result allgather(const void* in, void* out, size_t n) override {
        if (rank_ == 0) {
            char* o = static_cast<char*>(out);
            if (n) std::memcpy(o, in, n);
            for (int r = 1; r < world_; ++r) {
                if (!expect(conns_[r], kAllgather, n, r)) return Result::BootstrapError;
                if (n && !RecvAll(conns_[r], o + r * n, n)) return fail("allgather: recv failed");
            }
            for (int r = 1; r < world_; ++r)
                if (n && !SendAll(conns_[r], o, n * world_)) return fail("allgather: send failed");
        } else {
            if (!announce(kAllgather, n)) return Result::BootstrapError;
            if (n && !SendAll(conns_[0], in, n)) return fail("allgather: send failed");
            if (n && !RecvAll(conns_[0], out, n * world_)) return fail("allgather: recv failed (a rank left?)");
        }
        return Result::Success;
    }

    Result broadcast(void* buf, size_t n, int root) override {
        if (root < 0 || root >= world_) return Result::InvalidArg;
        // Route through rank 0: root -> 0 -> everyone.
        if (rank_ == 0) {
            if (root != 0) {
                if (!expect(conns_[root], kBroadcast, n, root)) return Result::BootstrapError;
                if (n && !RecvAll(conns_[root], buf, n)) return fail("broadcast: recv failed");
            }
            for (int r = 1; r < world_; ++r) {
                if (r == root) continue;
                if (n && !SendAll(conns_[r], buf, n)) return fail("broadcast: send failed");
            }
        } else if (rank_ == root) {
            if (!announce(kBroadcast, n)) return Result::BootstrapError;
            if (n && !SendAll(conns_[0], buf, n)) return fail("broadcast: send failed");
        } else {
            if (n && !RecvAll(conns_[0], buf, n)) return fail("broadcast: recv failed (a rank left?)");
        }
        return Result::Success;
    }

    Result barrier() override {
        char token = 0;
        std::vector<char> all(world_);
        return allgather(&token, all.data(), 1);
    }

    Result allgather_fd(int my_fd, std::vector<int>* out) override {
        out->assign(world_, -1);
        if (rank_ == 0) {
            (*out)[0] = dup(my_fd);
            for (int r = 1; r < world_; ++r) {
                if (!expect(conns_[r], kFdGather, 1, r)) return Result::BootstrapError;
                if (!RecvFds(conns_[r], &(*out)[r], 1)) return fail("allgather_fd: recv failed");
            }
            for (int r = 1; r < world_; ++r)
                if (!SendFds(conns_[r], out->data(), world_)) return fail("allgather_fd: send failed");
        } else {
            if (!announce(kFdGather, 1)) return Result::BootstrapError;
            if (!SendFds(conns_[0], &my_fd, 1)) return fail("allgather_fd: send failed");
            if (!RecvFds(conns_[0], out->data(), world_)) return fail("allgather_fd: recv failed (a rank left?)");
        }
        return Result::Success;
    }

    Result broadcast_fd(int* fd, int root) override {
        if (root != 0) return Result::InvalidArg;  // only the root-0 form is needed by the library
        if (rank_ == 0) {
            for (int r = 1; r < world_; ++r)
                if (!SendFds(conns_[r], fd, 1)) return fail("broadcast_fd: send failed");
            *fd = dup(*fd);
        } else {
            if (!RecvFds(conns_[0], fd, 1)) return fail("broadcast_fd: recv failed (a rank left?)");
        }
        return Result::Success;
    }

   private:
    Result fail(const std::string& what) {
        err_ = "bootstrap rank " + std::to_string(rank_) + ": " + what;
        return Result::BootstrapError;
    }
    bool announce(uint32_t op, size_t n) {
        Frame f = {kMagic, op, static_cast<uint64_t>(n), static_cast<uint32_t>(rank_), static_cast<uint32_t>(world_)};
        if (!SendAll(conns_[0], &f, sizeof(f))) {
            fail("could not reach rank 0");
            return false;
        }
        return true;
    }
    bool expect(int fd, uint32_t op, size_t n, int from) {
        Frame f;
        if (!RecvAll(fd, &f, sizeof(f))) {
            fail("rank " + std::to_string(from) + " left or timed out");
            return false;
        }
        if (f.magic != kMagic || f.op != op || f.bytes != n || static_cast<int>(f.rank) != from) {
            fail("rank " + std::to_string(from) + " is in a different collective (op " + std::to_string(f.op) +
                 ", " + std::to_string(f.bytes) + " bytes; expected op " + std::to_string(op) + ", " +
                 std::to_string(n) + " bytes)");
            return false;
        }
        return true;
    }

    int rank_, world_, local_rank_;
    int listen_fd_ = -1;
    std::vector<int> conns_;  // rank 0: per rank; others: [0] = connection to rank 0
};

int EnvInt(const char* const* names, int dflt) {
    for (int i = 0; names[i]; ++i) {
        const char* v = std::getenv(names[i]);
        if (v && *v) return std::atoi(v);
    }
    return dflt;
}

std::atomic<int> g_env_comm_counter{0};

}  // namespace

std::unique_ptr<Bootstrap> MakeSelfBootstrap() { return std::unique_ptr<Bootstrap>(new SelfBootstrap()); }

std::unique_ptr<Bootstrap> MakeSocketBootstrap(int rank, int world, int local_rank, const std::string& job_id,
                                               int timeout_ms, Result* res, std::string* err) {
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) {
        if (res) *res = Result::InvalidArg;
        if (err) *err = "rank/world out of range (1.." + std::to_string(kMaxRanks) + " ranks)";
        return nullptr;
    }
    if (world == 1) {
        if (res) *res = Result::Success;
        return MakeSelfBootstrap();
    }
    std::unique_ptr<SocketBootstrap> b(new SocketBootstrap(rank, world, local_rank));
    Result r = b->connect_all(job_id, timeout_ms);
    if (res) *res = r;
    if (r != Result::Success) {
        if (err) *err = b->last_error();
        return nullptr;
    }
    return b;
}

int LocalRankFromEnv() {
    static const char* const names[] = {"LOCAL_RANK", "OMPI_COMM_WORLD_LOCAL_RANK", "MPI_LOCALRANKID",
                                        "SLURM_LOCALID", "MV2_COMM_WORLD_LOCAL_RANK", nullptr};
    return EnvInt(names, -1);
}

std::unique_ptr<Bootstrap> MakeEnvBootstrap(Result* res, std::string* err) {
    static const char* const rank_names[] = {"RANK", "OMPI_COMM_WORLD_RANK", "PMI_RANK", "SLURM_PROCID", nullptr};
    static const char* const world_names[] = {"WORLD_SIZE", "OMPI_COMM_WORLD_SIZE", "PMI_SIZE", "SLURM_NTASKS",
                                              nullptr};
    int rank = EnvInt(rank_names, -1);
    int world = EnvInt(world_names, 1);
    if (rank < 0 || world <= 1) {
        if (res) *res = Result::Success;
        return MakeSelfBootstrap();
    }
    int local = LocalRankFromEnv();
    if (local < 0) local = rank;
    std::string job = env::GetStr("YALI_JOB_ID", "");
    if (job.empty()) job = "port" + env::GetStr("MASTER_PORT", "29500");
    job += "-" + std::to_string(g_env_comm_counter.fetch_add(1));
    int timeout_ms = static_cast<int>(env::GetInt("YALI_BOOTSTRAP_TIMEOUT_MS", 60000));
    return MakeSocketBootstrap(rank, world, local, job, timeout_ms, res, err);
}

}  // namespace yali
