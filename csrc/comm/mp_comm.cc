#include "mp_comm.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "bootstrap.h"
#include "cuda_driver.h"

using yali::Bootstrap;

namespace {
Bootstrap* BS(YaliMPComm* c) { return static_cast<Bootstrap*>(c->bootstrap); }

// Imported base pointers are remembered so that closing works on interior pointers, and an
// allocation that is imported more than once (several exported pointers inside one allocation
// share its handle) is opened only once per process: a second cudaIpcOpenMemHandle of the same
// handle is an error.
struct Imported {
    void* user;
    void* base;
};
struct Opened {
    cudaIpcMemHandle_t handle;
    void* base;
    int refs;
};
std::vector<Imported>& ImportTable() {
    static std::vector<Imported> t;
    return t;
}
std::vector<Opened>& OpenTable() {
    static std::vector<Opened> t;
    return t;
}
}  // namespace

extern "C" {

int yaliGetLocalRankFromEnv(void) {
    int r = yali::LocalRankFromEnv();
    return r < 0 ? 0 : r;
}

YaliMPComm* yaliMPCommCreate(int* argc, char*** argv) {
    (void)argc;
    (void)argv;
    yali::Result res = yali::Result::Success;
    std::string err;
    std::unique_ptr<Bootstrap> bs;
    int use_mpi = 0;
#ifdef YALI_MPI_SUPPORT
    bs = yali::MakeMpiBootstrap(argc, argv, &res, &err);
    use_mpi = 1;
#else
    bs = yali::MakeEnvBootstrap(&res, &err);
#endif
    if (!bs) {
        std::fprintf(stderr, "yaliMPCommCreate: %s\n", err.c_str());
        return nullptr;
    }
    YaliMPComm* c = static_cast<YaliMPComm*>(std::calloc(1, sizeof(YaliMPComm)));
    if (!c) return nullptr;
    c->rank = bs->rank();
    c->worldSize = bs->world();
    c->localRank = bs->local_rank();
    c->localSize = bs->world();  // single node
    c->useMpi = use_mpi;
    c->peerHandles = static_cast<cudaIpcMemHandle_t*>(std::calloc(c->worldSize, sizeof(cudaIpcMemHandle_t)));
    c->peerPtrs = static_cast<void**>(std::calloc(c->worldSize, sizeof(void*)));
    uint64_t id = 0;
    if (c->rank == 0) id = (static_cast<uint64_t>(std::rand()) << 32) ^ static_cast<uint64_t>(reinterpret_cast<uintptr_t>(c));
    bs->broadcast(&id, sizeof(id), 0);
    c->uniqueId = id;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) == cudaSuccess && ndev > 0) {
        cudaSetDevice(c->localRank % ndev);
        cudaStreamCreate(&c->stream);
    } else {
        (void)cudaGetLastError();
    }
    c->bootstrap = bs.release();
    return c;
}

void yaliMPCommDestroy(YaliMPComm* c) {
    if (!c) return;
    yaliIpcCloseAll(c);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete BS(c);
    std::free(c->peerHandles);
    std::free(c->peerPtrs);
    std::free(c);
}

void yaliMPCommBarrier(YaliMPComm* c) {
    if (!c) return;
    if (c->stream) cudaStreamSynchronize(c->stream);
    BS(c)->barrier();
}

void yaliMPCommBroadcast(YaliMPComm* c, void* data, size_t bytes) {
    if (!c) return;
    BS(c)->broadcast(data, bytes, 0);
}

int yaliMPCommAllgather(YaliMPComm* c, const void* in, void* out, size_t bytes) {
    if (!c) return -1;
    return BS(c)->allgather(in, out, bytes) == yali::Result::Success ? 0 : -1;
}

cudaError_t yaliIpcExport(void* devPtr, size_t size, YaliIpcHandle* h) {
    if (!devPtr || !h) return cudaErrorInvalidValue;
    std::memset(h, 0, sizeof(*h));
    // The IPC handle names the whole allocation; remember where devPtr sits inside it.
    void* base = devPtr;
    std::string derr;
    if (const yali::DriverApi* d = yali::DriverApi::Get(&derr)) {
        CUdeviceptr b = 0;
        size_t range = 0;
        if (d->MemGetAddressRange(&b, &range, reinterpret_cast<CUdeviceptr>(devPtr)) == CUDA_SUCCESS)
            base = reinterpret_cast<void*>(b);
    }
    cudaError_t e = cudaIpcGetMemHandle(&h->handle, base);
    if (e != cudaSuccess) return e;
    h->size = size;
    h->offset = static_cast<size_t>(static_cast<char*>(devPtr) - static_cast<char*>(base));
    h->srcRank = -1;
    return cudaSuccess;
}

cudaError_t yaliIpcImport(const YaliIpcHandle* h, void** devPtr) {
    if (!h || !devPtr) return cudaErrorInvalidValue;
    void* base = nullptr;
    for (Opened& o : OpenTable()) {
        if (std::memcmp(&o.handle, &h->handle, sizeof(cudaIpcMemHandle_t)) == 0) {
            base = o.base;
            ++o.refs;
            break;
        }
    }
    if (!base) {
        cudaError_t e = cudaIpcOpenMemHandle(&base, h->handle, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return e;
        OpenTable().push_back({h->handle, base, 1});
    }
    *devPtr = static_cast<char*>(base) + h->offset;
    ImportTable().push_back({*devPtr, base});
    return cudaSuccess;
}

cudaError_t yaliIpcClose(void* importedPtr) {
    if (!importedPtr) return cudaSuccess;
    auto& t = ImportTable();
    for (size_t i = 0; i < t.size(); ++i) {
        if (t[i].user == importedPtr) {
            void* base = t[i].base;
            t.erase(t.begin() + i);
            auto& open = OpenTable();
            for (size_t k = 0; k < open.size(); ++k) {
                if (open[k].base == base) {
                    if (--open[k].refs > 0) return cudaSuccess;  // other imports still use the mapping
                    open.erase(open.begin() + k);
                    break;
                }
            }
            return cudaIpcCloseMemHandle(base);
        }
    }
    return cudaIpcCloseMemHandle(importedPtr);
}

int yaliIpcExchangeBuffers(YaliMPComm* c, void* localBuf, size_t size) {
    if (!c || !localBuf) return -1;
    cudaDeviceSynchronize();
    YaliIpcHandle mine;
    char ok = yaliIpcExport(localBuf, size, &mine) == cudaSuccess;
    mine.srcRank = c->rank;
    std::vector<YaliIpcHandle> all(c->worldSize);
    std::vector<char> oks(c->worldSize);
    if (BS(c)->allgather(&ok, oks.data(), 1) != yali::Result::Success) return -1;
    for (char o : oks)
        if (!o) return -1;
    if (BS(c)->allgather(&mine, all.data(), sizeof(mine)) != yali::Result::Success) return -1;
    char open_ok = 1;
    for (int r = 0; r < c->worldSize; ++r) {
        c->peerHandles[r] = all[r].handle;
        if (r == c->rank) {
            c->peerPtrs[r] = localBuf;
        } else if (yaliIpcImport(&all[r], &c->peerPtrs[r]) != cudaSuccess) {
            (void)cudaGetLastError();
            c->peerPtrs[r] = nullptr;
            open_ok = 0;
        }
    }
    if (BS(c)->allgather(&open_ok, oks.data(), 1) != yali::Result::Success) return -1;
    for (char o : oks) {
        if (!o) {
            yaliIpcCloseAll(c);
            return -1;
        }
    }
    return 0;
}

void yaliIpcCloseAll(YaliMPComm* c) {
    if (!c || !c->peerPtrs) return;
    for (int r = 0; r < c->worldSize; ++r) {
        if (r != c->rank && c->peerPtrs[r]) yaliIpcClose(c->peerPtrs[r]);
        c->peerPtrs[r] = nullptr;
    }
}

int yaliIpcExchangeRingBuffers(YaliMPComm* c, const YaliRingDesc* rings, int numLanes, void*** peerSequence,
                               void*** peerGating, void*** peerData) {
    if (!c || !rings || numLanes <= 0 || !peerSequence || !peerGating || !peerData) return -1;
    cudaDeviceSynchronize();
    const int W = c->worldSize;
    std::vector<YaliIpcHandle> mine(3 * numLanes), all(static_cast<size_t>(3) * numLanes * W);
    char ok = 1;
    for (int l = 0; l < numLanes; ++l) {
        ok = ok && yaliIpcExport(rings[l].sequence, rings[l].sequenceBytes, &mine[3 * l]) == cudaSuccess &&
             yaliIpcExport(rings[l].gating, rings[l].gatingBytes, &mine[3 * l + 1]) == cudaSuccess &&
             yaliIpcExport(rings[l].data, rings[l].dataBytes, &mine[3 * l + 2]) == cudaSuccess;
    }
    std::vector<char> oks(W);
    if (BS(c)->allgather(&ok, oks.data(), 1) != yali::Result::Success) return -1;
    for (char o : oks)
        if (!o) return -1;
    if (BS(c)->allgather(mine.data(), all.data(), sizeof(YaliIpcHandle) * mine.size()) != yali::Result::Success)
        return -1;
    void** seq = static_cast<void**>(std::calloc(static_cast<size_t>(W) * numLanes, sizeof(void*)));
    void** gat = static_cast<void**>(std::calloc(static_cast<size_t>(W) * numLanes, sizeof(void*)));
    void** dat = static_cast<void**>(std::calloc(static_cast<size_t>(W) * numLanes, sizeof(void*)));
    char open_ok = seq && gat && dat;
    for (int r = 0; r < W && open_ok; ++r) {
        for (int l = 0; l < numLanes && open_ok; ++l) {
            const size_t i = static_cast<size_t>(r) * numLanes + l;
            if (r == c->rank) {
                seq[i] = rings[l].sequence;
                gat[i] = rings[l].gating;
                dat[i] = rings[l].data;
                continue;
            }
            const YaliIpcHandle* h = &all[(static_cast<size_t>(r) * numLanes + l) * 3];
            open_ok = yaliIpcImport(&h[0], &seq[i]) == cudaSuccess && yaliIpcImport(&h[1], &gat[i]) == cudaSuccess &&
                      yaliIpcImport(&h[2], &dat[i]) == cudaSuccess;
        }
    }
    if (!open_ok) (void)cudaGetLastError();
    if (BS(c)->allgather(&open_ok, oks.data(), 1) != yali::Result::Success) open_ok = 0;
    for (char o : oks)
        if (!o) open_ok = 0;
    if (!open_ok) {
        yaliIpcCloseRingBuffers(c, numLanes, seq, gat, dat);
        return -1;
    }
    *peerSequence = seq;
    *peerGating = gat;
    *peerData = dat;
    return 0;
}

void yaliIpcCloseRingBuffers(YaliMPComm* c, int numLanes, void** seq, void** gat, void** dat) {
    if (!c) return;
    for (int r = 0; r < c->worldSize; ++r) {
        if (r == c->rank) continue;
        for (int l = 0; l < numLanes; ++l) {
            const size_t i = static_cast<size_t>(r) * numLanes + l;
            if (seq && seq[i]) yaliIpcClose(seq[i]);
            if (gat && gat[i]) yaliIpcClose(gat[i]);
            if (dat && dat[i]) yaliIpcClose(dat[i]);
        }
    }
    std::free(seq);
    std::free(gat);
    std::free(dat);
}

}  // extern "C"
