// Thin PyTorch layer: the communicator and its collectives over torch tensors on
// the current CUDA stream, buffer utilities, topology and tuning queries.
// The functional torch.ops.yali.* operators are registered from Python on top of
// these entry points (yali_b200/ops/registry.py).
//
// Parity: the reference has no framework layer (its README.md:199-203 lists the
// C++ headers as the only interface); this file is an addition.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <memory>
#include <string>
#include <vector>

#include "comm/communicator.h"
#include "comm/topology.h"
#include "ops/buffer_ops.h"
#include "ops/fused_linear.h"
#include "ops/host_pipeline.h"
#include "ops/tuning.h"

namespace py = pybind11;
using namespace yali;

namespace {

Dtype ToDtype(at::ScalarType t) {
    switch (t) {
        case at::kFloat: return Dtype::FP32;
        case at::kHalf: return Dtype::FP16;
        case at::kBFloat16: return Dtype::BF16;
        default: TORCH_CHECK(false, "yali: unsupported dtype ", t, " (fp32, fp16, bf16 only)");
    }
}

KernelMode ToMode(const std::string& s) {
    KernelMode m;
    TORCH_CHECK(ParseKernelMode(s.c_str(), &m), "yali: unknown kernel mode '", s, "'");
    return m;
}

void Throw(Result r, const std::string& what) {
    if (r == Result::Success) return;
    std::string msg = std::string("yali: ") + GetErrorString(r) + (what.empty() ? "" : ": " + what);
    if (r == Result::Timeout) throw std::runtime_error("YaliTimeout: " + msg);
    throw std::runtime_error(msg);
}

class PyComm {
   public:
    static std::shared_ptr<PyComm> SingleProcess(std::vector<int> devices, uint64_t heap_bytes, bool want_mc,
                                                 int64_t timeout_ms) {
        auto p = std::make_shared<PyComm>();
        CommOptions o;
        o.heap_bytes = heap_bytes;
        o.want_multicast = want_mc;
        o.timeout_ms = timeout_ms;
        std::string err;
        Throw(Communicator::CreateSingleProcess(devices, o, &p->c_, &err), err);
        return p;
    }
    static std::shared_ptr<PyComm> Emulated(int world, int device, uint64_t heap_bytes, int64_t timeout_ms) {
        auto p = std::make_shared<PyComm>();
        CommOptions o;
        o.heap_bytes = heap_bytes;
        o.want_multicast = false;
        o.timeout_ms = timeout_ms;
        std::string err;
        Throw(Communicator::CreateEmulated(world, device, o, &p->c_, &err), err);
        return p;
    }
    static std::shared_ptr<PyComm> FromEnv(int device, uint64_t heap_bytes, bool want_mc, int64_t timeout_ms) {
        auto p = std::make_shared<PyComm>();
        Result r = Result::Success;
        std::string err;
        std::unique_ptr<Bootstrap> bs;
        {
            py::gil_scoped_release nogil;
            bs = MakeEnvBootstrap(&r, &err);
        }
        if (!bs) Throw(r == Result::Success ? Result::BootstrapError : r, err);
        if (device < 0) {
            int ndev = 0;
            TORCH_CHECK(cudaGetDeviceCount(&ndev) == cudaSuccess && ndev > 0, "yali: no CUDA device");
            device = bs->local_rank() % ndev;
        }
        CommOptions o;
        o.heap_bytes = heap_bytes;
        o.want_multicast = want_mc;
        o.timeout_ms = timeout_ms;
        {
            py::gil_scoped_release nogil;
            r = Communicator::CreateMultiProcess(std::move(bs), device, o, &p->c_, &err);
        }
        Throw(r, err);
        return p;
    }

    void Close() {
        py::gil_scoped_release nogil;
        host_pipe_.reset();
        c_.reset();
    }
    Communicator& c() {
        TORCH_CHECK(c_ != nullptr, "yali: communicator is closed");
        return *c_;
    }

    int world() { return c().world(); }
    int nlocal() { return c().nlocal(); }
    int rank(int i) { return c().rank_of(i); }
    int device(int i) { return c().device_of(i); }
    bool emulated() { return c().emulated(); }
    bool has_multicast() { return c().has_multicast(); }
    std::string heap_kind() { return c().heap_kind(); }
    uint64_t launches() { return c().last_call().launches; }
    py::dict layout() {
        const HeapLayout& l = c().layout();
        py::dict d;
        d["total_bytes"] = l.total_bytes;
        d["flash_cap"] = l.flash_cap;
        d["ring_bytes"] = l.ring_bytes;
        d["nvls_cap"] = l.nvls_cap;
        d["gemm_cap"] = l.gemm_cap;
        d["user_bytes"] = l.user_bytes;
        return d;
    }
    py::dict last_call() {
        const LastCallInfo& l = c().last_call();
        py::dict d;
        d["variant"] = VariantName(l.variant);
        d["ctas"] = l.ctas;
        d["slot_bytes"] = l.slot_bytes;
        d["stages"] = l.stages;
        d["flags"] = l.flags;
        d["launches"] = l.launches;
        return d;
    }

    void SetTrace(bool on) { c().SetTrace(on); }
    // Device-side timeline of local rank `local_index`: (traced calls so far, [(start_ns, end_ns), ...])
    // for the most recent calls, oldest first.  Synchronise before reading.
    py::tuple ReadTrace(int local_index, int max_entries) {
        std::vector<uint64_t> buf(static_cast<size_t>(std::max(max_entries, 1)) * 2);
        uint64_t calls = 0;
        const int n = c().ReadTrace(local_index, buf.data(), max_entries, &calls);
        py::list out;
        for (int k = 0; k < n; ++k) out.append(py::make_tuple(buf[2 * k], buf[2 * k + 1]));
        return py::make_tuple(calls, out);
    }

    void CheckTensors(const std::vector<at::Tensor>& ts, const char* what, at::ScalarType* dt, int64_t* numel) {
        TORCH_CHECK(static_cast<int>(ts.size()) == c().nlocal(), "yali: expected ", c().nlocal(), " ", what,
                    " tensors (one per local rank), got ", ts.size());
        for (int i = 0; i < c().nlocal(); ++i) {
            const at::Tensor& t = ts[i];
            TORCH_CHECK(t.is_cuda(), "yali: ", what, "[", i, "] is not a CUDA tensor");
            TORCH_CHECK(t.is_contiguous(), "yali: ", what, "[", i, "] is not contiguous");
            TORCH_CHECK(t.get_device() == c().device_of(i), "yali: ", what, "[", i, "] lives on GPU ", t.get_device(),
                        ", rank ", c().rank_of(i), " owns GPU ", c().device_of(i));
            if (i == 0) {
                *dt = t.scalar_type();
                *numel = t.numel();
            } else {
                TORCH_CHECK(t.scalar_type() == *dt && t.numel() == *numel, "yali: ", what,
                            " tensors differ in dtype or size");
            }
        }
    }
    std::vector<cudaStream_t> Streams() {
        std::vector<cudaStream_t> s(c().nlocal());
        for (int i = 0; i < c().nlocal(); ++i) s[i] = at::cuda::getCurrentCUDAStream(c().device_of(i)).stream();
        return s;
    }

    void AllReduce(std::vector<at::Tensor> send, std::vector<at::Tensor> recv, const std::string& mode,
                   c10::optional<double> scale, int ctas, int slot_bytes, int skip_rank) {
        at::ScalarType sd, rd;
        int64_t sn, rn;
        CheckTensors(send, "send", &sd, &sn);
        CheckTensors(recv, "recv", &rd, &rn);
        TORCH_CHECK(sn == rn, "yali: send and recv differ in size");
        OpOptions o;
        o.mode = ToMode(mode);
        o.ctas = ctas;
        o.slot_bytes = slot_bytes;
        o.skip_rank = skip_rank;
        if (scale.has_value() || sd != rd) {
            o.epilogue = kEpiScaleCast;
            o.scale = static_cast<float>(scale.value_or(1.0));
        }
        std::vector<const void*> s(send.size());
        std::vector<void*> r(recv.size());
        for (size_t i = 0; i < send.size(); ++i) {
            s[i] = send[i].data_ptr();
            r[i] = recv[i].data_ptr();
        }
        auto st = Streams();
        c10::cuda::OptionalCUDAGuard guard(c().device_of(0));
        Result res = c().AllReduce(s.data(), r.data(), sn, ToDtype(sd), ToDtype(rd), o, st.data());
        Throw(res, c().last_error());
    }

    void AllReduceRmsNorm(std::vector<at::Tensor> send, std::vector<at::Tensor> recv,
                          c10::optional<std::vector<at::Tensor>> residual,
                          c10::optional<std::vector<at::Tensor>> residual_out, std::vector<at::Tensor> weight,
                          double eps, const std::string& mode, int ctas) {
        at::ScalarType sd, rd, wd;
        int64_t sn, rn, wn;
        CheckTensors(send, "send", &sd, &sn);
        CheckTensors(recv, "recv", &rd, &rn);
        CheckTensors(weight, "weight", &wd, &wn);
        TORCH_CHECK(sd == rd && sd == wd && sn == rn, "yali: rmsnorm tensors must agree in dtype and size");
        TORCH_CHECK(wn > 0 && sn % wn == 0, "yali: input size is not a multiple of the hidden size");
        OpOptions o;
        o.mode = ToMode(mode);
        o.ctas = ctas;
        o.epilogue = kEpiResidualRmsNorm;
        o.hidden = static_cast<int>(wn);
        o.eps = static_cast<float>(eps);
        const int n = c().nlocal();
        std::vector<const void*> s(n), w(n), res(n, nullptr);
        std::vector<void*> r(n), ro(n, nullptr);
        for (int i = 0; i < n; ++i) {
            s[i] = send[i].data_ptr();
            r[i] = recv[i].data_ptr();
            w[i] = weight[i].data_ptr();
        }
        if (residual.has_value()) {
            at::ScalarType d;
            int64_t m;
            CheckTensors(*residual, "residual", &d, &m);
            TORCH_CHECK(d == sd && m == sn, "yali: residual must match the input");
            for (int i = 0; i < n; ++i) res[i] = (*residual)[i].data_ptr();
            o.residual = res.data();
        }
        if (residual_out.has_value()) {
            at::ScalarType d;
            int64_t m;
            CheckTensors(*residual_out, "residual_out", &d, &m);
            TORCH_CHECK(d == sd && m == sn, "yali: residual_out must match the input");
            for (int i = 0; i < n; ++i) ro[i] = (*residual_out)[i].data_ptr();
            o.residual_out = ro.data();
        }
        o.weight = w.data();
        auto st = Streams();
        c10::cuda::OptionalCUDAGuard guard(c().device_of(0));
        Throw(c().AllReduce(s.data(), r.data(), sn, ToDtype(sd), ToDtype(rd), o, st.data()), c().last_error());
    }

    // send: full message per rank; recv: ShardElems(count, world) elements per rank.
    void ReduceScatter(std::vector<at::Tensor> send, std::vector<at::Tensor> recv, int ctas, int slot_bytes) {
        at::ScalarType sd, rd;
        int64_t sn, rn;
        CheckTensors(send, "send", &sd, &sn);
        CheckTensors(recv, "recv", &rd, &rn);
        TORCH_CHECK(sd == rd, "yali: dtype mismatch");
        TORCH_CHECK(static_cast<uint64_t>(rn) >= ShardElems(sn, c().world()) || c().world() == 1,
                    "yali: recv needs shard_elems(count, world) elements");
        Run(send, recv, sn, ToDtype(sd), ctas, slot_bytes, true);
    }
    // send: ShardElems elements per rank; recv: `count` elements.
    void AllGather(std::vector<at::Tensor> send, std::vector<at::Tensor> recv, int ctas, int slot_bytes) {
        at::ScalarType sd, rd;
        int64_t sn, rn;
        CheckTensors(send, "send", &sd, &sn);
        CheckTensors(recv, "recv", &rd, &rn);
        TORCH_CHECK(sd == rd, "yali: dtype mismatch");
        TORCH_CHECK(static_cast<uint64_t>(sn) >= ShardElems(rn, c().world()) || c().world() == 1,
                    "yali: send needs shard_elems(count, world) elements");
        Run(send, recv, rn, ToDtype(sd), ctas, slot_bytes, false);
    }
    void Run(std::vector<at::Tensor>& send, std::vector<at::Tensor>& recv, int64_t count, Dtype dt, int ctas,
             int slot_bytes, bool rs) {
        OpOptions o;
        o.ctas = ctas;
        o.slot_bytes = slot_bytes;
        std::vector<const void*> s(send.size());
        std::vector<void*> r(recv.size());
        for (size_t i = 0; i < send.size(); ++i) {
            s[i] = send[i].data_ptr();
            r[i] = recv[i].data_ptr();
        }
        auto st = Streams();
        c10::cuda::OptionalCUDAGuard guard(c().device_of(0));
        Result res = rs ? c().ReduceScatter(s.data(), r.data(), count, dt, o, st.data())
                        : c().AllGather(s.data(), r.data(), count, dt, o, st.data());
        Throw(res, c().last_error());
    }

    // out = RMSNorm(residual + sum_r x_r @ w_r^T) * norm_weight, one kernel per rank.
    void FusedLinear(std::vector<at::Tensor> x, std::vector<at::Tensor> w, std::vector<at::Tensor> norm_weight,
                     std::vector<at::Tensor> out, c10::optional<std::vector<at::Tensor>> residual,
                     c10::optional<std::vector<at::Tensor>> residual_out, double eps, int force_oneshot, int ctas,
                     c10::optional<std::vector<at::Tensor>> trace, int nvls, int decode) {
        at::ScalarType d;
        int64_t n;
        CheckTensors(x, "x", &d, &n);
        TORCH_CHECK(d == at::kBFloat16, "yali: fused linear takes bf16 tensors");
        CheckTensors(w, "w", &d, &n);
        TORCH_CHECK(d == at::kBFloat16, "yali: fused linear takes bf16 tensors");
        CheckTensors(norm_weight, "norm_weight", &d, &n);
        TORCH_CHECK(d == at::kBFloat16, "yali: fused linear takes bf16 tensors");
        CheckTensors(out, "out", &d, &n);
        TORCH_CHECK(d == at::kBFloat16, "yali: fused linear takes bf16 tensors");
        TORCH_CHECK(x[0].dim() == 2 && w[0].dim() == 2 && out[0].dim() == 2, "yali: x [T,K], w [N,K], out [T,N]");
        const int64_t T = x[0].size(0), K = x[0].size(1), N = w[0].size(0);
        TORCH_CHECK(w[0].size(1) == K && out[0].size(0) == T && out[0].size(1) == N && norm_weight[0].numel() == N,
                    "yali: fused linear shape mismatch");
        const int nl = c().nlocal();
        std::vector<FusedLinearDesc> descs(nl);
        for (int i = 0; i < nl; ++i) {
            descs[i].x = x[i].data_ptr();
            descs[i].w = w[i].data_ptr();
            descs[i].norm_weight = norm_weight[i].data_ptr();
            descs[i].out = out[i].data_ptr();
        }
        if (residual.has_value()) {
            CheckTensors(*residual, "residual", &d, &n);
            TORCH_CHECK(d == at::kBFloat16 && n == T * N, "yali: residual must be bf16 [T,N]");
            for (int i = 0; i < nl; ++i) descs[i].residual = (*residual)[i].data_ptr();
        }
        if (residual_out.has_value()) {
            CheckTensors(*residual_out, "residual_out", &d, &n);
            TORCH_CHECK(d == at::kBFloat16 && n == T * N, "yali: residual_out must be bf16 [T,N]");
            for (int i = 0; i < nl; ++i) descs[i].residual_out = (*residual_out)[i].data_ptr();
        }
        FusedLinearOptions o;
        o.force_oneshot = force_oneshot;
        o.ctas = ctas;
        o.nvls = nvls;
        o.decode = decode;
        o.eps = static_cast<float>(eps);
        std::vector<unsigned long long*> tr(nl, nullptr);
        if (trace.has_value()) {
            TORCH_CHECK(static_cast<int>(trace->size()) == nl, "yali: one trace tensor per local rank");
            for (int i = 0; i < nl; ++i) {
                TORCH_CHECK((*trace)[i].scalar_type() == at::kLong && (*trace)[i].numel() >= 8 && (*trace)[i].is_cuda(),
                            "yali: trace tensors are int64 CUDA tensors with 8 elements");
                tr[i] = reinterpret_cast<unsigned long long*>((*trace)[i].data_ptr());
            }
            o.trace = tr.data();
        }
        auto st = Streams();
        c10::cuda::OptionalCUDAGuard guard(c().device_of(0));
        Throw(FusedLinearAllReduceRmsNorm(c(), descs.data(), static_cast<uint32_t>(T), static_cast<uint32_t>(N),
                                          static_cast<uint32_t>(K), o, st.data()),
              c().last_error());
    }

    // One tensor per local rank, at the same offset of every rank's heap.  The tensors alias
    // heap memory: they stay valid until the communicator is closed.
    std::vector<at::Tensor> SymmEmpty(std::vector<int64_t> shape, at::ScalarType dtype) {
        int64_t n = 1;
        for (int64_t d : shape) n *= d;
        std::vector<void*> ptrs;
        Throw(c().SymmAlloc(static_cast<uint64_t>(n) * c10::elementSize(dtype), &ptrs), c().last_error());
        std::vector<at::Tensor> out;
        for (int i = 0; i < c().nlocal(); ++i) {
            auto opts = at::TensorOptions().dtype(dtype).device(at::kCUDA, c().device_of(i));
            out.push_back(at::from_blob(ptrs[i], shape, [](void*) {}, opts));
        }
        return out;
    }
    void SymmReset() {
        if (host_pipe_) host_pipe_->Invalidate();
        c().SymmReset();
    }

    // dst = scale * sum over ranks of src, both in pinned host memory; copies and all-reduce
    // overlap chunk by chunk (ops/host_pipeline.h).
    void AllReduceHost(std::vector<at::Tensor> src, std::vector<at::Tensor> dst, int64_t chunk_bytes,
                       c10::optional<double> scale, const std::string& mode, bool copies_only) {
        const int nl = c().nlocal();
        TORCH_CHECK(static_cast<int>(src.size()) == nl && static_cast<int>(dst.size()) == nl,
                    "yali: one src and one dst tensor per local rank");
        const at::ScalarType d = src[0].scalar_type();
        const int64_t n = src[0].numel();
        std::vector<const void*> s(nl);
        std::vector<void*> r(nl);
        for (int i = 0; i < nl; ++i) {
            for (const at::Tensor& t : {src[i], dst[i]}) {
                TORCH_CHECK(!t.is_cuda() && t.is_pinned() && t.is_contiguous(),
                            "yali: all_reduce_host takes contiguous tensors in pinned host memory");
                TORCH_CHECK(t.scalar_type() == d && t.numel() == n, "yali: src and dst must agree in size and dtype");
            }
            s[i] = src[i].data_ptr();
            r[i] = dst[i].data_ptr();
        }
        OpOptions o;
        o.mode = ToMode(mode);
        if (scale.has_value()) {
            o.epilogue = kEpiScaleCast;
            o.scale = static_cast<float>(*scale);
        }
        if (!host_pipe_) host_pipe_ = std::make_unique<HostPipeline>(c());
        auto st = Streams();
        c10::cuda::OptionalCUDAGuard guard(c().device_of(0));
        Throw(host_pipe_->AllReduce(s.data(), r.data(), static_cast<uint64_t>(n), ToDtype(d), o,
                                    static_cast<uint64_t>(chunk_bytes <= 0 ? 0 : std::max<int64_t>(chunk_bytes, 4096)), st.data(), copies_only),
              c().last_error());
    }

    void Sync() {
        auto st = Streams();
        Result r;
        {
            py::gil_scoped_release nogil;
            r = c().Sync(st.data());
        }
        Throw(r, c().last_error());
    }
    void Check() { Throw(c().Check(), c().last_error()); }
    void Reset() {
        Result r;
        {
            py::gil_scoped_release nogil;
            r = c().Reset();
        }
        Throw(r, c().last_error());
    }
    void Barrier() {
        Result r;
        {
            py::gil_scoped_release nogil;
            r = c().Barrier();
        }
        Throw(r, c().last_error());
    }
    std::string Status() { return c().DescribeStatus(); }

    // Host-side collectives over the control plane (small Python objects, test plumbing).
    py::bytes AllgatherBytes(const std::string& mine) {
        Bootstrap* bs = c().bootstrap();
        if (!bs) return py::bytes(mine);
        std::string out(mine.size() * bs->world(), '\0');
        Result r;
        {
            py::gil_scoped_release nogil;
            r = bs->allgather(mine.data(), &out[0], mine.size());
        }
        Throw(r, bs->last_error());
        return py::bytes(out);
    }

    std::unique_ptr<Communicator> c_;
    std::unique_ptr<HostPipeline> host_pipe_;
};

void FillRandomT(at::Tensor t, int dist, uint64_t seed) {
    TORCH_CHECK(t.is_cuda() && t.is_contiguous(), "yali: fill_random needs a contiguous CUDA tensor");
    c10::cuda::CUDAGuard g(t.device());
    cudaError_t e = FillRandom(t.data_ptr(), t.numel(), ToDtype(t.scalar_type()), dist, seed,
                               at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(e == cudaSuccess, "yali: fill_random: ", cudaGetErrorString(e));
}

void FillConstantT(at::Tensor t, double v) {
    TORCH_CHECK(t.is_cuda() && t.is_contiguous(), "yali: fill_constant needs a contiguous CUDA tensor");
    c10::cuda::CUDAGuard g(t.device());
    cudaError_t e = FillConstant(t.data_ptr(), t.numel(), ToDtype(t.scalar_type()), static_cast<float>(v),
                                 at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(e == cudaSuccess, "yali: fill_constant: ", cudaGetErrorString(e));
}

py::dict ValidateSumT(at::Tensor out, at::ScalarType in_dtype, int dist, uint64_t seed_base, int world, double scale,
                      c10::optional<double> rtol, c10::optional<double> atol, uint64_t index_offset) {
    TORCH_CHECK(out.is_cuda() && out.is_contiguous(), "yali: validate_sum needs a contiguous CUDA tensor");
    c10::cuda::CUDAGuard g(out.device());
    double rt, at_;
    DefaultTolerance(ToDtype(out.scalar_type()), world, &rt, &at_);
    if (std::fabs(scale) > 1.0) at_ *= std::fabs(scale);
    if (rtol.has_value()) rt = *rtol;
    if (atol.has_value()) at_ = *atol;
    ValidateReport h = {0ull, ~0ull, 0.0};
    ValidateReport* d = nullptr;
    TORCH_CHECK(cudaMalloc(reinterpret_cast<void**>(&d), sizeof(h)) == cudaSuccess, "yali: cudaMalloc failed");
    cudaStream_t s = at::cuda::getCurrentCUDAStream().stream();
    cudaMemcpyAsync(d, &h, sizeof(h), cudaMemcpyHostToDevice, s);
    cudaError_t e = ValidateSumAsync(out.data_ptr(), out.numel(), index_offset, ToDtype(in_dtype),
                                     ToDtype(out.scalar_type()), dist, seed_base, world, static_cast<float>(scale), rt,
                                     at_, d, s);
    cudaMemcpyAsync(&h, d, sizeof(h), cudaMemcpyDeviceToHost, s);
    cudaError_t e2 = cudaStreamSynchronize(s);
    cudaFree(d);
    TORCH_CHECK(e == cudaSuccess && e2 == cudaSuccess, "yali: validate_sum failed: ",
                cudaGetErrorString(e != cudaSuccess ? e : e2));
    py::dict r;
    r["mismatches"] = h.mismatches;
    r["first_mismatch"] = h.mismatches ? py::cast(h.first_mismatch) : py::none();
    r["max_abs_err"] = h.max_abs_err;
    r["rtol"] = rt;
    r["atol"] = at_;
    return r;
}

py::dict TopologyDict() {
    TopologyInfo t = QueryTopology();
    py::dict d;
    d["device_count"] = t.device_count;
    d["all_pairs_connected"] = t.AllPairsConnected();
    d["connected_pairs"] = t.ConnectedPairs();
    py::list mc, fab, names;
    for (int i = 0; i < t.device_count; ++i) {
        mc.append(static_cast<bool>(t.multicast_supported[i]));
        fab.append(static_cast<bool>(t.fabric_handle_supported[i]));
        names.append(t.names[i]);
    }
    d["multicast_supported"] = mc;
    d["fabric_handle_supported"] = fab;
    d["names"] = names;
    return d;
}

}  // namespace

PYBIND11_MODULE(_C, m) {
    m.doc() = "yali_b200 native bindings";
    py::class_<PyComm, std::shared_ptr<PyComm>>(m, "Comm")
        .def_static("single_process", &PyComm::SingleProcess, py::arg("devices"), py::arg("heap_bytes") = 0,
                    py::arg("want_multicast") = true, py::arg("timeout_ms") = -1)
        .def_static("emulated", &PyComm::Emulated, py::arg("world"), py::arg("device") = 0, py::arg("heap_bytes") = 0,
                    py::arg("timeout_ms") = -1)
        .def_static("from_env", &PyComm::FromEnv, py::arg("device") = -1, py::arg("heap_bytes") = 0,
                    py::arg("want_multicast") = true, py::arg("timeout_ms") = -1)
        .def("close", &PyComm::Close)
        .def_property_readonly("world", &PyComm::world)
        .def_property_readonly("nlocal", &PyComm::nlocal)
        .def("rank", &PyComm::rank, py::arg("local_index") = 0)
        .def("device", &PyComm::device, py::arg("local_index") = 0)
        .def_property_readonly("is_emulated", &PyComm::emulated)
        .def_property_readonly("has_multicast", &PyComm::has_multicast)
        .def_property_readonly("heap_kind", &PyComm::heap_kind)
        .def_property_readonly("launches", &PyComm::launches)
        .def("layout", &PyComm::layout)
        .def("last_call", &PyComm::last_call)
        .def("set_trace", &PyComm::SetTrace, py::arg("on"))
        .def("read_trace", &PyComm::ReadTrace, py::arg("local_index") = 0, py::arg("max_entries") = 4096)
        .def("all_reduce", &PyComm::AllReduce, py::arg("send"), py::arg("recv"), py::arg("mode") = "auto",
             py::arg("scale") = py::none(), py::arg("ctas") = 0, py::arg("slot_bytes") = 0, py::arg("skip_rank") = -1)
        .def("all_reduce_rmsnorm", &PyComm::AllReduceRmsNorm, py::arg("send"), py::arg("recv"),
             py::arg("residual") = py::none(), py::arg("residual_out") = py::none(), py::arg("weight"),
             py::arg("eps") = 1e-5, py::arg("mode") = "auto", py::arg("ctas") = 0)
        .def("reduce_scatter", &PyComm::ReduceScatter, py::arg("send"), py::arg("recv"), py::arg("ctas") = 0,
             py::arg("slot_bytes") = 0)
        .def("all_gather", &PyComm::AllGather, py::arg("send"), py::arg("recv"), py::arg("ctas") = 0,
             py::arg("slot_bytes") = 0)
        .def("fused_linear", &PyComm::FusedLinear, py::arg("x"), py::arg("w"), py::arg("norm_weight"), py::arg("out"),
             py::arg("residual") = py::none(), py::arg("residual_out") = py::none(), py::arg("eps") = 1e-5,
             py::arg("force_oneshot") = -1, py::arg("ctas") = 0, py::arg("trace") = py::none(),
             py::arg("nvls") = -1, py::arg("decode") = -1)
        .def("symm_empty", &PyComm::SymmEmpty, py::arg("shape"), py::arg("dtype"))
        .def("symm_reset", &PyComm::SymmReset)
        .def("all_reduce_host", &PyComm::AllReduceHost, py::arg("src"), py::arg("dst"), py::arg("chunk_bytes") = 0,
             py::arg("scale") = py::none(), py::arg("mode") = "auto", py::arg("copies_only") = false)
        .def("sync", &PyComm::Sync)
        .def("check", &PyComm::Check)
        .def("reset", &PyComm::Reset)
        .def("barrier", &PyComm::Barrier)
        .def("status", &PyComm::Status)
        .def("allgather_bytes", &PyComm::AllgatherBytes)
        .def("raw", [](PyComm& p) { return reinterpret_cast<uintptr_t>(&p.c()); });

    m.def("fill_random", &FillRandomT, py::arg("tensor"), py::arg("dist"), py::arg("seed"));
    m.def("fill_constant", &FillConstantT, py::arg("tensor"), py::arg("value"));
    m.def("validate_sum", &ValidateSumT, py::arg("out"), py::arg("in_dtype"), py::arg("dist"), py::arg("seed_base"),
          py::arg("world"), py::arg("scale") = 1.0, py::arg("rtol") = py::none(), py::arg("atol") = py::none(),
          py::arg("index_offset") = 0);
    m.def("topology", &TopologyDict);
    m.def("shard_elems", [](uint64_t count, int world) { return ShardElems(count, world); });
}
