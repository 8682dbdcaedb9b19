// Result codes, data types and small POD configuration structs of the library.
//
// Parity: the reference declares Result/Dtype in src/include/yali.h:27-76 and
// DataType/ReduceOp/KernelMode/AllReduceConfig/AllReduceResult in
// src/all_reduce/all_reduce.h:18-92.  The enumerators kept here have the same
// names; Timeout/Unsupported/BootstrapError and the NVLS kernel mode are new
// because this library bounds every device-side wait and has a multicast path.
#pragma once

#include <cstddef>
#include <cstdint>

namespace yali {

enum class Result : int {
    Success = 0,
    InvalidArg,
    CudaError,
    PeerAccessFailed,
    NotInitialized,
    Timeout,         // a device-side wait ran out; the communicator is poisoned until reset()
    Unsupported,     // shape / dtype / feature not available on this box
    BootstrapError,  // rendezvous or handle exchange between ranks failed
};

inline const char* GetErrorString(Result r) {
    switch (r) {
        case Result::Success: return "Success";
        case Result::InvalidArg: return "Invalid argument";
        case Result::CudaError: return "CUDA error";
        case Result::PeerAccessFailed: return "Peer access failed";
        case Result::NotInitialized: return "Not initialized";
        case Result::Timeout: return "Device-side wait timed out";
        case Result::Unsupported: return "Unsupported";
        case Result::BootstrapError: return "Bootstrap error";
    }
    return "Unknown error";
}

enum class Dtype : int { FP32 = 0, FP16 = 1, BF16 = 2 };

inline size_t DtypeSize(Dtype d) { return d == Dtype::FP32 ? 4 : 2; }
inline const char* DtypeName(Dtype d) {
    switch (d) {
        case Dtype::FP32: return "fp32";
        case Dtype::FP16: return "fp16";
        case Dtype::BF16: return "bf16";
    }
    return "unknown";
}
// Parses "fp32"/"f32"/"float", "fp16"/"f16"/"half", "bf16"/"bfloat16"; returns false on anything else.
bool ParseDtype(const char* s, Dtype* out);

// Interface-level aliases with the spelling of the reference's all_reduce.h.
enum class DataType : int { Float32 = 0, Float16 = 1, BFloat16 = 2 };
enum class ReduceOp : int { Sum = 0 };
// FlashPull / StreamDirect force the pipelined kernels that read the peers' inputs in place
// (they need buffers every rank can address); Auto picks them when they apply.  CopyEngine lets
// cudaMemcpyAsync move the payload between the GPUs and keeps kernels for the additions and the flags.
enum class KernelMode : int { Auto = 0, Flash = 1, Stream = 2, NVLS = 3, FlashPull = 4, StreamDirect = 5, CopyEngine = 6 };

inline Dtype ToDtype(DataType d) { return static_cast<Dtype>(static_cast<int>(d)); }
inline DataType ToDataType(Dtype d) { return static_cast<DataType>(static_cast<int>(d)); }
inline size_t ElementSize(DataType d) { return DtypeSize(ToDtype(d)); }
inline const char* DataTypeName(DataType d) { return DtypeName(ToDtype(d)); }
inline const char* KernelModeName(KernelMode m) {
    switch (m) {
        case KernelMode::Flash: return "flash";
        case KernelMode::Stream: return "stream";
        case KernelMode::NVLS: return "nvls";
        case KernelMode::FlashPull: return "flash_pull";
        case KernelMode::StreamDirect: return "stream_direct";
        case KernelMode::CopyEngine: return "copy_engine";
        case KernelMode::Auto: break;
    }
    return "auto";
}
bool ParseKernelMode(const char* s, KernelMode* out);

struct AllReduceConfig {
    int num_ranks = 2;
    int lanes = -1;          // -1: from the tuning table
    int ctas_per_lane = -1;  // -1: from the tuning table
    KernelMode kernel_mode = KernelMode::Auto;
    int warmup_iters = 1;
    int measure_iters = 5;
};

struct AllReduceResult {
    bool success;
    double latency_us;
    double bandwidth_gbps;  // NCCL-convention bus bandwidth
    double aggregate_gbps;  // bus bandwidth x ranks
    const char* error_msg;
};

constexpr int kMaxRanks = 8;

}  // namespace yali
