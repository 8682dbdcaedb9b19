// Host-side entry points of the kernel translation units.  Each returns the
// __global__ function for a (dtype, epilogue, world) combination so that the
// dispatcher can launch it with cudaLaunchKernel (one rank per launch) or, for
// an emulated communicator whose ranks share one GPU, with a cooperative launch
// of the *_emu twin (ranks = blockIdx.y), which guarantees that all CTAs that
// wait on one another are resident together.
//
// Parity: src/all_reduce/kernels.cuh:41-55 (LaunchFlashKernel) and the
// extern "C" YaliKernel symbols of src/kernels/stream.cu:104-111.
#pragma once

#include <cuda_runtime.h>

#include "../comm/layout.h"

namespace yali {

constexpr int kFlashThreads = 512;
constexpr int kStreamThreads = 512;
constexpr int kNvlsThreads = 512;
constexpr int kDirectThreads = 288;   // one producer warp + eight consumer warps
constexpr int kDirectMaxStages = kMaxPipelineStages;

// nullptr when the combination is not built.
const void* FlashKernelFor(Dtype in, Dtype out, int epilogue, int world, bool emu);
// Flag-in-data form of the one-shot kernel (equal in/out type, scale epilogue only).
const void* FlashLLKernelFor(Dtype dt, int world, bool emu);
const void* StreamKernelFor(Dtype in, Dtype out, int epilogue, int world, bool emu);
const void* NvlsKernelFor(Dtype dt, int world, bool two_shot);
// Pipelined direct kernel (all buffers peer-addressable): one-shot pull or two-shot pull + push.
const void* DirectKernelFor(Dtype in, Dtype out, int world, bool one_shot, bool emu);

}  // namespace yali
