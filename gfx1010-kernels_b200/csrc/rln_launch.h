// Internal launch interface between the C-ABI translation unit and the two
// kernel-instantiating translation units (split so they compile in parallel).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "rln_kernels.cuh"

namespace rln {

// Compile-time launch geometry per hidden size.  kWarps warps per CTA, each
// warp handles kRows consecutive rows per loop iteration (more rows in flight
// for narrow rows).  kCtasPerSm sizes the persistent backward grid; it is a
// constant (not an occupancy query) so that the deterministic partial layout
// depends only on (hidden, rows, SM count).
template <int H>
struct ForwardTune {
    static constexpr int kWarps = 4;
    static constexpr int kRows = H <= 128 ? 4 : (H <= 256 ? 2 : 1);
};

template <int H>
struct BackwardTune {
    static constexpr int kWarps = 4;
    static constexpr int kRows = H <= 128 ? 4 : (H <= 256 ? 2 : 1);
    static constexpr int kCtasPerSm = H <= 512 ? 6 : (H <= 768 ? 4 : 3);
};

// Number of CTAs of the persistent backward grid (pure function of its
// arguments; also the number of [2, hidden] partials in deterministic mode).
int backward_grid(int hidden, int64_t rows, int sm_count);

cudaError_t launch_forward(
    int hidden,
    bool branch_is_half,
    bool dropout,
    bool aligned,
    const ForwardParams& params,
    cudaStream_t stream);

cudaError_t launch_backward(
    int hidden,
    bool branch_is_half,
    bool dropout,
    bool parameters,
    bool aligned,
    const BackwardParams& params,
    int grid,
    cudaStream_t stream);

cudaError_t launch_reduce_partials(
    const float* partials,
    float* out,
    int partial_count,
    int columns,
    cudaStream_t stream);

}  // namespace rln
