// Backward entry of the launch interface, the persistent-grid rule, the
// float32-`grad_normalized` kernels and the two small helper kernels.
#include "rln_backward_dispatch.cuh"

namespace rln {
namespace {

template <int H>
int backward_grid_hidden(int64_t rows, int sm_count) {
    constexpr int64_t kRowsPerCta =
        static_cast<int64_t>(BackwardTune<H>::kWarps) * BackwardTune<H>::kRows;
    const int64_t needed = (rows + kRowsPerCta - 1) / kRowsPerCta;
    const int64_t resident = static_cast<int64_t>(sm_count) * BackwardTune<H>::kCtasPerSm;
    return static_cast<int>(needed < resident ? needed : resident);
}

}  // namespace

int backward_grid(int hidden, int64_t rows, int sm_count) {
    switch (hidden) {
        case 128: return backward_grid_hidden<128>(rows, sm_count);
        case 256: return backward_grid_hidden<256>(rows, sm_count);
        case 384: return backward_grid_hidden<384>(rows, sm_count);
        case 512: return backward_grid_hidden<512>(rows, sm_count);
        case 768: return backward_grid_hidden<768>(rows, sm_count);
        case 1024: return backward_grid_hidden<1024>(rows, sm_count);
        default: return 0;
    }
}

cudaError_t launch_backward(
    int hidden,
    int branch_kind,
    int normalized_kind,
    bool dropout,
    bool parameters,
    bool aligned,
    const BackwardParams& params,
    int grid,
    cudaStream_t stream) {
    switch (normalized_kind) {
        case 0:
            return launch_backward_normalized_as<float, false>(
                hidden, branch_kind, dropout, parameters, aligned, params, grid, stream);
        case 1:
            return launch_backward_normalized_half(
                hidden, branch_kind, dropout, parameters, aligned, params, grid, stream);
        case 2:
            return launch_backward_normalized_bfloat16(
                hidden, branch_kind, dropout, parameters, aligned, params, grid, stream);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_reduce_partials(
    const float* partials,
    float* out,
    int partial_count,
    int columns,
    cudaStream_t stream) {
    constexpr int kSegments = 32;  // one warp per range: 1,024 threads per 32 columns
    const int blocks = (columns + kWarpSize - 1) / kWarpSize;
    return launch_dependent(
        rln_reduce_partials_kernel<kSegments>,
        static_cast<unsigned>(blocks),
        kSegments * kWarpSize,
        stream,
        partials,
        out,
        partial_count,
        columns);
}

cudaError_t launch_zero(float* out, int count, cudaStream_t stream) {
    constexpr int kThreads = 256;
    const int count4 = count / 4;
    const int blocks = (count4 + kThreads - 1) / kThreads;
    return launch_dependent(
        rln_zero_kernel<kThreads>,
        static_cast<unsigned>(blocks > 0 ? blocks : 1),
        kThreads,
        stream,
        reinterpret_cast<float4*>(out),
        count4,
        static_cast<uint4*>(nullptr));
}

}  // namespace rln
