// Backward kernel instantiations, the persistent-grid rule and the dispatch ladder.
#include "rln_launch.h"

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

template <int H, typename BranchT, bool kDropout, bool kParams, bool kAligned>
cudaError_t launch_backward_typed(const BackwardParams& params, int grid, cudaStream_t stream) {
    constexpr int kWarps = BackwardTune<H>::kWarps;
    constexpr int kRows = BackwardTune<H>::kRows;
    return launch_dependent(
        rln_backward_kernel<H, BranchT, kDropout, kParams, kAligned, kWarps, kRows,
                            BackwardTune<H>::kCtasPerSm>,
        static_cast<unsigned>(grid),
        kWarps * kWarpSize,
        stream,
        params);
}

template <int H, typename BranchT, bool kAligned>
cudaError_t launch_backward_branch(
    bool dropout,
    bool parameters,
    const BackwardParams& params,
    int grid,
    cudaStream_t stream) {
    if (dropout) {
        return parameters
            ? launch_backward_typed<H, BranchT, true, true, kAligned>(params, grid, stream)
            : launch_backward_typed<H, BranchT, true, false, kAligned>(params, grid, stream);
    }
    return parameters
        ? launch_backward_typed<H, BranchT, false, true, kAligned>(params, grid, stream)
        : launch_backward_typed<H, BranchT, false, false, kAligned>(params, grid, stream);
}

template <int H, bool kAligned>
cudaError_t launch_backward_hidden(
    int branch_kind,
    bool dropout,
    bool parameters,
    const BackwardParams& params,
    int grid,
    cudaStream_t stream) {
    switch (branch_kind) {
        case 0:
            return launch_backward_branch<H, float, kAligned>(
                dropout, parameters, params, grid, stream);
        case 1:
            return launch_backward_branch<H, __half, kAligned>(
                dropout, parameters, params, grid, stream);
        case 2:
            return launch_backward_branch<H, __nv_bfloat16, kAligned>(
                dropout, parameters, params, grid, stream);
        default: return cudaErrorInvalidValue;
    }
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
    bool dropout,
    bool parameters,
    bool aligned,
    const BackwardParams& params,
    int grid,
    cudaStream_t stream) {
#define RLN_BWD_HIDDEN(HIDDEN)                                                               \
    case HIDDEN:                                                                             \
        return aligned                                                                       \
            ? launch_backward_hidden<HIDDEN, true>(                                          \
                  branch_kind, dropout, parameters, params, grid, stream)                 \
            : launch_backward_hidden<HIDDEN, false>(                                         \
                  branch_kind, dropout, parameters, params, grid, stream);
    switch (hidden) {
        RLN_BWD_HIDDEN(128)
        RLN_BWD_HIDDEN(256)
        RLN_BWD_HIDDEN(384)
        RLN_BWD_HIDDEN(512)
        RLN_BWD_HIDDEN(768)
        RLN_BWD_HIDDEN(1024)
        default: return cudaErrorInvalidValue;
    }
#undef RLN_BWD_HIDDEN
}

cudaError_t launch_reduce_partials(
    const float* partials,
    float* out,
    int partial_count,
    int columns,
    cudaStream_t stream) {
    constexpr int kSegments = 8;
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
        static_cast<unsigned>(blocks),
        kThreads,
        stream,
        reinterpret_cast<float4*>(out),
        count4);
}

}  // namespace rln
