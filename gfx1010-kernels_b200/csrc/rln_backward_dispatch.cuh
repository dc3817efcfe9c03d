// Backward dispatch ladder, parameterised on the element type of
// `grad_normalized` (the type the forward stored `normalized` in).  float32 is
// instantiated in rln_backward.cu, float16 / bfloat16 in rln_backward_narrow.cu.
#pragma once

#include "rln_launch.h"

namespace rln {

template <int H, typename BranchT, typename NormT, bool kDropout, bool kParams, bool kAligned>
cudaError_t launch_backward_typed(const BackwardParams& params, int grid, cudaStream_t stream) {
    constexpr int kWarps = BackwardTune<H>::kWarps;
    constexpr int kRows = BackwardTune<H>::kRows;
    return launch_dependent(
        rln_backward_kernel<H, BranchT, kDropout, kParams, kAligned, kWarps, kRows,
                            BackwardTune<H>::kCtasPerSm, false, NormT>,
        static_cast<unsigned>(grid),
        kWarps * kWarpSize,
        stream,
        params);
}

template <int H, typename BranchT, typename NormT, bool kAligned>
cudaError_t launch_backward_branch(
    bool dropout,
    bool parameters,
    const BackwardParams& params,
    int grid,
    cudaStream_t stream) {
    if (dropout) {
        return parameters
            ? launch_backward_typed<H, BranchT, NormT, true, true, kAligned>(params, grid, stream)
            : launch_backward_typed<H, BranchT, NormT, true, false, kAligned>(params, grid, stream);
    }
    return parameters
        ? launch_backward_typed<H, BranchT, NormT, false, true, kAligned>(params, grid, stream)
        : launch_backward_typed<H, BranchT, NormT, false, false, kAligned>(params, grid, stream);
}

template <int H, typename NormT, bool kAligned>
cudaError_t launch_backward_hidden(
    int branch_kind,
    bool dropout,
    bool parameters,
    const BackwardParams& params,
    int grid,
    cudaStream_t stream) {
    switch (branch_kind) {
        case 0:
            return launch_backward_branch<H, float, NormT, kAligned>(
                dropout, parameters, params, grid, stream);
        case 1:
            return launch_backward_branch<H, __half, NormT, kAligned>(
                dropout, parameters, params, grid, stream);
        case 2:
            return launch_backward_branch<H, __nv_bfloat16, NormT, kAligned>(
                dropout, parameters, params, grid, stream);
        default: return cudaErrorInvalidValue;
    }
}

// kAlignedOnly: the narrow gradient types are instantiated for 16-byte aligned
// pointers only (the C-ABI layer rejects the other case earlier).
template <typename NormT, bool kAlignedOnly>
cudaError_t launch_backward_normalized_as(
    int hidden,
    int branch_kind,
    bool dropout,
    bool parameters,
    bool aligned,
    const BackwardParams& params,
    int grid,
    cudaStream_t stream) {
    if (kAlignedOnly && !aligned) {
        return cudaErrorNotSupported;
    }
#define RLN_BWD_HIDDEN(HIDDEN)                                                    \
    case HIDDEN:                                                                  \
        if constexpr (kAlignedOnly) {                                             \
            return launch_backward_hidden<HIDDEN, NormT, true>(                   \
                branch_kind, dropout, parameters, params, grid, stream);          \
        } else {                                                                  \
            return aligned                                                        \
                ? launch_backward_hidden<HIDDEN, NormT, true>(                    \
                      branch_kind, dropout, parameters, params, grid, stream)     \
                : launch_backward_hidden<HIDDEN, NormT, false>(                   \
                      branch_kind, dropout, parameters, params, grid, stream);    \
        }
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

}  // namespace rln
