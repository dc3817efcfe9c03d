// Forward dispatch ladder, parameterised on the element type of `normalized`.
// Each translation unit that includes this header instantiates the kernels of
// one NormT (they compile in parallel): float32 in rln_forward.cu, float16 and
// bfloat16 in rln_forward_narrow.cu.
#pragma once

#include "rln_launch.h"

namespace rln {

template <int H, typename BranchT, typename NormT, bool kDropout, bool kAligned,
          bool kDeviceRng = false>
cudaError_t launch_forward_typed(const ForwardParams& params, int sm_count, cudaStream_t stream) {
    constexpr int kWarps = ForwardTune<H>::kWarps;
    constexpr int kRows = ForwardTune<H>::kRows;
    constexpr int kLanes = ForwardTune<H>::kLanes;
    constexpr int kMinCtas = ForwardTune<H>::kMinCtas;
    constexpr int64_t kRowsPerCta =
        static_cast<int64_t>(kWarps) * (kLanes == kWarpSize ? kRows : kWarpSize / kLanes);
    int64_t blocks = (params.rows + kRowsPerCta - 1) / kRowsPerCta;
    if (ForwardTune<H>::kPersistent) {
        const int64_t resident = static_cast<int64_t>(sm_count) * kMinCtas;
        blocks = blocks < resident ? blocks : resident;
    }
    if (blocks > 0x7fffffff) {
        blocks = 0x7fffffff;  // the kernels grid-stride over the remainder
    }
    if constexpr (kLanes == kWarpSize) {
        return launch_dependent(
            rln_forward_kernel<H, BranchT, kDropout, kAligned, kWarps, kRows, kMinCtas,
                               kDeviceRng, false, NormT, ForwardTune<H>::kPacked>,
            static_cast<unsigned>(blocks),
            kWarps * kWarpSize,
            stream,
            params);
    } else {
        return launch_dependent(
            rln_forward_subwarp_kernel<H, BranchT, kDropout, kAligned, kWarps, kLanes, kMinCtas,
                                       kDeviceRng, false, NormT, ForwardTune<H>::kPacked>,
            static_cast<unsigned>(blocks),
            kWarps * kWarpSize,
            stream,
            params);
    }
}

// kAlignedOnly: the narrow `normalized` types are instantiated for 16-byte
// aligned pointers only (the C-ABI layer rejects the other case earlier).
template <int H, typename BranchT, typename NormT, bool kAlignedOnly>
cudaError_t launch_forward_branch(
    bool dropout,
    bool aligned,
    const ForwardParams& params,
    int sm_count,
    cudaStream_t stream) {
    if (params.device_seed != nullptr) {
        // Philox state behind device pointers (graph capture): instantiated for
        // the vectorised dropout kernels only.
        if (!dropout || !aligned) {
            return cudaErrorNotSupported;
        }
        return launch_forward_typed<H, BranchT, NormT, true, true, true>(params, sm_count, stream);
    }
    if constexpr (kAlignedOnly) {
        if (!aligned) {
            return cudaErrorNotSupported;
        }
        return dropout
            ? launch_forward_typed<H, BranchT, NormT, true, true>(params, sm_count, stream)
            : launch_forward_typed<H, BranchT, NormT, false, true>(params, sm_count, stream);
    } else {
        if (dropout) {
            return aligned
                ? launch_forward_typed<H, BranchT, NormT, true, true>(params, sm_count, stream)
                : launch_forward_typed<H, BranchT, NormT, true, false>(params, sm_count, stream);
        }
        return aligned
            ? launch_forward_typed<H, BranchT, NormT, false, true>(params, sm_count, stream)
            : launch_forward_typed<H, BranchT, NormT, false, false>(params, sm_count, stream);
    }
}

template <int H, typename NormT, bool kAlignedOnly>
cudaError_t launch_forward_hidden(
    int branch_kind,
    bool dropout,
    bool aligned,
    const ForwardParams& params,
    int sm_count,
    cudaStream_t stream) {
    switch (branch_kind) {
        case 0:
            return launch_forward_branch<H, float, NormT, kAlignedOnly>(
                dropout, aligned, params, sm_count, stream);
        case 1:
            return launch_forward_branch<H, __half, NormT, kAlignedOnly>(
                dropout, aligned, params, sm_count, stream);
        case 2:
            return launch_forward_branch<H, __nv_bfloat16, NormT, kAlignedOnly>(
                dropout, aligned, params, sm_count, stream);
        default: return cudaErrorInvalidValue;
    }
}

template <typename NormT, bool kAlignedOnly>
cudaError_t launch_forward_normalized_as(
    int hidden,
    int branch_kind,
    bool dropout,
    bool aligned,
    const ForwardParams& params,
    int sm_count,
    cudaStream_t stream) {
#define RLN_FWD_HIDDEN(HIDDEN)                                       \
    case HIDDEN:                                                     \
        return launch_forward_hidden<HIDDEN, NormT, kAlignedOnly>(   \
            branch_kind, dropout, aligned, params, sm_count, stream);
    switch (hidden) {
        RLN_FWD_HIDDEN(128)
        RLN_FWD_HIDDEN(256)
        RLN_FWD_HIDDEN(384)
        RLN_FWD_HIDDEN(512)
        RLN_FWD_HIDDEN(768)
        RLN_FWD_HIDDEN(1024)
        default: return cudaErrorInvalidValue;
    }
#undef RLN_FWD_HIDDEN
}

}  // namespace rln
