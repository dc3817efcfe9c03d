// Forward kernel instantiations and their dispatch ladder.
#include "rln_launch.h"

namespace rln {
namespace {

template <int H, typename BranchT, bool kDropout, bool kAligned, bool kDeviceRng = false>
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
                               kDeviceRng>,
            static_cast<unsigned>(blocks),
            kWarps * kWarpSize,
            stream,
            params);
    } else {
        return launch_dependent(
            rln_forward_subwarp_kernel<H, BranchT, kDropout, kAligned, kWarps, kLanes, kMinCtas,
                                       kDeviceRng>,
            static_cast<unsigned>(blocks),
            kWarps * kWarpSize,
            stream,
            params);
    }
}

template <int H, typename BranchT>
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
        return launch_forward_typed<H, BranchT, true, true, true>(params, sm_count, stream);
    }
    if (dropout) {
        return aligned ? launch_forward_typed<H, BranchT, true, true>(params, sm_count, stream)
                       : launch_forward_typed<H, BranchT, true, false>(params, sm_count, stream);
    }
    return aligned ? launch_forward_typed<H, BranchT, false, true>(params, sm_count, stream)
                   : launch_forward_typed<H, BranchT, false, false>(params, sm_count, stream);
}

template <int H>
cudaError_t launch_forward_hidden(
    int branch_kind,
    bool dropout,
    bool aligned,
    const ForwardParams& params,
    int sm_count,
    cudaStream_t stream) {
    switch (branch_kind) {
        case 0: return launch_forward_branch<H, float>(dropout, aligned, params, sm_count, stream);
        case 1: return launch_forward_branch<H, __half>(dropout, aligned, params, sm_count, stream);
        case 2:
            return launch_forward_branch<H, __nv_bfloat16>(
                dropout, aligned, params, sm_count, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

cudaError_t launch_forward(
    int hidden,
    int branch_kind,
    bool dropout,
    bool aligned,
    const ForwardParams& params,
    int sm_count,
    cudaStream_t stream) {
    switch (hidden) {
        case 128: return launch_forward_hidden<128>(branch_kind, dropout, aligned, params, sm_count, stream);
        case 256: return launch_forward_hidden<256>(branch_kind, dropout, aligned, params, sm_count, stream);
        case 384: return launch_forward_hidden<384>(branch_kind, dropout, aligned, params, sm_count, stream);
        case 512: return launch_forward_hidden<512>(branch_kind, dropout, aligned, params, sm_count, stream);
        case 768: return launch_forward_hidden<768>(branch_kind, dropout, aligned, params, sm_count, stream);
        case 1024: return launch_forward_hidden<1024>(branch_kind, dropout, aligned, params, sm_count, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace rln
