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

template <int H>
cudaError_t launch_forward_hidden(
    bool branch_is_half,
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
        return branch_is_half
            ? launch_forward_typed<H, __half, true, true, true>(params, sm_count, stream)
            : launch_forward_typed<H, float, true, true, true>(params, sm_count, stream);
    }
#define RLN_FWD_CASE(HALF, DROP, ALIGNED)                                                   \
    if (branch_is_half == HALF && dropout == DROP && aligned == ALIGNED) {                  \
        if constexpr (HALF) {                                                               \
            return launch_forward_typed<H, __half, DROP, ALIGNED>(params, sm_count, stream);          \
        } else {                                                                            \
            return launch_forward_typed<H, float, DROP, ALIGNED>(params, sm_count, stream);           \
        }                                                                                   \
    }
    RLN_FWD_CASE(true, true, true)
    RLN_FWD_CASE(true, false, true)
    RLN_FWD_CASE(false, true, true)
    RLN_FWD_CASE(false, false, true)
    RLN_FWD_CASE(true, true, false)
    RLN_FWD_CASE(true, false, false)
    RLN_FWD_CASE(false, true, false)
    RLN_FWD_CASE(false, false, false)
#undef RLN_FWD_CASE
    return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_forward(
    int hidden,
    bool branch_is_half,
    bool dropout,
    bool aligned,
    const ForwardParams& params,
    int sm_count,
    cudaStream_t stream) {
    switch (hidden) {
        case 128: return launch_forward_hidden<128>(branch_is_half, dropout, aligned, params, sm_count, stream);
        case 256: return launch_forward_hidden<256>(branch_is_half, dropout, aligned, params, sm_count, stream);
        case 384: return launch_forward_hidden<384>(branch_is_half, dropout, aligned, params, sm_count, stream);
        case 512: return launch_forward_hidden<512>(branch_is_half, dropout, aligned, params, sm_count, stream);
        case 768: return launch_forward_hidden<768>(branch_is_half, dropout, aligned, params, sm_count, stream);
        case 1024: return launch_forward_hidden<1024>(branch_is_half, dropout, aligned, params, sm_count, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace rln
