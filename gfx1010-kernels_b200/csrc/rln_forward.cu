// Forward entry of the launch interface and the float32-`normalized` kernels.
#include "rln_forward_dispatch.cuh"

namespace rln {

cudaError_t launch_forward(
    int hidden,
    int branch_kind,
    int normalized_kind,
    bool dropout,
    bool aligned,
    const ForwardParams& params,
    int sm_count,
    cudaStream_t stream) {
    switch (normalized_kind) {
        case 0:
            return launch_forward_normalized_as<float, false>(
                hidden, branch_kind, dropout, aligned, params, sm_count, stream);
        case 1:
            return launch_forward_normalized_half(
                hidden, branch_kind, dropout, aligned, params, sm_count, stream);
        case 2:
            return launch_forward_normalized_bfloat16(
                hidden, branch_kind, dropout, aligned, params, sm_count, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace rln
