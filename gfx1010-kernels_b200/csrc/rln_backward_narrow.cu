// Backward kernels that read `grad_normalized` as float16 or bfloat16 (the
// gradient of a `normalized` output stored in that type).  Vectorised
// (16-byte aligned) instantiations only.
#include "rln_backward_dispatch.cuh"

namespace rln {

cudaError_t launch_backward_normalized_half(
    int hidden,
    int branch_kind,
    bool dropout,
    bool parameters,
    bool aligned,
    const BackwardParams& params,
    int grid,
    cudaStream_t stream) {
    return launch_backward_normalized_as<__half, true>(
        hidden, branch_kind, dropout, parameters, aligned, params, grid, stream);
}

cudaError_t launch_backward_normalized_bfloat16(
    int hidden,
    int branch_kind,
    bool dropout,
    bool parameters,
    bool aligned,
    const BackwardParams& params,
    int grid,
    cudaStream_t stream) {
    return launch_backward_normalized_as<__nv_bfloat16, true>(
        hidden, branch_kind, dropout, parameters, aligned, params, grid, stream);
}

}  // namespace rln
