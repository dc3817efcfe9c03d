// Forward kernels that store `normalized` as float16 or bfloat16 (rounded once
// from the float32 result), for consumers that feed it to a half-precision
// GEMM.  Vectorised (16-byte aligned) instantiations only.
#include "rln_forward_dispatch.cuh"

namespace rln {

cudaError_t launch_forward_normalized_half(
    int hidden,
    int branch_kind,
    bool dropout,
    bool aligned,
    const ForwardParams& params,
    int sm_count,
    cudaStream_t stream) {
    return launch_forward_normalized_as<__half, true>(
        hidden, branch_kind, dropout, aligned, params, sm_count, stream);
}

cudaError_t launch_forward_normalized_bfloat16(
    int hidden,
    int branch_kind,
    bool dropout,
    bool aligned,
    const ForwardParams& params,
    int sm_count,
    cudaStream_t stream) {
    return launch_forward_normalized_as<__nv_bfloat16, true>(
        hidden, branch_kind, dropout, aligned, params, sm_count, stream);
}

}  // namespace rln
