// Internal launch interface between the C-ABI translation unit and the two
// kernel-instantiating translation units (split so they compile in parallel).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "rln_kernels.cuh"

namespace rln {

// Compile-time launch geometry per hidden size, chosen from measurements on
// B200 (87,381 x 768 and equal-volume shapes of the other widths):
//   kWarps    warps per CTA;
//   kRows     consecutive rows a warp keeps in flight per loop iteration;
//   kMinCtas  __launch_bounds__ minimum, i.e. the register budget
//             65536 / (32 * kWarps * kMinCtas) per thread.  16 to 32 resident
//             warps per SM is the sweet spot for the forward: fewer warps leave
//             HBM latency exposed, more warps cut the registers a warp can keep
//             in flight;
//   kPersistent (forward) launch exactly sm_count * kMinCtas CTAs that
//             grid-stride, instead of one CTA per kWarps * kRows rows.  Not
//             used by the current table: with several rows per warp even the
//             narrowest rows are fastest with one short-lived CTA per row group.
template <int H>
struct ForwardTune {
    // kLanes lanes own one row: 32 = one warp per row (rln_forward_kernel);
    // 8 / 16 = several rows per warp (rln_forward_subwarp_kernel), which wins
    // for the two narrowest widths (H=128: +14 %, H=256: +1 %) and loses from
    // H=384 up.
    static constexpr int kLanes = H <= 128 ? 8 : (H <= 256 ? 16 : 32);
    // The forward has no CTA-wide step at all, so the CTA is only a scheduling
    // unit.  For wide rows the smallest unit wins in a sustained
    // forward+backward chain on random data: a one-warp CTA frees its slot the
    // moment its row is stored instead of waiting for the slowest of four
    // warps (step time, same board: H=1024 -3.4 %, H=768 -3.1 % against
    // 4 warps x 4 / 5 CTAs; H=512 and 384 gain about 1 % with two warps).
    static constexpr int kWarps = H <= 256 ? 4 : (H <= 512 ? 2 : 1);
    static constexpr int kRows = 1;
    static constexpr int kMinCtas =
        H <= 256 ? 6 : (H <= 384 ? 16 : (H <= 512 ? 12 : (H <= 768 ? 18 : 16)));
    static constexpr bool kPersistent = false;
    // Two-wide fp32 arithmetic (kPacked of the kernels): H = 384 runs 32 warps
    // per SM on 64 registers each and is the one width whose forward gains from
    // the halved instruction count (same board, back to back: 174,762 rows
    // 0.1574 -> 0.1466 ms, 32,768 rows 0.0318 -> 0.0299 ms); H = 512 and the
    // sub-warp widths do not move, H = 768 / 1024 lose 4-5 % (more spills under
    // their 96-register budget).
    static constexpr bool kPacked = H == 384;
};

// The backward grid is persistent (register-resident parameter-gradient
// accumulators): exactly sm_count * kCtasPerSm CTAs, all resident because
// kCtasPerSm is also the __launch_bounds__ minimum.  It is a constant (not an
// occupancy query) so that the deterministic partial layout depends only on
// (hidden, rows, SM count).
template <int H>
struct BackwardTune {
    // Chosen in a sustained forward+backward chain on random data (the board at
    // its power cap); short bursts of the backward alone rank some neighbours
    // differently by 1-2 %.
    // H=1024: three warps x two CTAs (six warps per SM, up to 255 registers
    // each) beat four warps x two by 2 % of the step.
    static constexpr int kWarps = H == 1024 ? 3 : 4;
    static constexpr int kRows = H == 128 ? 2 : 1;
    static constexpr int kCtasPerSm =
        H <= 128 ? 6 : (H <= 256 ? 5 : (H <= 512 ? 4 : 2));
};

// Launch with the programmatic-stream-serialization attribute: the kernel may
// be scheduled while its predecessor in the stream drains.  Every kernel of
// this library executes griddepcontrol.wait before its first memory access, so
// this is safe after any predecessor; it removes the launch gap between the
// forward, the zeroing kernel and the backward of one training step.
template <typename... KernelArgs, typename... Args>
cudaError_t launch_dependent(
    void (*kernel)(KernelArgs...),
    unsigned grid,
    unsigned block,
    cudaStream_t stream,
    Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid);
    config.blockDim = dim3(block);
    config.dynamicSmemBytes = 0;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, args...);
}

// Remembers a failing CUDA call for rln_sm100_last_cuda_error (per thread) and
// returns RLN_ERR_CUDA.
int record_cuda_error(cudaError_t error);

// One backward call as it crosses the C ABI (every backward entry point fills
// this and goes through the same two functions, so their argument rules cannot
// drift apart).
struct BackwardCall {
    const float* grad_updated;
    const void* grad_normalized;
    const float* updated;
    const float* weight;
    const float* mean;
    const float* rstd;
    const uint32_t* dropout_mask;
    float* grad_x;
    void* grad_branch;
    float* grad_parameters;     // NULL = parameter gradients not requested
    bool parameters_required;   // entry points that exist to reduce them
    int64_t rows;
    int32_t hidden;
    int32_t branch_dtype;
    int32_t normalized_dtype;
    int32_t dropout_active;
    float dropout_p;
};

// RLN_OK or the RLN_ERR_* code of the first violated rule; on RLN_OK
// *vector_ok says whether the 16-byte-vector kernels apply.
int check_backward_call(const BackwardCall& call, bool* vector_ok);

// Zeroing kernel (fast path), backward kernel and, for `deterministic`, the
// fixed-order reduction over the partials in `scratch`; a scratch that is
// missing, misaligned or too small for the partials returns `scratch_error`.
// Without `deterministic` the scratch is not used.
int launch_backward_call(
    const BackwardCall& call,
    bool vector_ok,
    int sm_count,
    bool deterministic,
    void* scratch,
    int64_t scratch_bytes,
    int scratch_error,
    cudaStream_t stream);

// Number of CTAs of the persistent backward grid (pure function of its
// arguments; also the number of [2, hidden] partials in deterministic mode).
int backward_grid(int hidden, int64_t rows, int sm_count);

// branch_kind / normalized_kind: RLN_DTYPE_FLOAT32 / FLOAT16 / BFLOAT16
// (0 / 1 / 2).  normalized_kind is the element type of `normalized` (forward)
// and of `grad_normalized` (backward); kinds 1 and 2 exist for 16-byte aligned
// pointers only and return cudaErrorNotSupported otherwise.
cudaError_t launch_forward(
    int hidden,
    int branch_kind,
    int normalized_kind,
    bool dropout,
    bool aligned,
    const ForwardParams& params,
    int sm_count,
    cudaStream_t stream);

cudaError_t launch_backward(
    int hidden,
    int branch_kind,
    int normalized_kind,
    bool dropout,
    bool parameters,
    bool aligned,
    const BackwardParams& params,
    int grid,
    cudaStream_t stream);

// The narrow-`normalized` halves of the two ladders live in translation units
// of their own (rln_forward_narrow.cu, rln_backward_narrow.cu).
cudaError_t launch_forward_normalized_half(
    int hidden, int branch_kind, bool dropout, bool aligned,
    const ForwardParams& params, int sm_count, cudaStream_t stream);
cudaError_t launch_forward_normalized_bfloat16(
    int hidden, int branch_kind, bool dropout, bool aligned,
    const ForwardParams& params, int sm_count, cudaStream_t stream);
cudaError_t launch_backward_normalized_half(
    int hidden, int branch_kind, bool dropout, bool parameters, bool aligned,
    const BackwardParams& params, int grid, cudaStream_t stream);
cudaError_t launch_backward_normalized_bfloat16(
    int hidden, int branch_kind, bool dropout, bool parameters, bool aligned,
    const BackwardParams& params, int grid, cudaStream_t stream);

// Zeroes `count` floats (count % 4 == 0, 16-byte aligned) with a kernel instead
// of a memset node, which keeps the step's launches kernel -> kernel.
cudaError_t launch_zero(float* out, int count, cudaStream_t stream);

cudaError_t launch_reduce_partials(
    const float* partials,
    float* out,
    int partial_count,
    int columns,
    cudaStream_t stream);

}  // namespace rln
