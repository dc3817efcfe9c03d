// Backward with the fixed-order parameter reduction, for callers that cannot
// allocate device memory: the per-CTA partials go to a scratch array that is
// part of this library's device image instead of a caller-provided workspace.
//
// Who needs this: hosts that own all device memory themselves (a serving
// runtime or plugin host that handed the whole GPU to its own pool and forbids
// allocation calls inside an operator), and loops that cannot afford the
// device-wide synchronisation a cudaMalloc/cudaFree may imply.  Such a caller
// has nowhere to get the [grid, 2, hidden] partial buffer that
// rln_sm100_backward wants in deterministic mode, and no way to size one ahead
// of time without calling into this library first.
#include "rln_sm100.h"

#include <cuda_runtime.h>

#include <mutex>

#include "rln_launch.h"

// The scratch itself.  It lives in every device's copy of the module image
// from the moment the module is loaded there until the process exits.
static __device__ __align__(256) unsigned char static_scratch[RLN_STATIC_SCRATCH_BYTES];

namespace {

constexpr int kCachedDevices = 64;
std::mutex scratch_mutex;
void* scratch_address[kCachedDevices] = {nullptr};
int sm_counts[kCachedDevices] = {0};

// Device address of `static_scratch` on the CURRENT device.  In host code the
// array's name is only a handle for the runtime, not a device address, so it
// is never passed to a kernel: the address is asked for once per device, with
// that device current, and remembered.
int scratch_on_current_device(void** address, int* sm_count) {
    int device = 0;
    cudaError_t error = cudaGetDevice(&device);
    if (error != cudaSuccess) {
        return rln::record_cuda_error(error);
    }
    const bool cacheable = device >= 0 && device < kCachedDevices;
    std::lock_guard<std::mutex> lock(scratch_mutex);
    if (cacheable && scratch_address[device] != nullptr) {
        *address = scratch_address[device];
        *sm_count = sm_counts[device];
        return RLN_OK;
    }
    void* found = nullptr;
    error = cudaGetSymbolAddress(&found, static_scratch);
    if (error != cudaSuccess) {
        return rln::record_cuda_error(error);
    }
    if (found == nullptr) {
        return rln::record_cuda_error(cudaErrorInvalidSymbol);
    }
    int count = 0;
    error = cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
    if (error != cudaSuccess) {
        return rln::record_cuda_error(error);
    }
    if (cacheable) {
        scratch_address[device] = found;
        sm_counts[device] = count;
    }
    *address = found;
    *sm_count = count;
    return RLN_OK;
}

bool aligned_to(const void* pointer, uintptr_t bytes) {
    return (reinterpret_cast<uintptr_t>(pointer) & (bytes - 1)) == 0;
}

}  // namespace

extern "C" int rln_sm100_backward_static_scratch(
    const float* grad_updated,
    const float* grad_normalized,
    const float* updated,
    const float* weight,
    const float* mean,
    const float* rstd,
    const uint32_t* dropout_mask,
    float* grad_x,
    void* grad_branch,
    float* grad_parameters,
    int64_t rows,
    int32_t hidden,
    int32_t branch_dtype,
    int32_t dropout_active,
    float dropout_p,
    void* stream_pointer) {
    if (!(hidden == 128 || hidden == 256 || hidden == 384 || hidden == 512 || hidden == 768
          || hidden == 1024)) {
        return RLN_ERR_HIDDEN_SIZE;
    }
    if (branch_dtype != RLN_BRANCH_FLOAT32 && branch_dtype != RLN_BRANCH_FLOAT16
        && branch_dtype != RLN_BRANCH_BFLOAT16) {
        return RLN_ERR_BRANCH_DTYPE;
    }
    if (rows <= 0) {
        return RLN_ERR_ROW_COUNT;
    }
    if (!(dropout_p >= 0.0f && dropout_p < 1.0f)) {
        return RLN_ERR_DROPOUT_P;
    }
    if (grad_updated == nullptr || grad_normalized == nullptr || updated == nullptr
        || weight == nullptr || mean == nullptr || rstd == nullptr || grad_x == nullptr
        || grad_branch == nullptr || grad_parameters == nullptr
        || (dropout_active && dropout_mask == nullptr)) {
        return RLN_ERR_NULL_POINTER;
    }
    const uintptr_t branch_element = branch_dtype == RLN_BRANCH_FLOAT32 ? 4 : 2;
    if (!aligned_to(grad_updated, 4) || !aligned_to(grad_normalized, 4) || !aligned_to(updated, 4)
        || !aligned_to(weight, 4) || !aligned_to(mean, 4) || !aligned_to(rstd, 4)
        || !aligned_to(grad_x, 4) || !aligned_to(grad_branch, branch_element)
        || !aligned_to(grad_parameters, 4) || (dropout_active && !aligned_to(dropout_mask, 4))) {
        return RLN_ERR_ALIGNMENT;
    }
    const bool vector_ok = aligned_to(grad_updated, 16) && aligned_to(grad_normalized, 16)
        && aligned_to(updated, 16) && aligned_to(weight, 16) && aligned_to(grad_x, 16)
        && aligned_to(grad_branch, branch_element * 4) && aligned_to(grad_parameters, 16);

    void* scratch = nullptr;
    int sm_count = 0;
    const int status = scratch_on_current_device(&scratch, &sm_count);
    if (status != RLN_OK) {
        return status;
    }
    const int grid = rln::backward_grid(hidden, rows, sm_count);
    const int64_t needed =
        static_cast<int64_t>(grid) * 2 * hidden * static_cast<int64_t>(sizeof(float));
    if (needed > static_cast<int64_t>(RLN_STATIC_SCRATCH_BYTES)) {
        return RLN_ERR_LIMIT;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_pointer);

    rln::BackwardParams params;
    params.grad_updated = grad_updated;
    params.grad_normalized = grad_normalized;
    params.updated = updated;
    params.weight = weight;
    params.mean = mean;
    params.rstd = rstd;
    params.mask = dropout_mask;
    params.grad_x = grad_x;
    params.grad_branch = grad_branch;
    params.grad_parameters = grad_parameters;
    params.partials = static_cast<float*>(scratch);
    params.rows = rows;
    params.scale = dropout_active ? 1.0f / (1.0f - dropout_p) : 1.0f;
    params.deterministic = 1;

    // Nothing in the scratch has to start at zero: every CTA of the grid stores
    // its whole [2, hidden] partial before the reduction reads partials
    // 0 .. grid-1, and entries left over from an earlier, larger call lie
    // beyond `grid` and are never read.
    cudaError_t error = rln::launch_backward(
        hidden,
        branch_dtype,
        RLN_DTYPE_FLOAT32,  // this entry takes a float32 grad_normalized only
        dropout_active != 0,
        /*parameters=*/true,
        vector_ok,
        params,
        grid,
        stream);
    if (error != cudaSuccess) {
        return rln::record_cuda_error(error);
    }
    error = rln::launch_reduce_partials(
        static_cast<const float*>(scratch), grad_parameters, grid, 2 * hidden, stream);
    if (error != cudaSuccess) {
        return rln::record_cuda_error(error);
    }
    return RLN_OK;
}
