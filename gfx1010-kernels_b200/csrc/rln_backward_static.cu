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
    rln::BackwardCall call;
    call.grad_updated = grad_updated;
    call.grad_normalized = grad_normalized;  // this entry takes float32 only
    call.updated = updated;
    call.weight = weight;
    call.mean = mean;
    call.rstd = rstd;
    call.dropout_mask = dropout_mask;
    call.grad_x = grad_x;
    call.grad_branch = grad_branch;
    call.grad_parameters = grad_parameters;
    call.parameters_required = true;
    call.rows = rows;
    call.hidden = hidden;
    call.branch_dtype = branch_dtype;
    call.normalized_dtype = RLN_DTYPE_FLOAT32;
    call.dropout_active = dropout_active;
    call.dropout_p = dropout_p;
    bool vector_ok = false;
    int status = rln::check_backward_call(call, &vector_ok);
    if (status != RLN_OK) {
        return status;
    }
    void* scratch = nullptr;
    int sm_count = 0;
    status = scratch_on_current_device(&scratch, &sm_count);
    if (status != RLN_OK) {
        return status;
    }
    // Nothing in the scratch has to start at zero: every CTA of the grid stores
    // its whole [2, hidden] partial before the reduction reads partials
    // 0 .. grid-1, and entries left over from an earlier, larger call lie
    // beyond `grid` and are never read.  A grid whose partials do not fit in
    // the array gets RLN_ERR_LIMIT.
    return rln::launch_backward_call(
        call, vector_ok, sm_count, /*deterministic=*/true, scratch,
        static_cast<int64_t>(RLN_STATIC_SCRATCH_BYTES), RLN_ERR_LIMIT,
        static_cast<cudaStream_t>(stream_pointer));
}
