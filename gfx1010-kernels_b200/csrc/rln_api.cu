// C ABI of the sm_100a residual LayerNorm path: argument checks, dropout
// constants, alignment-based kernel selection and launches.  No torch here.
#include "rln_sm100.h"

#include <cuda_runtime.h>

#include <atomic>

#include "rln_launch.h"

namespace {

thread_local int tls_last_cuda_error = 0;

int cuda_failed(cudaError_t error) {
    tls_last_cuda_error = static_cast<int>(error);
    return RLN_ERR_CUDA;
}

}  // namespace

int rln::record_cuda_error(cudaError_t error) { return cuda_failed(error); }

namespace {

bool supported_hidden(int32_t hidden) {
    return hidden == 128 || hidden == 256 || hidden == 384 || hidden == 512
        || hidden == 768 || hidden == 1024;
}

bool supported_dtype(int32_t dtype) {
    return dtype == RLN_DTYPE_FLOAT32 || dtype == RLN_DTYPE_FLOAT16 || dtype == RLN_DTYPE_BFLOAT16;
}

uintptr_t element_bytes(int32_t dtype) { return dtype == RLN_DTYPE_FLOAT32 ? 4 : 2; }

bool aligned_to(const void* pointer, uintptr_t bytes) {
    return (reinterpret_cast<uintptr_t>(pointer) & (bytes - 1)) == 0;
}

// SM count of the current device, cached per device ordinal.
int current_sm_count(int* out) {
    static std::atomic<int> cached[64];
    int device = 0;
    cudaError_t error = cudaGetDevice(&device);
    if (error != cudaSuccess) {
        return cuda_failed(error);
    }
    const bool cacheable = device >= 0 && device < 64;
    if (cacheable) {
        const int known = cached[device].load(std::memory_order_relaxed);
        if (known > 0) {
            *out = known;
            return RLN_OK;
        }
    }
    int count = 0;
    error = cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
    if (error != cudaSuccess) {
        return cuda_failed(error);
    }
    if (cacheable) {
        cached[device].store(count, std::memory_order_relaxed);
    }
    *out = count;
    return RLN_OK;
}

// threshold and scale exactly as the reference computes them
// (csrc/residual_layer_norm_kernel.hip:896-899): p is narrowed to fp32 first.
uint32_t dropout_threshold(float dropout_p) {
    return static_cast<uint32_t>(static_cast<double>(dropout_p) * 4294967296.0);
}

float dropout_scale(float dropout_p, bool active) {
    return active ? 1.0f / (1.0f - dropout_p) : 1.0f;
}

}  // namespace

extern "C" int rln_sm100_abi_version(void) { return RLN_SM100_ABI_VERSION; }

extern "C" const char* rln_sm100_status_string(int status) {
    switch (status) {
        case RLN_OK: return "ok";
        case RLN_ERR_NULL_POINTER: return "a required pointer is NULL";
        case RLN_ERR_HIDDEN_SIZE: return "unsupported native hidden size";
        case RLN_ERR_ROW_COUNT: return "empty tensors are unsupported";
        case RLN_ERR_DROPOUT_P: return "dropout_p must be in [0, 1)";
        case RLN_ERR_EPS: return "eps must be positive";
        case RLN_ERR_ALIGNMENT: return "a pointer is not aligned to its element size";
        case RLN_ERR_WORKSPACE: return "workspace is missing or too small";
        case RLN_ERR_CUDA: return "a CUDA runtime call failed";
        case RLN_ERR_HOST_BUFFERS: return "invalid host-buffer pipeline arguments";
        case RLN_ERR_LIMIT: return "size exceeds a fixed maximum of this entry point";
        case RLN_ERR_BRANCH_DTYPE: return "branch must use float32, float16 or bfloat16";
        case RLN_ERR_NORMALIZED_DTYPE:
            return "normalized must use float32, float16 or bfloat16";
        default: return "unknown status";
    }
}

extern "C" int rln_sm100_last_cuda_error(void) { return tls_last_cuda_error; }

namespace {

int forward_launch(
    const float* x,
    const void* branch,
    const float* weight,
    const float* bias,
    float* updated,
    void* normalized,
    float* mean,
    float* rstd,
    uint32_t* dropout_mask,
    int64_t rows,
    int32_t hidden,
    int32_t branch_dtype,
    int32_t normalized_dtype,
    int32_t dropout_active,
    float dropout_p,
    float eps,
    uint64_t seed,
    uint64_t offset,
    const int64_t* device_seed,
    const int64_t* device_offset,
    int64_t row_base,
    void* stream) {
    if (!supported_hidden(hidden)) {
        return RLN_ERR_HIDDEN_SIZE;
    }
    if (!supported_dtype(branch_dtype)) {
        return RLN_ERR_BRANCH_DTYPE;
    }
    if (!supported_dtype(normalized_dtype)) {
        return RLN_ERR_NORMALIZED_DTYPE;
    }
    if (rows <= 0) {
        return RLN_ERR_ROW_COUNT;
    }
    if (!(dropout_p >= 0.0f && dropout_p < 1.0f)) {
        return RLN_ERR_DROPOUT_P;
    }
    if (!(eps > 0.0f)) {
        return RLN_ERR_EPS;
    }
    if (x == nullptr || branch == nullptr || weight == nullptr || bias == nullptr
        || updated == nullptr || normalized == nullptr || mean == nullptr || rstd == nullptr
        || (dropout_active && dropout_mask == nullptr)) {
        return RLN_ERR_NULL_POINTER;
    }
    const uintptr_t branch_element = element_bytes(branch_dtype);
    const uintptr_t normalized_element = element_bytes(normalized_dtype);
    if (!aligned_to(x, 4) || !aligned_to(branch, branch_element) || !aligned_to(weight, 4)
        || !aligned_to(bias, 4) || !aligned_to(updated, 4)
        || !aligned_to(normalized, normalized_element)
        || !aligned_to(mean, 4) || !aligned_to(rstd, 4)
        || (dropout_active && !aligned_to(dropout_mask, 4))) {
        return RLN_ERR_ALIGNMENT;
    }
    const bool vector_ok = aligned_to(x, 16) && aligned_to(branch, branch_element * 4)
        && aligned_to(weight, 16) && aligned_to(bias, 16) && aligned_to(updated, 16)
        && aligned_to(normalized, normalized_element * 4);

    rln::ForwardParams params;
    params.x = x;
    params.branch = branch;
    params.weight = weight;
    params.bias = bias;
    params.updated = updated;
    params.normalized = normalized;
    params.mean = mean;
    params.rstd = rstd;
    params.mask = dropout_mask;
    params.rows = rows;
    params.row_base = row_base;
    params.scale = dropout_scale(dropout_p, dropout_active != 0);
    params.eps = eps;
    params.threshold = dropout_threshold(dropout_p);
    params.seed_lo = static_cast<uint32_t>(seed);
    params.seed_hi = static_cast<uint32_t>(seed >> 32);
    // The generator's offset counts 32-bit words; a Philox call yields four, so
    // the counter's low half is the block index offset / 4 -- the convention of
    // torch's (and the reference's hipRAND) generators, under which a later
    // random op, whose offset is at least four words further on, can never land
    // on a counter this call used.
    params.offset_lo = static_cast<uint32_t>(offset >> 2);
    params.offset_hi = static_cast<uint32_t>(offset >> 34);
    params.device_seed = device_seed;
    params.device_offset = device_offset;
    params.device_offset_extra = device_seed != nullptr ? offset : 0;
    params.zero_buffer = nullptr;
    params.zero_count4 = 0;
    if ((device_seed != nullptr || normalized_dtype != RLN_DTYPE_FLOAT32) && !vector_ok) {
        // the device-state kernels and the narrow-`normalized` kernels exist in
        // the vectorised form only
        return RLN_ERR_ALIGNMENT;
    }

    int sm_count = 0;
    const int status = current_sm_count(&sm_count);
    if (status != RLN_OK) {
        return status;
    }
    const cudaError_t error = rln::launch_forward(
        hidden,
        branch_dtype,
        normalized_dtype,
        dropout_active != 0,
        vector_ok,
        params,
        sm_count,
        static_cast<cudaStream_t>(stream));
    return error == cudaSuccess ? RLN_OK : cuda_failed(error);
}

}  // namespace

extern "C" int rln_sm100_forward(
    const float* x,
    const void* branch,
    const float* weight,
    const float* bias,
    float* updated,
    void* normalized,
    float* mean,
    float* rstd,
    uint32_t* dropout_mask,
    int64_t rows,
    int32_t hidden,
    int32_t branch_dtype,
    int32_t normalized_dtype,
    int32_t dropout_active,
    float dropout_p,
    float eps,
    uint64_t seed,
    uint64_t offset,
    int64_t row_base,
    void* stream) {
    return forward_launch(
        x, branch, weight, bias, updated, normalized, mean, rstd, dropout_mask, rows, hidden,
        branch_dtype, normalized_dtype, dropout_active, dropout_p, eps, seed, offset, nullptr,
        nullptr, row_base, stream);
}

extern "C" int rln_sm100_forward_device_rng(
    const float* x,
    const void* branch,
    const float* weight,
    const float* bias,
    float* updated,
    void* normalized,
    float* mean,
    float* rstd,
    uint32_t* dropout_mask,
    int64_t rows,
    int32_t hidden,
    int32_t branch_dtype,
    int32_t normalized_dtype,
    int32_t dropout_active,
    float dropout_p,
    float eps,
    const int64_t* device_seed,
    const int64_t* device_offset,
    uint64_t offset_extra,
    int64_t row_base,
    void* stream) {
    if (dropout_active && (device_seed == nullptr || device_offset == nullptr)) {
        return RLN_ERR_NULL_POINTER;
    }
    if (dropout_active
        && (!aligned_to(device_seed, 8) || !aligned_to(device_offset, 8))) {
        return RLN_ERR_ALIGNMENT;
    }
    return forward_launch(
        x, branch, weight, bias, updated, normalized, mean, rstd, dropout_mask, rows, hidden,
        branch_dtype, normalized_dtype, dropout_active, dropout_p, eps, 0, offset_extra,
        dropout_active ? device_seed : nullptr, dropout_active ? device_offset : nullptr,
        row_base, stream);
}

extern "C" int64_t rln_sm100_backward_workspace_bytes(
    int64_t rows,
    int32_t hidden,
    int32_t deterministic) {
    if (!supported_hidden(hidden)) {
        return RLN_ERR_HIDDEN_SIZE;
    }
    if (rows <= 0) {
        return RLN_ERR_ROW_COUNT;
    }
    if (!deterministic) {
        return 0;
    }
    int sm_count = 0;
    const int status = current_sm_count(&sm_count);
    if (status != RLN_OK) {
        return status;
    }
    const int grid = rln::backward_grid(hidden, rows, sm_count);
    return static_cast<int64_t>(grid) * 2 * hidden * static_cast<int64_t>(sizeof(float));
}

// Argument rules shared by every backward entry point.
int rln::check_backward_call(const rln::BackwardCall& call, bool* vector_ok) {
    if (!supported_hidden(call.hidden)) {
        return RLN_ERR_HIDDEN_SIZE;
    }
    if (!supported_dtype(call.branch_dtype)) {
        return RLN_ERR_BRANCH_DTYPE;
    }
    if (!supported_dtype(call.normalized_dtype)) {
        return RLN_ERR_NORMALIZED_DTYPE;
    }
    if (call.rows <= 0) {
        return RLN_ERR_ROW_COUNT;
    }
    if (!(call.dropout_p >= 0.0f && call.dropout_p < 1.0f)) {
        return RLN_ERR_DROPOUT_P;
    }
    const bool dropout = call.dropout_active != 0;
    if (call.grad_updated == nullptr || call.grad_normalized == nullptr
        || call.updated == nullptr || call.weight == nullptr || call.mean == nullptr
        || call.rstd == nullptr || call.grad_x == nullptr || call.grad_branch == nullptr
        || (dropout && call.dropout_mask == nullptr)
        || (call.parameters_required && call.grad_parameters == nullptr)) {
        return RLN_ERR_NULL_POINTER;
    }
    const uintptr_t branch_element = element_bytes(call.branch_dtype);
    const uintptr_t normalized_element = element_bytes(call.normalized_dtype);
    if (!aligned_to(call.grad_updated, 4)
        || !aligned_to(call.grad_normalized, normalized_element)
        || !aligned_to(call.updated, 4) || !aligned_to(call.weight, 4)
        || !aligned_to(call.mean, 4) || !aligned_to(call.rstd, 4)
        || !aligned_to(call.grad_x, 4) || !aligned_to(call.grad_branch, branch_element)
        || (dropout && !aligned_to(call.dropout_mask, 4))
        || (call.grad_parameters != nullptr && !aligned_to(call.grad_parameters, 4))) {
        return RLN_ERR_ALIGNMENT;
    }
    *vector_ok = aligned_to(call.grad_updated, 16)
        && aligned_to(call.grad_normalized, normalized_element * 4)
        && aligned_to(call.updated, 16) && aligned_to(call.weight, 16)
        && aligned_to(call.grad_x, 16) && aligned_to(call.grad_branch, branch_element * 4)
        && (call.grad_parameters == nullptr || aligned_to(call.grad_parameters, 16));
    if (call.normalized_dtype != RLN_DTYPE_FLOAT32 && !*vector_ok) {
        // the narrow-gradient kernels exist in the vectorised form only
        return RLN_ERR_ALIGNMENT;
    }
    return RLN_OK;
}

// Launches of one checked backward call.  `scratch` holds the per-CTA partials
// (deterministic != 0; too small -> `scratch_error`).
int rln::launch_backward_call(
    const rln::BackwardCall& call,
    bool vector_ok,
    int sm_count,
    bool deterministic,
    void* scratch,
    int64_t scratch_bytes,
    int scratch_error,
    cudaStream_t stream) {
    const bool parameters = call.grad_parameters != nullptr;
    const int grid = rln::backward_grid(call.hidden, call.rows, sm_count);
    const bool two_pass = parameters && deterministic;
    if (two_pass) {
        const int64_t needed = static_cast<int64_t>(grid) * 2 * call.hidden
            * static_cast<int64_t>(sizeof(float));
        if (scratch == nullptr || scratch_bytes < needed || !aligned_to(scratch, 16)) {
            return scratch_error;
        }
    }
    rln::BackwardParams params;
    params.grad_updated = call.grad_updated;
    params.grad_normalized = call.grad_normalized;
    params.updated = call.updated;
    params.weight = call.weight;
    params.mean = call.mean;
    params.rstd = call.rstd;
    params.mask = call.dropout_mask;
    params.grad_x = call.grad_x;
    params.grad_branch = call.grad_branch;
    params.grad_parameters = call.grad_parameters;
    params.partials = two_pass ? static_cast<float*>(scratch) : nullptr;
    params.rows = call.rows;
    params.scale = dropout_scale(call.dropout_p, call.dropout_active != 0);
    params.deterministic = two_pass ? 1 : 0;
    params.row_counter = nullptr;
    params.dynamic_begin = 0;

    if (parameters && !two_pass) {
        // the atomics accumulate into a zeroed buffer
        const cudaError_t error = aligned_to(call.grad_parameters, 16)
            ? rln::launch_zero(call.grad_parameters, 2 * call.hidden, stream)
            : cudaMemsetAsync(
                  call.grad_parameters, 0, static_cast<size_t>(2) * call.hidden * sizeof(float),
                  stream);
        if (error != cudaSuccess) {
            return cuda_failed(error);
        }
    }
    cudaError_t error = rln::launch_backward(
        call.hidden,
        call.branch_dtype,
        call.normalized_dtype,
        call.dropout_active != 0,
        parameters,
        vector_ok,
        params,
        grid,
        stream);
    if (error != cudaSuccess) {
        return cuda_failed(error);
    }
    if (two_pass) {
        error = rln::launch_reduce_partials(
            static_cast<const float*>(scratch), call.grad_parameters, grid, 2 * call.hidden,
            stream);
        if (error != cudaSuccess) {
            return cuda_failed(error);
        }
    }
    return RLN_OK;
}

extern "C" int rln_sm100_backward(
    const float* grad_updated,
    const void* grad_normalized,
    const float* updated,
    const float* weight,
    const float* mean,
    const float* rstd,
    const uint32_t* dropout_mask,
    float* grad_x,
    void* grad_branch,
    float* grad_parameters,
    void* workspace,
    int64_t workspace_bytes,
    int64_t rows,
    int32_t hidden,
    int32_t branch_dtype,
    int32_t normalized_dtype,
    int32_t dropout_active,
    float dropout_p,
    int32_t deterministic,
    void* stream_pointer) {
    rln::BackwardCall call;
    call.grad_updated = grad_updated;
    call.grad_normalized = grad_normalized;
    call.updated = updated;
    call.weight = weight;
    call.mean = mean;
    call.rstd = rstd;
    call.dropout_mask = dropout_mask;
    call.grad_x = grad_x;
    call.grad_branch = grad_branch;
    call.grad_parameters = grad_parameters;
    call.parameters_required = false;
    call.rows = rows;
    call.hidden = hidden;
    call.branch_dtype = branch_dtype;
    call.normalized_dtype = normalized_dtype;
    call.dropout_active = dropout_active;
    call.dropout_p = dropout_p;
    bool vector_ok = false;
    int status = rln::check_backward_call(call, &vector_ok);
    if (status != RLN_OK) {
        return status;
    }
    int sm_count = 0;
    status = current_sm_count(&sm_count);
    if (status != RLN_OK) {
        return status;
    }
    return rln::launch_backward_call(
        call, vector_ok, sm_count, deterministic != 0, workspace, workspace_bytes,
        RLN_ERR_WORKSPACE, static_cast<cudaStream_t>(stream_pointer));
}
