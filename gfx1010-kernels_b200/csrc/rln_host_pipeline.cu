// Host-buffer pipeline of the residual LayerNorm training step: chunked
// host->device copies, forward + backward kernels and device->host copies on
// three streams, so that both PCIe directions and the SMs work at once.
#include "rln_sm100.h"

#include <cuda_runtime.h>

#include <initializer_list>
#include <new>

#include "rln_launch.h"

namespace {

constexpr int kMaxDepth = 8;

// total = first ? slot : total + slot, over 2 * hidden floats.  Chunks are
// accumulated in chunk order on one stream, so the sum order is fixed.
__global__ void accumulate_parameters_kernel(
    float* __restrict__ total,
    const float* __restrict__ slot,
    int count,
    int first) {
    const int index = blockIdx.x * blockDim.x + threadIdx.x;
    if (index < count) {
        total[index] = first ? slot[index] : total[index] + slot[index];
    }
}

constexpr int kStepsTracked = 8;

struct Slot {
    float* x = nullptr;
    void* branch = nullptr;
    float* grad_updated = nullptr;
    void* grad_normalized = nullptr;
    float* updated = nullptr;
    void* normalized = nullptr;
    float* grad_x = nullptr;
    void* grad_branch = nullptr;
    float* mean = nullptr;
    float* rstd = nullptr;
    uint32_t* mask = nullptr;
    float* grad_parameters = nullptr;
    void* workspace = nullptr;
    cudaEvent_t in_ready = nullptr;   // inputs of the slot have arrived
    cudaEvent_t computed = nullptr;   // kernels of the slot are done (inputs reusable)
    cudaEvent_t drained = nullptr;    // outputs of the slot have left (outputs reusable)
    bool used = false;
};

}  // namespace

struct RlnHostPipeline {
    int device = 0;
    int32_t hidden = 0;
    int32_t branch_dtype = 0;
    int32_t normalized_dtype = 0;
    int64_t chunk_rows = 0;
    int32_t depth = 0;
    int64_t workspace_bytes = 0;
    cudaStream_t stream_in = nullptr;
    cudaStream_t stream_compute = nullptr;
    cudaStream_t stream_out = nullptr;
    // Two sets, alternating from step to step: a step enqueued behind another
    // one copies its parameters in, and resets its gradient sums, while the
    // previous step's last kernels and last copy-out still use theirs.
    float* weight[2] = {nullptr, nullptr};
    float* bias[2] = {nullptr, nullptr};
    float* total[2] = {nullptr, nullptr};
    int64_t chunks_enqueued = 0;  // position in the slot ring; runs on across calls
    // Completion of the most recent steps: step n (1-based count of enqueued
    // steps) has landed once both events of entry n % kStepsTracked fired.
    int64_t steps_enqueued = 0;
    cudaEvent_t step_out[kStepsTracked] = {};       // last chunk copied out
    cudaEvent_t step_compute[kStepsTracked] = {};   // parameter gradients copied out
    Slot slots[kMaxDepth];
};

namespace {

void release(RlnHostPipeline* p) {
    if (p == nullptr) {
        return;
    }
    for (int s = 0; s < kMaxDepth; ++s) {
        Slot& slot = p->slots[s];
        cudaFree(slot.x);
        cudaFree(slot.branch);
        cudaFree(slot.grad_updated);
        cudaFree(slot.grad_normalized);
        cudaFree(slot.updated);
        cudaFree(slot.normalized);
        cudaFree(slot.grad_x);
        cudaFree(slot.grad_branch);
        cudaFree(slot.mean);
        cudaFree(slot.rstd);
        cudaFree(slot.mask);
        cudaFree(slot.grad_parameters);
        cudaFree(slot.workspace);
        if (slot.in_ready) cudaEventDestroy(slot.in_ready);
        if (slot.computed) cudaEventDestroy(slot.computed);
        if (slot.drained) cudaEventDestroy(slot.drained);
    }
    for (int n = 0; n < kStepsTracked; ++n) {
        if (p->step_out[n]) cudaEventDestroy(p->step_out[n]);
        if (p->step_compute[n]) cudaEventDestroy(p->step_compute[n]);
    }
    for (int set = 0; set < 2; ++set) {
        cudaFree(p->weight[set]);
        cudaFree(p->bias[set]);
        cudaFree(p->total[set]);
    }
    if (p->stream_in) cudaStreamDestroy(p->stream_in);
    if (p->stream_compute) cudaStreamDestroy(p->stream_compute);
    if (p->stream_out) cudaStreamDestroy(p->stream_out);
    delete p;
}

// Returns the first failing call's error as it is (the caller releases what was
// allocated so far, which issues further CUDA calls: asking the runtime for its
// last error after that could name a different failure).
#define RLN_TRY(call)                                  \
    do {                                               \
        const cudaError_t rln_try_error = (call);      \
        if (rln_try_error != cudaSuccess) {            \
            return rln_try_error;                      \
        }                                              \
    } while (0)

cudaError_t allocate(RlnHostPipeline* p) {
    const size_t elements = static_cast<size_t>(p->chunk_rows) * p->hidden;
    const size_t branch_bytes = elements * (p->branch_dtype == RLN_DTYPE_FLOAT32 ? 4 : 2);
    const size_t normalized_bytes = elements * (p->normalized_dtype == RLN_DTYPE_FLOAT32 ? 4 : 2);
    RLN_TRY(cudaStreamCreateWithFlags(&p->stream_in, cudaStreamNonBlocking));
    RLN_TRY(cudaStreamCreateWithFlags(&p->stream_compute, cudaStreamNonBlocking));
    RLN_TRY(cudaStreamCreateWithFlags(&p->stream_out, cudaStreamNonBlocking));
    for (int set = 0; set < 2; ++set) {
        RLN_TRY(cudaMalloc(&p->weight[set], p->hidden * sizeof(float)));
        RLN_TRY(cudaMalloc(&p->bias[set], p->hidden * sizeof(float)));
        RLN_TRY(cudaMalloc(&p->total[set], 2 * p->hidden * sizeof(float)));
    }
    for (int n = 0; n < kStepsTracked; ++n) {
        RLN_TRY(cudaEventCreateWithFlags(&p->step_out[n], cudaEventDisableTiming));
        RLN_TRY(cudaEventCreateWithFlags(&p->step_compute[n], cudaEventDisableTiming));
    }
    for (int s = 0; s < p->depth; ++s) {
        Slot& slot = p->slots[s];
        RLN_TRY(cudaMalloc(&slot.x, elements * 4));
        RLN_TRY(cudaMalloc(&slot.branch, branch_bytes));
        RLN_TRY(cudaMalloc(&slot.grad_updated, elements * 4));
        RLN_TRY(cudaMalloc(&slot.grad_normalized, normalized_bytes));
        RLN_TRY(cudaMalloc(&slot.updated, elements * 4));
        RLN_TRY(cudaMalloc(&slot.normalized, normalized_bytes));
        RLN_TRY(cudaMalloc(&slot.grad_x, elements * 4));
        RLN_TRY(cudaMalloc(&slot.grad_branch, branch_bytes));
        RLN_TRY(cudaMalloc(&slot.mean, p->chunk_rows * sizeof(float)));
        RLN_TRY(cudaMalloc(&slot.rstd, p->chunk_rows * sizeof(float)));
        RLN_TRY(cudaMalloc(&slot.mask, elements / 8));
        RLN_TRY(cudaMalloc(&slot.grad_parameters, 2 * p->hidden * sizeof(float)));
        if (p->workspace_bytes > 0) {
            RLN_TRY(cudaMalloc(&slot.workspace, p->workspace_bytes));
        }
        RLN_TRY(cudaEventCreateWithFlags(&slot.in_ready, cudaEventDisableTiming));
        RLN_TRY(cudaEventCreateWithFlags(&slot.computed, cudaEventDisableTiming));
        RLN_TRY(cudaEventCreateWithFlags(&slot.drained, cudaEventDisableTiming));
    }
    return cudaSuccess;
}

}  // namespace

extern "C" int rln_sm100_host_pipeline_create(
    RlnHostPipeline** pipeline,
    int32_t hidden,
    int32_t branch_dtype,
    int32_t normalized_dtype,
    int64_t chunk_rows,
    int32_t depth) {
    if (pipeline == nullptr) {
        return RLN_ERR_NULL_POINTER;
    }
    *pipeline = nullptr;
    if (chunk_rows <= 0 || chunk_rows > (1 << 24) || depth < 2 || depth > kMaxDepth) {
        return RLN_ERR_HOST_BUFFERS;
    }
    if (branch_dtype != RLN_DTYPE_FLOAT32 && branch_dtype != RLN_DTYPE_FLOAT16
        && branch_dtype != RLN_DTYPE_BFLOAT16) {
        return RLN_ERR_BRANCH_DTYPE;
    }
    if (normalized_dtype != RLN_DTYPE_FLOAT32 && normalized_dtype != RLN_DTYPE_FLOAT16
        && normalized_dtype != RLN_DTYPE_BFLOAT16) {
        return RLN_ERR_NORMALIZED_DTYPE;
    }
    // the deterministic workspace for the largest chunk; also validates hidden
    const int64_t workspace_bytes = rln_sm100_backward_workspace_bytes(chunk_rows, hidden, 1);
    if (workspace_bytes < 0) {
        return static_cast<int>(workspace_bytes);
    }
    RlnHostPipeline* p = new (std::nothrow) RlnHostPipeline();
    if (p == nullptr) {
        return RLN_ERR_HOST_BUFFERS;
    }
    const cudaError_t device_error = cudaGetDevice(&p->device);
    if (device_error != cudaSuccess) {
        delete p;
        return rln::record_cuda_error(device_error);
    }
    p->hidden = hidden;
    p->branch_dtype = branch_dtype;
    p->normalized_dtype = normalized_dtype;
    p->chunk_rows = chunk_rows;
    p->depth = depth;
    p->workspace_bytes = workspace_bytes;
    const cudaError_t allocation_error = allocate(p);
    if (allocation_error != cudaSuccess) {
        release(p);
        (void)cudaGetLastError();  // clear the runtime's sticky copy of the same failure
        return rln::record_cuda_error(allocation_error);
    }
    *pipeline = p;
    return RLN_OK;
}

extern "C" int rln_sm100_host_pipeline_destroy(RlnHostPipeline* pipeline) {
    if (pipeline == nullptr) {
        return RLN_OK;
    }
    cudaStreamSynchronize(pipeline->stream_in);
    cudaStreamSynchronize(pipeline->stream_compute);
    cudaStreamSynchronize(pipeline->stream_out);
    release(pipeline);
    return RLN_OK;
}

#undef RLN_TRY
#define RLN_TRY(call)                                  \
    do {                                               \
        const cudaError_t rln_try_error = (call);      \
        if (rln_try_error != cudaSuccess) {            \
            return rln::record_cuda_error(rln_try_error); \
        }                                              \
    } while (0)

namespace {

// Enqueues the whole step on the pipeline's three streams.  Returns at the
// first failing call; the caller drains the streams in either case.
int enqueue_step(
    RlnHostPipeline* p,
    const float* x,
    const void* branch,
    const float* weight,
    const float* bias,
    const float* grad_updated,
    const void* grad_normalized,
    float* updated,
    void* normalized,
    float* grad_x,
    void* grad_branch,
    float* grad_parameters,
    int64_t rows,
    int32_t dropout_active,
    float dropout_p,
    float eps,
    uint64_t seed,
    uint64_t offset,
    int64_t row_base,
    int32_t deterministic,
    bool streaming) {
    if (p == nullptr || x == nullptr || branch == nullptr || weight == nullptr || bias == nullptr
        || grad_updated == nullptr || grad_normalized == nullptr || updated == nullptr
        || normalized == nullptr || grad_x == nullptr || grad_branch == nullptr
        || grad_parameters == nullptr) {
        return RLN_ERR_NULL_POINTER;
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
    int device = -1;
    RLN_TRY(cudaGetDevice(&device));
    if (device != p->device) {
        return RLN_ERR_HOST_BUFFERS;
    }
    const int64_t hidden = p->hidden;
    const size_t branch_element = p->branch_dtype == RLN_DTYPE_FLOAT32 ? 4 : 2;
    const size_t normalized_element = p->normalized_dtype == RLN_DTYPE_FLOAT32 ? 4 : 2;
    const char* branch_bytes = static_cast<const char*>(branch);
    char* grad_branch_bytes = static_cast<char*>(grad_branch);
    const char* grad_normalized_bytes = static_cast<const char*>(grad_normalized);
    char* normalized_bytes = static_cast<char*>(normalized);

    // The slot ring and its events carry over from the previous call: a step
    // enqueued behind another one (rln_sm100_host_forward_backward_enqueue) reuses
    // a slot only after that slot's kernels ran and its results left.
    const int64_t step = p->steps_enqueued + 1;
    const int tracked = static_cast<int>(step % kStepsTracked);
    if (p->steps_enqueued >= kStepsTracked) {
        // the completion entry is reused: the step that held it must have landed
        RLN_TRY(cudaEventSynchronize(p->step_out[tracked]));
        RLN_TRY(cudaEventSynchronize(p->step_compute[tracked]));
    }
    // Every copy goes through one of the two copy streams and the compute
    // stream holds kernels only.  (A small copy on the compute stream queues
    // behind whatever the copy engine of its direction already holds -- the
    // previous step's last chunks -- and would stall the kernels behind it
    // until then, which serialises consecutive steps.)
    const int set = static_cast<int>(step & 1);
    float* const device_weight = p->weight[set];
    float* const device_bias = p->bias[set];
    float* const device_total = p->total[set];
    if (step > 2) {
        // this set was used by step - 2: its kernels must be done before the
        // parameters are overwritten, its sums copied out before they are reset
        const int before = static_cast<int>((step - 2) % kStepsTracked);
        RLN_TRY(cudaStreamWaitEvent(p->stream_in, p->step_compute[before], 0));
        RLN_TRY(cudaStreamWaitEvent(p->stream_compute, p->step_out[before], 0));
    }
    RLN_TRY(cudaMemcpyAsync(
        device_weight, weight, hidden * sizeof(float), cudaMemcpyHostToDevice, p->stream_in));
    RLN_TRY(cudaMemcpyAsync(
        device_bias, bias, hidden * sizeof(float), cudaMemcpyHostToDevice, p->stream_in));
    // (the kernels of the first chunk wait for that chunk's in_ready event, which
    // the copy-in stream records after these two copies)

    // Copy-in of the chunk that starts at row `begin` into the next slot of the ring.
    auto enqueue_copy_in = [&](int64_t begin, Slot** taken) -> int {
        const int64_t count = rows - begin < p->chunk_rows ? rows - begin : p->chunk_rows;
        const size_t elements = static_cast<size_t>(count) * hidden;
        const size_t first = static_cast<size_t>(begin) * hidden;
        Slot& slot = p->slots[p->chunks_enqueued % p->depth];
        ++p->chunks_enqueued;
        // the slot's inputs are free once its previous kernels ran
        if (slot.used) {
            RLN_TRY(cudaStreamWaitEvent(p->stream_in, slot.computed, 0));
        }
        RLN_TRY(cudaMemcpyAsync(
            slot.x, x + first, elements * 4, cudaMemcpyHostToDevice, p->stream_in));
        RLN_TRY(cudaMemcpyAsync(
            slot.branch, branch_bytes + first * branch_element, elements * branch_element,
            cudaMemcpyHostToDevice, p->stream_in));
        RLN_TRY(cudaMemcpyAsync(
            slot.grad_updated, grad_updated + first, elements * 4, cudaMemcpyHostToDevice,
            p->stream_in));
        RLN_TRY(cudaMemcpyAsync(
            slot.grad_normalized, grad_normalized_bytes + first * normalized_element,
            elements * normalized_element, cudaMemcpyHostToDevice, p->stream_in));
        RLN_TRY(cudaEventRecord(slot.in_ready, p->stream_in));
        *taken = &slot;
        return RLN_OK;
    };

    // The copy-in runs one chunk ahead of the loop below.  For steps that stream
    // one behind the other (`streaming`, the enqueue entry) the copy-out of a
    // chunk additionally waits until the NEXT chunk has arrived.  Both PCIe
    // directions move a chunk in about the same time, so without that rule they
    // fall into lockstep: chunk c+1 arrives just as chunk c has left, and the
    // copy-out engine then idles for the kernels of chunk c+1 plus two
    // cross-stream hand-overs before it has anything to send, once per chunk.
    // With the rule the kernels of chunk c+1 run while chunk c leaves (measured
    // on streamed steps of 87,381 x 768: -2 % with 8,192-row chunks, -6 % with
    // 2,048-row chunks).  A lone step does not get the rule: it would start its
    // copy-out one chunk later and finish later (+4 % with 8,192-row chunks).
    Slot* current = nullptr;
    {
        const int status = enqueue_copy_in(0, &current);
        if (status != RLN_OK) {
            return status;
        }
    }
    int64_t chunk_index = 0;
    for (int64_t begin = 0; begin < rows; begin += p->chunk_rows, ++chunk_index) {
        const int64_t count = rows - begin < p->chunk_rows ? rows - begin : p->chunk_rows;
        const size_t elements = static_cast<size_t>(count) * hidden;
        const size_t first = static_cast<size_t>(begin) * hidden;
        Slot* next = nullptr;
        if (begin + p->chunk_rows < rows) {
            const int status = enqueue_copy_in(begin + p->chunk_rows, &next);
            if (status != RLN_OK) {
                return status;
            }
        }
        Slot& slot = *current;

        // compute (the slot's outputs are free once its previous results left)
        RLN_TRY(cudaStreamWaitEvent(p->stream_compute, slot.in_ready, 0));
        if (slot.used) {
            RLN_TRY(cudaStreamWaitEvent(p->stream_compute, slot.drained, 0));
        }
        int status = rln_sm100_forward(
            slot.x, slot.branch, device_weight, device_bias, slot.updated, slot.normalized,
            slot.mean, slot.rstd, slot.mask, count, p->hidden, p->branch_dtype,
            p->normalized_dtype, dropout_active, dropout_p, eps, seed, offset, row_base + begin,
            p->stream_compute);
        if (status != RLN_OK) {
            return status;
        }
        status = rln_sm100_backward(
            slot.grad_updated, slot.grad_normalized, slot.updated, device_weight, slot.mean,
            slot.rstd, slot.mask, slot.grad_x, slot.grad_branch, slot.grad_parameters,
            slot.workspace, p->workspace_bytes, count, p->hidden, p->branch_dtype,
            p->normalized_dtype, dropout_active, dropout_p, deterministic, p->stream_compute);
        if (status != RLN_OK) {
            return status;
        }
        const int parameter_count = static_cast<int>(2 * hidden);
        accumulate_parameters_kernel<<<(parameter_count + 255) / 256, 256, 0, p->stream_compute>>>(
            device_total, slot.grad_parameters, parameter_count, chunk_index == 0 ? 1 : 0);
        RLN_TRY(cudaGetLastError());
        RLN_TRY(cudaEventRecord(slot.computed, p->stream_compute));

        // copy out
        RLN_TRY(cudaStreamWaitEvent(p->stream_out, slot.computed, 0));
        if (streaming && next != nullptr) {
            RLN_TRY(cudaStreamWaitEvent(p->stream_out, next->in_ready, 0));
        }
        RLN_TRY(cudaMemcpyAsync(
            updated + first, slot.updated, elements * 4, cudaMemcpyDeviceToHost, p->stream_out));
        RLN_TRY(cudaMemcpyAsync(
            normalized_bytes + first * normalized_element, slot.normalized,
            elements * normalized_element, cudaMemcpyDeviceToHost, p->stream_out));
        RLN_TRY(cudaMemcpyAsync(
            grad_x + first, slot.grad_x, elements * 4, cudaMemcpyDeviceToHost, p->stream_out));
        RLN_TRY(cudaMemcpyAsync(
            grad_branch_bytes + first * branch_element, slot.grad_branch,
            elements * branch_element, cudaMemcpyDeviceToHost, p->stream_out));
        RLN_TRY(cudaEventRecord(slot.drained, p->stream_out));
        slot.used = true;
        current = next;
    }
    // the sums leave on the copy-out stream, behind the last chunk's results
    RLN_TRY(cudaEventRecord(p->step_compute[tracked], p->stream_compute));
    RLN_TRY(cudaStreamWaitEvent(p->stream_out, p->step_compute[tracked], 0));
    RLN_TRY(cudaMemcpyAsync(
        grad_parameters, device_total, 2 * hidden * sizeof(float), cudaMemcpyDeviceToHost,
        p->stream_out));
    RLN_TRY(cudaEventRecord(p->step_out[tracked], p->stream_out));
    ++p->steps_enqueued;
    return RLN_OK;
}

}  // namespace

namespace {

// Waits for everything the pipeline has enqueued; first failure wins.
int drain(RlnHostPipeline* p) {
    const cudaError_t drained_in = cudaStreamSynchronize(p->stream_in);
    const cudaError_t drained_compute = cudaStreamSynchronize(p->stream_compute);
    const cudaError_t drained_out = cudaStreamSynchronize(p->stream_out);
    for (const cudaError_t error : {drained_in, drained_compute, drained_out}) {
        if (error != cudaSuccess) {
            return rln::record_cuda_error(error);
        }
    }
    return RLN_OK;
}

}  // namespace

extern "C" int rln_sm100_host_forward_backward_enqueue(
    RlnHostPipeline* p,
    const float* x,
    const void* branch,
    const float* weight,
    const float* bias,
    const float* grad_updated,
    const void* grad_normalized,
    float* updated,
    void* normalized,
    float* grad_x,
    void* grad_branch,
    float* grad_parameters,
    int64_t rows,
    int32_t dropout_active,
    float dropout_p,
    float eps,
    uint64_t seed,
    uint64_t offset,
    int64_t row_base,
    int32_t deterministic) {
    if (p == nullptr) {
        return RLN_ERR_NULL_POINTER;
    }
    const int status = enqueue_step(
        p, x, branch, weight, bias, grad_updated, grad_normalized, updated, normalized, grad_x,
        grad_branch, grad_parameters, rows, dropout_active, dropout_p, eps, seed, offset,
        row_base, deterministic, /*streaming=*/true);
    if (status != RLN_OK) {
        // A step that failed half-way has copies in flight that target the
        // caller's host buffers; they must not outlive this call.
        (void)drain(p);
    }
    return status;
}

extern "C" int rln_sm100_host_pipeline_wait(RlnHostPipeline* p) {
    if (p == nullptr) {
        return RLN_ERR_NULL_POINTER;
    }
    return drain(p);
}

extern "C" int64_t rln_sm100_host_pipeline_steps_enqueued(const RlnHostPipeline* p) {
    return p == nullptr ? RLN_ERR_NULL_POINTER : p->steps_enqueued;
}

extern "C" int rln_sm100_host_pipeline_wait_step(RlnHostPipeline* p, int64_t step) {
    if (p == nullptr) {
        return RLN_ERR_NULL_POINTER;
    }
    if (step <= 0 || step > p->steps_enqueued) {
        return RLN_ERR_HOST_BUFFERS;
    }
    if (p->steps_enqueued - step >= kStepsTracked) {
        return RLN_OK;  // its completion entry was reused, which waited for it
    }
    const int tracked = static_cast<int>(step % kStepsTracked);
    RLN_TRY(cudaEventSynchronize(p->step_out[tracked]));
    RLN_TRY(cudaEventSynchronize(p->step_compute[tracked]));
    return RLN_OK;
}

extern "C" int rln_sm100_host_forward_backward(
    RlnHostPipeline* p,
    const float* x,
    const void* branch,
    const float* weight,
    const float* bias,
    const float* grad_updated,
    const void* grad_normalized,
    float* updated,
    void* normalized,
    float* grad_x,
    void* grad_branch,
    float* grad_parameters,
    int64_t rows,
    int32_t dropout_active,
    float dropout_p,
    float eps,
    uint64_t seed,
    uint64_t offset,
    int64_t row_base,
    int32_t deterministic) {
    if (p == nullptr) {
        return RLN_ERR_NULL_POINTER;
    }
    const int status = enqueue_step(
        p, x, branch, weight, bias, grad_updated, grad_normalized, updated, normalized, grad_x,
        grad_branch, grad_parameters, rows, dropout_active, dropout_p, eps, seed, offset,
        row_base, deterministic, /*streaming=*/false);
    // Drain the streams whatever happened: copies that were already enqueued
    // still target the caller's host buffers and must not outlive this call.
    const int drained = drain(p);
    return status != RLN_OK ? status : drained;
}
