/*
 * C ABI of the sm_100a (B200) fused residual-add + dropout + LayerNorm path.
 *
 * Plain pointers and sizes only: no torch, ATen or C++ types cross this
 * boundary.  Every pointer named "device" must be a device address valid on
 * the CUDA device that is current when the call is made; the work is enqueued
 * on `stream` (a cudaStream_t passed as void*, NULL = the legacy default
 * stream) and the call returns without synchronising.  No entry point
 * allocates or frees device memory unless its comment says so.
 *
 * These entry points replace, one to one, the two host functions that the
 * reference project (T-vaccari/gfx1010-kernels) exposes to its binding in
 * csrc/residual_layer_norm.h:10-42 and implements in
 * csrc/residual_layer_norm_kernel.hip:1720-2036.  The reference mixes tensor
 * allocation, validation and launch in those functions; here allocation and
 * tensor validation stay in the binding and the launch is what crosses the ABI.
 *
 * Return value: RLN_OK (0) or a negative RLN_ERR_* code.  Nothing throws.
 */
#ifndef RLN_SM100_H_
#define RLN_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define RLN_API __attribute__((visibility("default")))
#else
#define RLN_API
#endif

#define RLN_OK 0
#define RLN_ERR_NULL_POINTER (-1)       /* a required pointer is NULL */
#define RLN_ERR_HIDDEN_SIZE (-2)        /* hidden not in {128,256,384,512,768,1024} */
#define RLN_ERR_ROW_COUNT (-3)          /* rows <= 0 ("empty tensors are unsupported") */
#define RLN_ERR_DROPOUT_P (-4)          /* dropout_p outside [0, 1) */
#define RLN_ERR_EPS (-5)                /* eps <= 0 */
#define RLN_ERR_ALIGNMENT (-6)          /* pointer not aligned to its element size */
#define RLN_ERR_WORKSPACE (-7)          /* workspace missing or too small */
#define RLN_ERR_CUDA (-8)               /* a CUDA runtime call failed; see rln_sm100_last_cuda_error */
#define RLN_ERR_HOST_BUFFERS (-9)       /* host-buffer pipeline: bad chunk size or context */
#define RLN_ERR_LIMIT (-10)             /* size beyond a documented fixed maximum */
#define RLN_ERR_BRANCH_DTYPE (-11)      /* branch_dtype is not one of RLN_DTYPE_* */
#define RLN_ERR_NORMALIZED_DTYPE (-12)  /* normalized_dtype is not one of RLN_DTYPE_* */

/* Element type of `branch` / `grad_branch`.  0 and 1 are the reference's two
 * cases (its entry points carry a bool "branch is half",
 * csrc/residual_layer_norm.h:36); bfloat16 is an addition for mixed-precision
 * training on this hardware.  Rounding rule for all three: the dropped branch
 * is float32(b) * keep * scale rounded once to the branch type, grad_branch is
 * the float32 gradient * keep * scale rounded once to the branch type. */
#define RLN_DTYPE_FLOAT32 0
#define RLN_DTYPE_FLOAT16 1
#define RLN_DTYPE_BFLOAT16 2
#define RLN_BRANCH_FLOAT32 RLN_DTYPE_FLOAT32
#define RLN_BRANCH_FLOAT16 RLN_DTYPE_FLOAT16
#define RLN_BRANCH_BFLOAT16 RLN_DTYPE_BFLOAT16

/* Element type of `normalized` (forward) and of `grad_normalized` (backward),
 * the same RLN_DTYPE_* codes.  RLN_DTYPE_FLOAT32 is the reference's contract
 * (csrc/residual_layer_norm_kernel.hip:1746-1747: both outputs float32).  The
 * two 16-bit types are an addition for a consumer that feeds `normalized` to a
 * half-precision GEMM: the float32 result is rounded once (to nearest even) on
 * store, the incoming gradient is widened on load, everything in between is
 * the same float32 arithmetic, and the operator moves 2 bytes less per element
 * in each direction.  They need the 16-byte pointer alignment of the
 * vectorised kernels (8-byte for the 16-bit tensors): RLN_ERR_ALIGNMENT
 * otherwise. */

/* ABI version of this header; bumped on any signature change. */
#define RLN_SM100_ABI_VERSION 4
RLN_API int rln_sm100_abi_version(void);

/* Human-readable text for a status code (static storage, never NULL). */
RLN_API const char* rln_sm100_status_string(int status);

/* cudaError_t value of the most recent failing CUDA call made by this library
 * on the calling thread (0 if none). */
RLN_API int rln_sm100_last_cuda_error(void);

/*
 * Forward: updated = x + dropout(branch); normalized = LayerNorm(updated).
 *
 * Replaces residual_layer_norm_forward_hip
 * (csrc/residual_layer_norm.h:10-24, csrc/residual_layer_norm_kernel.hip:1720-1827)
 * and the kernels it dispatches (forward kernel :425-545, vector4 kernel :353-422).
 *
 *   x            device, float32 [rows, hidden]
 *   branch       device, float32 / float16 / bfloat16 per branch_dtype (RLN_DTYPE_*), [rows, hidden]
 *   weight, bias device, float32 [hidden]
 *   updated      device out, float32 [rows, hidden]
 *   normalized   device out, float32 / float16 / bfloat16 per normalized_dtype, [rows, hidden]
 *   mean, rstd   device out, float32 [rows]   (rstd = rsqrt(centred variance + eps))
 *   dropout_mask device out, uint32 [rows * hidden/32]; bit (col & 31) of word
 *                row*(hidden/32) + col/32 is 1 when the element was kept
 *                (layout of :500-511).  Ignored (may be NULL) when
 *                dropout_active == 0.
 *   dropout_active  the caller's (training && dropout_p > 0)
 *   seed, offset Philox4x32-10 key and per-call position.  `offset` counts
 *                32-bit words of the generator's stream, as torch's CUDA
 *                generator does; a Philox call yields four words, so the
 *                counter holds the block index b = offset / 4 (pass multiples
 *                of 4: the low two bits are dropped).  Element group
 *                g = ((row_base + row) * hidden + col) / 4 uses counter
 *                (lo32(b), hi32(b), lo32(g), hi32(g)), key
 *                (lo32(seed), hi32(seed)); output word j decides column 4g+j;
 *                keep <=> word >= (uint32)((double)dropout_p * 2^32)  (:896-899).
 *                One call uses block b only, so a consumer that starts at
 *                offset + 4 or later never reuses its words.
 *   row_base     global index of this call's first row.  A row shard that
 *                passes its global offset reproduces the mask of the unsharded
 *                call bit for bit.  0 for an unsharded call.
 *
 * Pointers that are 16-byte aligned (8-byte for a 16-bit branch) take the
 * vectorised kernels; otherwise a scalar kernel with identical results in
 * exact arithmetic is used (the reference's alignment predicate :1084-1120).
 */
RLN_API int rln_sm100_forward(
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
    void* stream);

/*
 * Forward whose Philox (seed, offset) is read from DEVICE memory when the
 * kernel runs: seed = *device_seed, offset = *device_offset + offset_extra
 * (in words; the block index is that sum / 4, as in rln_sm100_forward).
 * Everything else as rln_sm100_forward.
 *
 * This is the form a launch recorded into a CUDA graph needs: the reference
 * refuses dropout under graph capture because its kernel takes the generator
 * state by value (csrc/residual_layer_norm_kernel.hip:1758-1777); with the
 * state behind pointers every replay uses whatever the framework has stored
 * there (torch's graph-safe generator keeps exactly such a seed/offset pair and
 * hands out an intra-graph offset for each consumer).  This form needs the
 * 16-byte pointer alignment of the vectorised kernels (RLN_ERR_ALIGNMENT
 * otherwise).
 */
RLN_API int rln_sm100_forward_device_rng(
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
    void* stream);

/*
 * Bytes of device scratch the backward needs for the fixed-order (deterministic)
 * parameter reduction on the current device: one [2, hidden] float32 partial
 * per CTA of the persistent grid.  0 when deterministic == 0 or when parameter
 * gradients are not requested.  Negative RLN_ERR_* on invalid arguments.
 *
 * Stands where the reference allocates its [2, ceil(rows/block_rows), hidden]
 * partial tensor (csrc/residual_layer_norm_kernel.hip:1870-1878).
 */
RLN_API int64_t rln_sm100_backward_workspace_bytes(
    int64_t rows,
    int32_t hidden,
    int32_t deterministic);

/*
 * Backward: grad_x, grad_branch and (optionally) grad_weight/grad_bias in one
 * pass over the row data.
 *
 * Replaces residual_layer_norm_backward_hip
 * (csrc/residual_layer_norm.h:27-42, csrc/residual_layer_norm_kernel.hip:1830-2036)
 * and its kernels: backward-input :548-618 / :621-724, deterministic partials +
 * reduce :727-786, atomic parameter kernels :789-869.
 *
 *   grad_updated, updated                    device, float32 [rows, hidden]
 *   grad_normalized                          device, [rows, hidden] in the type
 *                                            the forward stored `normalized` in
 *                                            (normalized_dtype, RLN_DTYPE_*)
 *   weight                                   device, float32 [hidden]
 *   mean, rstd                               device, float32 [rows]
 *   dropout_mask     device, uint32 [rows*hidden/32] (ignored when dropout_active == 0)
 *   grad_x           device out, float32 [rows, hidden]
 *   grad_branch      device out, [rows, hidden] in the branch type
 *   grad_parameters  device out, float32 [2, hidden]: row 0 = grad_weight
 *                    (sum over rows of grad_normalized * xhat), row 1 = grad_bias
 *                    (sum over rows of grad_normalized).  NULL = not requested
 *                    (the reference's compute_parameter_gradients == false).
 *   deterministic    0: per-CTA shared-memory partials + fp32 atomics into
 *                       grad_parameters (zeroed by this call on `stream`);
 *                    1: per-CTA partials stored to `workspace`, then summed in
 *                       CTA-index order by a second kernel.  The grid is a pure
 *                       function of (hidden, rows, device), so two calls with
 *                       the same inputs give bitwise-identical results.
 *   workspace        device scratch of at least
 *                    rln_sm100_backward_workspace_bytes(...) bytes, 16-byte
 *                    aligned; may be NULL when that size is 0.
 */
RLN_API int rln_sm100_backward(
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
    void* stream);

/*
 * Backward for callers that must not allocate: same outputs as
 * rln_sm100_backward(..., normalized_dtype = RLN_DTYPE_FLOAT32,
 * deterministic = 1) with parameter gradients, but the
 * per-CTA partials are kept in a scratch array built into this library's
 * device image, so no workspace is passed and nothing is allocated -- not by
 * this call and not by anything it calls.
 *
 * It has no counterpart in the reference, whose backward always allocates its
 * partial tensor through torch.  It exists for hosts that cannot do that:
 * runtimes that gave all device memory to their own pool and forbid allocation
 * calls inside an operator, plugin interfaces whose run step may not allocate,
 * and loops where the device-wide synchronisation of a cudaMalloc or cudaFree
 * is not acceptable.  The caller still provides every input and output buffer.
 *
 * Limits and rules:
 *   - The scratch is RLN_STATIC_SCRATCH_BYTES (4 MiB) per GPU, held by every
 *     GPU that loads the library until the process exits.  A call needs
 *     grid * 2 * hidden * 4 bytes (grid = the persistent backward grid, at
 *     most 6 CTAs per SM): at most 2.4 MB on a 148-SM B200 for every supported
 *     width and any row count.  A device on which a call would need more gets
 *     RLN_ERR_LIMIT ("size exceeds a fixed maximum of this entry point").
 *   - The first call on each device looks the scratch address up (one
 *     cudaGetSymbolAddress with that device current, then cached).  Make that
 *     first call during set-up, before any stream capture.
 *   - All calls on a device share the one array, and it keeps whatever the
 *     last call left there.  Nothing in it needs clearing (each call overwrites
 *     every partial it later reads), but two calls that overlap on the GPU --
 *     different streams, or different host threads -- race on it and give
 *     wrong grad_parameters.  Serialise calls per device.
 *   - grad_parameters is required (this is the variant that reduces them).
 *   - The cached scratch address belongs to the device's primary context.  It
 *     does not survive cudaDeviceReset (or any other teardown of that context):
 *     do not reset a device while this library is loaded and this entry point
 *     is still going to be called on it.
 *
 * Arguments as in rln_sm100_backward.
 */
#define RLN_STATIC_SCRATCH_BYTES (4u << 20)

RLN_API int rln_sm100_backward_static_scratch(
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
    void* stream);

/*
 * Host-buffer pipeline: one training step (forward + backward) over rows that
 * live in HOST memory, results returned to HOST memory.
 *
 * The reference has no counterpart: its entry points take device tensors only
 * (csrc/residual_layer_norm.h:10-42) and a caller with host data pays a full
 * copy in, a full copy out and the kernels back to back.  This entry overlaps
 * the three: rows are cut into chunks; while chunk c is computed on the
 * device, chunk c+1 is copied in and chunk c-1 is copied out on separate
 * streams (both PCIe directions busy at once).  Results are identical to one
 * rln_sm100_forward + rln_sm100_backward call over all rows: every chunk passes
 * its global row offset to the Philox counter, and grad_weight/grad_bias are
 * summed over chunks in chunk order.
 *
 * rln_sm100_host_pipeline_create ALLOCATES device staging buffers
 * (cudaMalloc, about depth * chunk_rows * hidden * 30 bytes), streams and
 * events on the current device; _destroy frees them.  A pipeline is bound to
 * the device it was created on and serves one call at a time.
 *
 * Host pointers should be page-locked (cudaHostAlloc / cudaHostRegister /
 * torch pin_memory); pageable memory works but the copies then do not overlap.
 * rln_sm100_host_forward_backward returns after every output has landed in
 * host memory (it synchronises its own streams, nothing else).
 *
 * rln_sm100_host_forward_backward_enqueue takes the same arguments and returns
 * as soon as the step is enqueued; rln_sm100_host_pipeline_wait returns once
 * everything enqueued so far has landed, rln_sm100_host_pipeline_wait_step(p, n)
 * once the n-th step enqueued on this pipeline has (n counts from 1;
 * rln_sm100_host_pipeline_steps_enqueued gives the number so far, i.e. the n of
 * the step just enqueued; an n outside 1..that number is RLN_ERR_HOST_BUFFERS).
 * At most 8 steps are tracked: enqueueing a ninth first waits for the oldest.
 * Steps enqueued back to back overlap:
 * the first chunks of step i+1 are copied in while the last chunks of step i
 * are computed and copied out, so neither PCIe direction idles between steps
 * (a lone step leaves each direction idle for one chunk).  Rules for enqueued
 * steps: every host buffer of a step -- inputs, weight, bias and outputs --
 * must stay valid and untouched until a wait that covers the step has returned;
 * steps in flight must not share output buffers; one thread per pipeline.  If _enqueue returns an
 * error it has already waited for the copies that were in flight.
 *
 *   x, branch, grad_updated, grad_normalized   host in,  [rows, hidden]
 *   weight, bias                                host in,  float32 [hidden]
 *   updated, normalized, grad_x, grad_branch    host out, [rows, hidden]
 *   grad_parameters                             host out, float32 [2, hidden]
 *   other arguments as in rln_sm100_forward / rln_sm100_backward.
 * branch / grad_branch have the pipeline's branch_dtype, normalized /
 * grad_normalized its normalized_dtype (RLN_DTYPE_*); the step is bound by the
 * PCIe link, so a 16-bit `normalized` shortens it by the bytes it saves
 * (2 of 14 per element in each direction).
 */
typedef struct RlnHostPipeline RlnHostPipeline;

RLN_API int rln_sm100_host_pipeline_create(
    RlnHostPipeline** pipeline,
    int32_t hidden,
    int32_t branch_dtype,
    int32_t normalized_dtype,
    int64_t chunk_rows,
    int32_t depth);

RLN_API int rln_sm100_host_pipeline_destroy(RlnHostPipeline* pipeline);

RLN_API int rln_sm100_host_forward_backward(
    RlnHostPipeline* pipeline,
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
    int32_t deterministic);

RLN_API int rln_sm100_host_forward_backward_enqueue(
    RlnHostPipeline* pipeline,
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
    int32_t deterministic);

RLN_API int rln_sm100_host_pipeline_wait(RlnHostPipeline* pipeline);

RLN_API int64_t rln_sm100_host_pipeline_steps_enqueued(const RlnHostPipeline* pipeline);

RLN_API int rln_sm100_host_pipeline_wait_step(RlnHostPipeline* pipeline, int64_t step);

#ifdef __cplusplus
}
#endif

#endif  /* RLN_SM100_H_ */
