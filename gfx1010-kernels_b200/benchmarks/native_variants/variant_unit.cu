// One build of the kernel templates of csrc/rln_kernels.cuh with the switches
// and the launch geometry given on the compiler command line, behind a
// four-function C interface.  benchmark_native_variants.py compiles this file
// once per variant into a shared library of its own and drives all of them
// from one process, so that every variant is timed on the same board, on the
// same buffers, inside the same warmed-up run.
//
// Command-line macros (all optional; unset = what the shipped library uses):
//   VARIANT_PACKED_FWD, VARIANT_PACKED_BWD   0 / 1: two-wide fp32 arithmetic (kPacked)
//   RLN_FWD_MASK_REDUX                       mask words combined with redux.sync
//   RLN_LOAD_POLICY, RLN_STORE_POLICY        cache policy of the hinted accesses
//   VARIANT_STREAM_HINTS   1: instantiate the kernels with the hinted accesses
//   VARIANT_FWD_WARPS, VARIANT_FWD_MIN_CTAS, VARIANT_FWD_LANES
//   VARIANT_BWD_WARPS, VARIANT_BWD_ROWS, VARIANT_BWD_CTAS_PER_SM
//   VARIANT_BWD_DYNAMIC    N > 0: the last N rounds of the backward's rows are claimed
//                          through a counter (a huge N = every row but a warp's first)
//   VARIANT_ZERO_IN_FORWARD  1: the forward's first CTA clears the [2, H] gradient buffer and
//                          the step launches no zeroing kernel (step mode only is meaningful)
//   VARIANT_HIDDEN         instantiate this width only (faster builds)
//
// fp16 branch, float32 normalized, dropout on, parameter gradients on, 16-byte
// aligned pointers: the configuration the headline numbers are quoted on.
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "rln_launch.h"

#ifndef VARIANT_STREAM_HINTS
#define VARIANT_STREAM_HINTS 0
#endif
#ifndef VARIANT_BWD_DYNAMIC
#define VARIANT_BWD_DYNAMIC 0
#endif
#ifndef VARIANT_ZERO_IN_FORWARD
#define VARIANT_ZERO_IN_FORWARD 0
#endif

#if defined(__GNUC__)
#define VARIANT_API extern "C" __attribute__((visibility("default")))
#else
#define VARIANT_API extern "C"
#endif

// Everything one step needs; filled by the Python driver through ctypes.
struct VariantArgs {
    const float* x;
    const void* branch;
    const float* weight;
    const float* bias;
    float* updated;
    float* normalized;
    float* mean;
    float* rstd;
    uint32_t* mask;
    const float* grad_updated;
    const float* grad_normalized;
    float* grad_x;
    void* grad_branch;
    float* grad_parameters;   // [2, hidden]
    float* partials;          // deterministic scratch, [grid, 2, hidden]
    unsigned int* row_counter;  // 16 bytes
    int64_t rows;
    int32_t hidden;
    int32_t deterministic;
    float dropout_p;
    float eps;
    uint64_t seed;
    uint64_t offset;
    int32_t sm_count;
    int32_t reserved;
};

namespace {

using namespace rln;

template <int H>
struct Geometry {
#ifdef VARIANT_FWD_WARPS
    static constexpr int kFwdWarps = VARIANT_FWD_WARPS;
#else
    static constexpr int kFwdWarps = ForwardTune<H>::kWarps;
#endif
#ifdef VARIANT_FWD_MIN_CTAS
    static constexpr int kFwdMinCtas = VARIANT_FWD_MIN_CTAS;
#else
    static constexpr int kFwdMinCtas = ForwardTune<H>::kMinCtas;
#endif
#ifdef VARIANT_FWD_LANES
    static constexpr int kFwdLanes = VARIANT_FWD_LANES;
#else
    static constexpr int kFwdLanes = ForwardTune<H>::kLanes;
#endif
#ifdef VARIANT_PACKED_FWD
    static constexpr bool kFwdPacked = VARIANT_PACKED_FWD != 0;
#else
    static constexpr bool kFwdPacked = ForwardTune<H>::kPacked;
#endif
#ifdef VARIANT_PACKED_BWD
    static constexpr bool kBwdPacked = VARIANT_PACKED_BWD != 0;
#else
    static constexpr bool kBwdPacked = false;
#endif
#ifdef VARIANT_BWD_WARPS
    static constexpr int kBwdWarps = VARIANT_BWD_WARPS;
#else
    static constexpr int kBwdWarps = BackwardTune<H>::kWarps;
#endif
#ifdef VARIANT_BWD_ROWS
    static constexpr int kBwdRows = VARIANT_BWD_ROWS;
#else
    static constexpr int kBwdRows = BackwardTune<H>::kRows;
#endif
#ifdef VARIANT_BWD_CTAS_PER_SM
    static constexpr int kBwdCtas = VARIANT_BWD_CTAS_PER_SM;
#else
    static constexpr int kBwdCtas = BackwardTune<H>::kCtasPerSm;
#endif
};

ForwardParams forward_params(const VariantArgs& a) {
    ForwardParams p = {};
    p.x = a.x;
    p.branch = a.branch;
    p.weight = a.weight;
    p.bias = a.bias;
    p.updated = a.updated;
    p.normalized = a.normalized;
    p.mean = a.mean;
    p.rstd = a.rstd;
    p.mask = a.mask;
    p.rows = a.rows;
    p.row_base = 0;
    p.scale = 1.0f / (1.0f - a.dropout_p);
    p.eps = a.eps;
    p.threshold = static_cast<uint32_t>(static_cast<double>(a.dropout_p) * 4294967296.0);
    p.seed_lo = static_cast<uint32_t>(a.seed);
    p.seed_hi = static_cast<uint32_t>(a.seed >> 32);
    p.offset_lo = static_cast<uint32_t>(a.offset >> 2);   // Philox block index = word offset / 4
    p.offset_hi = static_cast<uint32_t>(a.offset >> 34);
#if VARIANT_ZERO_IN_FORWARD
    p.zero_buffer = reinterpret_cast<float4*>(a.grad_parameters);
    p.zero_count4 = 2 * a.hidden / 4;
#endif
    return p;
}

template <int H>
int backward_grid_of(const VariantArgs& a) {
    using G = Geometry<H>;
    const int64_t per_cta = static_cast<int64_t>(G::kBwdWarps) * G::kBwdRows;
    const int64_t needed = (a.rows + per_cta - 1) / per_cta;
    const int64_t resident = static_cast<int64_t>(a.sm_count) * G::kBwdCtas;
    return static_cast<int>(needed < resident ? needed : resident);
}

BackwardParams backward_params(const VariantArgs& a, bool dynamic) {
    BackwardParams p = {};
    p.grad_updated = a.grad_updated;
    p.grad_normalized = a.grad_normalized;
    p.updated = a.updated;
    p.weight = a.weight;
    p.mean = a.mean;
    p.rstd = a.rstd;
    p.mask = a.mask;
    p.grad_x = a.grad_x;
    p.grad_branch = a.grad_branch;
    p.grad_parameters = a.grad_parameters;
    p.partials = a.partials;
    p.rows = a.rows;
    p.scale = 1.0f / (1.0f - a.dropout_p);
    p.deterministic = a.deterministic;
    p.row_counter = dynamic ? a.row_counter : nullptr;
    p.dynamic_begin = 0;
    return p;
}

template <int H>
cudaError_t forward_of(const VariantArgs& a, cudaStream_t stream) {
    using G = Geometry<H>;
    const ForwardParams p = forward_params(a);
    if constexpr (G::kFwdLanes == kWarpSize) {
        const int64_t blocks = (a.rows + G::kFwdWarps - 1) / G::kFwdWarps;
        return launch_dependent(
            rln_forward_kernel<H, __half, true, true, G::kFwdWarps, 1, G::kFwdMinCtas, false,
                               VARIANT_STREAM_HINTS != 0, float, G::kFwdPacked>,
            static_cast<unsigned>(blocks), G::kFwdWarps * kWarpSize, stream, p);
    } else {
        constexpr int kRowsPerCta = G::kFwdWarps * (kWarpSize / G::kFwdLanes);
        const int64_t blocks = (a.rows + kRowsPerCta - 1) / kRowsPerCta;
        return launch_dependent(
            rln_forward_subwarp_kernel<H, __half, true, true, G::kFwdWarps, G::kFwdLanes,
                                       G::kFwdMinCtas, false, VARIANT_STREAM_HINTS != 0, float,
                                       G::kFwdPacked>,
            static_cast<unsigned>(blocks), G::kFwdWarps * kWarpSize, stream, p);
    }
}

// zeroing kernel + backward (+ fixed-order reduction in deterministic mode)
template <int H>
cudaError_t backward_of(const VariantArgs& a, cudaStream_t stream, bool fused_step) {
    using G = Geometry<H>;
    const int grid = backward_grid_of<H>(a);
    constexpr bool kDynamic = VARIANT_BWD_DYNAMIC != 0;
    const bool dynamic = kDynamic && !a.deterministic;
    BackwardParams p = backward_params(a, dynamic);
    {
        // all but the last VARIANT_BWD_DYNAMIC rounds of the grid are static
        const int64_t stride = static_cast<int64_t>(grid) * G::kBwdWarps * G::kBwdRows;
        const int64_t rounds = (a.rows + stride - 1) / stride;
        const int64_t static_rounds =
            rounds > VARIANT_BWD_DYNAMIC ? rounds - VARIANT_BWD_DYNAMIC : 1;
        p.dynamic_begin = static_rounds * stride;
    }
    cudaError_t error = cudaSuccess;
    if (!a.deterministic && !(VARIANT_ZERO_IN_FORWARD && fused_step)) {
        error = launch_dependent(
            rln_zero_kernel<256>, 1u + (2 * H / 4 - 1) / 256, 256u, stream,
            reinterpret_cast<float4*>(a.grad_parameters), 2 * H / 4,
            dynamic ? reinterpret_cast<uint4*>(a.row_counter) : static_cast<uint4*>(nullptr));
        if (error != cudaSuccess) {
            return error;
        }
    }
    if (dynamic) {
        error = launch_dependent(
            rln_backward_kernel<H, __half, true, true, true, G::kBwdWarps, G::kBwdRows,
                                G::kBwdCtas, VARIANT_STREAM_HINTS != 0, float, kDynamic,
                                G::kBwdPacked>,
            static_cast<unsigned>(grid), G::kBwdWarps * kWarpSize, stream, p);
    } else {
        error = launch_dependent(
            rln_backward_kernel<H, __half, true, true, true, G::kBwdWarps, G::kBwdRows,
                                G::kBwdCtas, VARIANT_STREAM_HINTS != 0, float, false,
                                G::kBwdPacked>,
            static_cast<unsigned>(grid), G::kBwdWarps * kWarpSize, stream, p);
    }
    if (error != cudaSuccess || !a.deterministic) {
        return error;
    }
    return launch_dependent(
        rln_reduce_partials_kernel<32>, static_cast<unsigned>((2 * H + 31) / 32), 1024u, stream,
        static_cast<const float*>(a.partials), a.grad_parameters, grid, 2 * H);
}

template <typename Function>
int for_hidden(int hidden, Function function) {
    switch (hidden) {
#define VARIANT_CASE(HIDDEN) \
    case HIDDEN: return function(std::integral_constant<int, HIDDEN>());
#ifdef VARIANT_HIDDEN
        VARIANT_CASE(VARIANT_HIDDEN)
#else
        VARIANT_CASE(128)
        VARIANT_CASE(256)
        VARIANT_CASE(384)
        VARIANT_CASE(512)
        VARIANT_CASE(768)
        VARIANT_CASE(1024)
#endif
#undef VARIANT_CASE
        default: return -2;
    }
}

}  // namespace

// mode: 0 forward, 1 zero + backward, 2 forward + zero + backward; `steps`
// repetitions enqueued back to back on `stream`, each forward with a fresh
// Philox offset.  Returns 0, -2 (width not built in) or a positive cudaError_t.
VARIANT_API int rln_variant_run(const VariantArgs* args, int mode, int steps, void* stream_pointer) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_pointer);
    return for_hidden(args->hidden, [&](auto hidden_constant) -> int {
        constexpr int H = decltype(hidden_constant)::value;
        VariantArgs a = *args;
        for (int index = 0; index < steps; ++index) {
            a.offset = args->offset + 4ull * static_cast<uint64_t>(index);
            if (mode == 0 || mode == 2) {
                const cudaError_t error = forward_of<H>(a, stream);
                if (error != cudaSuccess) {
                    return static_cast<int>(error);
                }
            }
            if (mode == 1 || mode == 2) {
                const cudaError_t error = backward_of<H>(a, stream, mode == 2);
                if (error != cudaSuccess) {
                    return static_cast<int>(error);
                }
            }
        }
        return 0;
    });
}

// CTAs of the backward grid for these arguments (= partials in deterministic mode).
VARIANT_API int rln_variant_backward_grid(const VariantArgs* args) {
    return for_hidden(args->hidden, [&](auto hidden_constant) -> int {
        return backward_grid_of<decltype(hidden_constant)::value>(*args);
    });
}

VARIANT_API int rln_variant_args_bytes(void) { return static_cast<int>(sizeof(VariantArgs)); }
