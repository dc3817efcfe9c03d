// Device code of the sm_100a fused residual-add + dropout + LayerNorm path.
//
// Design (B200, 148 SMs, HBM3e): the operator has no contraction and does
// O(10) flops per element, so every kernel here is an HBM streaming kernel.
//   * One warp owns one row at a time.  All supported widths are multiples of
//     128, so lane l owns the float4 chunks l, l+32, l+64, ... of the row and
//     every global access of a warp is one fully coalesced 512-byte (fp32) or
//     256-byte (fp16 branch) transaction.  The whole row stays in registers
//     between the load and the store: row data is read from HBM exactly once.
//   * Row mean and the centred variance are two 5-step xor-shuffle butterflies;
//     there is no __syncthreads anywhere in the row loop.
//   * The dropout keep decision of the four columns of a chunk is one
//     Philox4x32-10 call keyed on (seed, offset, global element-group index);
//     eight neighbouring lanes OR their nibbles into one 32-bit mask word.
//   * The backward reads grad_updated, grad_normalized and updated once,
//     writes grad_x and grad_branch, and accumulates the grad_weight/grad_bias
//     partial sums of the rows a warp visits in registers (persistent grid).
//     The warps of a CTA combine in shared memory in warp order; the CTA then
//     either issues vector fp32 atomics or stores its partial for the
//     fixed-order second pass.
//
// The arithmetic follows the reference project's HIP kernels
// (csrc/residual_layer_norm_kernel.hip): forward :483-545, backward-input
// :572-617, parameter sums :741-760; the launch geometry, the Philox counter
// layout and the single-pass backward do not.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rln {

constexpr int kWarpSize = 32;
constexpr unsigned kFullMask = 0xffffffffu;

struct ForwardParams {
    const float* x;
    const void* branch;
    const float* weight;
    const float* bias;
    float* updated;
    void* normalized;  // float32, or float16 / bfloat16 for kernels instantiated with that NormT
    float* mean;
    float* rstd;
    uint32_t* mask;
    int64_t rows;
    int64_t row_base;
    float scale;
    float eps;
    uint32_t threshold;
    uint32_t seed_lo;
    uint32_t seed_hi;
    uint32_t offset_lo;   // Philox block index = word offset / 4 (low, high half)
    uint32_t offset_hi;
    // Philox state kept on the device (set when the launch is recorded into a
    // CUDA graph, so that each replay sees the generator's current state):
    // seed = *device_seed, offset = *device_offset + device_offset_extra.
    // Read only by kernels instantiated with kDeviceRng.
    const int64_t* device_seed;
    const int64_t* device_offset;
    uint64_t device_offset_extra;
    // Optional (set by the variant benchmark only; the library passes NULL): a
    // small buffer (16-byte aligned, zero_count4 float4 words) that the first
    // CTA clears -- the [2, H] target of the following backward's atomics, so
    // that no zeroing kernel stands between forward and backward.  Measured
    // gain: about 1 us per step (the zeroing kernel is already hidden by
    // programmatic dependent launch), too little to carry a buffer that the
    // backward allocates today through the forward's interface.
    float4* zero_buffer;
    int zero_count4;
};

// The forward kernels' side job (see ForwardParams::zero_buffer).
__device__ __forceinline__ void clear_side_buffer(const ForwardParams& p) {
    if (p.zero_buffer != nullptr && blockIdx.x == 0) {
        for (int i = threadIdx.x; i < p.zero_count4; i += blockDim.x) {
            p.zero_buffer[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    }
}

struct PhiloxState {
    uint32_t seed_lo;
    uint32_t seed_hi;
    uint32_t offset_lo;
    uint32_t offset_hi;
};

struct BackwardParams {
    const float* grad_updated;
    const void* grad_normalized;  // element type = the forward's NormT
    const float* updated;
    const float* weight;
    const float* mean;
    const float* rstd;
    const uint32_t* mask;
    float* grad_x;
    void* grad_branch;
    float* grad_parameters;  // [2, H]; atomics target (fast path)
    float* partials;         // [gridDim.x, 2, H]; deterministic path
    int64_t rows;
    float scale;
    int deterministic;
    // Kernels instantiated with kDynamicRows (variant benchmark only): rows
    // below dynamic_begin (a multiple of the grid's stride, at least one stride)
    // are split statically, the rows from there on are claimed from
    // row_counter, which is zeroed before the launch.
    unsigned int* row_counter;
    int64_t dynamic_begin;
};

// ---------------------------------------------------------------------------
// Programmatic dependent launch (sm_90+).  Every kernel first allows the next
// kernel of the stream to be scheduled while this one drains, then waits until
// the previous kernel has completed and its writes are visible.  Both are
// no-ops for a launch without the programmatic-serialization attribute.
// Nothing is read or written before the wait, so any predecessor is safe.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void grid_dependency_sync() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Zeroes a small buffer; stands in for cudaMemsetAsync so that the kernel
// chain of a training step stays kernel -> kernel (a memset node would break
// the programmatic dependency between the forward and the backward).
template <int kThreads>
__global__ void __launch_bounds__(kThreads)
rln_zero_kernel(float4* __restrict__ out, int count4, uint4* __restrict__ extra) {
    grid_dependency_sync();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < count4; i += gridDim.x * blockDim.x) {
        out[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    // the backward's row counter (one 16-byte word somewhere else), if any
    if (extra != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
        *extra = make_uint4(0u, 0u, 0u, 0u);
    }
}

// ---------------------------------------------------------------------------
// Philox4x32-10 (Salmon et al., SC'11), written out; one call = 4 random words.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint4 philox4x32_10(uint4 counter, uint32_t key0, uint32_t key1) {
    constexpr uint32_t kM0 = 0xD2511F53u;
    constexpr uint32_t kM1 = 0xCD9E8D57u;
    constexpr uint32_t kW0 = 0x9E3779B9u;
    constexpr uint32_t kW1 = 0xBB67AE85u;
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        const uint32_t hi0 = __umulhi(kM0, counter.x);
        const uint32_t lo0 = kM0 * counter.x;
        const uint32_t hi1 = __umulhi(kM1, counter.z);
        const uint32_t lo1 = kM1 * counter.z;
        counter = make_uint4(hi1 ^ counter.y ^ key0, lo1, hi0 ^ counter.w ^ key1, lo0);
        key0 += kW0;
        key1 += kW1;
    }
    return counter;
}

// (seed, offset) of this launch: immediate, or read from device memory.
__device__ __forceinline__ PhiloxState resolve_philox_state(const ForwardParams& p) {
    const uint64_t seed = static_cast<uint64_t>(__ldg(p.device_seed));
    // word offset -> Philox block index (four words per call), as on the host side
    const uint64_t offset =
        (static_cast<uint64_t>(__ldg(p.device_offset)) + p.device_offset_extra) >> 2;
    PhiloxState state;
    state.seed_lo = static_cast<uint32_t>(seed);
    state.seed_hi = static_cast<uint32_t>(seed >> 32);
    state.offset_lo = static_cast<uint32_t>(offset);
    state.offset_hi = static_cast<uint32_t>(offset >> 32);
    return state;
}

// ---------------------------------------------------------------------------
// Global-memory access.  kAligned == false is the 4-byte-aligned fallback with
// the same lane->column mapping and therefore bit-identical arithmetic.  Row
// data is touched once; streaming cache hints are available as an option (see
// kStream below) but are not what ships.
// ---------------------------------------------------------------------------
// Cache policy of the hinted accesses (compile-time tunables, used when kStream is on).
//   RLN_LOAD_POLICY : 0 plain, 1 ld.global.nc (__ldg), 2 evict-first (__ldcs),
//                     3 ld.global.nc.L1::no_allocate
//   RLN_STORE_POLICY: 0 plain, 1 evict-first (__stcs), 2 write-through (__stwt)
#ifndef RLN_LOAD_POLICY
#define RLN_LOAD_POLICY 2
#endif
#ifndef RLN_STORE_POLICY
#define RLN_STORE_POLICY 1
#endif

__device__ __forceinline__ float4 stream_load(const float4* p) {
#if RLN_LOAD_POLICY == 0
    return *p;
#elif RLN_LOAD_POLICY == 1
    return __ldg(p);
#elif RLN_LOAD_POLICY == 2
    return __ldcs(p);
#else
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
#endif
}
__device__ __forceinline__ uint2 stream_load(const uint2* p) {
#if RLN_LOAD_POLICY == 0
    return *p;
#elif RLN_LOAD_POLICY == 1
    return __ldg(p);
#elif RLN_LOAD_POLICY == 2
    return __ldcs(p);
#else
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];"
                 : "=r"(v.x), "=r"(v.y)
                 : "l"(p));
    return v;
#endif
}
__device__ __forceinline__ void stream_store(float4* p, float4 v) {
#if RLN_STORE_POLICY == 0
    *p = v;
#elif RLN_STORE_POLICY == 1
    __stcs(p, v);
#else
    __stwt(p, v);
#endif
}
__device__ __forceinline__ void stream_store(uint2* p, uint2 v) {
#if RLN_STORE_POLICY == 0
    *p = v;
#elif RLN_STORE_POLICY == 1
    __stcs(p, v);
#else
    __stwt(p, v);
#endif
}

// kStream selects the streaming cache hints above.  Both kernels take the
// choice as a template parameter (kStreamHints) and ship with plain accesses:
// timed alone in short bursts the backward is ~4 % faster with the hints, but
// in a sustained forward+backward chain on random data (the board at its power
// cap, which is how the operator runs in training) plain accesses in both
// kernels are 2 % faster per step than hints in both, and mixed settings lie
// in between.
template <bool kAligned, bool kStream = true>
__device__ __forceinline__ float4 load_f4(const float* base, int64_t chunk) {
    if constexpr (kAligned) {
        if constexpr (kStream) {
            return stream_load(reinterpret_cast<const float4*>(base) + chunk);
        } else {
            return *(reinterpret_cast<const float4*>(base) + chunk);
        }
    } else {
        const float* p = base + chunk * 4;
        return make_float4(p[0], p[1], p[2], p[3]);
    }
}

template <bool kAligned, bool kStream = true>
__device__ __forceinline__ void store_f4(float* base, int64_t chunk, float4 v) {
    if constexpr (kAligned) {
        if constexpr (kStream) {
            stream_store(reinterpret_cast<float4*>(base) + chunk, v);
        } else {
            *(reinterpret_cast<float4*>(base) + chunk) = v;
        }
    } else {
        float* p = base + chunk * 4;
        p[0] = v.x;
        p[1] = v.y;
        p[2] = v.z;
        p[3] = v.w;
    }
}

// Small, reused vectors (weight, bias): default caching so they stay in L1.
__device__ __forceinline__ float4 load_param4(const float* base, int chunk) {
    // weight/bias come from the caching allocator or cudaMalloc: 16-byte
    // alignment is checked on the host, scalar fallback otherwise.
    return __ldg(reinterpret_cast<const float4*>(base) + chunk);
}
__device__ __forceinline__ float4 load_param4_scalar(const float* base, int chunk) {
    const float* p = base + chunk * 4;
    return make_float4(__ldg(p), __ldg(p + 1), __ldg(p + 2), __ldg(p + 3));
}
template <bool kAligned>
__device__ __forceinline__ float4 load_param(const float* base, int chunk) {
    if constexpr (kAligned) {
        return load_param4(base, chunk);
    } else {
        return load_param4_scalar(base, chunk);
    }
}

// Branch-typed access: four consecutive elements of the branch tensor.
template <typename T>
struct BranchIO;

template <>
struct BranchIO<float> {
    template <bool kAligned, bool kStream = true>
    static __device__ __forceinline__ float4 load(const void* base, int64_t chunk) {
        return load_f4<kAligned, kStream>(static_cast<const float*>(base), chunk);
    }
    template <bool kAligned, bool kStream = true>
    static __device__ __forceinline__ void store(void* base, int64_t chunk, float4 v) {
        store_f4<kAligned, kStream>(static_cast<float*>(base), chunk, v);
    }
    static __device__ __forceinline__ float round(float v) { return v; }
    static __device__ __forceinline__ float4 round4(float4 v) { return v; }
};

template <>
struct BranchIO<__half> {
    template <bool kAligned, bool kStream = true>
    static __device__ __forceinline__ float4 load(const void* base, int64_t chunk) {
        if constexpr (kAligned) {
            const uint2 raw = kStream ? stream_load(static_cast<const uint2*>(base) + chunk)
                                      : *(static_cast<const uint2*>(base) + chunk);
            const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
            const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
            return make_float4(lo.x, lo.y, hi.x, hi.y);
        } else {
            const __half* p = static_cast<const __half*>(base) + chunk * 4;
            return make_float4(
                __half2float(p[0]), __half2float(p[1]), __half2float(p[2]), __half2float(p[3]));
        }
    }
    template <bool kAligned, bool kStream = true>
    static __device__ __forceinline__ void store(void* base, int64_t chunk, float4 v) {
        if constexpr (kAligned) {
            const __half2 lo = __floats2half2_rn(v.x, v.y);
            const __half2 hi = __floats2half2_rn(v.z, v.w);
            uint2 raw;
            raw.x = *reinterpret_cast<const uint32_t*>(&lo);
            raw.y = *reinterpret_cast<const uint32_t*>(&hi);
            if constexpr (kStream) {
                stream_store(static_cast<uint2*>(base) + chunk, raw);
            } else {
                *(static_cast<uint2*>(base) + chunk) = raw;
            }
        } else {
            __half* p = static_cast<__half*>(base) + chunk * 4;
            p[0] = __float2half_rn(v.x);
            p[1] = __float2half_rn(v.y);
            p[2] = __float2half_rn(v.z);
            p[3] = __float2half_rn(v.w);
        }
    }
    static __device__ __forceinline__ float round(float v) {
        return __half2float(__float2half_rn(v));
    }
    // four values through float16 and back: two packed conversions down, two up
    static __device__ __forceinline__ float4 round4(float4 v) {
        const float2 lo = __half22float2(__floats2half2_rn(v.x, v.y));
        const float2 hi = __half22float2(__floats2half2_rn(v.z, v.w));
        return make_float4(lo.x, lo.y, hi.x, hi.y);
    }
};

// bfloat16 branch (what mixed-precision training on this hardware produces;
// the reference, written for a GPU without bf16, stops at fp16).  Same access
// pattern as fp16: four elements = one 64-bit word per lane.
template <>
struct BranchIO<__nv_bfloat16> {
    template <bool kAligned, bool kStream = true>
    static __device__ __forceinline__ float4 load(const void* base, int64_t chunk) {
        if constexpr (kAligned) {
            const uint2 raw = kStream ? stream_load(static_cast<const uint2*>(base) + chunk)
                                      : *(static_cast<const uint2*>(base) + chunk);
            // a bfloat16 is the upper half of the float32 with the same value
            return make_float4(
                __uint_as_float(raw.x << 16),
                __uint_as_float(raw.x & 0xffff0000u),
                __uint_as_float(raw.y << 16),
                __uint_as_float(raw.y & 0xffff0000u));
        } else {
            const __nv_bfloat16* p = static_cast<const __nv_bfloat16*>(base) + chunk * 4;
            return make_float4(
                __bfloat162float(p[0]), __bfloat162float(p[1]), __bfloat162float(p[2]),
                __bfloat162float(p[3]));
        }
    }
    template <bool kAligned, bool kStream = true>
    static __device__ __forceinline__ void store(void* base, int64_t chunk, float4 v) {
        if constexpr (kAligned) {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y);
            const __nv_bfloat162 hi = __floats2bfloat162_rn(v.z, v.w);
            uint2 raw;
            raw.x = *reinterpret_cast<const uint32_t*>(&lo);
            raw.y = *reinterpret_cast<const uint32_t*>(&hi);
            if constexpr (kStream) {
                stream_store(static_cast<uint2*>(base) + chunk, raw);
            } else {
                *(static_cast<uint2*>(base) + chunk) = raw;
            }
        } else {
            __nv_bfloat16* p = static_cast<__nv_bfloat16*>(base) + chunk * 4;
            p[0] = __float2bfloat16_rn(v.x);
            p[1] = __float2bfloat16_rn(v.y);
            p[2] = __float2bfloat16_rn(v.z);
            p[3] = __float2bfloat16_rn(v.w);
        }
    }
    static __device__ __forceinline__ float round(float v) {
        return __bfloat162float(__float2bfloat16_rn(v));
    }
    static __device__ __forceinline__ float4 round4(float4 v) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(v.z, v.w);
        const uint32_t a = *reinterpret_cast<const uint32_t*>(&lo);
        const uint32_t b = *reinterpret_cast<const uint32_t*>(&hi);
        return make_float4(
            __uint_as_float(a << 16), __uint_as_float(a & 0xffff0000u),
            __uint_as_float(b << 16), __uint_as_float(b & 0xffff0000u));
    }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int delta = 16; delta > 0; delta >>= 1) {
        v += __shfl_xor_sync(kFullMask, v, delta);
    }
    return v;
}

// ---------------------------------------------------------------------------
// Two optional forms of the arithmetic core, a template parameter of the
// kernels and a macro (the variant benchmark times the combinations; the launch
// tables in rln_launch.h say what ships).
//   kPacked     two-wide fp32 instructions (add/mul/fma .f32x2 of sm_100) on
//               the (x, y) and (z, w) halves of a chunk.  Every lane-local
//               operation keeps its rounding (round-to-nearest, no flush) and
//               the residual add stays scalar (see add_residual), so `updated`
//               and the affine output are the bits of the scalar form; only
//               the association of the per-lane partial sums differs.  Pays
//               where the forward runs at 32 warps per SM on a 64-register
//               budget (H = 384: +5 %); neutral or slower elsewhere.
//   RLN_FWD_MASK_REDUX (macro, 0)  the eight lanes of a mask word combine their
//               nibbles with one redux.sync.or over the lane group instead of
//               three shuffle + or steps.  Measured 25 % slower for the forward
//               (a redux over a partial member mask is far from one shuffle's
//               cost), so it stays off.
// ---------------------------------------------------------------------------
#ifndef RLN_FWD_MASK_REDUX
#define RLN_FWD_MASK_REDUX 0
#endif

__device__ __forceinline__ float2 lo2(float4 v) { return make_float2(v.x, v.y); }
__device__ __forceinline__ float2 hi2(float4 v) { return make_float2(v.z, v.w); }
__device__ __forceinline__ float4 join4(float2 lo, float2 hi) {
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ float2 splat2(float v) { return make_float2(v, v); }

// OR of `word` over the aligned group of eight lanes this lane belongs to.
__device__ __forceinline__ uint32_t or_over_eight_lanes(uint32_t word, int lane) {
#if RLN_FWD_MASK_REDUX
    return __reduce_or_sync(0xffu << (lane & 24), word);
#else
    word |= __shfl_xor_sync(kFullMask, word, 1);
    word |= __shfl_xor_sync(kFullMask, word, 2);
    word |= __shfl_xor_sync(kFullMask, word, 4);
    return word;
#endif
}

// keep ? scale : 0 for the four columns of a chunk, times v, one rounding each.
template <bool kPacked>
__device__ __forceinline__ float4 scale_kept(float4 v, uint32_t nibble, float scale) {
    if constexpr (kPacked) {
        return join4(
            __fmul2_rn(lo2(v), make_float2((nibble & 1u) ? scale : 0.0f,
                                           (nibble & 2u) ? scale : 0.0f)),
            __fmul2_rn(hi2(v), make_float2((nibble & 4u) ? scale : 0.0f,
                                           (nibble & 8u) ? scale : 0.0f)));
    } else {
        return make_float4(__fmul_rn(v.x, (nibble & 1u) ? scale : 0.0f),
                           __fmul_rn(v.y, (nibble & 2u) ? scale : 0.0f),
                           __fmul_rn(v.z, (nibble & 4u) ? scale : 0.0f),
                           __fmul_rn(v.w, (nibble & 8u) ? scale : 0.0f));
    }
}

// dropped = round_to_branch(float(b) * keep * scale) for the four columns of a
// chunk; `nibble` holds their keep bits.  One multiply by (keep ? scale : 0)
// gives the same bits as the two multiplies of the torch decomposition
// evaluated with this mask -- b * 1 * scale == b * scale and
// b * 0 * scale == b * 0 including the sign of zero, and a non-finite b times
// zero is NaN either way -- and the sum is never contracted into an fma.
template <typename BranchT, bool kPacked>
__device__ __forceinline__ float4 drop_four(float4 b, uint32_t nibble, float scale) {
    return BranchIO<BranchT>::round4(scale_kept<kPacked>(b, nibble, scale));
}

// Lane-local pieces of the row arithmetic, shared by the two forward kernels.
// u = x + dropped, never contracted into an fma with the dropout multiply:
// always the scalar __fadd_rn.  The two-wide add is NOT safe here -- with a
// float32 branch nothing stands between the two-wide multiply of the dropout
// and this add, and the compiler fuses the pair into a two-wide fma, which
// changes the last bit of `updated` (caught by the float32-branch parity test).
__device__ __forceinline__ float4 add_residual(float4 x, float4 dropped) {
    return make_float4(__fadd_rn(x.x, dropped.x), __fadd_rn(x.y, dropped.y),
                       __fadd_rn(x.z, dropped.z), __fadd_rn(x.w, dropped.w));
}

// A lane's running sum over its chunks (values, or squares of centred values).
template <bool kPacked>
struct LaneSum;

template <>
struct LaneSum<true> {
    float2 acc = {0.0f, 0.0f};
    __device__ __forceinline__ void add(float4 v) {
        acc = __fadd2_rn(acc, __fadd2_rn(lo2(v), hi2(v)));
    }
    __device__ __forceinline__ void add_centred_square(float4 v, float mean) {
        const float2 shift = splat2(-mean);
        const float2 a = __fadd2_rn(lo2(v), shift);
        const float2 b = __fadd2_rn(hi2(v), shift);
        acc = __ffma2_rn(a, a, acc);
        acc = __ffma2_rn(b, b, acc);
    }
    __device__ __forceinline__ float total() const { return acc.x + acc.y; }
};

template <>
struct LaneSum<false> {
    float acc = 0.0f;
    __device__ __forceinline__ void add(float4 v) { acc += (v.x + v.y) + (v.z + v.w); }
    __device__ __forceinline__ void add_centred_square(float4 v, float mean) {
        const float cx = v.x - mean;
        const float cy = v.y - mean;
        const float cz = v.z - mean;
        const float cw = v.w - mean;
        acc += (cx * cx + cy * cy) + (cz * cz + cw * cw);
    }
    __device__ __forceinline__ float total() const { return acc; }
};

// (u - mean) * rstd * gamma + beta for the four columns of a chunk.
template <bool kPacked>
__device__ __forceinline__ float4 normalize_affine(
    float4 u, float mean, float rstd, float4 gamma, float4 beta) {
    if constexpr (kPacked) {
        const float2 shift = splat2(-mean);
        const float2 scale = splat2(rstd);
        const float2 lo = __ffma2_rn(
            __fmul2_rn(__fadd2_rn(lo2(u), shift), scale), lo2(gamma), lo2(beta));
        const float2 hi = __ffma2_rn(
            __fmul2_rn(__fadd2_rn(hi2(u), shift), scale), hi2(gamma), hi2(beta));
        return join4(lo, hi);
    } else {
        float4 out;
        out.x = (u.x - mean) * rstd * gamma.x + beta.x;
        out.y = (u.y - mean) * rstd * gamma.y + beta.y;
        out.z = (u.z - mean) * rstd * gamma.z + beta.z;
        out.w = (u.w - mean) * rstd * gamma.w + beta.w;
        return out;
    }
}

// ---------------------------------------------------------------------------
// Forward.  grid-stride over groups of kRows consecutive rows per warp.
// ---------------------------------------------------------------------------
template <int H, typename BranchT, bool kDropout, bool kAligned, int kWarps, int kRows,
          int kMinCtas = 1, bool kDeviceRng = false, bool kStreamHints = false,
          typename NormT = float, bool kPacked = false>
__global__ void __launch_bounds__(kWarps * kWarpSize, kMinCtas)
rln_forward_kernel(const ForwardParams p) {
    static_assert(H % 128 == 0, "hidden must be a multiple of 128");
    constexpr int V = H / 128;          // float4 chunks per lane
    constexpr int kChunksPerRow = H / 4;
    constexpr int kWordsPerRow = H / 32;
    constexpr float kInvH = 1.0f / static_cast<float>(H);
    using IO = BranchIO<BranchT>;

    const int lane = threadIdx.x & (kWarpSize - 1);
    const int warp = threadIdx.x / kWarpSize;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kWarps * kRows;
    grid_dependency_sync();
    clear_side_buffer(p);
    // Device state (graph capture): two loads, four registers.  Immediate
    // state: the four words are used straight from the kernel parameters
    // (constant-bank operands), see the Philox call below.
    PhiloxState rng = {0u, 0u, 0u, 0u};
    if constexpr (kDropout && kDeviceRng) {
        rng = resolve_philox_state(p);
    }

    for (int64_t first = (static_cast<int64_t>(blockIdx.x) * kWarps + warp) * kRows;
         first < p.rows; first += stride) {
        float4 u[kRows][V];
        float4 b[kRows][V];
        uint32_t nibble[kRows][V];

        // 1. issue every load of this warp's rows
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const int64_t row = first + r;
            if (row < p.rows) {
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    const int64_t chunk = row * kChunksPerRow + lane + k * kWarpSize;
                    u[r][k] = load_f4<kAligned, kStreamHints>(p.x, chunk);
                    b[r][k] = IO::template load<kAligned, kStreamHints>(p.branch, chunk);
                }
            }
        }

        // 2. keep decisions (independent of the loads: overlaps their latency)
        if constexpr (kDropout) {
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                const int64_t row = first + r;
                if (row < p.rows) {
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        const uint64_t group =
                            static_cast<uint64_t>(p.row_base + row) * kChunksPerRow
                            + static_cast<uint64_t>(lane + k * kWarpSize);
                        const uint4 random = philox4x32_10(
                            make_uint4(
                                kDeviceRng ? rng.offset_lo : p.offset_lo,
                                kDeviceRng ? rng.offset_hi : p.offset_hi,
                                static_cast<uint32_t>(group),
                                static_cast<uint32_t>(group >> 32)),
                            kDeviceRng ? rng.seed_lo : p.seed_lo,
                            kDeviceRng ? rng.seed_hi : p.seed_hi);
                        nibble[r][k] =
                            (random.x >= p.threshold ? 1u : 0u)
                            | (random.y >= p.threshold ? 2u : 0u)
                            | (random.z >= p.threshold ? 4u : 0u)
                            | (random.w >= p.threshold ? 8u : 0u);
                    }
                }
            }
        }

        // 3. per row: residual add, statistics, affine, stores
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const int64_t row = first + r;
            if (row >= p.rows) {
                continue;  // warp-uniform
            }
            LaneSum<kPacked> sum;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                float4 dropped = b[r][k];
                if constexpr (kDropout) {
                    dropped = drop_four<BranchT, kPacked>(dropped, nibble[r][k], p.scale);
                }
                const float4 value = add_residual(u[r][k], dropped);
                u[r][k] = value;
                const int64_t chunk = row * kChunksPerRow + lane + k * kWarpSize;
                store_f4<kAligned, kStreamHints>(p.updated, chunk, value);
                sum.add(value);
            }
            const float row_mean = warp_sum(sum.total()) * kInvH;
            LaneSum<kPacked> square_sum;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                square_sum.add_centred_square(u[r][k], row_mean);
            }
            const float variance = warp_sum(square_sum.total()) * kInvH;
            const float row_rstd = rsqrtf(variance + p.eps);
            if (lane == 0) {
                p.mean[row] = row_mean;
                p.rstd[row] = row_rstd;
            }
#pragma unroll
            for (int k = 0; k < V; ++k) {
                const int pchunk = lane + k * kWarpSize;
                const float4 gamma = load_param<kAligned>(p.weight, pchunk);
                const float4 beta = load_param<kAligned>(p.bias, pchunk);
                const float4 out = normalize_affine<kPacked>(u[r][k], row_mean, row_rstd, gamma, beta);
                // rounded once to NormT (identity for float32)
                BranchIO<NormT>::template store<kAligned, kStreamHints>(
                    p.normalized, row * kChunksPerRow + pchunk, out);
            }
            if constexpr (kDropout) {
                // chunk c = lane + 32k covers columns 4c..4c+3 -> nibble
                // (lane & 7) of mask word 4k + lane/8.
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    const uint32_t word =
                        or_over_eight_lanes(nibble[r][k] << (4 * (lane & 7)), lane);
                    if ((lane & 7) == 0) {
                        p.mask[row * kWordsPerRow + 4 * k + (lane >> 3)] = word;
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Forward for narrow rows.  A group of kLanes (8 or 16) lanes owns one row, so
// a warp works on 32/kLanes rows at once: the shuffle butterflies shrink to
// log2(kLanes) steps and every shuffle, compare and store instruction serves
// several rows.  Same arithmetic per element, same lane-group mask packing
// (8 lanes -> one word), so results are bit-identical to the one-warp-per-row
// kernel.  Row validity is per lane group here (not warp-uniform): loads and
// stores are predicated, shuffles are executed by the whole warp.
// ---------------------------------------------------------------------------
template <int H, typename BranchT, bool kDropout, bool kAligned, int kWarps, int kLanes,
          int kMinCtas = 1, bool kDeviceRng = false, bool kStreamHints = false,
          typename NormT = float, bool kPacked = false>
__global__ void __launch_bounds__(kWarps * kWarpSize, kMinCtas)
rln_forward_subwarp_kernel(const ForwardParams p) {
    static_assert(kLanes == 8 || kLanes == 16, "a row is owned by 8 or 16 lanes");
    static_assert(H % (4 * kLanes) == 0, "hidden must be a multiple of 4 * kLanes");
    constexpr int V = H / (4 * kLanes);  // float4 chunks per lane
    constexpr int kRowsPerWarp = kWarpSize / kLanes;
    constexpr int kChunksPerRow = H / 4;
    constexpr int kWordsPerRow = H / 32;
    constexpr float kInvH = 1.0f / static_cast<float>(H);
    using IO = BranchIO<BranchT>;

    const int lane = threadIdx.x & (kWarpSize - 1);
    const int warp = threadIdx.x / kWarpSize;
    const int lane_in_row = lane & (kLanes - 1);
    const int row_in_warp = lane / kLanes;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kWarps * kRowsPerWarp;
    grid_dependency_sync();
    clear_side_buffer(p);
    // Device state (graph capture): two loads, four registers.  Immediate
    // state: the four words are used straight from the kernel parameters
    // (constant-bank operands), see the Philox call below.
    PhiloxState rng = {0u, 0u, 0u, 0u};
    if constexpr (kDropout && kDeviceRng) {
        rng = resolve_philox_state(p);
    }

    for (int64_t first = (static_cast<int64_t>(blockIdx.x) * kWarps + warp) * kRowsPerWarp;
         first < p.rows; first += stride) {
        const int64_t row = first + row_in_warp;
        const bool valid = row < p.rows;
        float4 u[V];
        float4 b[V];
        uint32_t nibble[V];

#pragma unroll
        for (int k = 0; k < V; ++k) {
            u[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            b[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            nibble[k] = 0u;
            if (valid) {
                const int64_t chunk = row * kChunksPerRow + lane_in_row + k * kLanes;
                u[k] = load_f4<kAligned, kStreamHints>(p.x, chunk);
                b[k] = IO::template load<kAligned, kStreamHints>(p.branch, chunk);
            }
        }
        if constexpr (kDropout) {
#pragma unroll
            for (int k = 0; k < V; ++k) {
                const uint64_t group =
                    static_cast<uint64_t>(p.row_base + row) * kChunksPerRow
                    + static_cast<uint64_t>(lane_in_row + k * kLanes);
                const uint4 random = philox4x32_10(
                    make_uint4(
                        kDeviceRng ? rng.offset_lo : p.offset_lo,
                        kDeviceRng ? rng.offset_hi : p.offset_hi,
                        static_cast<uint32_t>(group),
                        static_cast<uint32_t>(group >> 32)),
                    kDeviceRng ? rng.seed_lo : p.seed_lo,
                    kDeviceRng ? rng.seed_hi : p.seed_hi);
                nibble[k] =
                    (random.x >= p.threshold ? 1u : 0u)
                    | (random.y >= p.threshold ? 2u : 0u)
                    | (random.z >= p.threshold ? 4u : 0u)
                    | (random.w >= p.threshold ? 8u : 0u);
            }
        }

        LaneSum<kPacked> lane_sum;
#pragma unroll
        for (int k = 0; k < V; ++k) {
            float4 dropped = b[k];
            if constexpr (kDropout) {
                dropped = drop_four<BranchT, kPacked>(dropped, nibble[k], p.scale);
            }
            const float4 value = add_residual(u[k], dropped);
            u[k] = value;
            if (valid) {
                store_f4<kAligned, kStreamHints>(
                    p.updated, row * kChunksPerRow + lane_in_row + k * kLanes, value);
            }
            lane_sum.add(value);
        }
        float sum = lane_sum.total();
#pragma unroll
        for (int delta = kLanes / 2; delta > 0; delta >>= 1) {
            sum += __shfl_xor_sync(kFullMask, sum, delta);
        }
        const float row_mean = sum * kInvH;
        LaneSum<kPacked> lane_squares;
#pragma unroll
        for (int k = 0; k < V; ++k) {
            lane_squares.add_centred_square(u[k], row_mean);
        }
        float square_sum = lane_squares.total();
#pragma unroll
        for (int delta = kLanes / 2; delta > 0; delta >>= 1) {
            square_sum += __shfl_xor_sync(kFullMask, square_sum, delta);
        }
        const float row_rstd = rsqrtf(square_sum * kInvH + p.eps);
        if (valid && lane_in_row == 0) {
            p.mean[row] = row_mean;
            p.rstd[row] = row_rstd;
        }
#pragma unroll
        for (int k = 0; k < V; ++k) {
            const int pchunk = lane_in_row + k * kLanes;
            const float4 gamma = load_param<kAligned>(p.weight, pchunk);
            const float4 beta = load_param<kAligned>(p.bias, pchunk);
            const float4 out = normalize_affine<kPacked>(u[k], row_mean, row_rstd, gamma, beta);
            if (valid) {
                BranchIO<NormT>::template store<kAligned, kStreamHints>(
                    p.normalized, row * kChunksPerRow + pchunk, out);
            }
        }
        if constexpr (kDropout) {
            // chunk c = lane_in_row + kLanes*k -> nibble (c & 7) of word c / 8
#pragma unroll
            for (int k = 0; k < V; ++k) {
                const uint32_t word = or_over_eight_lanes(nibble[k] << (4 * (lane & 7)), lane);
                if (valid && (lane & 7) == 0) {
                    p.mask[row * kWordsPerRow + (lane_in_row + k * kLanes) / 8] = word;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Backward.  Persistent grid.  Two ways of handing rows to warps:
//   static   (kDynamicRows == false) each warp walks groups of kRows
//            consecutive rows with a fixed stride, so the set and order of
//            rows a warp (and a CTA) sums is a pure function of (rows,
//            gridDim) -- the basis of the bitwise-replay mode;
//   dynamic  (kDynamicRows == true; instantiated by the variant benchmark only)
//            rows below p.dynamic_begin are split statically as above, the
//            groups from there on are claimed from a global counter, the claim
//            issued right after the loads of the current group so that its
//            latency hides behind them.  Measured on B200: claiming every row
//            costs one atomic per row on a single address (1-2 ns each), which
//            caps the grid below the row rate the static kernel reaches (8 %
//            slower at H = 768, 50 % at H = 384); claiming only the last one to
//            six rounds gains up to 4 % for the backward of 32,768 x 1,024 and
//            87,381 x 768 and loses 1-7 % at H = 128, 384 and 512, so the
//            library ships the static split only.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void red_add_f4(float* address, float4 v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                 :
                 : "l"(address), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}

// A lane's partial sums of q = g * gamma and of q * xhat over its chunks.
template <bool kPacked>
struct BackwardLaneSums;

template <>
struct BackwardLaneSums<true> {
    float2 q = {0.0f, 0.0f};
    float2 qx = {0.0f, 0.0f};
    __device__ __forceinline__ float total_q() const { return q.x + q.y; }
    __device__ __forceinline__ float total_qx() const { return qx.x + qx.y; }
};

template <>
struct BackwardLaneSums<false> {
    float q = 0.0f;
    float qx = 0.0f;
    __device__ __forceinline__ float total_q() const { return q; }
    __device__ __forceinline__ float total_qx() const { return qx; }
};

// First pass over a chunk: xhat = (u - mean) * rstd, the parameter-gradient
// accumulators, q = g * gamma and the lane's partial sums of q and q * xhat.
// Returns xhat in `u` and q in `g`.
template <bool kParams, bool kPacked>
__device__ __forceinline__ void backward_first_pass(
    float4& u, float4& g, float4 gamma, float mean, float rstd,
    float4& acc_weight, float4& acc_bias, BackwardLaneSums<kPacked>& sums) {
    if constexpr (kPacked) {
        const float2 shift = splat2(-mean);
        const float2 scale = splat2(rstd);
        const float2 xhat_lo = __fmul2_rn(__fadd2_rn(lo2(u), shift), scale);
        const float2 xhat_hi = __fmul2_rn(__fadd2_rn(hi2(u), shift), scale);
        const float2 g_lo = lo2(g);
        const float2 g_hi = hi2(g);
        if constexpr (kParams) {
            acc_weight = join4(__ffma2_rn(g_lo, xhat_lo, lo2(acc_weight)),
                               __ffma2_rn(g_hi, xhat_hi, hi2(acc_weight)));
            acc_bias = join4(__fadd2_rn(lo2(acc_bias), g_lo), __fadd2_rn(hi2(acc_bias), g_hi));
        }
        const float2 q_lo = __fmul2_rn(g_lo, lo2(gamma));
        const float2 q_hi = __fmul2_rn(g_hi, hi2(gamma));
        sums.q = __fadd2_rn(sums.q, __fadd2_rn(q_lo, q_hi));
        sums.qx = __ffma2_rn(q_lo, xhat_lo, sums.qx);
        sums.qx = __ffma2_rn(q_hi, xhat_hi, sums.qx);
        g = join4(q_lo, q_hi);
        u = join4(xhat_lo, xhat_hi);
    } else {
        float4 xhat;
        xhat.x = (u.x - mean) * rstd;
        xhat.y = (u.y - mean) * rstd;
        xhat.z = (u.z - mean) * rstd;
        xhat.w = (u.w - mean) * rstd;
        if constexpr (kParams) {
            acc_weight.x += g.x * xhat.x;
            acc_weight.y += g.y * xhat.y;
            acc_weight.z += g.z * xhat.z;
            acc_weight.w += g.w * xhat.w;
            acc_bias.x += g.x;
            acc_bias.y += g.y;
            acc_bias.z += g.z;
            acc_bias.w += g.w;
        }
        float4 q;
        q.x = g.x * gamma.x;
        q.y = g.y * gamma.y;
        q.z = g.z * gamma.z;
        q.w = g.w * gamma.w;
        sums.q += (q.x + q.y) + (q.z + q.w);
        sums.qx += (q.x * xhat.x + q.y * xhat.y) + (q.z * xhat.z + q.w * xhat.w);
        g = q;
        u = xhat;
    }
}

// Second pass: grad_x = grad_updated + rstd * (q - mean(q) - xhat * mean(q * xhat)).
template <bool kPacked>
__device__ __forceinline__ float4 backward_input_gradient(
    float4 grad_updated, float4 q, float4 xhat, float rstd, float mean_q, float mean_qx) {
    if constexpr (kPacked) {
        const float2 minus_mean_q = splat2(-mean_q);
        const float2 minus_mean_qx = splat2(-mean_qx);
        const float2 scale = splat2(rstd);
        const float2 lo = __ffma2_rn(
            __ffma2_rn(lo2(xhat), minus_mean_qx, __fadd2_rn(lo2(q), minus_mean_q)), scale,
            lo2(grad_updated));
        const float2 hi = __ffma2_rn(
            __ffma2_rn(hi2(xhat), minus_mean_qx, __fadd2_rn(hi2(q), minus_mean_q)), scale,
            hi2(grad_updated));
        return join4(lo, hi);
    } else {
        float4 total;
        total.x = grad_updated.x + rstd * (q.x - mean_q - xhat.x * mean_qx);
        total.y = grad_updated.y + rstd * (q.y - mean_q - xhat.y * mean_qx);
        total.z = grad_updated.z + rstd * (q.z - mean_q - xhat.z * mean_qx);
        total.w = grad_updated.w + rstd * (q.w - mean_q - xhat.w * mean_qx);
        return total;
    }
}

template <int H, typename BranchT, bool kDropout, bool kParams, bool kAligned, int kWarps, int kRows,
          int kMinCtas = 1, bool kStreamHints = false, typename NormT = float,
          bool kDynamicRows = false, bool kPacked = false>
__global__ void __launch_bounds__(kWarps * kWarpSize, kMinCtas)
rln_backward_kernel(const BackwardParams p) {
    static_assert(H % 128 == 0, "hidden must be a multiple of 128");
    constexpr int V = H / 128;
    constexpr int kChunksPerRow = H / 4;
    constexpr int kWordsPerRow = H / 32;
    constexpr float kInvH = 1.0f / static_cast<float>(H);
    using IO = BranchIO<BranchT>;

    const int lane = threadIdx.x & (kWarpSize - 1);
    const int warp = threadIdx.x / kWarpSize;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kWarps * kRows;

    grid_dependency_sync();

    float4 acc_weight[kParams ? V : 1];
    float4 acc_bias[kParams ? V : 1];
    if constexpr (kParams) {
#pragma unroll
        for (int k = 0; k < V; ++k) {
            acc_weight[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            acc_bias[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    }

    int64_t first = (static_cast<int64_t>(blockIdx.x) * kWarps + warp) * kRows;
    while (first < p.rows) {
        float4 gy[kRows][V];
        float4 uu[kRows][V];
        float4 gu[kRows][V];
        uint32_t words[kRows][V];
        float row_mean[kRows];
        float row_rstd[kRows];

#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const int64_t row = first + r;
            if (row < p.rows) {
                row_mean[r] = __ldg(p.mean + row);
                row_rstd[r] = __ldg(p.rstd + row);
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    const int64_t chunk = row * kChunksPerRow + lane + k * kWarpSize;
                    gy[r][k] = BranchIO<NormT>::template load<kAligned, kStreamHints>(
                        p.grad_normalized, chunk);
                    uu[r][k] = load_f4<kAligned, kStreamHints>(p.updated, chunk);
                    gu[r][k] = load_f4<kAligned, kStreamHints>(p.grad_updated, chunk);
                    if constexpr (kDropout) {
                        words[r][k] = __ldg(p.mask + row * kWordsPerRow + 4 * k + (lane >> 3));
                    }
                }
            }
        }
        // claim the next group now; the answer is needed after this group's stores
        unsigned int ticket = 0u;
        bool claimed = false;  // warp-uniform
        if constexpr (kDynamicRows) {
            claimed = first + stride >= p.dynamic_begin;
            if (claimed && lane == 0) {
                ticket = atomicAdd(p.row_counter, static_cast<unsigned int>(kRows));
            }
        }

#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const int64_t row = first + r;
            if (row >= p.rows) {
                continue;  // warp-uniform
            }
            const float mu = row_mean[r];
            const float rs = row_rstd[r];
            BackwardLaneSums<kPacked> sums;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                const float4 gamma = load_param<kAligned>(p.weight, lane + k * kWarpSize);
                // afterwards uu holds the normalised value, gy the weighted gradient
                backward_first_pass<kParams, kPacked>(
                    uu[r][k], gy[r][k], gamma, mu, rs,
                    acc_weight[kParams ? k : 0], acc_bias[kParams ? k : 0], sums);
            }
            float sum_q = sums.total_q();
            float sum_qx = sums.total_qx();
#pragma unroll
            for (int delta = 16; delta > 0; delta >>= 1) {
                sum_q += __shfl_xor_sync(kFullMask, sum_q, delta);
                sum_qx += __shfl_xor_sync(kFullMask, sum_qx, delta);
            }
            const float mean_q = sum_q * kInvH;
            const float mean_qx = sum_qx * kInvH;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                const int64_t chunk = row * kChunksPerRow + lane + k * kWarpSize;
                float4 total = backward_input_gradient<kPacked>(
                    gu[r][k], gy[r][k], uu[r][k], rs, mean_q, mean_qx);
                store_f4<kAligned, kStreamHints>(p.grad_x, chunk, total);
                if constexpr (kDropout) {
                    const uint32_t n = words[r][k] >> (4 * (lane & 7));
                    // g * keep * scale as one multiply (same bits, see drop_four)
                    total = scale_kept<kPacked>(total, n, p.scale);
                }
                IO::template store<kAligned, kStreamHints>(p.grad_branch, chunk, total);
            }
        }
        if (kDynamicRows && claimed) {
            first = p.dynamic_begin + static_cast<int64_t>(__shfl_sync(kFullMask, ticket, 0));
        } else {
            first += stride;
        }
    }

    if constexpr (kParams) {
        // Combine the warps of this CTA in warp order (fixed order => the CTA
        // partial is reproducible), then hand the [2, H] partial on.
        __shared__ float4 combined[2 * kChunksPerRow];
#pragma unroll 1
        for (int turn = 0; turn < kWarps; ++turn) {
            if (warp == turn) {
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    const int c = lane + k * kWarpSize;
                    if (turn == 0) {
                        combined[c] = acc_weight[k];
                        combined[kChunksPerRow + c] = acc_bias[k];
                    } else {
                        float4 w = combined[c];
                        float4 bsum = combined[kChunksPerRow + c];
                        w.x += acc_weight[k].x;
                        w.y += acc_weight[k].y;
                        w.z += acc_weight[k].z;
                        w.w += acc_weight[k].w;
                        bsum.x += acc_bias[k].x;
                        bsum.y += acc_bias[k].y;
                        bsum.z += acc_bias[k].z;
                        bsum.w += acc_bias[k].w;
                        combined[c] = w;
                        combined[kChunksPerRow + c] = bsum;
                    }
                }
            }
            __syncthreads();
        }
        if (p.deterministic) {
            float4* out = reinterpret_cast<float4*>(p.partials)
                + static_cast<int64_t>(blockIdx.x) * (2 * kChunksPerRow);
            for (int c = threadIdx.x; c < 2 * kChunksPerRow; c += kWarps * kWarpSize) {
                out[c] = combined[c];
            }
        } else {
            for (int c = threadIdx.x; c < 2 * kChunksPerRow; c += kWarps * kWarpSize) {
                const float4 v = combined[c];
                if constexpr (kAligned) {
                    red_add_f4(p.grad_parameters + 4 * c, v);
                } else {
                    atomicAdd(p.grad_parameters + 4 * c + 0, v.x);
                    atomicAdd(p.grad_parameters + 4 * c + 1, v.y);
                    atomicAdd(p.grad_parameters + 4 * c + 2, v.z);
                    atomicAdd(p.grad_parameters + 4 * c + 3, v.w);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Deterministic stage 2: out[c] = sum over CTA partials in a fixed order.
// 32 columns x kSegments contiguous partial ranges per CTA; each range is
// summed serially in index order, the ranges are combined in range order.
// The partials were written a moment ago and sit in L2, so the kernel is bound
// by load latency, not bandwidth: many short ranges (one warp each) and four
// loads in flight per thread -- issued together, added in index order, so the
// sum is the serial one -- keep the chains short (888 partials at H = 128:
// 28 per range, 7 batches).
// ---------------------------------------------------------------------------
template <int kSegments>
__global__ void __launch_bounds__(kSegments * kWarpSize)
rln_reduce_partials_kernel(
    const float* __restrict__ partials,
    float* __restrict__ out,
    int partial_count,
    int columns) {
    __shared__ float staged[kSegments][kWarpSize];
    const int lane = threadIdx.x & (kWarpSize - 1);
    const int segment = threadIdx.x / kWarpSize;
    const int column = blockIdx.x * kWarpSize + lane;
    grid_dependency_sync();
    const int per_segment = (partial_count + kSegments - 1) / kSegments;
    const int begin = segment * per_segment;
    const int end = min(partial_count, begin + per_segment);
    float sum = 0.0f;
    if (column < columns) {
        const float* cursor = partials + static_cast<int64_t>(begin) * columns + column;
        int index = begin;
        for (; index + 4 <= end; index += 4) {
            const float a = cursor[0];
            const float b = cursor[columns];
            const float c = cursor[2 * static_cast<int64_t>(columns)];
            const float d = cursor[3 * static_cast<int64_t>(columns)];
            sum += a;
            sum += b;
            sum += c;
            sum += d;
            cursor += 4 * static_cast<int64_t>(columns);
        }
        for (; index < end; ++index) {
            sum += cursor[0];
            cursor += columns;
        }
    }
    staged[segment][lane] = sum;
    __syncthreads();
    if (segment == 0 && column < columns) {
        float total = staged[0][lane];
#pragma unroll
        for (int s = 1; s < kSegments; ++s) {
            total += staged[s][lane];
        }
        out[column] = total;
    }
}

}  // namespace rln
