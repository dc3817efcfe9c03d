/*
 * Scalar C restatement of the residual-add + dropout + LayerNorm arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY: built into oracle/_build/librln_oracle.so and
 * loaded by tests; never linked into, imported by or called from the shipped
 * package.
 *
 * It follows the reference project's HIP kernels (T-vaccari/gfx1010-kernels,
 * csrc/residual_layer_norm_kernel.hip) element by element, one row at a time:
 *   forward          :483-545  dropped = round_branch(b * keep * scale); u = x + dropped;
 *                              mean; centred variance; rstd = 1/sqrt(var + eps);
 *                              y = (u - mean) * rstd * gamma + beta; ballot mask :500-511
 *   backward-input   :572-617  xhat, q = g_y * gamma, g = g_u + rstd * (q - mean(q) - xhat * mean(q xhat)),
 *                              grad_branch = round_branch(g * keep * scale)
 *   parameter sums   :741-760  grad_weight = sum_rows g_y * xhat, grad_bias = sum_rows g_y
 *   threshold, scale :896-899
 * Row reductions are accumulated in double (the kernels use fp32 trees whose
 * order is an implementation detail); everything an output depends on
 * bit-for-bit (the dropped branch, `updated`, the mask) is done in the
 * kernels' exact fp32/fp16 arithmetic.
 *
 * The dropout bits come from Philox4x32-10 (Salmon et al., SC'11) with the
 * counter layout of the sm_100a kernel: group g = ((row_base + row) * H + col) / 4,
 * block b = offset / 4 (the offset counts 32-bit words, a call yields four),
 * counter (lo32(b), hi32(b), lo32(g), hi32(g)), key (lo32(seed), hi32(seed)),
 * word j -> column 4g + j, keep <=> word >= threshold.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

static void philox4x32_10(uint32_t counter[4], uint32_t key0, uint32_t key1) {
    for (int round = 0; round < 10; ++round) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * counter[0];
        const uint64_t p1 = (uint64_t)0xCD9E8D57u * counter[2];
        const uint32_t c0 = (uint32_t)(p1 >> 32) ^ counter[1] ^ key0;
        const uint32_t c1 = (uint32_t)p1;
        const uint32_t c2 = (uint32_t)(p0 >> 32) ^ counter[3] ^ key1;
        const uint32_t c3 = (uint32_t)p0;
        counter[0] = c0; counter[1] = c1; counter[2] = c2; counter[3] = c3;
        key0 += 0x9E3779B9u;
        key1 += 0xBB67AE85u;
    }
}

void rln_oracle_philox(const uint32_t counter_in[4], const uint32_t key[2], uint32_t out[4]) {
    for (int i = 0; i < 4; ++i) out[i] = counter_in[i];
    philox4x32_10(out, key[0], key[1]);
}

static float round_half(float v) { return (float)(_Float16)v; }

/* float32 -> bfloat16 -> float32, round to nearest even (NaN kept quiet). */
static float round_bfloat16(float v) {
    union { float f; uint32_t u; } bits;
    bits.f = v;
    if ((bits.u & 0x7fffffffu) > 0x7f800000u) {
        bits.u |= 0x00400000u;
    } else {
        bits.u += 0x7fffu + ((bits.u >> 16) & 1u);
    }
    bits.u &= 0xffff0000u;
    return bits.f;
}

/* branch_kind: 0 float32 (no rounding), 1 float16, 2 bfloat16. */
static float round_branch(float v, int32_t branch_kind) {
    if (branch_kind == 1) return round_half(v);
    if (branch_kind == 2) return round_bfloat16(v);
    return v;
}

/* In place: values[i] = widen(round_to_kind(values[i])).  Used for a
 * `normalized` output stored as float16 / bfloat16 (an addition of the sm_100a
 * build; the reference stores float32): rounded once, to nearest even. */
void rln_oracle_round(float* values, int64_t count, int32_t kind) {
    for (int64_t i = 0; i < count; ++i) values[i] = round_branch(values[i], kind);
}

/* keep[rows * hidden] (0/1 bytes) and mask words [rows * hidden / 32]. */
void rln_oracle_keep_mask(
    int64_t rows, int32_t hidden, float dropout_p, uint64_t seed, uint64_t offset,
    int64_t row_base, uint8_t* keep, uint32_t* mask_words) {
    const uint32_t threshold = (uint32_t)((double)dropout_p * 4294967296.0);
    for (int64_t i = 0; i < rows * (hidden / 32); ++i) mask_words[i] = 0;
    for (int64_t row = 0; row < rows; ++row) {
        for (int32_t col = 0; col < hidden; col += 4) {
            const uint64_t group = ((uint64_t)(row_base + row) * (uint64_t)hidden + (uint64_t)col) / 4;
            const uint64_t block = offset >> 2;
            uint32_t counter[4] = {(uint32_t)block, (uint32_t)(block >> 32),
                                   (uint32_t)group, (uint32_t)(group >> 32)};
            philox4x32_10(counter, (uint32_t)seed, (uint32_t)(seed >> 32));
            for (int j = 0; j < 4; ++j) {
                const int kept = counter[j] >= threshold;
                keep[row * hidden + col + j] = (uint8_t)kept;
                if (kept) {
                    mask_words[row * (hidden / 32) + (col + j) / 32] |= 1u << ((col + j) & 31);
                }
            }
        }
    }
}

/* branch is float32 values already widened; branch_kind selects the rounding. */
void rln_oracle_forward(
    const float* x, const float* branch, const float* weight, const float* bias,
    const uint8_t* keep /* NULL = dropout inactive */, float dropout_p, float eps,
    int32_t branch_kind, int64_t rows, int32_t hidden,
    float* updated, float* normalized, float* mean, float* rstd) {
    const float scale = keep ? 1.0f / (1.0f - dropout_p) : 1.0f;
    for (int64_t row = 0; row < rows; ++row) {
        const int64_t base = row * hidden;
        double sum = 0.0;
        for (int32_t c = 0; c < hidden; ++c) {
            float b = branch[base + c];
            if (keep) {
                volatile float kept = b * (float)keep[base + c];   /* two un-fused products */
                b = kept * scale;
                b = round_branch(b, branch_kind);
            }
            volatile float u = x[base + c] + b;
            updated[base + c] = u;
            sum += u;
        }
        const float row_mean = (float)(sum / hidden);
        double square = 0.0;
        for (int32_t c = 0; c < hidden; ++c) {
            const double centred = (double)updated[base + c] - row_mean;
            square += centred * centred;
        }
        const float row_rstd = (float)(1.0 / sqrt(square / hidden + (double)eps));
        mean[row] = row_mean;
        rstd[row] = row_rstd;
        for (int32_t c = 0; c < hidden; ++c) {
            normalized[base + c] =
                (updated[base + c] - row_mean) * row_rstd * weight[c] + bias[c];
        }
    }
}

void rln_oracle_backward(
    const float* grad_updated, const float* grad_normalized, const float* updated,
    const float* weight, const float* mean, const float* rstd,
    const uint8_t* keep /* NULL = dropout inactive */, float dropout_p,
    int32_t branch_kind, int64_t rows, int32_t hidden,
    float* grad_x, float* grad_branch /* widened to float32 */,
    float* grad_weight, float* grad_bias) {
    const float scale = keep ? 1.0f / (1.0f - dropout_p) : 1.0f;
    double* sum_weight = (double*)calloc((size_t)hidden, sizeof(double));
    double* sum_bias = (double*)calloc((size_t)hidden, sizeof(double));
    for (int64_t row = 0; row < rows; ++row) {
        const int64_t base = row * hidden;
        const float mu = mean[row];
        const float rs = rstd[row];
        double sum_q = 0.0, sum_qx = 0.0;
        for (int32_t c = 0; c < hidden; ++c) {
            const float xhat = (updated[base + c] - mu) * rs;
            const float q = grad_normalized[base + c] * weight[c];
            sum_q += q;
            sum_qx += (double)q * xhat;
            sum_weight[c] += (double)grad_normalized[base + c] * xhat;
            sum_bias[c] += grad_normalized[base + c];
        }
        const float mean_q = (float)(sum_q / hidden);
        const float mean_qx = (float)(sum_qx / hidden);
        for (int32_t c = 0; c < hidden; ++c) {
            const float xhat = (updated[base + c] - mu) * rs;
            const float q = grad_normalized[base + c] * weight[c];
            const float total = grad_updated[base + c] + rs * (q - mean_q - xhat * mean_qx);
            grad_x[base + c] = total;
            float b = total;
            if (keep) {
                volatile float kept = total * (float)keep[base + c];
                b = kept * scale;
            }
            grad_branch[base + c] = round_branch(b, branch_kind);
        }
    }
    for (int32_t c = 0; c < hidden; ++c) {
        grad_weight[c] = (float)sum_weight[c];
        grad_bias[c] = (float)sum_bias[c];
    }
    free(sum_weight);
    free(sum_bias);
}
