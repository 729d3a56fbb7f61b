// csrc/seq_moe.cu — mixture-of-experts feed-forward of the ragged token batch: routing and the experts' activation as one kernel.
// The router's logits, the experts' up projections of every token (all experts side by side, one wide product) and the layer's input
// arrive; per token the kernel takes the softmax over all router outputs (fp32), adds a per-expert correction to the scores for the
// CHOICE only, picks the `top` largest, and writes act(up) * score for the chosen real experts (zeros for the others) as the operand of
// ONE down product over the concatenated experts. The last `identity` router outputs are experts without weights whose output is the
// input itself: their scores are summed and the kernel leaves (sum * input) in the output rows, to which the down product is added.
// Variants, chosen by bits of the `mode` argument beside the activation: scores that are the sigmoid of each router output by itself
// (SLLM_MOE_SIGMOID) instead of a softmax over all; gated experts (SLLM_MOE_GATED: an expert's `up` columns are [gate ff | up ff] and
// it computes act(gate) * up); a score that multiplies what the expert reads instead of what it returns (SLLM_MOE_SCALE_INPUT: the
// products are linear, so gate and up are multiplied after the product in the dense form, the gathered rows before it).
#include "seq_common.cuh"

namespace sllm {

constexpr int kMoeGated = 4, kMoeScaleInput = 8, kMoeSigmoid = 16;   // SLLM_MOE_* of the header

__device__ __forceinline__ float moe_act(float z, int kind) {
    kind &= 3;
    if (kind == 0) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752f));   // exact gelu
    if (kind == 1) return seq_gelu_tanh(z);
    return z * seq_sigmoid(z);                                                   // silu
}

// one CTA per token; shared: scores [n_route], weights [n_route]
__global__ void seq_moe_act_kernel(const float* __restrict__ logits, int ldl, int n_route, int experts, int top, const float* __restrict__ correction,
                                   const float* __restrict__ up, int ldu, int ff, int act, const float* __restrict__ h, int ldh, int d,
                                   float* __restrict__ out, uint16_t* __restrict__ out16, float* __restrict__ y, int ldy, float* __restrict__ route_w) {
    extern __shared__ float msm[];
    float* s_score = msm;
    float* s_choice = msm + n_route;
    float* s_w = msm + 2 * n_route;
    __shared__ float s_identity;
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    const float* z = logits + (size_t)t * ldl;
    if (threadIdx.x < 32) {
        float inv = 1.0f;
        if (act & kMoeSigmoid) {
            for (int e = lane; e < n_route; e += 32) s_score[e] = seq_sigmoid(z[e]);
        } else {
            float mx = -INFINITY;
            for (int e = lane; e < n_route; e += 32) mx = fmaxf(mx, z[e]);
            mx = warp_max(mx);
            float sum = 0.0f;
            for (int e = lane; e < n_route; e += 32) {
                const float v = expf(z[e] - mx);
                s_score[e] = v;
                sum += v;
            }
            sum = warp_sum(sum);
            inv = 1.0f / sum;
        }
        for (int e = lane; e < n_route; e += 32) {
            const float s = s_score[e] * inv;
            s_score[e] = s;
            s_choice[e] = s + (correction ? correction[e] : 0.0f);
            s_w[e] = 0.0f;
        }
        __syncwarp();
        float ident = 0.0f;
        for (int k = 0; k < top; ++k) {                 // the largest remaining choice score; the lower index wins a tie
            float best = -INFINITY;
            int arg = n_route;
            for (int e = lane; e < n_route; e += 32) {
                const float c = s_choice[e];
                if (c > best) { best = c; arg = e; }
            }
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
                if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
            }
            if (arg < n_route && lane == 0) {
                s_choice[arg] = -INFINITY;
                s_w[arg] = s_score[arg];
                if (arg >= experts) ident += s_score[arg];
            }
            __syncwarp();
        }
        if (lane == 0) s_identity = ident;
    }
    __syncthreads();
    if (route_w)
        for (int e = threadIdx.x; e < n_route; e += blockDim.x) route_w[(size_t)t * n_route + e] = s_w[e];
    const float* ur = up + (size_t)t * ldu;
    const size_t orow = (size_t)t * experts * ff;
    const bool gated = act & kMoeGated, on_input = act & kMoeScaleInput;
    for (int i = threadIdx.x; i < experts * ff; i += blockDim.x) {
        const int e = i / ff;
        const float w = s_w[e];
        float v = 0.0f;
        if (w != 0.0f) {
            const float pre = on_input ? w : 1.0f, post = on_input ? 1.0f : w;
            if (gated) v = moe_act(ur[(size_t)e * 2 * ff + i % ff] * pre, act) * (ur[(size_t)e * 2 * ff + ff + i % ff] * pre) * post;
            else v = moe_act(ur[i] * pre, act) * post;
        }
        if (out) out[orow + i] = v;
        if (out16) out16[orow + i] = f32_to_bf16_bits(v);
    }
    const float ident = s_identity;
    for (int j = threadIdx.x; j < d; j += blockDim.x) y[(size_t)t * ldy + j] = ident * h[(size_t)t * ldh + j];
}

}  // namespace sllm

using namespace sllm;

extern "C" int sllm_seq_moe_act(const float* logits, int32_t ldl, int32_t n_route, int32_t experts, int32_t top, const float* correction, const float* up,
                                int32_t ldu, int32_t ff, int32_t act, const float* h, int32_t ldh, int32_t d, float* out, void* out16, float* y, int32_t ldy,
                                float* route_w, int32_t T, sllm_stream_t stream) {
    SLLM_REQUIRE(logits && up && h && y && (out || out16) && T > 0 && ff > 0 && d > 0, SLLM_EINVAL, "seq_moe_act: bad argument");
    SLLM_REQUIRE(experts >= 0 && n_route >= experts && n_route > 0 && top >= 1 && top <= n_route, SLLM_EINVAL, "seq_moe_act: %d of %d router outputs, %d experts with weights",
                 top, n_route, experts);
    SLLM_REQUIRE(act >= 0 && (act & 3) <= 2 && act < 32, SLLM_EINVAL, "seq_moe_act: activation 0 (gelu), 1 (tanh gelu) or 2 (silu), plus SLLM_MOE_* bits");
    SLLM_REQUIRE(n_route <= 4096, SLLM_ENOTSUP, "seq_moe_act: %d router outputs beyond 4096", n_route);
    const int work = std::max(experts * ff, d);
    const int threads = T >= 64 ? 256 : std::min(1024, std::max(128, (work + 31) / 32 * 32));
    seq_moe_act_kernel<<<T, threads, 3 * (size_t)n_route * sizeof(float), as_stream(stream)>>>(logits, ldl, n_route, experts, top, correction, up, ldu, ff, act, h, ldh,
                                                                                                d, out, (uint16_t*)out16, y, ldy, route_w);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

// ---- the same layer with the tokens gathered per expert (steps of many tokens) ------------------------------------------------------------
// Every expert gets a buffer of `cap` rows. The routing kernel gives each (token, chosen expert) pair a row of that expert's buffer
// (an atomic counter per expert: the ORDER of rows in a buffer is whatever the hardware makes it, the numbers in a row do not depend on
// it) and copies the token's input there; the up and down products then run per expert over the rows that are in use (the count stays on
// the device: sllm_seq_linear's rows_dev); the combine kernel adds each token's rows, times their scores, to (identity scores) * input.
namespace sllm {

__global__ void seq_moe_route_kernel(int act, const float* __restrict__ logits, int ldl, int n_route, int experts, int top, const float* __restrict__ correction,
                                     const float* __restrict__ h, int ldh, int d, int32_t* __restrict__ counts, int cap, int32_t* __restrict__ sel_e,
                                     int32_t* __restrict__ sel_pos, float* __restrict__ sel_w, float* __restrict__ ident_out, uint16_t* __restrict__ rows16,
                                     float* __restrict__ rows32) {
    extern __shared__ float msm[];
    float* s_score = msm;
    float* s_choice = msm + n_route;
    int* s_e = reinterpret_cast<int*>(msm + 2 * n_route);   // [top] expert of the k-th choice, -1 = an expert without weights
    int* s_pos = s_e + top;                                 // [top] its row in that expert's buffer
    float* s_in = reinterpret_cast<float*>(s_pos + top);    // [top] what the gathered row is multiplied by
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    const float* z = logits + (size_t)t * ldl;
    if (threadIdx.x < 32) {
        float inv = 1.0f;
        if (act & kMoeSigmoid) {
            for (int e = lane; e < n_route; e += 32) s_score[e] = seq_sigmoid(z[e]);
        } else {
            float mx = -INFINITY;
            for (int e = lane; e < n_route; e += 32) mx = fmaxf(mx, z[e]);
            mx = warp_max(mx);
            float sum = 0.0f;
            for (int e = lane; e < n_route; e += 32) {
                const float v = expf(z[e] - mx);
                s_score[e] = v;
                sum += v;
            }
            sum = warp_sum(sum);
            inv = 1.0f / sum;
        }
        for (int e = lane; e < n_route; e += 32) {
            const float s = s_score[e] * inv;
            s_score[e] = s;
            s_choice[e] = s + (correction ? correction[e] : 0.0f);
        }
        __syncwarp();
        float ident = 0.0f;
        for (int k = 0; k < top; ++k) {
            float best = -INFINITY;
            int arg = n_route;
            for (int e = lane; e < n_route; e += 32) {
                const float c = s_choice[e];
                if (c > best) { best = c; arg = e; }
            }
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
                if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
            }
            if (lane == 0) {
                int e_out = -1, pos = 0;
                float w = 0.0f;
                if (arg < n_route) {
                    s_choice[arg] = -INFINITY;
                    w = s_score[arg];
                    if (arg >= experts) ident += w;
                    else {
                        e_out = arg;
                        // without counters nothing is gathered: the pair keeps its own number, (token, choice) in order
                        pos = counts ? atomicAdd(counts + arg, 1) : t * top + k;
                        if (counts && pos >= cap) e_out = -1;      // cannot happen with cap >= the step's tokens; never write outside the buffer
                    }
                }
                s_e[k] = e_out;
                s_pos[k] = pos;
                sel_e[(size_t)t * top + k] = e_out;
                sel_pos[(size_t)t * top + k] = pos;
                // a score that multiplies the expert's input is applied to the gathered row; the combine kernel then adds the rows as they are
                sel_w[(size_t)t * top + k] = e_out >= 0 ? ((act & kMoeScaleInput) ? 1.0f : w) : 0.0f;
                s_in[k] = (act & kMoeScaleInput) ? w : 1.0f;
            }
            __syncwarp();
        }
        if (lane == 0) ident_out[t] = ident;
    }
    __syncthreads();
    if (!rows16 && !rows32) return;
    const float* hr = h + (size_t)t * ldh;
    for (int k = 0; k < top; ++k) {
        const int e = s_e[k];
        if (e < 0) continue;
        const size_t row = ((size_t)e * cap + s_pos[k]) * d;
        const float mul = s_in[k];
        for (int j = threadIdx.x; j < d; j += blockDim.x) {
            if (rows16) rows16[row + j] = f32_to_bf16_bits(hr[j] * mul);
            if (rows32) rows32[row + j] = hr[j] * mul;
        }
    }
}

// x <- act(x) over n floats
__global__ void seq_act_kernel(float* __restrict__ x, size_t n, int act) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] = moe_act(x[i], act);
}

// grid (cap, experts): rows in use only
__global__ void seq_moe_expert_act_kernel(const float* __restrict__ up, const int32_t* __restrict__ counts, int cap, int ff, int act,
                                          uint16_t* __restrict__ out16, float* __restrict__ out32) {
    const int e = blockIdx.y, r = blockIdx.x;
    if (r >= counts[e]) return;
    const size_t row = ((size_t)e * cap + r) * ff;
    const bool gated = act & kMoeGated;                  // rows of `up` then hold [gate ff | up ff]
    for (int j = threadIdx.x; j < ff; j += blockDim.x) {
        const float v = gated ? moe_act(up[2 * row + j], act) * up[2 * row + ff + j] : moe_act(up[row + j], act);
        if (out16) out16[row + j] = f32_to_bf16_bits(v);
        if (out32) out32[row + j] = v;
    }
}

// one CTA per (token, choice) pair, rows in the pairs' own order: out = act(s * up) or act(s * gate) * (s * up), with s the pair's score when
// the score multiplies what the expert reads (the products are linear: the score is applied to their results) and 1 otherwise;
// w_out takes what the combine kernel has to multiply the pair's down row by: 1 in the first case, the score in the second
__global__ void seq_moe_pair_act_kernel(const float* __restrict__ up, const float* __restrict__ sel_w, int ff, int act, float* __restrict__ out,
                                        float* __restrict__ w_out) {
    const int p = blockIdx.x;
    const bool gated = act & kMoeGated, on_input = act & kMoeScaleInput;
    const float score = sel_w[p], s = on_input ? score : 1.0f;
    const float* row = up + (size_t)p * ff * (gated ? 2 : 1);
    for (int j = threadIdx.x; j < ff; j += blockDim.x)
        out[(size_t)p * ff + j] = gated ? moe_act(s * row[j], act) * (s * row[ff + j]) : moe_act(s * row[j], act);
    if (threadIdx.x == 0) w_out[p] = on_input ? 1.0f : score;
}

__global__ void seq_moe_combine_kernel(const float* __restrict__ down, const int32_t* __restrict__ sel_e, const int32_t* __restrict__ sel_pos,
                                       const float* __restrict__ sel_w, int top, const float* __restrict__ ident, const float* __restrict__ h, int ldh,
                                       int cap, int d, float* __restrict__ y, int ldy) {
    extern __shared__ float csm[];                           // [top] score (0 = no row), [top] row offset
    float* s_w = csm;
    long long* s_row = reinterpret_cast<long long*>(csm + ((top + 1) & ~1));
    const int t = blockIdx.x;
    for (int k = threadIdx.x; k < top; k += blockDim.x) {
        const int e = sel_e[(size_t)t * top + k];
        s_w[k] = e >= 0 ? sel_w[(size_t)t * top + k] : 0.0f;
        s_row[k] = e >= 0 ? ((long long)e * cap + sel_pos[(size_t)t * top + k]) * d : -1;
    }
    __syncthreads();
    const float idw = ident[t];
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        float acc = idw * h[(size_t)t * ldh + j];
        for (int k = 0; k < top; ++k)                        // in the order of the choice: a fixed order of the sum
            if (s_row[k] >= 0) acc = fmaf(s_w[k], down[s_row[k] + j], acc);
        y[(size_t)t * ldy + j] = acc;
    }
}

}  // namespace sllm

extern "C" {

int sllm_seq_act(float* x, int64_t n, int32_t act, sllm_stream_t stream) {
    SLLM_REQUIRE(x && n > 0 && act >= 0 && act <= 2, SLLM_EINVAL, "seq_act: bad argument");
    seq_act_kernel<<<(int)std::min<size_t>(((size_t)n + 255) / 256, (size_t)sm_count() * 8), 256, 0, as_stream(stream)>>>(x, (size_t)n, act);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_zero(void* p, int64_t n_bytes, sllm_stream_t stream) {
    SLLM_REQUIRE(p && n_bytes > 0, SLLM_EINVAL, "seq_zero: bad argument");
    SLLM_CUDA(cudaMemsetAsync(p, 0, (size_t)n_bytes, as_stream(stream)));
    return SLLM_OK;
}

int sllm_seq_moe_route(const float* logits, int32_t ldl, int32_t n_route, int32_t experts, int32_t top, const float* correction, const float* h, int32_t ldh,
                       int32_t d, int32_t* counts, int32_t cap, int32_t* sel_e, int32_t* sel_pos, float* sel_w, float* ident, void* rows16, float* rows32,
                       int32_t T, int32_t mode, sllm_stream_t stream) {
    SLLM_REQUIRE(logits && h && sel_e && sel_pos && sel_w && ident && T > 0 && d > 0, SLLM_EINVAL, "seq_moe_route: bad argument");
    SLLM_REQUIRE((counts != nullptr) == (rows16 || rows32), SLLM_EINVAL, "seq_moe_route: counters and row buffers come together");
    SLLM_REQUIRE(experts >= 0 && n_route >= experts && n_route > 0 && top >= 1 && top <= n_route && cap >= T, SLLM_EINVAL,
                 "seq_moe_route: %d of %d router outputs, %d experts with weights, buffers of %d rows for %d tokens", top, n_route, experts, cap, T);
    SLLM_REQUIRE(n_route <= 4096 && top <= 1024, SLLM_ENOTSUP, "seq_moe_route: %d router outputs / top %d beyond what one CTA routes", n_route, top);
    const size_t smem = (2 * (size_t)n_route + 3 * (size_t)top) * sizeof(float);
    seq_moe_route_kernel<<<T, 256, smem, as_stream(stream)>>>(mode, logits, ldl, n_route, experts, top, correction, h, ldh, d, counts, cap, sel_e, sel_pos, sel_w, ident,
                                                               (uint16_t*)rows16, rows32);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_moe_expert_act(const float* up, const int32_t* counts, int32_t experts, int32_t cap, int32_t ff, int32_t act, void* out16, float* out32,
                            sllm_stream_t stream) {
    SLLM_REQUIRE(up && counts && (out16 || out32) && experts > 0 && cap > 0 && cap <= 65535 * 32 && ff > 0 && act >= 0 && (act & 3) <= 2, SLLM_EINVAL, "seq_moe_expert_act: bad argument");
    SLLM_REQUIRE(experts <= 65535, SLLM_ENOTSUP, "seq_moe_expert_act: %d experts", experts);
    seq_moe_expert_act_kernel<<<dim3(cap, experts), 256, 0, as_stream(stream)>>>(up, counts, cap, ff, act, (uint16_t*)out16, out32);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_moe_pair_act(const float* up, const float* sel_w, int32_t pairs, int32_t ff, int32_t act, float* out, float* w_out, sllm_stream_t stream) {
    SLLM_REQUIRE(up && sel_w && out && w_out && pairs > 0 && ff > 0 && act >= 0 && (act & 3) <= 2 && act < 32, SLLM_EINVAL, "seq_moe_pair_act: bad argument");
    seq_moe_pair_act_kernel<<<pairs, 256, 0, as_stream(stream)>>>(up, sel_w, ff, act, out, w_out);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_moe_combine(const float* down, const int32_t* sel_e, const int32_t* sel_pos, const float* sel_w, int32_t top, const float* ident, const float* h,
                         int32_t ldh, int32_t cap, int32_t d, float* y, int32_t ldy, int32_t T, sllm_stream_t stream) {
    SLLM_REQUIRE(down && sel_e && sel_pos && sel_w && ident && h && y && top >= 1 && T > 0 && d > 0, SLLM_EINVAL, "seq_moe_combine: bad argument");
    SLLM_REQUIRE(top <= 2048, SLLM_ENOTSUP, "seq_moe_combine: top %d beyond 2048", top);
    const int threads = T >= 64 ? 256 : std::min(1024, std::max(128, (d + 31) / 32 * 32));
    const size_t smem = (size_t)((top + 1) & ~1) * sizeof(float) + (size_t)top * sizeof(long long);
    seq_moe_combine_kernel<<<T, threads, smem, as_stream(stream)>>>(down, sel_e, sel_pos, sel_w, top, ident, h, ldh, cap, d, y, ldy);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

}  // extern "C"
