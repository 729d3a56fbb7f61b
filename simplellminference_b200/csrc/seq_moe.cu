// csrc/seq_moe.cu — mixture-of-experts feed-forward of the ragged token batch: routing and the experts' activation as one kernel.
// The router's logits, the experts' up projections of every token (all experts side by side, one wide product) and the layer's input
// arrive; per token the kernel takes the softmax over all router outputs (fp32), adds a per-expert correction to the scores for the
// CHOICE only, picks the `top` largest, and writes act(up) * score for the chosen real experts (zeros for the others) as the operand of
// ONE down product over the concatenated experts. The last `identity` router outputs are experts without weights whose output is the
// input itself: their scores are summed and the kernel leaves (sum * input) in the output rows, to which the down product is added.
#include "seq_common.cuh"

namespace sllm {

__device__ __forceinline__ float moe_act(float z, int kind) {
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
        const float inv = 1.0f / sum;
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
    for (int i = threadIdx.x; i < experts * ff; i += blockDim.x) {
        const float w = s_w[i / ff];
        const float v = w != 0.0f ? moe_act(ur[i], act) * w : 0.0f;
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
    SLLM_REQUIRE(act >= 0 && act <= 2, SLLM_EINVAL, "seq_moe_act: activation 0 (gelu), 1 (tanh gelu) or 2 (silu)");
    SLLM_REQUIRE(n_route <= 4096, SLLM_ENOTSUP, "seq_moe_act: %d router outputs beyond 4096", n_route);
    const int work = std::max(experts * ff, d);
    const int threads = T >= 64 ? 256 : std::min(1024, std::max(128, (work + 31) / 32 * 32));
    seq_moe_act_kernel<<<T, threads, 3 * (size_t)n_route * sizeof(float), as_stream(stream)>>>(logits, ldl, n_route, experts, top, correction, up, ldu, ff, act, h, ldh,
                                                                                                d, out, (uint16_t*)out16, y, ldy, route_w);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}
