// csrc/seq_sublayer.cu — the seam between two sublayers of a model whose sublayers are wrapped in scalar RMS norms and read their input
// through a short causal convolution: x <- x + g_post * y / rms(y) (the residual sum, fp32), then h = n + conv(n) with
// n = g_pre * x / rms(x) and conv a per-channel causal convolution over time, as ONE kernel. A norm here has one number as its weight.
// The same seam serves pre-norm layers: the sum may take y as it is (no norm on the sublayer's output), and the norm in front of the
// next sublayer may carry a weight per channel stored as its distance from a constant, n = g_pre * (offset + w[c]) * x / rms(x).
//
// The convolution reaches taps-1 tokens back. Inside a portion those are rows of this step: a CTA (one per token) recomputes the
// residual sum and the norm of its predecessors from the sublayer's input and output (x is therefore read from one buffer and written to
// another). Before the portion they come from the sequence's state: a ring of taps-1 normed rows per slot, position p at row
// p % (taps-1). A ring may not be written while other CTAs of the launch still read it, so the normed rows of a portion's last tokens
// go to a per-token stash, and the NEXT seam launch moves them into the ring (`flush_*`); the model's last seam (the final norm, no
// convolution) flushes the last ring.
#include "seq_common.cuh"

namespace sllm {

struct SeamArgs {
    sllm_seq_batch b;
    const float* x_in; float* x_out;          // residual stream before / after the sum (x_out unused when y is NULL)
    const float* y; float post_g;             // sublayer output and its norm's weight; NULL = no sum
    int has_pre; float pre_g, eps;            // 0 = only the sum
    const float* conv_w; int taps;            // [d][taps], last column = the current token; NULL = no convolution
    const float* ring;                        // [slots][taps-1][d]
    float* h; uint16_t* h16;                  // what the next sublayer reads, fp32 and (optionally) as bf16 operand rows
    float* stash;                             // [T][d]: normed rows of tokens that a later launch moves into `ring`
    float* flush_ring; int flush_taps;        // the ring that takes the stash the previous seam left
    int d;
    int post_norm;                            // 0 = y is added as it is
    const float* pre_w; float pre_off;        // [d] or NULL: channel c of the normed row is also multiplied by pre_off + pre_w[c]
};

__device__ __forceinline__ float seam_gain(const SeamArgs& p, int j) { return p.pre_w ? p.pre_off + p.pre_w[j] : 1.0f; }

// is token t among the last `keep` tokens of its portion?
__device__ __forceinline__ bool seam_is_last(const sllm_seq_batch& b, int t, int slot, int keep) {
    return keep > 0 && (t + keep >= b.T || b.tok_slot[t + keep] != slot);
}

__global__ void seq_seam_kernel(SeamArgs p) {
    extern __shared__ __align__(16) float seam_sm[];   // [d] the row at hand, [d] the convolution's sums
    __shared__ float red[33];
    float* s_row = seam_sm;
    float* s_acc = seam_sm + p.d;
    const sllm_seq_batch& b = p.b;
    const int t = blockIdx.x, d = p.d, slot = b.tok_slot[t], pos = b.tok_pos[t];
    // the stash of the previous seam goes into that seam's ring before this launch overwrites the stash row
    if (p.flush_ring && seam_is_last(b, t, slot, p.flush_taps - 1)) {
        float* dst = p.flush_ring + ((size_t)slot * (p.flush_taps - 1) + pos % (p.flush_taps - 1)) * d;
        for (int j = threadIdx.x; j < d; j += blockDim.x) dst[j] = p.stash[(size_t)t * d + j];
    }
    const int reach = (p.has_pre && p.conv_w) ? p.taps - 1 : 0;
    bool started = false;                                // does s_acc hold a sum yet? (the same answer in every thread)
    for (int back = reach; back >= 0; --back) {          // the current token last: its normed row stays in s_row
        if (pos - back < 0) continue;                    // before the sequence's start: zeros
        const bool here = back == 0 || (t - back >= 0 && b.tok_slot[t - back] == slot);
        if (!here) {
            const float* src = p.ring + ((size_t)slot * (p.taps - 1) + (pos - back) % (p.taps - 1)) * d;
            for (int j = threadIdx.x; j < d; j += blockDim.x) {
                s_acc[j] = fmaf(p.conv_w[(size_t)j * p.taps + p.taps - 1 - back], src[j], started ? s_acc[j] : 0.0f);
            }
            started = true;
            continue;
        }
        const size_t r = (size_t)(t - back) * d;
        float inv_y = 1.0f;
        if (p.y && p.post_norm) {
            float ss = 0.0f;
            for (int j = threadIdx.x; j < d; j += blockDim.x) ss = fmaf(p.y[r + j], p.y[r + j], ss);
            inv_y = p.post_g / sqrtf(block_sum(ss, red) / (float)d + p.eps);
        }
        float ss = 0.0f;
        for (int j = threadIdx.x; j < d; j += blockDim.x) {
            float v = p.x_in[r + j];
            if (p.y) {
                v = fmaf(p.y[r + j], inv_y, v);
                if (back == 0) p.x_out[r + j] = v;
            }
            s_row[j] = v;
            ss = fmaf(v, v, ss);
        }
        if (!p.has_pre) return;
        const float inv = p.pre_g / sqrtf(block_sum(ss, red) / (float)d + p.eps);
        if (!p.conv_w) {
            for (int j = threadIdx.x; j < d; j += blockDim.x) {
                const float v = s_row[j] * inv * seam_gain(p, j);
                p.h[r + j] = v;
                if (p.h16) p.h16[r + j] = f32_to_bf16_bits(v);
            }
            return;
        }
        const bool keep = back == 0 && seam_is_last(b, t, slot, p.taps - 1);
        for (int j = threadIdx.x; j < d; j += blockDim.x) {
            const float n = s_row[j] * inv * seam_gain(p, j);
            float acc = fmaf(p.conv_w[(size_t)j * p.taps + p.taps - 1 - back], n, started ? s_acc[j] : 0.0f);
            if (back == 0) {
                acc += n;
                p.h[r + j] = acc;
                if (p.h16) p.h16[r + j] = f32_to_bf16_bits(acc);
                if (keep) p.stash[r + j] = n;
            } else {
                s_acc[j] = acc;
            }
        }
        started = true;
    }
}

// ---- the same seam as two launches, for steps of many tokens: no row is normed more than once ------------------------------------------
// (1) one CTA per token: the residual sum and the scale of the next norm, scale[t] = g_pre / rms(x_new[t]);
// (2) element-wise over (token, channel): h = n + conv(n) with n = scale * x_new read from the step's rows (complete after launch 1) or
//     the ring, the stash and the flush as in the one-launch form.
__global__ void seq_seam_sum_kernel(SeamArgs p, float* __restrict__ scale) {
    extern __shared__ __align__(16) float seam_sm[];   // [d] the sublayer's output row
    __shared__ float red[33];
    const int t = blockIdx.x, d = p.d;
    const size_t r = (size_t)t * d;
    float ss = 0.0f;
    if (p.y) {
        float sy = 0.0f;
        for (int j = threadIdx.x; j < d; j += blockDim.x) {
            const float v = p.y[r + j];
            seam_sm[j] = v;
            sy = fmaf(v, v, sy);
        }
        const float inv_y = p.post_norm ? p.post_g / sqrtf(block_sum(sy, red) / (float)d + p.eps) : 1.0f;
        for (int j = threadIdx.x; j < d; j += blockDim.x) {
            const float v = fmaf(seam_sm[j], inv_y, p.x_in[r + j]);
            p.x_out[r + j] = v;
            ss = fmaf(v, v, ss);
        }
    } else {
        for (int j = threadIdx.x; j < d; j += blockDim.x) ss = fmaf(p.x_in[r + j], p.x_in[r + j], ss);
    }
    ss = block_sum(ss, red);
    if (threadIdx.x == 0) scale[t] = p.pre_g / sqrtf(ss / (float)d + p.eps);
}

constexpr int kSeamMaxTaps = 64;

// The rows a token's convolution reads are found once per CTA (the step's own rows with their scales, or ring rows), then the channels
// are walked four at a time with 16-byte loads where the row length allows.
__global__ void seq_seam_conv_kernel(SeamArgs p, const float* __restrict__ scale, int vec) {
    __shared__ const float* s_src[kSeamMaxTaps];   // [back] row that lies `back` positions before the token, NULL = before the sequence's start
    __shared__ float s_mul[kSeamMaxTaps];
    __shared__ bool back_is_step[kSeamMaxTaps];    // the row is one of this step's (not yet normed) rather than a ring row
    const sllm_seq_batch& b = p.b;
    const int t = blockIdx.x, d = p.d, slot = b.tok_slot[t], pos = b.tok_pos[t], taps = p.taps;
    const float* x = p.y ? p.x_out : p.x_in;             // the stream after the sum
    const bool flush = p.flush_ring && seam_is_last(b, t, slot, p.flush_taps - 1);
    const bool keep = seam_is_last(b, t, slot, taps - 1);
    float* fdst = flush ? p.flush_ring + ((size_t)slot * (p.flush_taps - 1) + pos % (p.flush_taps - 1)) * d : nullptr;
    const size_t r = (size_t)t * d;
    if ((int)threadIdx.x < taps) {
        const int back = threadIdx.x;
        const float* src = nullptr;
        float mul = 1.0f;
        bool in_step = false;
        if (pos - back >= 0) {
            if (back == 0 || (t - back >= 0 && b.tok_slot[t - back] == slot)) {
                src = x + r - (size_t)back * d;
                mul = scale[t - back];
                in_step = true;
            } else {
                src = p.ring + ((size_t)slot * (taps - 1) + (pos - back) % (taps - 1)) * d;
            }
        }
        s_src[back] = src;
        s_mul[back] = mul;
        back_is_step[back] = in_step;
    }
    __syncthreads();
    const float own = s_mul[0];
    if (vec) {
        for (int j = (blockIdx.y * blockDim.x + threadIdx.x) * 4; j < d; j += gridDim.y * blockDim.x * 4) {
            if (flush) *reinterpret_cast<float4*>(fdst + j) = *reinterpret_cast<const float4*>(p.stash + r + j);
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const float gn[4] = {seam_gain(p, j), seam_gain(p, j + 1), seam_gain(p, j + 2), seam_gain(p, j + 3)};
            for (int back = taps - 1; back >= 1; --back) {
                const float* src = s_src[back];
                if (!src) continue;
                const float4 v = *reinterpret_cast<const float4*>(src + j);
                const float m = s_mul[back];
                // a ring row is normed and weighted already (its multiplier is 1); a row of this step gets the channel's weight here
                const bool raw = back_is_step[back];
                const float n4[4] = {v.x * m * (raw ? gn[0] : 1.0f), v.y * m * (raw ? gn[1] : 1.0f), v.z * m * (raw ? gn[2] : 1.0f), v.w * m * (raw ? gn[3] : 1.0f)};
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[e] = fmaf(p.conv_w[(size_t)(j + e) * taps + taps - 1 - back], n4[e], acc[e]);
            }
            const float4 v = *reinterpret_cast<const float4*>(x + r + j);
            const float n4[4] = {v.x * own * gn[0], v.y * own * gn[1], v.z * own * gn[2], v.w * own * gn[3]};
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] = fmaf(p.conv_w[(size_t)(j + e) * taps + taps - 1], n4[e], acc[e]) + n4[e];
            *reinterpret_cast<float4*>(p.h + r + j) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            if (p.h16) {
                const uint2 packed = make_uint2((uint32_t)f32_to_bf16_bits(acc[0]) | ((uint32_t)f32_to_bf16_bits(acc[1]) << 16),
                                                (uint32_t)f32_to_bf16_bits(acc[2]) | ((uint32_t)f32_to_bf16_bits(acc[3]) << 16));
                *reinterpret_cast<uint2*>(p.h16 + r + j) = packed;
            }
            if (keep) *reinterpret_cast<float4*>(p.stash + r + j) = make_float4(n4[0], n4[1], n4[2], n4[3]);
        }
        return;
    }
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < d; j += gridDim.y * blockDim.x) {
        if (flush) fdst[j] = p.stash[r + j];
        float acc = 0.0f;
        const float gn = seam_gain(p, j);
        for (int back = taps - 1; back >= 1; --back) {
            const float* src = s_src[back];
            if (src) acc = fmaf(p.conv_w[(size_t)j * taps + taps - 1 - back], src[j] * s_mul[back] * (back_is_step[back] ? gn : 1.0f), acc);
        }
        const float n = x[r + j] * own * gn;
        acc = fmaf(p.conv_w[(size_t)j * taps + taps - 1], n, acc) + n;
        p.h[r + j] = acc;
        if (p.h16) p.h16[r + j] = f32_to_bf16_bits(acc);
        if (keep) p.stash[r + j] = n;
    }
}

}  // namespace sllm

using namespace sllm;

extern "C" int sllm_seq_seam(const sllm_seq_batch* b, const float* x_in, float* x_out, const float* y, float post_g, int32_t has_pre, float pre_g,
                             float eps, const float* conv_w, int32_t taps, const float* ring, float* h, void* h16, float* stash, float* flush_ring,
                             int32_t flush_taps, int32_t d, float* scales, int32_t post_norm, const float* pre_w, float pre_w_offset, sllm_stream_t stream) {
    SLLM_REQUIRE(b && b->T > 0 && b->tok_slot && b->tok_pos, SLLM_EINVAL, "seq_seam: incomplete batch description");
    SLLM_REQUIRE(x_in && d > 0 && (!y || (x_out && x_out != x_in)), SLLM_EINVAL, "seq_seam: the residual sum needs a second buffer for x");
    SLLM_REQUIRE(!has_pre || h, SLLM_EINVAL, "seq_seam: no output for the normed rows");
    SLLM_REQUIRE(!conv_w || (taps >= 1 && taps <= kSeamMaxTaps && (taps == 1 || (ring && stash))), SLLM_EINVAL, "seq_seam: a convolution (1..%d taps) needs its ring and a stash", kSeamMaxTaps);
    SLLM_REQUIRE(!flush_ring || (flush_taps >= 2 && stash), SLLM_EINVAL, "seq_seam: nothing to flush from");
    if (conv_w && taps == 1) ring = nullptr;
    const size_t smem = 2 * (size_t)d * sizeof(float);
    SLLM_REQUIRE(smem <= (size_t)smem_optin_bytes() - 1024, SLLM_ENOTSUP, "seq_seam: rows of %d floats do not fit shared memory", d);
    if (smem > 48 * 1024) SLLM_CUDA(cudaFuncSetAttribute(seq_seam_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    SeamArgs p{*b, x_in, x_out, y, post_g, has_pre, pre_g, eps, conv_w, taps, ring, h, (uint16_t*)h16, stash, flush_ring, flush_taps, d, post_norm, pre_w, pre_w_offset};
    const int threads = b->T >= 64 ? (d >= 2048 ? 256 : 128) : std::min(1024, std::max(128, (d + 31) / 32 * 32));
    if (scales && has_pre && conv_w && b->T >= 64 && b->T <= 65535) {       // many tokens: two launches, every row normed once
        seq_seam_sum_kernel<<<b->T, threads, smem / 2, as_stream(stream)>>>(p, scales);
        auto aligned = [](const void* q) { return q == nullptr || ((uintptr_t)q % 16) == 0; };
        const int vec = d % 4 == 0 && aligned(x_in) && aligned(x_out) && aligned(ring) && aligned(h) && aligned(stash) && aligned(flush_ring) &&
                        (h16 == nullptr || ((uintptr_t)h16 % 8) == 0);
        seq_seam_conv_kernel<<<dim3(b->T, std::max(1, std::min(4, d / 4096))), 256, 0, as_stream(stream)>>>(p, scales, vec);
        g_launches += 2;
        SLLM_LAUNCH_CHECK();
        return SLLM_OK;
    }
    seq_seam_kernel<<<b->T, threads, smem, as_stream(stream)>>>(p);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}
