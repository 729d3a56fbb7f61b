// csrc/seq_delta.cu — the gated delta rule over the ragged token batch, and the short causal convolution (with an activation) in front
// of it. Per head the state S [dk][dv] (fp32, one per sequence slot) follows
//     S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q     (o of the NEW state; computed as (g S_old)^T q + u (k . q))
// with q and k made unit vectors per head (q also times dk^-1/2), beta = sigmoid(b), g = exp(-exp(A_log) * softplus(a + dt_bias)).
// Everything that enters the recurrence is fp32. The columns of S are independent recurrences that share k, q, beta and g: a CTA takes
// up to 32 columns of one head, a thread owns a piece (32 key channels) of one column in registers; the pieces of a column sit in
// adjacent lanes and meet by shuffles. More CTAs per head means more of the machine per sequence: the token loop itself is serial.
//
// The same kernel, instantiated without the correction term, runs the state-space-duality recurrence (Mamba-2): per head
//     S <- g S + dt B x^T;  y = S^T C + D x,   dt = softplus(a + dt_bias), g = exp(-exp(A_log) dt)
// with B in the place of k, C in the place of q (neither made a unit vector), x in the place of v, and the heads of a group sharing B and C.
//
// The convolution keeps its last taps-1 inputs per sequence in a ring (position p at row p % (taps-1)); the recurrence kernel, which
// runs after the convolution has read the ring, stores the portion's last inputs there.
#include <cstdlib>

#include "seq_common.cuh"

namespace sllm {

// thread = (token, channel): out = act(cb[c] + sum_j w[c][j] * x[t - taps + 1 + j][c]); act 0 = none, 1 = silu
__global__ void seq_conv_ring_kernel(sllm_seq_batch b, const float* __restrict__ x, int ldx, int channels, int taps, const float* __restrict__ w,
                                     const float* __restrict__ cb, const float* __restrict__ ring, int act, float* __restrict__ out, int ldo) {
    const int t = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int slot = b.tok_slot[t], pos = b.tok_pos[t];
    float acc = fmaf(w[(size_t)c * taps + taps - 1], x[(size_t)t * ldx + c], cb ? cb[c] : 0.0f);
    for (int back = 1; back < taps; ++back) {
        if (pos - back < 0) break;
        const float xv = (t - back >= 0 && b.tok_slot[t - back] == slot) ? x[(size_t)(t - back) * ldx + c]
                                                                          : ring[((size_t)slot * (taps - 1) + (pos - back) % (taps - 1)) * channels + c];
        acc = fmaf(w[(size_t)c * taps + taps - 1 - back], xv, acc);
    }
    if (act == 1) acc = acc * seq_sigmoid(acc);
    out[(size_t)t * ldo + c] = acc;
}

struct DeltaArgs {
    sllm_seq_batch b;
    const float *q, *k, *v; int ldq, ldk, ldv;          // after convolution and activation; q / k [kv_heads][dk], v [heads][dv] per token
    const float *bl, *al; int ldb, lda;                 // logits of beta and of the decay's step, [heads] per token
    const float *A_log, *dt_bias;                       // [heads]
    int heads, kv_heads, dk, dv;
    float unit_eps, qscale;
    float* state;                                       // [slots][heads][dk][dv]
    float* o; int ldo;                                  // [T][heads * dv]
    const float* conv_x; int ldx, channels, taps; float* ring;   // inputs of the convolution, stored to the ring for the next step (NULL = not)
    int chunk, PP, CB, vec;
    const float* skip;                                  // state-space form: [heads] weight of the input added to the output (NULL = none)
    float* ws; int nrange;                              // state-space form in three passes: per range and head [dk][dv] states, then the sums of dt
};

// The state-space recurrence is linear in the state and its decay over a run of tokens is exp(-rate * (sum of the run's dt)): steps that
// hold a long portion run it as three passes over ranges of kSsdRange tokens — every range from a zero state (end state Q, sum of dt), the
// ranges of a portion in order per state element (start of range r+1 = exp(-rate sum_r) start_r + Q_r; the last is the sequence's new
// state), every range again from its start state with the outputs. Ranges are numbered in segment order; segment s starts at
// seg_tile0[s] / 4 + s (a range is four query tiles of 32 tokens, so that number never runs into the next segment's).
constexpr int kSsdRange = 128;
__device__ __forceinline__ size_t ssd_range_id(const sllm_seq_batch& b, int seg, int rg) { return (size_t)(b.seg_tile0[seg] / 4 + seg + rg); }
__host__ __device__ __forceinline__ size_t ssd_range_count(int n_qtiles, int nseg) { return (size_t)(n_qtiles / 4 + nseg + 1); }

// key channels of a thread: 16 for key heads of up to 512 channels (measured best of 8 / 16 / 32 at 128-wide heads), 32 for wider ones.
// A piece's stride in shared memory is 4 floats more: 16-byte loads, pieces of the same index in different banks.
constexpr int kDeltaCB = 32;      // value columns of a CTA, at most

__device__ __forceinline__ uint32_t delta_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// global -> shared without passing through registers; `take` false writes zeros and reads nothing
__device__ __forceinline__ void delta_cp16(void* dst, const void* src, bool take) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(delta_smem(dst)), "l"(src), "r"(take ? 16 : 0) : "memory");
}
__device__ __forceinline__ void delta_cp4(void* dst, const void* src, bool take) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(delta_smem(dst)), "l"(src), "r"(take ? 4 : 0) : "memory");
}

// CTA = (segment, head, block of CB value columns); thread = (value column j, piece `part` of the key channels), part = tid % PP
// kForm 0: the delta rule. 1: the state-space form (no correction by the old state, no unit vectors, the step size multiplies the input)
// over whole portions; 2 / 3: its first and third pass over ranges (2: from zero, no outputs; 3: from the range's start state, no state store)
template <int kDeltaKP, int kMaxThreads, int kForm>
__global__ void __launch_bounds__(kMaxThreads) seq_delta_kernel(DeltaArgs p) {
    constexpr int kDeltaRS = kDeltaKP + 4;
    constexpr bool kSsd = kForm != 0, kRanges = kForm >= 2;
    extern __shared__ __align__(16) float dsm[];
    const sllm_seq_batch& b = p.b;
    const int seg = kRanges ? blockIdx.x / p.nrange : blockIdx.x, rg = kRanges ? blockIdx.x % p.nrange : 0;
    const int h = blockIdx.y, kvh = h / (p.heads / p.kv_heads);
    const int seg_len = b.seg_len[seg], r0 = rg * kSsdRange;
    if (kRanges && r0 >= seg_len) return;
    const int start = b.seg_start[seg] + r0, len = kRanges ? min(kSsdRange, seg_len - r0) : seg_len, slot = b.seg_slot[seg];
    const int dk = p.dk, dv = p.dv, PP = p.PP, C = p.chunk, RS = PP * kDeltaRS, CB = p.CB;
    const int part = threadIdx.x % PP, jl = threadIdx.x / PP, j = blockIdx.z * CB + jl;   // jl: the column inside the CTA's block
    const bool live = jl < CB && j < dv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    // two stages of inputs (the next chunk of tokens travels while this one is walked), then what both share
    const int CBp = (CB + 3) & ~3;                     // every array of a stage starts at a 16-byte boundary
    const int stage_floats = C * (2 * RS + CBp + 4);   // per token: k and q [RS] each, v [CB], the two logits
    float* s_o = dsm + 2 * stage_floats;               // [C][CB]
    float* s_beta = s_o + C * CB;                      // [C]
    float* s_g = s_beta + C;                           // [C]
    float* s_kq = s_g + C;                             // [C] k . q of the unit vectors
    const bool vec = p.vec;                            // 16-byte copies of q / k: dk a multiple of 4, rows 16-byte aligned
    auto issue = [&](int c0, int stage) {
        float* d_k = dsm + stage * stage_floats;
        float* d_q = d_k + C * RS;
        float* d_v = d_q + C * RS;
        float* d_l = d_v + C * CBp;                    // [C][2] logits of beta and of the step
        const int n = min(C, len - c0), groups = PP * kDeltaKP / 4;
        for (int i = threadIdx.x; i < n * groups; i += blockDim.x) {               // channels beyond dk are zeros
            const int tok = i / groups, kr = (i % groups) * 4;
            const size_t t = (size_t)(start + c0 + tok);
            const int at = tok * RS + (kr / kDeltaKP) * kDeltaRS + kr % kDeltaKP;
            const float* ks = p.k + t * p.ldk + (size_t)kvh * dk;
            const float* qs = p.q + t * p.ldq + (size_t)kvh * dk;
            if (vec) {
                delta_cp16(d_k + at, kr < dk ? ks + kr : ks, kr < dk);
                delta_cp16(d_q + at, kr < dk ? qs + kr : qs, kr < dk);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    delta_cp4(d_k + at + e, kr + e < dk ? ks + kr + e : ks, kr + e < dk);
                    delta_cp4(d_q + at + e, kr + e < dk ? qs + kr + e : qs, kr + e < dk);
                }
            }
        }
        for (int i = threadIdx.x; i < n * CB; i += blockDim.x) {
            const int col = blockIdx.z * CB + i % CB;
            const float* vs = p.v + (size_t)(start + c0 + i / CB) * p.ldv + (size_t)h * dv;
            delta_cp4(d_v + i, col < dv ? vs + col : vs, col < dv);
        }
        for (int i = threadIdx.x; i < 2 * n; i += blockDim.x) {
            const size_t t = (size_t)(start + c0 + (i >> 1));
            delta_cp4(d_l + i, (i & 1) ? p.al + t * p.lda + h : p.bl + t * p.ldb + h, true);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float* st = kRanges ? p.ws + (ssd_range_id(b, seg, rg) * p.heads + h) * dk * dv : p.state + ((size_t)slot * p.heads + h) * dk * dv;
    float S[kDeltaKP];
#pragma unroll
    for (int x = 0; x < kDeltaKP; ++x) {
        const int kr = part * kDeltaKP + x;
        S[x] = (kForm != 2 && live && kr < dk) ? st[(size_t)kr * dv + j] : 0.0f;
    }
    float dt_sum = 0.0f;
    const float rate = expf(p.A_log[h]), bias = p.dt_bias[h];
    const float skip = (kSsd && p.skip) ? p.skip[h] : 0.0f;
    issue(0, 0);
    int stage = 0;
    for (int c0 = 0; c0 < len; c0 += C, stage ^= 1) {
        const int n = min(C, len - c0);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                               // this chunk has landed for everyone, and everyone has left the chunk before
        if (c0 + C < len) issue(c0 + C, stage ^ 1);
        float* s_k = dsm + stage * stage_floats;       // [C][RS]
        float* s_q = s_k + C * RS;                     // [C][RS]
        const float* s_v = s_q + C * RS;               // [C][CB]
        const float* s_l = s_v + C * CBp;              // [C][2]
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const float dt = seq_softplus(s_l[2 * i + 1] + bias);
            s_beta[i] = kSsd ? dt : seq_sigmoid(s_l[2 * i]);
            s_g[i] = expf(-rate * dt);
        }
        for (int tok = warp; tok < n; tok += nwarps) {                             // unit vectors: a warp per token
            float sk = 0.0f, sq = 0.0f, skq = 0.0f;
            for (int kr = lane; kr < PP * kDeltaKP; kr += 32) {
                const int at = tok * RS + (kr / kDeltaKP) * kDeltaRS + kr % kDeltaKP;
                sk = fmaf(s_k[at], s_k[at], sk);
                sq = fmaf(s_q[at], s_q[at], sq);
                skq = fmaf(s_k[at], s_q[at], skq);
            }
            skq = warp_sum(skq);
            if (kSsd) {                                                             // B and C enter as they are
                if (lane == 0) s_kq[tok] = skq;
                continue;
            }
            const float ik = 1.0f / sqrtf(warp_sum(sk) + p.unit_eps), iq = p.qscale / sqrtf(warp_sum(sq) + p.unit_eps);
            if (lane == 0) s_kq[tok] = (skq * ik) * iq;
            for (int kr = lane; kr < PP * kDeltaKP; kr += 32) {
                const int at = tok * RS + (kr / kDeltaKP) * kDeltaRS + kr % kDeltaKP;
                s_k[at] *= ik;
                s_q[at] *= iq;
            }
        }
        __syncthreads();
        // One token: with D = g S the rule reads u = beta (v - D^T k), S' = D + k u^T, o = S'^T q = D^T q + u (k . q). Both products with the
        // OLD state run side by side (one pass over the piece, ONE round of shuffles for the two sums), and k . q is a number per token:
        // the serial chain of a token holds one reduction instead of two.
        for (int i = 0; i < n; ++i) {
            const float g = s_g[i], beta = s_beta[i], kq = s_kq[i];
            const float4* kk = reinterpret_cast<const float4*>(s_k + i * RS + part * kDeltaRS);
            if (kForm == 2) {                                                       // the end state only
                dt_sum += beta;
                const float u = beta * (live ? s_v[i * CB + jl] : 0.0f);
#pragma unroll
                for (int x = 0; x < kDeltaKP; x += 4) {
                    const float4 kv = kk[x >> 2];
                    S[x] = fmaf(kv.x, u, g * S[x]);
                    S[x + 1] = fmaf(kv.y, u, g * S[x + 1]);
                    S[x + 2] = fmaf(kv.z, u, g * S[x + 2]);
                    S[x + 3] = fmaf(kv.w, u, g * S[x + 3]);
                }
                continue;
            }
            const float4* qq = reinterpret_cast<const float4*>(s_q + i * RS + part * kDeltaRS);
            float kr[kDeltaKP];
            float d4[4] = {0.0f, 0.0f, 0.0f, 0.0f}, e4[4] = {0.0f, 0.0f, 0.0f, 0.0f};   // four running sums each: no long chain of dependent multiply-adds
#pragma unroll
            for (int x = 0; x < kDeltaKP; x += 4) {
                const float4 kv = kk[x >> 2], qv = qq[x >> 2];
                const float qr[4] = {qv.x, qv.y, qv.z, qv.w};
                kr[x] = kv.x; kr[x + 1] = kv.y; kr[x + 2] = kv.z; kr[x + 3] = kv.w;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (!kSsd) d4[e] = fmaf(S[x + e], kr[x + e], d4[e]);
                    e4[e] = fmaf(S[x + e], qr[e], e4[e]);
                }
            }
            float dot = (d4[0] + d4[1]) + (d4[2] + d4[3]), dq = (e4[0] + e4[1]) + (e4[2] + e4[3]);
            for (int o = PP >> 1; o > 0; o >>= 1) {
                if (!kSsd) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                dq += __shfl_xor_sync(0xffffffffu, dq, o);
            }
            const float vin = live ? s_v[i * CB + jl] : 0.0f;
            const float u = kSsd ? beta * vin : beta * (vin - g * dot);
            if (live && part == 0) s_o[i * CB + jl] = fmaf(u, kq, g * dq) + skip * vin;
#pragma unroll
            for (int x = 0; x < kDeltaKP; ++x) S[x] = fmaf(kr[x], u, g * S[x]);
        }
        __syncthreads();
        if (kForm != 2)
        for (int i = threadIdx.x; i < n * CB; i += blockDim.x) {
            const int col = blockIdx.z * CB + i % CB;
            if (col < dv) p.o[(size_t)(start + c0 + i / CB) * p.ldo + (size_t)h * dv + col] = s_o[i];
        }
    }
    if (kForm != 3 && live) {
#pragma unroll
        for (int x = 0; x < kDeltaKP; ++x) {
            const int kr = part * kDeltaKP + x;
            if (kr < dk) st[(size_t)kr * dv + j] = S[x];
        }
    }
    if (kForm == 2 && threadIdx.x == 0 && blockIdx.z == 0)
        p.ws[ssd_range_count(b.n_qtiles, b.nseg) * p.heads * dk * dv + ssd_range_id(b, seg, rg) * p.heads + h] = dt_sum;
    if (kForm != 2 && p.ring && p.taps > 1 && r0 + len == seg_len) {   // the heads of a segment share the job of storing its last inputs of the convolution
        const int seg_start = b.seg_start[seg], pos0 = b.seg_pos0[seg];
        const int keep = min(seg_len, p.taps - 1);
        for (int i = (h * gridDim.z + blockIdx.z) * blockDim.x + threadIdx.x; i < keep * p.channels; i += p.heads * gridDim.z * blockDim.x) {
            const int r = seg_len - keep + i / p.channels, c = i % p.channels;
            p.ring[((size_t)slot * (p.taps - 1) + (pos0 + r) % (p.taps - 1)) * p.channels + c] = p.conv_x[(size_t)(seg_start + r) * p.ldx + c];
        }
    }
}

// thread = one state element of one head of one portion: its ranges in order, end state from zero -> start state
__global__ void seq_ssd_carry_kernel(DeltaArgs p) {
    const sllm_seq_batch& b = p.b;
    const int seg = blockIdx.z, h = blockIdx.y, per = p.dk * p.dv, e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= per) return;
    const int ranges = (b.seg_len[seg] + kSsdRange - 1) / kSsdRange;
    const float rate = expf(p.A_log[h]);
    const float* sums = p.ws + ssd_range_count(b.n_qtiles, b.nseg) * p.heads * per;
    float* sp = p.state + ((size_t)b.seg_slot[seg] * p.heads + h) * per + e;
    float S = *sp;
    const size_t id0 = ssd_range_id(b, seg, 0);
    for (int r0 = 0; r0 < ranges; r0 += 4) {               // four ranges' loads in flight before the first store
        float Q[4], sum[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const bool has = r0 + u < ranges;
            Q[u] = has ? p.ws[((id0 + r0 + u) * p.heads + h) * per + e] : 0.0f;
            sum[u] = has ? sums[(id0 + r0 + u) * p.heads + h] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (r0 + u < ranges) {
                p.ws[((id0 + r0 + u) * p.heads + h) * per + e] = S;
                S = fmaf(expf(-rate * sum[u]), S, Q[u]);
            }
        }
    }
    *sp = S;
}

}  // namespace sllm

using namespace sllm;

extern "C" {

int sllm_seq_conv_ring(const sllm_seq_batch* b, const float* x, int32_t ldx, int32_t channels, int32_t taps, const float* w, const float* cb,
                       const float* ring, int32_t act, float* out, int32_t ldo, sllm_stream_t stream) {
    SLLM_REQUIRE(b && b->T > 0 && b->tok_slot && b->tok_pos, SLLM_EINVAL, "seq_conv_ring: incomplete batch description");
    SLLM_REQUIRE(x && w && out && channels > 0 && taps >= 1 && (taps == 1 || ring) && (act == 0 || act == 1), SLLM_EINVAL, "seq_conv_ring: bad argument");
    SLLM_REQUIRE(b->T <= 65535, SLLM_ENOTSUP, "seq_conv_ring: at most 65535 tokens per step");
    seq_conv_ring_kernel<<<dim3((channels + 127) / 128, b->T), 128, 0, as_stream(stream)>>>(*b, x, ldx, channels, taps, w, cb, ring, act, out, ldo);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

}  // extern "C"

// both recurrences: `ssd` = the state-space form (skip [heads] or NULL)
static int delta_run(bool ssd, const float* skip, const sllm_seq_batch* b, const float* q, int32_t ldq, const float* k, int32_t ldk, const float* v, int32_t ldv,
                     const float* beta_logit, int32_t ldb, const float* step_logit, int32_t lda, const float* A_log, const float* dt_bias, int32_t heads,
                     int32_t kv_heads, int32_t dk, int32_t dv, float unit_eps, float qscale, float* state, float* o, int32_t ldo, const float* conv_x,
                     int32_t ldx, int32_t channels, int32_t taps, float* ring, float* scratch, sllm_stream_t stream) {
    SLLM_REQUIRE(b && b->T > 0 && b->nseg > 0 && b->seg_start && b->seg_len && b->seg_slot && b->seg_pos0, SLLM_EINVAL, "seq_delta_rule: incomplete batch description");
    SLLM_REQUIRE(q && k && v && beta_logit && step_logit && A_log && dt_bias && state && o, SLLM_EINVAL, "seq_delta_rule / seq_ssd_scan: bad argument");
    SLLM_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dk > 0 && dv > 0, SLLM_EINVAL, "seq_delta_rule: %d heads over %d key heads", heads, kv_heads);
    SLLM_REQUIRE(!ring || (conv_x && channels > 0 && taps >= 1), SLLM_EINVAL, "seq_delta_rule: the ring needs the convolution's inputs");
    static const int tune_kp = getenv("SLLM_DELTA_KP") ? atoi(getenv("SLLM_DELTA_KP")) : 0;      // measurement aids: 8 / 16 / 32 channels per thread,
    static const int tune_cb = getenv("SLLM_DELTA_CB") ? atoi(getenv("SLLM_DELTA_CB")) : 0;      // columns per CTA
    int KP = dk <= 512 ? 16 : 32;
    if ((tune_kp == 8 || tune_kp == 16 || tune_kp == 32) && (dk + tune_kp - 1) / tune_kp <= 32) KP = tune_kp;
    const int RSh = KP + 4;
    const int parts = (dk + KP - 1) / KP;
    int PP = 1;
    while (PP < parts) PP *= 2;
    SLLM_REQUIRE(PP <= 32, SLLM_ENOTSUP, "seq_delta_rule: key heads of %d channels beyond 1024", dk);
    // value columns per CTA: 32 measured best whatever the number of heads (the token loop is serial and bound by its own latency:
    // narrower CTAs only add warps that wait)
    int CB = std::min(dv, kDeltaCB);
    if (tune_cb > 0) CB = std::min(dv, tune_cb);
    const int blocks = (dv + CB - 1) / CB;
    const int threads = (CB * PP + 31) / 32 * 32;
    const int per_tok = 2 * (2 * PP * RSh + ((CB + 3) & ~3) + 4) + CB + 3;      // two stages of inputs, one of outputs
    // tokens per stage: every stage costs a round trip to memory and three barriers whatever its size (measured: 12 tokens per stage spent
    // most of the time there), so portions use up to 160 KB of shared memory; steps of single tokens keep the stages small
    static const int tune_chunk = getenv("SLLM_DELTA_CHUNK") ? atoi(getenv("SLLM_DELTA_CHUNK")) : 0;
    const int longest = b->T - b->nseg + 1;                                   // no portion is longer than this
    int chunk = std::max(1, std::min(std::min(64, longest), 40960 / per_tok));
    if (tune_chunk > 0) chunk = std::max(1, std::min(tune_chunk, 50000 / per_tok));
    // the state-space form with some portion spanning several ranges (and a batch description that numbers the query tiles): three passes.
    // Its CTAs are many and independent: stages small enough for four of them per SM, so that one's round trips hide behind another's walk
    // (taken while the whole-portion form would leave SMs without a CTA: the passes walk every token twice, which pays as long as the
    // machine is not full — measured on B200 at 2048 tokens: 32 heads of 128 x 64 2.2 x faster, 64 heads equal, 128 heads 3 % slower)
    static const int tune_ranges = getenv("SLLM_SSD_RANGES") ? atoi(getenv("SLLM_SSD_RANGES")) : -1;   // measurement aid: 0 never, 1 whenever possible
    const bool ranges = ssd && scratch && longest > kSsdRange && b->seg_tile0 && b->n_qtiles > 0 && tune_ranges != 0 &&
                        (tune_ranges == 1 || (long long)b->nseg * heads * blocks <= sm_count());
    if (ranges && tune_chunk <= 0) chunk = std::max(4, std::min(chunk, 14336 / per_tok));
    const size_t smem = (size_t)chunk * per_tok * sizeof(float);
    SLLM_REQUIRE(smem <= (size_t)smem_optin_bytes() - 2048, SLLM_ENOTSUP, "seq_delta_rule: one token of a %d x %d head needs %zu bytes of shared memory", dk, dv, smem);
    const int vec = dk % 4 == 0 && ldq % 4 == 0 && ldk % 4 == 0 && ((uintptr_t)q % 16) == 0 && ((uintptr_t)k % 16) == 0;
    DeltaArgs p{*b, q, k, v, ldq, ldk, ldv, beta_logit, step_logit, ldb, lda, A_log, dt_bias, heads, kv_heads, dk, dv, unit_eps, qscale, state, o, ldo,
                conv_x, ldx, channels, taps, ring, chunk, PP, CB, vec, skip, scratch, (longest + kSsdRange - 1) / kSsdRange};
    SLLM_REQUIRE(!ranges || (long long)b->nseg * p.nrange <= 0x7fffffffLL, SLLM_ENOTSUP, "seq_ssd_scan: %d portions of up to %d ranges", b->nseg, p.nrange);
    const dim3 grid(ranges ? b->nseg * p.nrange : b->nseg, heads, blocks);
#define SLLM_DELTA_LAUNCH_AS(KPV, MAXT, FORM)                                                                                                             \
    do {                                                                                                                                                  \
        if (smem > 48 * 1024) SLLM_CUDA(cudaFuncSetAttribute(seq_delta_kernel<KPV, MAXT, FORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        seq_delta_kernel<KPV, MAXT, FORM><<<grid, threads, smem, as_stream(stream)>>>(p);                                                                 \
        ++g_launches;                                                                                                                                     \
        SLLM_LAUNCH_CHECK();                                                                                                                              \
    } while (0)
#define SLLM_DELTA_LAUNCH(KPV, MAXT)                                                                                                  \
    do {                                                                                                                              \
        if (ranges) {                                                                                                                 \
            SLLM_DELTA_LAUNCH_AS(KPV, MAXT, 2);                                                                                       \
            seq_ssd_carry_kernel<<<dim3((dk * dv + 255) / 256, heads, b->nseg), 256, 0, as_stream(stream)>>>(p);                      \
            ++g_launches;                                                                                                             \
            SLLM_LAUNCH_CHECK();                                                                                                      \
            SLLM_DELTA_LAUNCH_AS(KPV, MAXT, 3);                                                                                       \
        } else if (ssd) SLLM_DELTA_LAUNCH_AS(KPV, MAXT, 1);                                                                           \
        else SLLM_DELTA_LAUNCH_AS(KPV, MAXT, 0);                                                                                      \
    } while (0)
    if (KP == 8) SLLM_DELTA_LAUNCH(8, 1024);
    else if (KP == 16) SLLM_DELTA_LAUNCH(16, 512);
    else if (threads <= 256) SLLM_DELTA_LAUNCH(32, 256);
    else SLLM_DELTA_LAUNCH(32, 1024);
#undef SLLM_DELTA_LAUNCH
#undef SLLM_DELTA_LAUNCH_AS
    return SLLM_OK;
}

extern "C" {

int sllm_seq_delta_rule(const sllm_seq_batch* b, const float* q, int32_t ldq, const float* k, int32_t ldk, const float* v, int32_t ldv, const float* beta_logit,
                        int32_t ldb, const float* step_logit, int32_t lda, const float* A_log, const float* dt_bias, int32_t heads, int32_t kv_heads,
                        int32_t dk, int32_t dv, float unit_eps, float qscale, float* state, float* o, int32_t ldo, const float* conv_x, int32_t ldx,
                        int32_t channels, int32_t taps, float* ring, sllm_stream_t stream) {
    return delta_run(false, nullptr, b, q, ldq, k, ldk, v, ldv, beta_logit, ldb, step_logit, lda, A_log, dt_bias, heads, kv_heads, dk, dv, unit_eps, qscale, state,
                     o, ldo, conv_x, ldx, channels, taps, ring, nullptr, stream);
}

int sllm_seq_ssd_scan(const sllm_seq_batch* b, const float* x, int32_t ldx, const float* B, int32_t ldb, const float* C, int32_t ldc, const float* step_logit,
                      int32_t lda, const float* A_log, const float* dt_bias, const float* skip, int32_t heads, int32_t groups, int32_t n_state, int32_t dv,
                      float* state, float* y, int32_t ldy, const float* conv_x, int32_t ld_conv, int32_t channels, int32_t taps, float* ring,
                      float* scratch, sllm_stream_t stream) {
    return delta_run(true, skip, b, C, ldc, B, ldb, x, ldx, step_logit, lda, step_logit, lda, A_log, dt_bias, heads, groups, n_state, dv, 0.0f, 1.0f, state, y, ldy,
                     conv_x, ld_conv, channels, taps, ring, scratch, stream);
}

}  // extern "C"
