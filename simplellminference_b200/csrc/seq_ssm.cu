// csrc/seq_ssm.cu — the selective scan (Mamba) over the ragged token batch, and the store of a convolution's last inputs.
// Every channel c of the block carries its own state of N numbers (fp32, one set per sequence slot):
//     S[c][n] <- exp(dt_c A[c][n]) S[c][n] + dt_c x_c B_n;   y_c = sum_n S[c][n] C_n + D_c x_c;   out_c = y_c * silu(z_c)
// with dt = softplus(step logit) per channel and token, A = -exp(A_log), and B, C shared by all channels of a token. Everything that
// enters the recurrence is fp32. The channels are independent recurrences that share B and C: a CTA takes 32 channels of one portion,
// eight adjacent lanes own the states of one channel in registers (lane l holds states l, l + 8, ...) and meet by shuffles; the tokens
// of a portion are staged in shared memory a chunk at a time and walked in order.
//
// The recurrence is linear in the state, with a decay whose product over a run of tokens is exp(A * (sum of the run's dt)). Steps that hold
// a long portion therefore run as three passes over ranges of kScanRange tokens: (1) every range, in parallel, from a zero state: its end
// state Q and its sum of dt; (2) per state element, the ranges of a portion in order: start of range r+1 = exp(A * sum_r) * start_r + Q_r,
// the last one being the sequence's new state; (3) every range again, in parallel, from its start state, writing the outputs.
#include "seq_common.cuh"

namespace sllm {

constexpr int kScanLanes = 8;       // lanes that share a channel's states
constexpr int kScanChannels = 32;   // channels of a CTA (256 threads)
constexpr int kScanRange = 128;     // tokens of a range of the three-pass form (four query tiles of the batch description)

struct ScanArgs {
    sllm_seq_batch b;
    const float *x, *dtl, *Bm, *Cm, *z; int ldx, lddt, ldb, ldc, ldz;   // per token: x, step logits, z [inner]; B, C [N]
    const float *A_log, *D;                                             // [inner][N], [inner]
    int inner, N;
    float* state;                                                       // [slots][inner][N]
    float* out; int ldo; uint16_t* out16;                               // [T][inner] fp32 and / or dense bf16 rows
    const float* conv_x; int ld_conv, taps; float* ring;                // the convolution's inputs [T][inner] -> ring [slots][taps-1][inner]
    int chunk;
    float* ws; int nrange;                                              // three passes: per range [inner][N] states, then [inner] sums of dt
};

// where range `rg` of segment `seg` keeps its summary: ranges are numbered by the first query tile (32 tokens) of the segment
__device__ __forceinline__ size_t scan_range_id(const sllm_seq_batch& b, int seg, int rg) { return (size_t)b.seg_tile0[seg] + rg; }

// R: states per lane, N <= 8 * R. MODE 0: a CTA walks a whole portion from the sequence's state and stores the state back; MODE 1: a range
// from zero, leaving its end state and its sum of dt in the workspace; MODE 2: a range from the start state the carry kernel left there.
template <int R, int MODE>
__global__ void __launch_bounds__(kScanLanes * kScanChannels) seq_selective_scan_kernel(ScanArgs p) {
    extern __shared__ __align__(16) float ssm_sm[];
    const sllm_seq_batch& b = p.b;
    const int seg = MODE == 0 ? blockIdx.x : blockIdx.x / p.nrange, rg = MODE == 0 ? 0 : blockIdx.x % p.nrange, c0 = blockIdx.y * kScanChannels;
    const int seg_len = b.seg_len[seg], r0 = rg * kScanRange;
    if (MODE != 0 && r0 >= seg_len) return;
    const int start = b.seg_start[seg] + r0, len = MODE == 0 ? seg_len : min(kScanRange, seg_len - r0), slot = b.seg_slot[seg];
    const int N = p.N, C = p.chunk;
    const int cl = threadIdx.x / kScanLanes, sub = threadIdx.x % kScanLanes, c = c0 + cl;
    const bool live = c < p.inner;
    // per staged token: B [N], C [N], then dt, x, z and the result of the CTA's channels
    const int per_tok = 2 * N + 4 * kScanChannels;
    float A[R], S[R];
    float* st = MODE == 0 ? p.state + ((size_t)slot * p.inner + (live ? c : 0)) * N
                          : p.ws + (scan_range_id(b, seg, rg) * p.inner + (live ? c : 0)) * N;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int n = sub + r * kScanLanes;
        const bool has = live && n < N;
        A[r] = has ? -expf(p.A_log[(size_t)c * N + n]) : 0.0f;
        S[r] = (has && MODE != 1) ? st[n] : 0.0f;
    }
    const float skip = live ? p.D[c] : 0.0f;
    float dt_sum = 0.0f;
    for (int t0 = 0; t0 < len; t0 += C) {
        const int n_tok = min(C, len - t0);
        __syncthreads();                                   // everyone has left the chunk before
        for (int i = threadIdx.x; i < n_tok * 2 * N; i += blockDim.x) {
            const int tok = i / (2 * N), j = i % (2 * N);
            const size_t t = (size_t)(start + t0 + tok);
            ssm_sm[tok * per_tok + j] = j < N ? p.Bm[t * p.ldb + j] : p.Cm[t * p.ldc + j - N];
        }
        for (int i = threadIdx.x; i < n_tok * kScanChannels; i += blockDim.x) {
            const int tok = i / kScanChannels, ch = i % kScanChannels;
            const size_t t = (size_t)(start + t0 + tok);
            const bool ok = c0 + ch < p.inner;
            float* row = ssm_sm + tok * per_tok + 2 * N;
            row[ch] = ok ? seq_softplus(p.dtl[t * p.lddt + c0 + ch]) : 0.0f;
            row[kScanChannels + ch] = ok ? p.x[t * p.ldx + c0 + ch] : 0.0f;
            if (MODE != 1) row[2 * kScanChannels + ch] = ok ? p.z[t * p.ldz + c0 + ch] : 0.0f;
        }
        __syncthreads();
        for (int i = 0; i < n_tok; ++i) {
            const float* sB = ssm_sm + i * per_tok;
            const float* sC = sB + N;
            float* row = ssm_sm + i * per_tok + 2 * N;
            const float dt = row[cl], xv = row[kScanChannels + cl];
            const float dx = dt * xv;
            float acc = 0.0f;
            if (MODE == 1) {                               // the end state only
                dt_sum += dt;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int n = sub + r * kScanLanes;
                    if (n < N) S[r] = fmaf(expf(dt * A[r]), S[r], dx * sB[n]);
                }
                continue;
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int n = sub + r * kScanLanes;
                if (n < N) {
                    S[r] = fmaf(expf(dt * A[r]), S[r], dx * sB[n]);
                    acc = fmaf(S[r], sC[n], acc);
                }
            }
#pragma unroll
            for (int o = kScanLanes >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (sub == 0) {
                const float zv = row[2 * kScanChannels + cl];
                row[3 * kScanChannels + cl] = fmaf(skip, xv, acc) * (zv * seq_sigmoid(zv));
            }
        }
        __syncthreads();
        if (MODE != 1)
        for (int i = threadIdx.x; i < n_tok * kScanChannels; i += blockDim.x) {
            const int tok = i / kScanChannels, ch = i % kScanChannels;
            if (c0 + ch >= p.inner) continue;
            const size_t t = (size_t)(start + t0 + tok);
            const float v = ssm_sm[tok * per_tok + 2 * N + 3 * kScanChannels + ch];
            if (p.out) p.out[t * p.ldo + c0 + ch] = v;
            if (p.out16) p.out16[t * p.inner + c0 + ch] = f32_to_bf16_bits(v);
        }
    }
    if (MODE != 2) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int n = sub + r * kScanLanes;
            if (live && n < N) st[n] = S[r];
        }
    }
    if (MODE == 1 && live && sub == 0) p.ws[(size_t)b.n_qtiles * p.inner * N + scan_range_id(b, seg, rg) * p.inner + c] = dt_sum;
    if (MODE != 1 && p.ring && p.taps > 1 && r0 + len == seg_len) {           // the portion's last inputs of the convolution, this CTA's channels
        const int seg_start = b.seg_start[seg], pos0 = b.seg_pos0[seg];
        const int keep = min(seg_len, p.taps - 1);
        for (int i = threadIdx.x; i < keep * kScanChannels; i += blockDim.x) {
            const int r = seg_len - keep + i / kScanChannels, ch = c0 + i % kScanChannels;
            if (ch < p.inner) p.ring[((size_t)slot * (p.taps - 1) + (pos0 + r) % (p.taps - 1)) * p.inner + ch] = p.conv_x[(size_t)(seg_start + r) * p.ld_conv + ch];
        }
    }
}

// thread = one state element (channel c, state n) of one portion: its ranges in order, end state from zero -> start state; the last
// start state, moved on over the last range, is the sequence's new state
__global__ void seq_selective_scan_carry_kernel(ScanArgs p) {
    const sllm_seq_batch& b = p.b;
    const int seg = blockIdx.y;
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x, per = (size_t)p.inner * p.N;
    if (e >= per) return;
    const int c = (int)(e / p.N);
    const int ranges = (b.seg_len[seg] + kScanRange - 1) / kScanRange;
    const float A = -expf(p.A_log[e]);
    float* sp = p.state + (size_t)b.seg_slot[seg] * per + e;
    const float* sums = p.ws + (size_t)b.n_qtiles * per;
    float S = *sp;
    const size_t id0 = scan_range_id(b, seg, 0);
    for (int r0 = 0; r0 < ranges; r0 += 4) {               // four ranges' loads in flight before the first store
        float Q[4], sum[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const bool has = r0 + u < ranges;
            Q[u] = has ? p.ws[(id0 + r0 + u) * per + e] : 0.0f;
            sum[u] = has ? sums[(id0 + r0 + u) * p.inner + c] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (r0 + u < ranges) {
                p.ws[(id0 + r0 + u) * per + e] = S;
                S = fmaf(expf(A * sum[u]), S, Q[u]);
            }
        }
    }
    *sp = S;
}

// ring[slot][p % (taps-1)][c] <- x[t][c] for the last taps-1 tokens of every portion (position p); grid (nseg, blocks of channels)
__global__ void seq_ring_store_kernel(sllm_seq_batch b, const float* __restrict__ x, int ldx, int channels, int taps, float* __restrict__ ring) {
    const int seg = blockIdx.x;
    const int start = b.seg_start[seg], len = b.seg_len[seg], slot = b.seg_slot[seg], pos0 = b.seg_pos0[seg];
    const int keep = min(len, taps - 1);
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < keep * channels; i += gridDim.y * blockDim.x) {
        const int r = len - keep + i / channels, c = i % channels;
        ring[((size_t)slot * (taps - 1) + (pos0 + r) % (taps - 1)) * channels + c] = x[(size_t)(start + r) * ldx + c];
    }
}

}  // namespace sllm

using namespace sllm;

extern "C" {

int sllm_seq_selective_scan(const sllm_seq_batch* b, const float* x, int32_t ldx, const float* step_logit, int32_t lddt, const float* B, int32_t ldb,
                            const float* C, int32_t ldc, const float* z, int32_t ldz, const float* A_log, const float* D, int32_t inner, int32_t n_state,
                            float* state, float* out, int32_t ldo, void* out16, const float* conv_x, int32_t ld_conv, int32_t taps, float* ring,
                            float* scratch, sllm_stream_t stream) {
    SLLM_REQUIRE(b && b->T > 0 && b->nseg > 0 && b->seg_start && b->seg_len && b->seg_slot && b->seg_pos0, SLLM_EINVAL, "seq_selective_scan: incomplete batch description");
    SLLM_REQUIRE(x && step_logit && B && C && z && A_log && D && state && (out || out16) && inner > 0 && n_state > 0, SLLM_EINVAL, "seq_selective_scan: bad argument");
    SLLM_REQUIRE(!ring || (conv_x && taps >= 1), SLLM_EINVAL, "seq_selective_scan: the ring needs the convolution's inputs");
    SLLM_REQUIRE(n_state <= 32 * kScanLanes, SLLM_ENOTSUP, "seq_selective_scan: %d states per channel beyond %d", n_state, 32 * kScanLanes);
    const int blocks = (inner + kScanChannels - 1) / kScanChannels;
    SLLM_REQUIRE(blocks <= 65535, SLLM_ENOTSUP, "seq_selective_scan: %d channels", inner);
    const int per_tok = 2 * n_state + 4 * kScanChannels;
    const int longest = b->T - b->nseg + 1;                                   // no portion is longer than this
    const int chunk = std::max(1, std::min(std::min(64, longest), 10240 / per_tok));   // 40 KB of stages at most
    const size_t smem = (size_t)chunk * per_tok * sizeof(float);
    ScanArgs p{*b, x, step_logit, B, C, z, ldx, lddt, ldb, ldc, ldz, A_log, D, inner, n_state, state, out, ldo, (uint16_t*)out16, conv_x, ld_conv, taps, ring, chunk,
               scratch, (longest + kScanRange - 1) / kScanRange};
    const int threads = kScanLanes * kScanChannels;
    cudaStream_t st = as_stream(stream);
    const int per_lane = (n_state + kScanLanes - 1) / kScanLanes;
#define SLLM_SCAN_LAUNCH(MODE, GRID)                                                          \
    do {                                                                                      \
        if (per_lane <= 1) seq_selective_scan_kernel<1, MODE><<<GRID, threads, smem, st>>>(p);       \
        else if (per_lane <= 2) seq_selective_scan_kernel<2, MODE><<<GRID, threads, smem, st>>>(p);  \
        else if (per_lane <= 4) seq_selective_scan_kernel<4, MODE><<<GRID, threads, smem, st>>>(p);  \
        else if (per_lane <= 8) seq_selective_scan_kernel<8, MODE><<<GRID, threads, smem, st>>>(p);  \
        else if (per_lane <= 16) seq_selective_scan_kernel<16, MODE><<<GRID, threads, smem, st>>>(p); \
        else seq_selective_scan_kernel<32, MODE><<<GRID, threads, smem, st>>>(p);                    \
        ++g_launches;                                                                         \
        SLLM_LAUNCH_CHECK();                                                                  \
    } while (0)
    // some portion spans several ranges (and the batch description numbers the query tiles): three passes
    if (scratch && longest > kScanRange && b->seg_tile0 && b->n_qtiles > 0 && (long long)b->nseg * p.nrange <= 0x7fffffffLL) {
        const dim3 grid(b->nseg * p.nrange, blocks);
        SLLM_SCAN_LAUNCH(1, grid);
        const size_t per = (size_t)inner * n_state;
        seq_selective_scan_carry_kernel<<<dim3((unsigned)((per + 255) / 256), b->nseg), 256, 0, st>>>(p);
        ++g_launches;
        SLLM_LAUNCH_CHECK();
        SLLM_SCAN_LAUNCH(2, grid);
        return SLLM_OK;
    }
    const dim3 grid(b->nseg, blocks);
    SLLM_SCAN_LAUNCH(0, grid);
#undef SLLM_SCAN_LAUNCH
    return SLLM_OK;
}

int sllm_seq_ring_store(const sllm_seq_batch* b, const float* x, int32_t ldx, int32_t channels, int32_t taps, float* ring, sllm_stream_t stream) {
    SLLM_REQUIRE(b && b->nseg > 0 && b->seg_start && b->seg_len && b->seg_slot && b->seg_pos0, SLLM_EINVAL, "seq_ring_store: incomplete batch description");
    SLLM_REQUIRE(x && channels > 0 && taps >= 1 && (taps == 1 || ring), SLLM_EINVAL, "seq_ring_store: bad argument");
    if (taps == 1) return SLLM_OK;
    const int blocks = std::max(1, std::min(64, ((taps - 1) * channels + 255) / 256));
    seq_ring_store_kernel<<<dim3(b->nseg, blocks), 256, 0, as_stream(stream)>>>(*b, x, ldx, channels, taps, ring);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

}  // extern "C"
