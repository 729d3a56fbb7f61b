// csrc/seq_elem.cu — row-wise building blocks of the ragged token batch (sllm_seq_*): embedding into residual streams, the
// hyper-connection read (weighted sum of the streams + grouped RMS norm) and write (stream mixing + sublayer output), PolyNorm,
// row gather and the per-head norm with a SiLU gate; layer norm (weight and bias), the depth-weighted average of a model whose layers
// read a learned mix of ALL earlier layers' results, and a clamped gated-linear-unit activation. Everything here is fp32: norms and the
// residual sum are never rounded.
#include "seq_common.cuh"

namespace sllm {

__global__ void seq_embed_kernel(const int32_t* __restrict__ ids, const void* __restrict__ table, int w_dtype, int vocab, int d, int streams,
                                 float scale, float* __restrict__ out, int T) {
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        const float v = seq_ldw(table, w_dtype, (size_t)id * d + j) * scale;
        for (int s = 0; s < streams; ++s) out[((size_t)s * T + t) * d + j] = v;
    }
}

// grid (T, groups): one CTA normalises one part of one token's vector
__global__ void seq_hyper_read_kernel(const float* __restrict__ x, int streams, int T, int d, const float* __restrict__ coef,
                                      const float* __restrict__ norm_w, int groups, float eps, float* __restrict__ y) {
    __shared__ float red[33];
    const int t = blockIdx.x, g = blockIdx.y, n = d / groups, j0 = g * n;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
        float u = 0.0f;
        for (int s = 0; s < streams; ++s) u = fmaf(coef ? coef[s] : 1.0f, x[((size_t)s * T + t) * d + j0 + j], u);
        y[(size_t)t * d + j0 + j] = u;
        ss = fmaf(u, u, ss);
    }
    if (!norm_w) return;
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    for (int j = threadIdx.x; j < n; j += blockDim.x) {   // each thread re-reads what it wrote itself
        const size_t i = (size_t)t * d + j0 + j;
        y[i] = (y[i] * inv) * norm_w[j0 + j];
    }
}

constexpr int kMaxStreams = 8;

__global__ void seq_hyper_write_kernel(float* __restrict__ x, int streams, int T, int d, const float* __restrict__ mix,
                                       const float* __restrict__ outc, const float* __restrict__ y) {
    const size_t n = (size_t)T * d;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float old[kMaxStreams];
        for (int s = 0; s < streams; ++s) old[s] = x[(size_t)s * n + i];
        const float yv = y[i];
        for (int to = 0; to < streams; ++to) {
            float v;
            if (mix) {
                v = 0.0f;
                for (int s = 0; s < streams; ++s) v = fmaf(mix[s * streams + to], old[s], v);
            } else {
                v = old[to];
            }
            x[(size_t)to * n + i] = fmaf(outc ? outc[to] : 1.0f, yv, v);
        }
    }
}

// hyper-connection write of one sublayer and read (+ grouped norm) of the next in one pass over the streams: grid (T, groups), a CTA owns
// one part of one token's vector in every stream — it stores the mixed streams and normalises their weighted sum for the next sublayer
__global__ void seq_hyper_write_read_kernel(float* __restrict__ x, int streams, int T, int d, const float* __restrict__ mix, const float* __restrict__ outc,
                                            const float* __restrict__ y_in, const float* __restrict__ coef, const float* __restrict__ norm_w, int groups,
                                            float eps, float* __restrict__ y_out) {
    __shared__ float red[33];
    __shared__ float s_mix[kMaxStreams * kMaxStreams], s_outc[kMaxStreams], s_coef[kMaxStreams];   // the small matrices once per CTA, not per element
    const int t = blockIdx.x, g = blockIdx.y, n = d / groups, j0 = g * n;
    const size_t plane = (size_t)T * d;
    if (threadIdx.x < streams * streams) s_mix[threadIdx.x] = mix ? mix[threadIdx.x] : ((int)threadIdx.x / streams == (int)threadIdx.x % streams ? 1.0f : 0.0f);
    if (threadIdx.x < streams) {
        s_outc[threadIdx.x] = outc ? outc[threadIdx.x] : 1.0f;
        s_coef[threadIdx.x] = coef ? coef[threadIdx.x] : 1.0f;
    }
    __syncthreads();
    float ss = 0.0f;
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
        const size_t i = (size_t)t * d + j0 + j;
        float old[kMaxStreams];
        for (int s = 0; s < streams; ++s) old[s] = x[(size_t)s * plane + i];
        const float yv = y_in[i];
        float u = 0.0f;
        for (int to = 0; to < streams; ++to) {
            float v;
            if (mix) {
                v = 0.0f;
                for (int s = 0; s < streams; ++s) v = fmaf(s_mix[s * streams + to], old[s], v);
            } else {
                v = old[to];
            }
            v = fmaf(s_outc[to], yv, v);
            x[(size_t)to * plane + i] = v;
            u = fmaf(s_coef[to], v, u);
        }
        y_out[i] = u;
        ss = fmaf(u, u, ss);
    }
    if (!norm_w) return;
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
        const size_t i = (size_t)t * d + j0 + j;
        y_out[i] = (y_out[i] * inv) * norm_w[j0 + j];
    }
}

__global__ void seq_polynorm_kernel(const float* z, int ldz, const float* __restrict__ coef, float eps, float* out,
                                    int ldo, int n) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    const float* zr = z + (size_t)t * ldz;
    float s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
        const float v = zr[j], v2 = v * v, v3 = v2 * v;
        s1 = fmaf(v, v, s1);
        s2 = fmaf(v2, v2, s2);
        s3 = fmaf(v3, v3, s3);
    }
    s1 = block_sum(s1, red);
    s2 = block_sum(s2, red);
    s3 = block_sum(s3, red);
    const float i1 = 1.0f / sqrtf(s1 / (float)n + eps), i2 = 1.0f / sqrtf(s2 / (float)n + eps), i3 = 1.0f / sqrtf(s3 / (float)n + eps);
    const float c0 = coef[0], c1 = coef[1], c2 = coef[2], c3 = coef[3];
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
        const float v = zr[j], v2 = v * v, v3 = v2 * v;
        out[(size_t)t * ldo + j] = c0 * (v * i1) + c1 * (v2 * i2) + c2 * (v3 * i3) + c3;
    }
}

__global__ void seq_gather_rows_kernel(const float* __restrict__ x, int ldx, const int32_t* __restrict__ rows, int d, float* __restrict__ out) {
    const int i = blockIdx.x;
    const float* src = x + (size_t)rows[i] * ldx;
    for (int j = threadIdx.x; j < d; j += blockDim.x) out[(size_t)i * d + j] = src[j];
}

// one warp per (token, head)
__global__ void seq_headnorm_gate_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ g, int ldg, const float* __restrict__ w,
                                         int heads, int dv, float eps, float* __restrict__ out, int ldout, uint16_t* __restrict__ out16, int T, int mode) {
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= T * heads) return;
    const int t = item / heads, h = item % heads;
    const float* orow = o + (size_t)t * ldo + (size_t)h * dv;
    const float* grow = g + (size_t)t * ldg + (size_t)h * dv;
    const float* wrow = (mode & 2) ? w + (size_t)h * dv : w;      // a weight per channel of the whole row, or one set shared by the parts
    const bool gate_first = mode & 1;                             // the gate multiplies before the root mean square is taken
    float ss = 0.0f;
    for (int j = lane; j < dv; j += 32) {
        const float gv = grow[j];
        const float v = gate_first ? orow[j] * (gv / (1.0f + expf(-gv))) : orow[j];
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
    for (int j = lane; j < dv; j += 32) {
        const float gv = grow[j];
        const float sg = gv / (1.0f + expf(-gv));
        const float v = gate_first ? ((orow[j] * sg) * inv) * wrow[j] : ((orow[j] * inv) * wrow[j]) * sg;
        if (out) out[(size_t)t * ldout + (size_t)h * dv + j] = v;
        if (out16) out16[(size_t)t * heads * dv + (size_t)h * dv + j] = f32_to_bf16_bits(v);
    }
}

// the same with one CTA per (token, part), for parts too wide for a warp (a norm over a few parts of a wide row): the part's gated values
// wait in registers between the sum of squares and the scaling, kNormPer per thread
constexpr int kNormPer = 8;
__global__ void __launch_bounds__(256) seq_headnorm_gate_wide_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ g, int ldg,
                                                                     const float* __restrict__ w, int heads, int dv, float eps, float* __restrict__ out, int ldout,
                                                                     uint16_t* __restrict__ out16, int mode) {
    __shared__ float red[33];
    const int t = blockIdx.x / heads, h = blockIdx.x % heads;
    const float* orow = o + (size_t)t * ldo + (size_t)h * dv;
    const float* grow = g + (size_t)t * ldg + (size_t)h * dv;
    const float* wrow = (mode & 2) ? w + (size_t)h * dv : w;
    const bool gate_first = mode & 1;
    float v[kNormPer], sg[kNormPer];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < kNormPer; ++i) {
        const int j = threadIdx.x + i * blockDim.x;
        v[i] = 0.0f;
        sg[i] = 0.0f;
        if (j < dv) {
            const float gv = grow[j];
            sg[i] = gv / (1.0f + expf(-gv));
            v[i] = gate_first ? orow[j] * sg[i] : orow[j];
            ss = fmaf(v[i], v[i], ss);
        }
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)dv + eps);
#pragma unroll
    for (int i = 0; i < kNormPer; ++i) {
        const int j = threadIdx.x + i * blockDim.x;
        if (j < dv) {
            const float r = gate_first ? (v[i] * inv) * wrow[j] : ((v[i] * inv) * wrow[j]) * sg[i];
            if (out) out[(size_t)t * ldout + (size_t)h * dv + j] = r;
            if (out16) out16[(size_t)t * heads * dv + (size_t)h * dv + j] = f32_to_bf16_bits(r);
        }
    }
}

// (row - mean) / sqrt(variance + eps) * w + b of one row that the CTA's threads hold strided; the variance is the mean of the squared
// deviations (two passes: the mean first), as the definition says
__device__ __forceinline__ void seq_layernorm_row(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias, float eps,
                                                  float* __restrict__ y, uint16_t* __restrict__ y16, int d, float* red) {
    float s = 0.0f;
    for (int j = threadIdx.x; j < d; j += blockDim.x) s += x[j];
    const float mean = block_sum(s, red) / (float)d;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        const float c = x[j] - mean;
        ss = fmaf(c, c, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        const float v = ((x[j] - mean) * inv) * w[j] + (bias ? bias[j] : 0.0f);
        y[j] = v;
        if (y16) y16[j] = f32_to_bf16_bits(v);
    }
}

__global__ void seq_layernorm_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ w, const float* __restrict__ bias, float eps,
                                     float* __restrict__ y, int ldy, uint16_t* __restrict__ y16, int d) {
    __shared__ float red[33];
    seq_layernorm_row(x + (size_t)blockIdx.x * ldx, w, bias, eps, y + (size_t)blockIdx.x * ldy, y16 ? y16 + (size_t)blockIdx.x * d : nullptr, d, red);
}

constexpr int kMaxDepth = 256;

// One CTA per token: hist[n_prev] <- x + y (this layer's own result); x <- sum_{j <= n_prev} coef[j] * hist[j]; h <- layer norm of x.
// The new row stays in shared memory for the norm's passes; with rows of a multiple of four floats everything moves as 16-byte words and
// the loads of the earlier results are issued together, before the store into the same array.
template <typename V>
__global__ void seq_depth_average_kernel(float* __restrict__ x, const float* __restrict__ y, float* hist, int n_prev, const float* __restrict__ coef,
                                         const float* __restrict__ norm_w, const float* __restrict__ norm_b, float eps, float* __restrict__ h, uint16_t* __restrict__ h16, int T, int d) {
    extern __shared__ __align__(16) float s_row[];   // [d]
    __shared__ float red[33];
    __shared__ float s_coef[kMaxDepth + 1];
    constexpr int E = sizeof(V) / sizeof(float);
    const int t = blockIdx.x;
    for (int j = threadIdx.x; j <= n_prev; j += blockDim.x) s_coef[j] = coef[j];
    __syncthreads();
    const size_t plane = (size_t)T * d / E, row = (size_t)t * d / E;
    V* xv = reinterpret_cast<V*>(x) + row;
    const V* yv = reinterpret_cast<const V*>(y) + row;
    V* hv = reinterpret_cast<V*>(hist) + row;
    float sum = 0.0f;
    for (int c = threadIdx.x; c < d / E; c += blockDim.x) {
        V own = xv[c];
        const V add = yv[c];
        float u[E];
#pragma unroll
        for (int e = 0; e < E; ++e) {
            reinterpret_cast<float*>(&own)[e] += reinterpret_cast<const float*>(&add)[e];
            u[e] = 0.0f;
        }
#pragma unroll 4
        for (int l = 0; l < n_prev; ++l) {
            const V old = hv[(size_t)l * plane + c];
#pragma unroll
            for (int e = 0; e < E; ++e) u[e] = fmaf(s_coef[l], reinterpret_cast<const float*>(&old)[e], u[e]);
        }
        hv[(size_t)n_prev * plane + c] = own;
        V out;
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const float v = fmaf(s_coef[n_prev], reinterpret_cast<const float*>(&own)[e], u[e]);
            reinterpret_cast<float*>(&out)[e] = v;
            s_row[c * E + e] = v;
            sum += v;
        }
        xv[c] = out;
    }
    if (!norm_w) return;
    const float mean = block_sum(sum, red) / (float)d;   // its barriers also publish s_row
    float ss = 0.0f;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        const float c = s_row[j] - mean;
        ss = fmaf(c, c, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
    float* hr = h + (size_t)t * d;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        const float v = ((s_row[j] - mean) * inv) * norm_w[j] + (norm_b ? norm_b[j] : 0.0f);
        hr[j] = v;
        if (h16) h16[(size_t)t * d + j] = f32_to_bf16_bits(v);
    }
}

// out = g * sigmoid(alpha * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit)
__global__ void seq_clamped_glu_kernel(const float* __restrict__ gate, int ldg, const float* __restrict__ up, int ldu, float limit, float alpha,
                                       float* __restrict__ out, int ldo, uint16_t* __restrict__ out16, int T, int n) {
    const size_t total = (size_t)T * n;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / n, j = i % n;
        const float g = fminf(gate[t * ldg + j], limit);
        const float u = fminf(fmaxf(up[t * ldu + j], -limit), limit);
        const float v = (g * seq_sigmoid(alpha * g)) * (u + 1.0f);
        if (out) out[t * ldo + j] = v;
        if (out16) out16[i] = f32_to_bf16_bits(v);
    }
}

// token embedding plus a hashed embedding of the (previous token, token) pair: row (prev * mul_prev + id * mul_cur) mod buckets of
// `pairs`, and row `buckets` (the table's last) for a sequence's first token (prev < 0)
__global__ void seq_embed_pair_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ prev, const void* __restrict__ table,
                                      const void* __restrict__ pairs, int w_dtype, int vocab, int d, int buckets, long long mul_prev, long long mul_cur,
                                      float* __restrict__ out) {
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const int pv = prev[t];
    const long long row = pv < 0 ? (long long)buckets : (((long long)pv * mul_prev + (long long)id * mul_cur) % buckets + buckets) % buckets;
    for (int j = threadIdx.x; j < d; j += blockDim.x)
        out[(size_t)t * d + j] = seq_ldw(table, w_dtype, (size_t)id * d + j) + seq_ldw(pairs, w_dtype, (size_t)row * d + j);
}

// one warp per row: y = x / sqrt(mean(x^2) + eps) * w (w NULL = no weight)
__global__ void seq_rmsnorm_rows_kernel(const float* x, int ldx, const float* __restrict__ w, float eps, float* y, int ldy, int T, int n) {   // y may be x
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T) return;
    const float* xr = x + (size_t)t * ldx;
    float ss = 0.0f;
    for (int j = lane; j < n; j += 32) ss = fmaf(xr[j], xr[j], ss);
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)n + eps);
    for (int j = lane; j < n; j += 32) y[(size_t)t * ldy + j] = (xr[j] * inv) * (w ? w[j] : 1.0f);
}

// the same with one CTA per row, for steps of few rows (one warp would walk a long row alone)
__global__ void seq_rmsnorm_row_cta_kernel(const float* x, int ldx, const float* __restrict__ w, float eps, float* y, int ldy, int n) {   // y may be x
    __shared__ float red[33];
    const float* xr = x + (size_t)blockIdx.x * ldx;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < n; j += blockDim.x) ss = fmaf(xr[j], xr[j], ss);
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
    for (int j = threadIdx.x; j < n; j += blockDim.x) y[(size_t)blockIdx.x * ldy + j] = (xr[j] * inv) * (w ? w[j] : 1.0f);
}

// out = act(gate) * up; act 0 = silu
__global__ void seq_gated_act_kernel(const float* __restrict__ gate, int ldg, const float* __restrict__ up, int ldu, int act, float* __restrict__ out,
                                     int ldo, uint16_t* __restrict__ out16, int T, int n) {
    const size_t total = (size_t)T * n;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / n, j = i % n;
        const float g = gate[t * ldg + j];
        const float v = (g * seq_sigmoid(g)) * up[t * ldu + j];
        if (out) out[t * ldo + j] = v;
        if (out16) out16[i] = f32_to_bf16_bits(v);
    }
}

// x <- cap * tanh(x / cap)
__global__ void seq_softcap_kernel(float* __restrict__ x, size_t n, float cap) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] = cap * tanhf(x[i] / cap);
}

// Threads of a one-CTA-per-row kernel: steps of few tokens have few CTAs, and a row walked by 128 threads is a chain of dependent
// memory latencies (32 of them at 4096 floats); with up to 1024 threads every thread touches the row once or twice.
static int row_threads(int T, int items, int many_rows_threads) {
    if (T >= 64) return many_rows_threads;
    return std::min(1024, std::max(128, (items + 31) / 32 * 32));
}

}  // namespace sllm

using namespace sllm;

extern "C" {

int sllm_seq_embed(const int32_t* ids, const void* table, int32_t w_dtype, int32_t vocab, int32_t d, int32_t streams, float scale, float* out,
                   int32_t T, sllm_stream_t stream) {
    SLLM_REQUIRE(ids && table && out && T > 0 && d > 0 && vocab > 0 && streams >= 1, SLLM_EINVAL, "seq_embed: bad argument");
    SLLM_REQUIRE(w_dtype == SLLM_F32 || w_dtype == SLLM_BF16, SLLM_ENOTSUP, "seq_embed: fp32 or bf16 tables");
    seq_embed_kernel<<<T, row_threads(T, d, 128), 0, as_stream(stream)>>>(ids, table, w_dtype, vocab, d, streams, scale, out, T);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_hyper_read(const float* x, int32_t streams, int32_t T, int32_t d, const float* coef, const float* norm_w, int32_t groups, float eps,
                        float* y, sllm_stream_t stream) {
    SLLM_REQUIRE(x && y && T > 0 && d > 0 && streams >= 1, SLLM_EINVAL, "seq_hyper_read: bad argument");
    if (!norm_w) groups = 1;
    SLLM_REQUIRE(groups >= 1 && d % groups == 0, SLLM_EINVAL, "seq_hyper_read: %d does not divide into %d parts", d, groups);
    const int n = d / groups, threads = n >= 1024 ? 256 : (n >= 256 ? 128 : 64);
    seq_hyper_read_kernel<<<dim3(T, groups), threads, 0, as_stream(stream)>>>(x, streams, T, d, coef, norm_w, groups, eps, y);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_hyper_write(float* x, int32_t streams, int32_t T, int32_t d, const float* mix, const float* outc, const float* y, sllm_stream_t stream) {
    SLLM_REQUIRE(x && y && T > 0 && d > 0, SLLM_EINVAL, "seq_hyper_write: bad argument");
    SLLM_REQUIRE(streams >= 1 && streams <= kMaxStreams, SLLM_ENOTSUP, "seq_hyper_write: 1..%d streams", kMaxStreams);
    const size_t n = (size_t)T * d;
    const int blocks = (int)std::min<size_t>((n + 255) / 256, (size_t)sm_count() * 8);
    seq_hyper_write_kernel<<<blocks, 256, 0, as_stream(stream)>>>(x, streams, T, d, mix, outc, y);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_hyper_write_read(float* x, int32_t streams, int32_t T, int32_t d, const float* mix, const float* outc, const float* y_in, const float* coef,
                              const float* norm_w, int32_t groups, float eps, float* y_out, sllm_stream_t stream) {
    SLLM_REQUIRE(x && y_in && y_out && y_in != y_out && T > 0 && d > 0, SLLM_EINVAL, "seq_hyper_write_read: bad argument");
    SLLM_REQUIRE(streams >= 1 && streams <= kMaxStreams, SLLM_ENOTSUP, "seq_hyper_write_read: 1..%d streams", kMaxStreams);
    if (!norm_w) groups = 1;
    SLLM_REQUIRE(groups >= 1 && d % groups == 0, SLLM_EINVAL, "seq_hyper_write_read: %d does not divide into %d parts", d, groups);
    const int n = d / groups, threads = n >= 1024 ? 256 : (n >= 256 ? 128 : 64);
    seq_hyper_write_read_kernel<<<dim3(T, groups), threads, 0, as_stream(stream)>>>(x, streams, T, d, mix, outc, y_in, coef, norm_w, groups, eps, y_out);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_polynorm(const float* z, int32_t ldz, const float* coef, float eps, float* out, int32_t ldo, int32_t T, int32_t n, sllm_stream_t stream) {
    SLLM_REQUIRE(z && coef && out && T > 0 && n > 0 && ldz >= n && ldo >= n, SLLM_EINVAL, "seq_polynorm: bad argument");
    seq_polynorm_kernel<<<T, n >= 8192 ? 1024 : (n >= 2048 ? 512 : 256), 0, as_stream(stream)>>>(z, ldz, coef, eps, out, ldo, n);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_gather_rows(const float* x, int32_t ldx, const int32_t* rows, int32_t n, int32_t d, float* out, sllm_stream_t stream) {
    SLLM_REQUIRE(x && rows && out && n > 0 && d > 0, SLLM_EINVAL, "seq_gather_rows: bad argument");
    seq_gather_rows_kernel<<<n, row_threads(n, d, 128), 0, as_stream(stream)>>>(x, ldx, rows, d, out);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_headnorm_gate(const float* o, int32_t ldo, const float* g, int32_t ldg, const float* w, int32_t heads, int32_t dv, float eps, float* out,
                           int32_t ldout, void* out16, int32_t T, int32_t mode, sllm_stream_t stream) {
    SLLM_REQUIRE(o && g && w && (out || out16) && heads > 0 && dv > 0 && T > 0 && mode >= 0 && mode <= 3, SLLM_EINVAL, "seq_headnorm_gate: bad argument");
    const int items = T * heads;
    if (dv >= 512 && dv <= 256 * kNormPer)       // a warp per part would walk such a part in 16 and more rounds, twice
        seq_headnorm_gate_wide_kernel<<<items, 256, 0, as_stream(stream)>>>(o, ldo, g, ldg, w, heads, dv, eps, out, ldout, (uint16_t*)out16, mode);
    else
        seq_headnorm_gate_kernel<<<(items + 3) / 4, 128, 0, as_stream(stream)>>>(o, ldo, g, ldg, w, heads, dv, eps, out, ldout, (uint16_t*)out16, T, mode);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_layernorm(const float* x, int32_t ldx, const float* w, const float* bias, float eps, float* y, int32_t ldy, void* y16, int32_t T,
                       int32_t d, sllm_stream_t stream) {
    SLLM_REQUIRE(x && w && y && T > 0 && d > 0 && ldx >= d && ldy >= d, SLLM_EINVAL, "seq_layernorm: bad argument");
    seq_layernorm_kernel<<<T, row_threads(T, d, d >= 2048 ? 256 : 128), 0, as_stream(stream)>>>(x, ldx, w, bias, eps, y, ldy, (uint16_t*)y16, d);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_depth_average(float* x, const float* y, float* hist, int32_t n_prev, const float* coef, const float* norm_w, const float* norm_b, float eps,
                           float* h, void* h16, int32_t T, int32_t d, sllm_stream_t stream) {
    SLLM_REQUIRE(x && y && hist && coef && T > 0 && d > 0 && n_prev >= 0 && (!norm_w || h), SLLM_EINVAL, "seq_depth_average: bad argument");
    SLLM_REQUIRE(n_prev <= kMaxDepth, SLLM_ENOTSUP, "seq_depth_average: %d earlier results beyond %d", n_prev, kMaxDepth);
    const size_t smem = (size_t)d * sizeof(float);
    SLLM_REQUIRE(smem <= (size_t)smem_optin_bytes() - 4096, SLLM_ENOTSUP, "seq_depth_average: rows of %d floats do not fit shared memory", d);
    const bool vec = d % 4 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0 && ((uintptr_t)hist % 16) == 0;
    const int threads = row_threads(T, vec ? d / 4 : d, d >= 2048 ? 256 : 128);
    if (vec) {
        if (smem > 48 * 1024) SLLM_CUDA(cudaFuncSetAttribute(seq_depth_average_kernel<float4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        seq_depth_average_kernel<float4><<<T, threads, smem, as_stream(stream)>>>(x, y, hist, n_prev, coef, norm_w, norm_b, eps, h, (uint16_t*)h16, T, d);
    } else {
        if (smem > 48 * 1024) SLLM_CUDA(cudaFuncSetAttribute(seq_depth_average_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        seq_depth_average_kernel<float><<<T, threads, smem, as_stream(stream)>>>(x, y, hist, n_prev, coef, norm_w, norm_b, eps, h, (uint16_t*)h16, T, d);
    }
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_clamped_glu(const float* gate, int32_t ldg, const float* up, int32_t ldu, float limit, float alpha, float* out, int32_t ldo, void* out16,
                         int32_t T, int32_t n, sllm_stream_t stream) {
    SLLM_REQUIRE(gate && up && (out || out16) && T > 0 && n > 0 && ldg >= n && ldu >= n && (!out || ldo >= n), SLLM_EINVAL, "seq_clamped_glu: bad argument");
    const size_t total = (size_t)T * n;
    seq_clamped_glu_kernel<<<(int)std::min<size_t>((total + 255) / 256, (size_t)sm_count() * 8), 256, 0, as_stream(stream)>>>(gate, ldg, up, ldu, limit, alpha, out,
                                                                                                                       ldo, (uint16_t*)out16, T, n);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_embed_pair(const int32_t* ids, const int32_t* prev_ids, const void* table, const void* pairs, int32_t w_dtype, int32_t vocab, int32_t d,
                        int32_t buckets, int64_t mul_prev, int64_t mul_cur, float* out, int32_t T, sllm_stream_t stream) {
    SLLM_REQUIRE(ids && prev_ids && table && pairs && out && T > 0 && d > 0 && vocab > 0 && buckets > 0, SLLM_EINVAL, "seq_embed_pair: bad argument");
    SLLM_REQUIRE(w_dtype == SLLM_F32 || w_dtype == SLLM_BF16, SLLM_ENOTSUP, "seq_embed_pair: fp32 or bf16 tables");
    seq_embed_pair_kernel<<<T, row_threads(T, d, 128), 0, as_stream(stream)>>>(ids, prev_ids, table, pairs, w_dtype, vocab, d, buckets, mul_prev, mul_cur, out);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_rmsnorm_rows(const float* x, int32_t ldx, const float* w, float eps, float* y, int32_t ldy, int32_t T, int32_t n, sllm_stream_t stream) {
    SLLM_REQUIRE(x && y && T > 0 && n > 0 && ldx >= n && ldy >= n, SLLM_EINVAL, "seq_rmsnorm_rows: bad argument");
    if (T < 64 && n > 128) seq_rmsnorm_row_cta_kernel<<<T, std::min(1024, (n + 31) / 32 * 32), 0, as_stream(stream)>>>(x, ldx, w, eps, y, ldy, n);
    else seq_rmsnorm_rows_kernel<<<(T + 3) / 4, 128, 0, as_stream(stream)>>>(x, ldx, w, eps, y, ldy, T, n);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_gated_act(const float* gate, int32_t ldg, const float* up, int32_t ldu, int32_t act, float* out, int32_t ldo, void* out16, int32_t T, int32_t n,
                       sllm_stream_t stream) {
    SLLM_REQUIRE(gate && up && (out || out16) && T > 0 && n > 0 && ldg >= n && ldu >= n && (!out || ldo >= n), SLLM_EINVAL, "seq_gated_act: bad argument");
    SLLM_REQUIRE(act == 0, SLLM_ENOTSUP, "seq_gated_act: activation 0 (silu)");
    const size_t total = (size_t)T * n;
    seq_gated_act_kernel<<<(int)std::min<size_t>((total + 255) / 256, (size_t)sm_count() * 8), 256, 0, as_stream(stream)>>>(gate, ldg, up, ldu, act, out, ldo,
                                                                                                                     (uint16_t*)out16, T, n);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_softcap(float* x, int64_t n, float cap, sllm_stream_t stream) {
    SLLM_REQUIRE(x && n > 0 && cap > 0.0f, SLLM_EINVAL, "seq_softcap: bad argument");
    seq_softcap_kernel<<<(int)std::min<size_t>(((size_t)n + 255) / 256, (size_t)sm_count() * 8), 256, 0, as_stream(stream)>>>(x, (size_t)n, cap);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

}  // extern "C"
