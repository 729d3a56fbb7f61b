// csrc/seq_linear.cu — sllm_seq_linear: C = alpha * (A . W^T + bias) (+ C) for the ragged token batch. Three bodies:
//   * rows_kernel  (T <= 8, decode-sized steps): 1 to 8 warps per output column stream that weight row once with 16-byte loads, two batches of two in
//     flight per lane, one accumulator per activation row — the bandwidth-bound shape of the one-sequence path's GEMV, any size (scalar
//     loads when unaligned);
//   * tile_kernel  (any shape): 64 x 64 x 16 shared-memory tiles, 4 x 4 outputs per thread, fp32 FMAs with fp32 accumulation. This is
//     the body of the all-fp32 mode, and of bf16 products whose shape the tensor-core tiles do not take;
//   * the tcgen05 GEMM of the prefill path (prefill_gemm.cu) for bf16 weights when the caller passes a bf16 scratch for A and the shape
//     fits its TMA boxes; without a scale the GEMM's own epilogue adds the bias and stores (or adds) into C, otherwise bias, alpha and accumulation
//     run as a short epilogue kernel over C.
// In bf16 mode (round_a) the activations are rounded to bf16 as they are loaded, so all three bodies multiply the same operands and
// differ only in summation order.
#include "prefill.cuh"
#include "seq_common.cuh"

namespace sllm {

struct LinArgs {
    const float* A; const void* W; const float* bias; float* C;
    int lda, ldw, ldc, T, N, K, w_dtype, accumulate, round_a;
    float alpha;
    long long a_bs, w_bs, bias_bs, c_bs;
    const int32_t* rows_dev;   // device memory or NULL: rows from *rows_dev on are not computed (tile body and tensor cores)
    const int32_t* w_index;    // rows body, device memory or NULL: product b of the batch uses matrix w_index[b] (W + w_index[b] * w_bs); -1 = no matrix, zeros
    int a_div;                 // rows body: product b reads the activations of batch element b / a_div (0 or 1: its own)
};

constexpr int kRowsMax = 8;
#ifndef SLLM_ROWS_INFLIGHT
#define SLLM_ROWS_INFLIGHT 2
#endif
#ifndef SLLM_ROWS_MINB
#define SLLM_ROWS_MINB 4   // resident CTAs per SM the register budget is cut for (measured: 4 streams 14 % faster than the unconstrained 3; 5 and more spill)
#endif
constexpr int kInFlight = SLLM_ROWS_INFLIGHT;   // 16-byte weight loads per batch and lane; two batches are in flight (measured: 2 x 2 at four resident CTAs beats 1 x 4 by 12 %)

// `wpr` warps (1, 2, 4 or 8) share one output column and cut K among them, so that a matrix with few rows and long rows still fills the
// machine; a lane keeps two batches of 16-byte weight loads in flight (the next batch travels while this one is multiplied). The partial sums of a column meet in shared memory in a fixed order.
template <int WD>
__global__ void __launch_bounds__(256, SLLM_ROWS_MINB) seq_linear_rows_kernel(LinArgs p, int vec, int wpr) {
    __shared__ float part_sum[8][kRowsMax];
    const int b = blockIdx.y;
    const int wb = p.w_index ? p.w_index[b] : b;             // which matrix of W; negative: none (the outputs are zeros)
    const float* A = p.A + (size_t)(p.a_div > 1 ? b / p.a_div : b) * p.a_bs;
    const float* bias = p.bias ? p.bias + (size_t)b * p.bias_bs : nullptr;
    float* C = p.C + (size_t)b * p.c_bs;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * 8 + warp, n = item / wpr, part = item % wpr;
    constexpr int E = WD == SLLM_BF16 ? 8 : 4;                 // weights per 16-byte load
    const int kper = ((p.K + wpr - 1) / wpr + E - 1) / E * E;  // this warp's share of K, a multiple of the load width
    const int k_lo = part * kper, k_hi = min(p.K, k_lo + kper);
    float acc[kRowsMax];
#pragma unroll
    for (int t = 0; t < kRowsMax; ++t) acc[t] = 0.0f;
    if (n < p.N && wb >= 0) {
        if (vec) {
            const uint8_t* w = reinterpret_cast<const uint8_t*>(p.W) + ((size_t)wb * p.w_bs + (size_t)n * p.ldw) * (16 / E);
            constexpr int kStep = kInFlight * 32 * E;
            auto load = [&](uint4 (&u)[kInFlight], int k0) {
#pragma unroll
                for (int j = 0; j < kInFlight; ++j) {
                    const int k = k0 + j * 32 * E;
                    u[j] = k < k_hi ? ldg_stream(w + (size_t)k * (16 / E)) : make_uint4(0u, 0u, 0u, 0u);
                }
            };
            auto consume = [&](const uint4 (&u)[kInFlight], int k0) {
#pragma unroll
                for (int j = 0; j < kInFlight; ++j) {
                    const int k = k0 + j * 32 * E;
                    if (k < k_hi) {
                        float wv[E];
                        if (WD == SLLM_BF16) {
                            wv[0] = bf16_lo(u[j].x); wv[1] = bf16_hi(u[j].x); wv[2] = bf16_lo(u[j].y); wv[3] = bf16_hi(u[j].y);
                            wv[E - 4] = bf16_lo(u[j].z); wv[E - 3] = bf16_hi(u[j].z); wv[E - 2] = bf16_lo(u[j].w); wv[E - 1] = bf16_hi(u[j].w);
                        } else {
                            wv[0] = __uint_as_float(u[j].x); wv[1] = __uint_as_float(u[j].y); wv[2] = __uint_as_float(u[j].z); wv[3] = __uint_as_float(u[j].w);
                        }
#pragma unroll
                        for (int t = 0; t < kRowsMax; ++t) {
                            if (t < p.T) {
                                const float* ar = A + (size_t)t * p.lda + k;
#pragma unroll
                                for (int e = 0; e < E; e += 4) {
                                    const float4 a4 = *reinterpret_cast<const float4*>(ar + e);
                                    const float av[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
                                    for (int i = 0; i < 4; ++i) acc[t] = fmaf(p.round_a ? seq_round_bf16(av[i]) : av[i], wv[e + i], acc[t]);
                                }
                            }
                        }
                    }
                }
            };
            // two batches of loads: the next one is in flight while the current one is multiplied
            int k0 = k_lo + lane * E;
            uint4 cur[kInFlight];
            load(cur, k0);
            for (; k0 < k_hi; k0 += kStep) {
                uint4 nxt[kInFlight];
                load(nxt, k0 + kStep);
                consume(cur, k0);
#pragma unroll
                for (int j = 0; j < kInFlight; ++j) cur[j] = nxt[j];
            }
        } else {
            for (int k = k_lo + lane; k < k_hi; k += 32) {
                const size_t wi = (size_t)wb * p.w_bs + (size_t)n * p.ldw + k;
                const float wv = WD == SLLM_BF16 ? seq_ld(reinterpret_cast<const uint16_t*>(p.W), wi) : reinterpret_cast<const float*>(p.W)[wi];
#pragma unroll
                for (int t = 0; t < kRowsMax; ++t)
                    if (t < p.T) {
                        const float a = A[(size_t)t * p.lda + k];
                        acc[t] = fmaf(p.round_a ? seq_round_bf16(a) : a, wv, acc[t]);
                    }
            }
        }
    }
#pragma unroll
    for (int t = 0; t < kRowsMax; ++t) {
        const float sum = warp_sum(acc[t]);
        if (lane == 0) part_sum[warp][t] = sum;
    }
    __syncthreads();
    if (part == 0 && n < p.N && lane < p.T) {
        float sum = 0.0f;
        for (int j = 0; j < wpr; ++j) sum += part_sum[warp + j][lane];
        const float v = p.alpha * (sum + (bias ? bias[n] : 0.0f));
        float* c = C + (size_t)lane * p.ldc + n;
        *c = p.accumulate ? *c + v : v;
    }
}

constexpr int kTM = 64, kTN = 64, kTK = 16;

template <int WD>
__global__ void __launch_bounds__(256) seq_linear_tile_kernel(LinArgs p) {
    __shared__ float As[kTK][kTM + 4];
    __shared__ float Ws[kTK][kTN + 4];
    const int b = blockIdx.z;
    const float* A = p.A + (size_t)b * p.a_bs;
    const float* bias = p.bias ? p.bias + (size_t)b * p.bias_bs : nullptr;
    float* C = p.C + (size_t)b * p.c_bs;
    const int m0 = blockIdx.y * kTM, n0 = blockIdx.x * kTN;
    if (p.rows_dev && m0 >= *p.rows_dev) return;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int lr = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;   // loader: row lr of the tile, k columns lk .. lk+3
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < p.K; k0 += kTK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = k0 + lk + e;
            float a = 0.0f, w = 0.0f;
            if (k < p.K) {
                if (m0 + lr < p.T) {
                    a = A[(size_t)(m0 + lr) * p.lda + k];
                    if (p.round_a) a = seq_round_bf16(a);
                }
                if (n0 + lr < p.N) {
                    const size_t wi = (size_t)b * p.w_bs + (size_t)(n0 + lr) * p.ldw + k;
                    w = WD == SLLM_BF16 ? seq_ld(reinterpret_cast<const uint16_t*>(p.W), wi) : reinterpret_cast<const float*>(p.W)[wi];
                }
            }
            As[lk + e][lr] = a;
            Ws[lk + e][lr] = w;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kTK; ++k) {
            const float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 wv = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
            const float a4[4] = {av.x, av.y, av.z, av.w}, w4[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a4[i], w4[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= p.T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= p.N) continue;
            const float v = p.alpha * (acc[i][j] + (bias ? bias[n] : 0.0f));
            float* c = C + (size_t)m * p.ldc + n;
            *c = p.accumulate ? *c + v : v;
        }
    }
}

// A (fp32, row stride lda) -> bf16 [T][K] dense
__global__ void seq_to_bf16_kernel(const float* __restrict__ A, int lda, uint16_t* __restrict__ out, int T, int K) {
    const size_t n = (size_t)T * K;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / K, k = i % K;
        out[i] = f32_to_bf16_bits(A[t * lda + k]);
    }
}

// C = alpha * (P + bias) (+ C) where P [T][N] dense holds the plain product
__global__ void seq_linear_epilogue_kernel(const float* __restrict__ P, const float* __restrict__ bias, float* __restrict__ C, int ldc, int T, int N,
                                           float alpha, int accumulate) {
    const size_t n = (size_t)T * N;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / N, j = i % N;
        const float v = alpha * (P[i] + (bias ? bias[j] : 0.0f));
        float* c = C + t * ldc + j;
        *c = accumulate ? *c + v : v;
    }
}

}  // namespace sllm

using namespace sllm;

// the rows body: up to 8 activation rows per product, `batch` products
static int launch_rows(const sllm::LinArgs& p, int batch, cudaStream_t st) {
    using namespace sllm;
    const int e = p.w_dtype == SLLM_BF16 ? 8 : 4;   // elements per 16-byte weight load
    const bool vec = p.K % e == 0 && p.ldw % e == 0 && (p.w_bs % e) == 0 && p.lda % 4 == 0 && (p.a_bs % 4) == 0 && ((uintptr_t)p.W % 16) == 0 &&
                     ((uintptr_t)p.A % 16) == 0;
    int wpr = 1;   // warps per output column: enough CTAs for ~4 per SM, and no warp with less than 256 weights
    while (wpr < 8 && (long long)p.N * batch * wpr / 8 < 4LL * sm_count() && p.K / (2 * wpr) >= 256) wpr *= 2;
    dim3 grid(((long long)p.N * wpr + 7) / 8, batch);
    if (p.w_dtype == SLLM_BF16) seq_linear_rows_kernel<SLLM_BF16><<<grid, 256, 0, st>>>(p, vec, wpr);
    else seq_linear_rows_kernel<SLLM_F32><<<grid, 256, 0, st>>>(p, vec, wpr);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

extern "C" int sllm_seq_linear_indexed(const float* A, int32_t lda, int64_t a_bs, int32_t a_div, const void* W, int32_t w_dtype, int32_t ldw, int64_t w_bs,
                                       const int32_t* w_index, float* C, int32_t ldc, int64_t c_bs, int32_t batch, int32_t N, int32_t K, int32_t round_a,
                                       sllm_stream_t stream) {
    using namespace sllm;
    SLLM_REQUIRE(A && W && C && w_index && batch > 0 && batch <= 65535 && N > 0 && K > 0 && a_div >= 1, SLLM_EINVAL, "seq_linear_indexed: bad argument");
    SLLM_REQUIRE(lda >= K && ldw >= K && ldc >= N, SLLM_EINVAL, "seq_linear_indexed: row strides shorter than the rows");
    SLLM_REQUIRE(w_dtype == SLLM_F32 || w_dtype == SLLM_BF16, SLLM_ENOTSUP, "seq_linear_indexed: fp32 or bf16 weights");
    LinArgs p{A, W, nullptr, C, lda, ldw, ldc, 1, N, K, w_dtype, 0, round_a, 1.0f, a_bs, w_bs, 0, c_bs, nullptr, w_index, a_div};
    return launch_rows(p, batch, as_stream(stream));
}

extern "C" int sllm_seq_linear_on_tensor_cores(int32_t T, int32_t N, int32_t K, int32_t w_dtype, int32_t ldw, int32_t batch, int32_t round_a) {
    // bf16 weights and operands, rows that TMA can address (16-byte multiples) and enough work to fill tiles
    return w_dtype == SLLM_BF16 && batch == 1 && round_a && T >= 64 && N >= 64 && K >= 64 && K % 8 == 0 && ldw == K && N % 4 == 0;
}

extern "C" int sllm_seq_linear(const float* A, int32_t lda, const void* W, int32_t w_dtype, int32_t ldw, const float* bias, float* C, int32_t ldc, int32_t T,
                               int32_t N, int32_t K, float alpha, int32_t accumulate, int32_t round_a, int32_t batch, int64_t a_bs, int64_t w_bs,
                               int64_t bias_bs, int64_t c_bs, void* a16, int32_t a16_ready, const int32_t* rows_dev, sllm_stream_t stream) {
    SLLM_REQUIRE(A && W && C && T > 0 && N > 0 && K > 0 && batch >= 1, SLLM_EINVAL, "seq_linear: bad argument");
    SLLM_REQUIRE(lda >= K && ldw >= K && ldc >= N, SLLM_EINVAL, "seq_linear: row strides shorter than the rows");
    SLLM_REQUIRE(w_dtype == SLLM_F32 || w_dtype == SLLM_BF16, SLLM_ENOTSUP, "seq_linear: fp32 or bf16 weights");
    cudaStream_t st = as_stream(stream);
    LinArgs p{A, W, bias, C, lda, ldw, ldc, T, N, K, w_dtype, accumulate, round_a, alpha, a_bs, w_bs, bias_bs, c_bs, rows_dev, nullptr, 0};
    if (T <= kRowsMax) return launch_rows(p, batch, st);
    // tensor cores: bf16 weights, a dense bf16 copy of A, rows that TMA can address (16-byte multiples) and enough work to fill tiles
    if (a16 && sllm_seq_linear_on_tensor_cores(T, N, K, w_dtype, ldw, batch, round_a) && ((uintptr_t)W % 16) == 0) {
        static PfCache* cache = pf_cache_create();
        if (!a16_ready) {   // else the kernel that produced A has left its bf16 rows in a16 already
            const size_t n = (size_t)T * K;
            seq_to_bf16_kernel<<<(int)std::min<size_t>((n + 255) / 256, (size_t)sm_count() * 8), 256, 0, st>>>(A, lda, reinterpret_cast<uint16_t*>(a16), T, K);
            ++g_launches;
            SLLM_LAUNCH_CHECK();
        }
        PfGemmArgs a{};
        a.A = a16; a.W = W; a.T = T; a.N = N; a.K = K; a.tiled = 0; a.bn = 0; a.n_valid = N; a.rows_dev = rows_dev;
        if (alpha == 1.0f && ((uintptr_t)C % 16) == 0) {
            // nothing but the bias to do after the product: the GEMM's own epilogue adds it and stores (or adds) straight into C
            a.bias = bias;
            a.epilogue = accumulate ? PF_EPI_RESID : PF_EPI_STORE; a.out = C; a.ld_out = ldc;
            return pf_gemm(cache, a, st);
        }
        float* P = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(a16) + (((size_t)T * K * 2 + 255) / 256) * 256);   // product scratch behind the bf16 rows
        a.epilogue = PF_EPI_STORE; a.out = P; a.ld_out = N;
        const int rc = pf_gemm(cache, a, st);
        if (rc != SLLM_OK) return rc;
        const size_t m = (size_t)T * N;
        seq_linear_epilogue_kernel<<<(int)std::min<size_t>((m + 255) / 256, (size_t)sm_count() * 8), 256, 0, st>>>(P, bias, C, ldc, T, N, alpha, accumulate);
        ++g_launches;
        SLLM_LAUNCH_CHECK();
        return SLLM_OK;
    }
    dim3 grid((N + kTN - 1) / kTN, (T + kTM - 1) / kTM, batch);
    if (w_dtype == SLLM_BF16) seq_linear_tile_kernel<SLLM_BF16><<<grid, 256, 0, st>>>(p);
    else seq_linear_tile_kernel<SLLM_F32><<<grid, 256, 0, st>>>(p);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}
