// csrc/seq_prep.cu — what happens between the input projection of an attention mixer and the attention itself, for mixers whose keys are
// not simply rotated: (1) sllm_seq_unit_kv — every query, key and value head divided by its root mean square (no weight), values
// optionally blended with the values an earlier layer computed for the same token, keys and values written to their page pools;
// (2) sllm_seq_latent_kv — latent attention: the low-rank row of a token is RMS-normed (with a weight) and cached together with ONE
// rotated key part that all heads share; the rotated part of every query head moves, rotated, behind that head's absorbed query.
// (3) sllm_seq_normed_rotary_kv — every query and key head RMS-normed with a weight of the head's width, then (partly) rotated by the
// position; the keys go to their pool, the values (which may be the key heads as they were before norm and rotation) to theirs;
// (4) sllm_seq_head_mix — after the attention: the heads' results mixed by a heads x heads matrix.
// All arithmetic is fp32 (angles in double); the pools hold fp32 or bf16.
#include "seq_common.cuh"

namespace sllm {

// grid (T, ceil(items / 4)), 4 warps: warp = one head of q, k or v of one token
template <typename KV>
__global__ void seq_unit_kv_kernel(sllm_seq_batch b, float* __restrict__ q, int ldq, int heads, int dk, const float* __restrict__ k, int ldk, int kv_heads,
                                   const float* __restrict__ v, int ldv, int dv, float eps, int unit, float* __restrict__ v_shared, int share, float lambda,
                                   float q_temp_coef, int q_temp_every, KV* __restrict__ k_pool, KV* __restrict__ v_pool) {
    const int t = blockIdx.x, item = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= heads + 2 * kv_heads) return;
    const int pos = b.tok_pos[t], slot = b.tok_slot[t];
    const int page = b.block_table[(size_t)slot * b.max_pages + pos / b.page_len], in_page = pos % b.page_len;
    if (item < heads) {                                  // a query head, in place
        // query temperature: queries grow with the logarithm of the position, in steps of q_temp_every positions
        const float temp = q_temp_every > 0 ? 1.0f + q_temp_coef * logf((float)((pos + 1) / q_temp_every) + 1.0f) : 1.0f;
        if (!(unit & 1) && temp == 1.0f) return;
        float* row = q + (size_t)t * ldq + (size_t)item * dk;
        float inv = temp;
        if (unit & 1) {
            float ss = 0.0f;
            for (int j = lane; j < dk; j += 32) ss = fmaf(row[j], row[j], ss);
            inv = temp / sqrtf(warp_sum(ss) / (float)dk + eps);
        }
        for (int j = lane; j < dk; j += 32) row[j] *= inv;
    } else if (item < heads + kv_heads) {                // a key head -> pool
        const int g = item - heads;
        const float* row = k + (size_t)t * ldk + (size_t)g * dk;
        float inv = 1.0f;
        if (unit & 2) {
            float ss = 0.0f;
            for (int j = lane; j < dk; j += 32) ss = fmaf(row[j], row[j], ss);
            inv = 1.0f / sqrtf(warp_sum(ss) / (float)dk + eps);
        }
        const size_t dst = seq_pool_row(page, kv_heads, g, b.page_len, in_page, dk);
        for (int j = lane; j < dk; j += 32) seq_st(k_pool, dst + j, row[j] * inv);
    } else {                                             // a value head -> (blend) -> pool
        const int g = item - heads - kv_heads;
        const float* row = v + (size_t)t * ldv + (size_t)g * dv;
        float inv = 1.0f;
        if (unit & 4) {
            float ss = 0.0f;
            for (int j = lane; j < dv; j += 32) ss = fmaf(row[j], row[j], ss);
            inv = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
        }
        const size_t dst = seq_pool_row(page, kv_heads, g, b.page_len, in_page, dv);
        float* sh = v_shared ? v_shared + ((size_t)t * kv_heads + g) * dv : nullptr;
        for (int j = lane; j < dv; j += 32) {
            float val = row[j] * inv;
            if (share == 1) sh[j] = val;
            else if (share == 2) val = (1.0f - lambda) * val + lambda * sh[j];
            seq_st(v_pool, dst + j, val);
        }
    }
}

// one CTA per token
template <typename KV>
__global__ void seq_latent_kv_kernel(sllm_seq_batch b, const float* __restrict__ q, int ldq, int heads, int dn, int dr, const float* __restrict__ low, int ldlow,
                                     int rank, const float* __restrict__ norm_w, float eps, const double* __restrict__ freq, int n_freq, float magnitude,
                                     float* __restrict__ q_out, int ldqo, KV* __restrict__ pool) {
    __shared__ float red[33];
    const int t = blockIdx.x, pos = b.tok_pos[t], slot = b.tok_slot[t];
    const int page = b.block_table[(size_t)slot * b.max_pages + pos / b.page_len], in_page = pos % b.page_len;
    const float* lr = low ? low + (size_t)t * ldlow : nullptr;   // no low-rank row: the layer reads another layer's cache, only its queries turn
    const size_t dst = seq_pool_row(page, 1, 0, b.page_len, in_page, rank + dr);
    const int items = low ? heads + 1 : heads;
    if (low) {
        float ss = 0.0f;
        for (int j = threadIdx.x; j < rank; j += blockDim.x) ss = fmaf(lr[j], lr[j], ss);
        ss = block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
        for (int j = threadIdx.x; j < rank; j += blockDim.x) seq_st(pool, dst + j, (lr[j] * inv) * norm_w[j]);
    }
    // rotated pairs: item 0 .. heads-1 = the query heads, item heads = the shared key part; the first 2 * n_freq dimensions turn
    for (int i = threadIdx.x; i < items * n_freq; i += blockDim.x) {
        const int h = i / n_freq, mi = i % n_freq;
        float sn, cs;
        seq_angle(pos, freq[mi], &sn, &cs);
        sn *= magnitude;
        cs *= magnitude;
        const float* src = h < heads ? q + (size_t)t * ldq + (size_t)h * (dn + dr) + dn : lr + rank;
        const float u = src[2 * mi], w = src[2 * mi + 1];
        const float a = u * cs - w * sn, c = w * cs + u * sn;
        if (h < heads) {
            float* o = q_out + (size_t)t * ldqo + (size_t)h * (rank + dr) + rank;
            o[2 * mi] = a;
            o[2 * mi + 1] = c;
        } else {
            seq_st(pool, dst + rank + 2 * mi, a);
            seq_st(pool, dst + rank + 2 * mi + 1, c);
        }
    }
    const int rest = dr - 2 * n_freq;                     // dimensions of the rotated part beyond the rotary ones pass unchanged
    for (int i = threadIdx.x; i < items * rest; i += blockDim.x) {
        const int h = i / rest, j = 2 * n_freq + i % rest;
        if (h < heads) q_out[(size_t)t * ldqo + (size_t)h * (rank + dr) + rank + j] = q[(size_t)t * ldq + (size_t)h * (dn + dr) + dn + j];
        else seq_st(pool, dst + rank + j, lr[rank + j]);
    }
}

// grid (T, ceil(items / 4)), 4 warps: warp = one query head (normed and rotated in place), one key head (normed, rotated -> pool) or one
// value head (-> pool as it is); the head's row sits in shared memory while its pairs turn
template <typename KV>
__global__ void seq_normed_rotary_kv_kernel(sllm_seq_batch b, float* __restrict__ q, int ldq, int heads, int dk, const float* __restrict__ k, int ldk, int kv_heads,
                                            const float* __restrict__ v, int ldv, int dv, const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                            const double* __restrict__ freq, int n_freq, int layout, KV* __restrict__ k_pool, KV* __restrict__ v_pool) {
    extern __shared__ float nr_sm[];                     // [4][dk]
    const int t = blockIdx.x, item = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= heads + 2 * kv_heads) return;
    const int pos = b.tok_pos[t], slot = b.tok_slot[t];
    const int page = b.block_table[(size_t)slot * b.max_pages + pos / b.page_len], in_page = pos % b.page_len;
    if (item >= heads + kv_heads) {                      // a value head
        const int g = item - heads - kv_heads;
        const float* row = v + (size_t)t * ldv + (size_t)g * dv;
        const size_t dst = seq_pool_row(page, kv_heads, g, b.page_len, in_page, dv);
        for (int j = lane; j < dv; j += 32) seq_st(v_pool, dst + j, row[j]);
        return;
    }
    const bool is_q = item < heads;
    const int g = is_q ? item : item - heads;
    const float* row = is_q ? q + (size_t)t * ldq + (size_t)g * dk : k + (size_t)t * ldk + (size_t)g * dk;
    const float* w = is_q ? q_w : k_w;
    float* s_row = nr_sm + (threadIdx.x >> 5) * dk;
    float ss = 0.0f;
    for (int j = lane; j < dk; j += 32) {
        const float x = row[j];
        s_row[j] = x;
        ss = fmaf(x, x, ss);
    }
    const float inv = w ? 1.0f / sqrtf(warp_sum(ss) / (float)dk + eps) : 1.0f;
    __syncwarp();
    const int half = n_freq;                             // layout 1 pairs dimension i with i + n_freq
    const size_t dst = is_q ? 0 : seq_pool_row(page, kv_heads, g, b.page_len, in_page, dk);
    float* qrow = q + (size_t)t * ldq + (size_t)g * dk;
    auto put = [&](int j, float val) {
        if (is_q) qrow[j] = val;
        else seq_st(k_pool, dst + j, val);
    };
    for (int i = lane; i < n_freq; i += 32) {
        const int ia = layout == 0 ? 2 * i : i, ib = layout == 0 ? 2 * i + 1 : i + half;
        const float u = s_row[ia] * inv * (w ? w[ia] : 1.0f), x = s_row[ib] * inv * (w ? w[ib] : 1.0f);
        float sn, cs;
        seq_angle(pos, freq[i], &sn, &cs);
        put(ia, u * cs - x * sn);
        put(ib, x * cs + u * sn);
    }
    for (int j = 2 * n_freq + lane; j < dk; j += 32) put(j, s_row[j] * inv * (w ? w[j] : 1.0f));
}

// thread = (token, head, column): out[t][h][c] = sum_g mix[h][g] * in[t][(h / group) * heads + g][c], group = heads / kv_heads: `in` holds,
// for every key/value head, the result of EVERY query head's weights on that head's values
__global__ void seq_head_mix_kernel(const float* __restrict__ in, int ldi, const float* __restrict__ mix, int heads, int kv_heads, int dv,
                                    float* __restrict__ out, int ldo, uint16_t* __restrict__ out16, int T) {
    extern __shared__ float hm_sm[];                     // [heads][heads]
    for (int i = threadIdx.x; i < heads * heads; i += blockDim.x) hm_sm[i] = mix[i];
    __syncthreads();
    const int t = blockIdx.x, group = heads / kv_heads;
    const float* row = in + (size_t)t * ldi;
    for (int i = threadIdx.x; i < heads * dv; i += blockDim.x) {
        const int h = i / dv, c = i % dv;
        const float* src = row + (size_t)(h / group) * heads * dv + c;
        float acc = 0.0f;
        for (int g = 0; g < heads; ++g) acc = fmaf(hm_sm[h * heads + g], src[(size_t)g * dv], acc);
        if (out) out[(size_t)t * ldo + i] = acc;
        if (out16) out16[(size_t)t * heads * dv + i] = f32_to_bf16_bits(acc);
    }
}

}  // namespace sllm

using namespace sllm;

extern "C" {

int sllm_seq_unit_kv(const sllm_seq_batch* b, float* q, int32_t ldq, int32_t heads, int32_t dk, const float* k, int32_t ldk, int32_t kv_heads,
                     const float* v, int32_t ldv, int32_t dv, float eps, int32_t unit, float* v_shared, int32_t share, float lambda, void* k_pool,
                     void* v_pool, int32_t kv_dtype, float q_temp_coef, int32_t q_temp_every, sllm_stream_t stream) {
    SLLM_REQUIRE(b && b->T > 0 && b->tok_slot && b->tok_pos && b->block_table, SLLM_EINVAL, "seq_unit_kv: incomplete batch description");
    SLLM_REQUIRE(q && k && v && k_pool && v_pool && heads > 0 && kv_heads > 0 && dk > 0 && dv > 0, SLLM_EINVAL, "seq_unit_kv: bad argument");
    SLLM_REQUIRE(share >= 0 && share <= 2 && (share == 0 || v_shared), SLLM_EINVAL, "seq_unit_kv: share 0 (none), 1 (write) or 2 (blend) with a buffer");
    SLLM_REQUIRE(kv_dtype == SLLM_F32 || kv_dtype == SLLM_BF16, SLLM_ENOTSUP, "seq_unit_kv: fp32 or bf16 pools");
    const dim3 grid(b->T, (heads + 2 * kv_heads + 3) / 4);
    if (kv_dtype == SLLM_F32)
        seq_unit_kv_kernel<float><<<grid, 128, 0, as_stream(stream)>>>(*b, q, ldq, heads, dk, k, ldk, kv_heads, v, ldv, dv, eps, unit, v_shared, share, lambda,
                                                                       q_temp_coef, q_temp_every, (float*)k_pool, (float*)v_pool);
    else
        seq_unit_kv_kernel<uint16_t><<<grid, 128, 0, as_stream(stream)>>>(*b, q, ldq, heads, dk, k, ldk, kv_heads, v, ldv, dv, eps, unit, v_shared, share, lambda,
                                                                          q_temp_coef, q_temp_every, (uint16_t*)k_pool, (uint16_t*)v_pool);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_latent_kv(const sllm_seq_batch* b, const float* q, int32_t ldq, int32_t heads, int32_t dn, int32_t dr, const float* low, int32_t ldlow,
                       int32_t rank, const float* norm_w, float eps, const double* freq, int32_t n_freq, float* q_out, int32_t ldqo, void* pool,
                       int32_t kv_dtype, float magnitude, sllm_stream_t stream) {
    SLLM_REQUIRE(b && b->T > 0 && b->tok_slot && b->tok_pos && b->block_table, SLLM_EINVAL, "seq_latent_kv: incomplete batch description");
    SLLM_REQUIRE(q && q_out && (!low || (norm_w && pool)) && heads > 0 && dn >= 0 && dr >= 0 && rank > 0, SLLM_EINVAL, "seq_latent_kv: bad argument");
    SLLM_REQUIRE(n_freq >= 0 && 2 * n_freq <= dr && (n_freq == 0 || freq), SLLM_EINVAL, "seq_latent_kv: %d rotary pairs do not fit %d dimensions", n_freq, dr);
    SLLM_REQUIRE(kv_dtype == SLLM_F32 || kv_dtype == SLLM_BF16, SLLM_ENOTSUP, "seq_latent_kv: fp32 or bf16 pools");
    const int threads = rank >= 512 ? 256 : 128;
    if (kv_dtype == SLLM_F32)
        seq_latent_kv_kernel<float><<<b->T, threads, 0, as_stream(stream)>>>(*b, q, ldq, heads, dn, dr, low, ldlow, rank, norm_w, eps, freq, n_freq, magnitude, q_out, ldqo,
                                                                             (float*)pool);
    else
        seq_latent_kv_kernel<uint16_t><<<b->T, threads, 0, as_stream(stream)>>>(*b, q, ldq, heads, dn, dr, low, ldlow, rank, norm_w, eps, freq, n_freq, magnitude, q_out,
                                                                                ldqo, (uint16_t*)pool);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_normed_rotary_kv(const sllm_seq_batch* b, float* q, int32_t ldq, int32_t heads, int32_t dk, const float* k, int32_t ldk, int32_t kv_heads,
                              const float* v, int32_t ldv, int32_t dv, const float* q_norm_w, const float* k_norm_w, float eps, const double* freq,
                              int32_t n_freq, int32_t layout, void* k_pool, void* v_pool, int32_t kv_dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(b && b->T > 0 && b->tok_slot && b->tok_pos && b->block_table, SLLM_EINVAL, "seq_normed_rotary_kv: incomplete batch description");
    SLLM_REQUIRE(q && k && v && k_pool && v_pool && heads > 0 && kv_heads > 0 && dk > 0 && dv > 0, SLLM_EINVAL, "seq_normed_rotary_kv: bad argument");
    SLLM_REQUIRE(n_freq >= 0 && 2 * n_freq <= dk && (n_freq == 0 || freq), SLLM_EINVAL, "seq_normed_rotary_kv: %d rotary pairs do not fit %d dimensions", n_freq, dk);
    SLLM_REQUIRE(layout == 0 || layout == 1, SLLM_EINVAL, "seq_normed_rotary_kv: layout 0 (interleaved) or 1 (halves)");
    SLLM_REQUIRE(kv_dtype == SLLM_F32 || kv_dtype == SLLM_BF16, SLLM_ENOTSUP, "seq_normed_rotary_kv: fp32 or bf16 pools");
    SLLM_REQUIRE(dk <= 8192, SLLM_ENOTSUP, "seq_normed_rotary_kv: heads of %d", dk);
    const dim3 grid(b->T, (heads + 2 * kv_heads + 3) / 4);
    const size_t smem = 4 * (size_t)dk * sizeof(float);
    if (kv_dtype == SLLM_F32)
        seq_normed_rotary_kv_kernel<float><<<grid, 128, smem, as_stream(stream)>>>(*b, q, ldq, heads, dk, k, ldk, kv_heads, v, ldv, dv, q_norm_w, k_norm_w, eps, freq,
                                                                                 n_freq, layout, (float*)k_pool, (float*)v_pool);
    else
        seq_normed_rotary_kv_kernel<uint16_t><<<grid, 128, smem, as_stream(stream)>>>(*b, q, ldq, heads, dk, k, ldk, kv_heads, v, ldv, dv, q_norm_w, k_norm_w, eps, freq,
                                                                                    n_freq, layout, (uint16_t*)k_pool, (uint16_t*)v_pool);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_head_mix(const float* in, int32_t ldi, const float* mix, int32_t heads, int32_t kv_heads, int32_t dv, float* out, int32_t ldo, void* out16,
                      int32_t T, sllm_stream_t stream) {
    SLLM_REQUIRE(in && mix && (out || out16) && T > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dv > 0, SLLM_EINVAL, "seq_head_mix: bad argument");
    SLLM_REQUIRE(heads <= 96, SLLM_ENOTSUP, "seq_head_mix: %d heads beyond 96", heads);
    const int threads = T >= 64 ? 256 : std::min(1024, std::max(128, (heads * dv + 31) / 32 * 32));
    seq_head_mix_kernel<<<T, threads, (size_t)heads * heads * sizeof(float), as_stream(stream)>>>(in, ldi, mix, heads, kv_heads, dv, out, ldo, (uint16_t*)out16, T);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

}  // extern "C"
