// csrc/seq_attn.cu — softmax attention of the ragged token batch over a paged cache, for portions of prompts and single decoded tokens in
// one launch: rotary positions on q / k (partial, interleaved or half-split pairs, scaled frequencies arrive as a table), values rotated by
// their own position before they are cached and turned back by the query's position afterwards, key and value heads of different widths,
// grouped query heads, a sigmoid gate per head. Scores, softmax weights and the weighted sum are fp32 whatever the cache holds.
// Options of a launch (sllm_seq_attn_opts): a sliding window that keeps the first positions of a sequence visible (key tiles that no query
// of the CTA can see are never loaded), scores capped by cap * tanh(score / cap), a charge per position of distance with one slope per
// head, values that are the leading columns of the key rows (one pool holds both: latent attention in its absorbed form), and in the
// merge one more term exp(sink) per head in the softmax's denominator.
//
// seq_attention_kernel: CTA = (tile of up to 32 consecutive queries of one segment, query head, share of the key tiles), 8 warps x 4
// queries. A tile of 32 keys and values of the head's kv head is staged in shared memory (fp32); a lane owns one key for the scores
// (16-byte shared loads, rows padded by 4 floats: conflict-free) and dv/32 output columns for the weighted sum; online softmax per query
// with warp reductions. The key tiles are dealt to `nsplit` CTAs in turn (long contexts with few queries: decode), every CTA leaves
// (max, sum, unnormalised output) and seq_attention_finish_kernel merges them.
#include <climits>

#include "seq_common.cuh"

namespace sllm {

extern int g_tune_seq_attn_mma;   // runtime.cu: 1 (default) = tensor-core attention body where it applies, 0 = always the fp32 body

constexpr int kBQ = 32, kBK = 32, kQW = 4;   // queries per CTA, keys per tile, queries per warp

struct AttnArgs {
    sllm_seq_batch b;
    const float* q; int ldq, heads, kv_heads, dk, dv; float scale;
    const void *k_pool, *v_pool;
    int nsplit; float* ws;
    int by_head;   // fp32 body, steps of single tokens: a CTA's "queries" are the query heads of ONE kv head at one token (they share its tiles)
    int window, keep_first;   // query i sees key j <= i when i - j < window or j < keep_first (window INT_MAX = everything before it)
    float softcap;            // > 0: score <- softcap * tanh(score / softcap)
    const float* slopes;      // [heads] or NULL: score <- score - slopes[h] * (i - j)
    int v_in_k;               // values = the first dv columns of the key rows (v_pool unused)
    const float* logdist;     // [2][heads] or NULL: score <- score - r1[h] * ln(1 + r2[h] * (i - j)), r1 = row 0, r2 = row 1
    // Every query head's weights on every key/value head's values: `heads` then counts kv_heads * q_heads results, result u = (value
    // head u / q_heads, query head u % q_heads); the query head reads the KEYS of its own key/value head as always. Otherwise q_heads = heads.
    int q_heads, cross;
};

// The key tiles a CTA whose queries lie at positions first .. last has to visit: the tiles of the kept first positions, then the tiles
// from the one that holds the oldest key inside the first query's window up to the last query's own tile.
struct TileList {
    int n_keep, lo, n;
    __device__ __forceinline__ TileList(int first, int last, int window, int keep_first, int tile) {
        const int nkt = last / tile + 1;
        const int oldest = window > first ? 0 : first - window + 1;
        lo = oldest / tile;
        n_keep = min(lo, (min(keep_first, oldest) + tile - 1) / tile);
        n = n_keep + nkt - lo;
    }
    __device__ __forceinline__ int tile_of(int idx) const { return idx < n_keep ? idx : lo + idx - n_keep; }
};

__device__ __forceinline__ float seq_score(float dot, float scale, float softcap, float slope, float r1, float r2, int qpos, int key) {
    float sc = dot * scale;
    if (softcap > 0.0f) sc = softcap * tanhf(sc / softcap);
    sc -= slope * (float)(qpos - key);
    if (r1 != 0.0f) sc -= r1 * log1pf(r2 * (float)(qpos - key));
    return sc;
}
__device__ __forceinline__ bool seq_sees(int qpos, int key, int window, int keep_first) {
    return key <= qpos && (qpos - key < window || key < keep_first);
}

template <typename KV, int kMaxDvChunks>   // dv <= 32 * kMaxDvChunks
__global__ void __launch_bounds__(256) seq_attention_kernel(AttnArgs p) {
    extern __shared__ __align__(16) float sm[];
    const int dk = p.dk, dv = p.dv, dkp = ((dk + 3) & ~3) + 4;   // padded row of q / k in floats
    float* sq = sm;                      // [kBQ][dkp]
    float* sk = sq + kBQ * dkp;          // [kBK][dkp]
    float* sv = p.v_in_k ? sk : sk + kBK * dkp;   // [kBK][dv], or the key rows themselves
    const int ldsv = p.v_in_k ? dkp : dv;
    const sllm_seq_batch& b = p.b;
    const int qt = blockIdx.x, split = blockIdx.z;
    const int seg = b.qt_seg[qt], off = b.qt_off[qt];
    const int group = p.q_heads / p.kv_heads;
    const int t0 = b.seg_start[seg] + off, pos0 = b.seg_pos0[seg] + off, slot = b.seg_slot[seg];
    // row r of the CTA's query tile is (token t0 + r, head blockIdx.y), or with by_head (token t0, query head r of the CTA's key head)
    const int nq = p.by_head ? group : min(kBQ, b.seg_len[seg] - off);
    // key head and value head; with cross values and by_head the grid's y counts (value head, key head) pairs
    const int g = p.by_head ? (int)blockIdx.y % p.kv_heads : ((int)blockIdx.y % p.q_heads) / group;
    const int gv = p.cross ? (p.by_head ? (int)blockIdx.y / p.kv_heads : (int)blockIdx.y / p.q_heads) : g;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const KV* kp = reinterpret_cast<const KV*>(p.k_pool);
    const KV* vp = reinterpret_cast<const KV*>(p.v_pool);
    auto row_token = [&](int r) { return p.by_head ? t0 : t0 + r; };
    auto row_qhead = [&](int r) { return p.by_head ? g * group + r : (int)blockIdx.y % p.q_heads; };      // the query head behind row r
    auto row_head = [&](int r) { return p.by_head ? (p.cross ? gv * p.q_heads : 0) + g * group + r : (int)blockIdx.y; };   // the result's number
    auto row_pos = [&](int r) { return p.by_head ? pos0 : pos0 + r; };

    for (int i = threadIdx.x; i < kBQ * dkp; i += blockDim.x) {
        const int r = i / dkp, c = i % dkp;
        sq[i] = (r < nq && c < dk) ? p.q[(size_t)row_token(r) * p.ldq + (size_t)row_qhead(r) * dk + c] : 0.0f;
    }
    float m[kQW], l[kQW], acc[kQW][kMaxDvChunks];
#pragma unroll
    for (int i = 0; i < kQW; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.0f;
#pragma unroll
        for (int c = 0; c < kMaxDvChunks; ++c) acc[i][c] = 0.0f;
    }
    float slope[kQW];
#pragma unroll
    for (int i = 0; i < kQW; ++i) slope[i] = (p.slopes && warp * kQW + i < nq) ? p.slopes[row_qhead(warp * kQW + i)] : 0.0f;
    float r1[kQW], r2[kQW];
#pragma unroll
    for (int i = 0; i < kQW; ++i) {
        const bool has = p.logdist && warp * kQW + i < nq;
        r1[i] = has ? p.logdist[row_qhead(warp * kQW + i)] : 0.0f;
        r2[i] = has ? p.logdist[p.q_heads + row_qhead(warp * kQW + i)] : 0.0f;
    }
    const int last_pos = row_pos(nq - 1);
    const TileList tiles(row_pos(0), last_pos, p.window, p.keep_first, kBK);
    for (int idx = split; idx < tiles.n; idx += p.nsplit) {
        const int j0 = tiles.tile_of(idx) * kBK;
        const int page = b.block_table[(size_t)slot * b.max_pages + j0 / b.page_len], in_page = j0 % b.page_len;
        const int valid = min(kBK, last_pos + 1 - j0);   // keys of this tile that exist
        __syncthreads();
        const size_t krow = seq_pool_row(page, p.kv_heads, g, b.page_len, in_page, dk), vrow = seq_pool_row(page, p.kv_heads, gv, b.page_len, in_page, dv);
        constexpr int E = 16 / sizeof(KV);   // elements per 16-byte load
        if (dk % E == 0 && (dv % E == 0 || p.v_in_k)) {
            // the tile's rows are consecutive in the pool: 16-byte loads, rows beyond `valid` zero-filled (dk is a multiple of 4 here, so the
            // padding columns of a row are never read)
            const int kgroups = dk / E, vgroups = dv / E;
            for (int i = threadIdx.x; i < kBK * kgroups; i += blockDim.x) {
                const int r = i / kgroups, c = (i % kgroups) * E;
                float vals[E];
                seq_ld16(kp + krow + (size_t)r * dk + c, r < valid, vals);
#pragma unroll
                for (int e = 0; e < E; e += 4) *reinterpret_cast<float4*>(sk + r * dkp + c + e) = make_float4(vals[e], vals[e + 1], vals[e + 2], vals[e + 3]);
            }
            for (int i = threadIdx.x; i < (p.v_in_k ? 0 : kBK * vgroups); i += blockDim.x) {
                const int r = i / vgroups;
                float vals[E];
                seq_ld16(vp + vrow + (size_t)i * E, r < valid, vals);
#pragma unroll
                for (int e = 0; e < E; e += 4) *reinterpret_cast<float4*>(sv + (size_t)i * E + e) = make_float4(vals[e], vals[e + 1], vals[e + 2], vals[e + 3]);
            }
        } else {
            for (int i = threadIdx.x; i < kBK * dkp; i += blockDim.x) {
                const int r = i / dkp, c = i % dkp;
                sk[i] = (r < valid && c < dk) ? seq_ld(kp, krow + (size_t)r * dk + c) : 0.0f;
            }
            for (int i = threadIdx.x; i < (p.v_in_k ? 0 : kBK * dv); i += blockDim.x) {
                const int r = i / dv;
                sv[i] = r < valid ? seq_ld(vp, vrow + i) : 0.0f;
            }
        }
        __syncthreads();
        // scores: lane = key j0 + lane, four queries of this warp
        float s[kQW] = {0.0f, 0.0f, 0.0f, 0.0f};
        const float* krowp = sk + lane * dkp;
        for (int c = 0; c < dk; c += 4) {
            const float4 kv = *reinterpret_cast<const float4*>(krowp + c);
#pragma unroll
            for (int i = 0; i < kQW; ++i) {
                const float4 qv = *reinterpret_cast<const float4*>(sq + (warp * kQW + i) * dkp + c);
                s[i] = fmaf(qv.x, kv.x, s[i]);
                s[i] = fmaf(qv.y, kv.y, s[i]);
                s[i] = fmaf(qv.z, kv.z, s[i]);
                s[i] = fmaf(qv.w, kv.w, s[i]);
            }
        }
        float pw[kQW];
#pragma unroll
        for (int i = 0; i < kQW; ++i) {
            const int qi = warp * kQW + i;
            const bool see = qi < nq && seq_sees(row_pos(qi), j0 + lane, p.window, p.keep_first);
            const float sc = see ? seq_score(s[i], p.scale, p.softcap, slope[i], r1[i], r2[i], row_pos(qi), j0 + lane) : -INFINITY;
            const float mn = fmaxf(m[i], warp_max(sc));
            const float corr = (mn == -INFINITY) ? 1.0f : expf(m[i] - mn);   // m = -inf: nothing accumulated yet, expf(-inf) = 0 is right too
            pw[i] = see ? expf(sc - mn) : 0.0f;
            l[i] = l[i] * corr + warp_sum(pw[i]);
            m[i] = mn;
#pragma unroll
            for (int c = 0; c < kMaxDvChunks; ++c) acc[i][c] *= corr;
        }
        for (int jj = 0; jj < valid; ++jj) {
            float pj[kQW];
#pragma unroll
            for (int i = 0; i < kQW; ++i) pj[i] = __shfl_sync(0xffffffffu, pw[i], jj);
#pragma unroll
            for (int c = 0; c < kMaxDvChunks; ++c) {
                if (c * 32 < dv) {
                    const int col = c * 32 + lane;
                    const float vv = col < dv ? sv[jj * ldsv + col] : 0.0f;
#pragma unroll
                    for (int i = 0; i < kQW; ++i) acc[i][c] = fmaf(pj[i], vv, acc[i][c]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < kQW; ++i) {
        const int qi = warp * kQW + i;
        if (qi >= nq) continue;
        float* rec = p.ws + (((size_t)row_token(qi) * p.heads + row_head(qi)) * p.nsplit + split) * (dv + 2);
        if (lane == 0) {
            rec[0] = m[i];
            rec[1] = l[i];
        }
#pragma unroll
        for (int c = 0; c < kMaxDvChunks; ++c) {
            const int col = c * 32 + lane;
            if (col < dv) rec[2 + col] = acc[i][c];
        }
    }
}


// ---- tensor-core body for bf16 pools (the bf16 mode) ------------------------------------------------------------------------------------
// CTA = (tile of up to 32 queries, head, share of the key tiles), two warps of 16 queries each. Scores = Q K^T with mma.sync m16n8k16
// (q rounded to bf16 as it is loaded, keys as cached, fp32 accumulation); the softmax runs on the accumulator fragments in fp32 (row
// maxima across the four lanes of a quad); the weights enter the second product as TWO bf16 terms (p = hi + lo, |p - hi - lo| < 2^-17 p),
// so that P V keeps the weights to fp32 working accuracy while the values come from the cache as they are. A fragment of S maps
// register-for-register onto an A fragment of P. K and V tiles are staged row-major as cached (rows padded by 16 bytes: conflict-free
// fragment loads; V's B fragments come out of ldmatrix.trans) by cp.async into two stages, the next tile in flight while this one is
// multiplied; four warps = two query heads of one kv head share a staged tile when the group size is even. Writes the same (max, sum, unnormalised output) records as the fp32 body.
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) { return (uint32_t)f32_to_bf16_bits(lo) | ((uint32_t)f32_to_bf16_bits(hi) << 16); }
// p = hi + lo with both terms bf16: hi = round(p), lo = round(p - hi)
__device__ __forceinline__ void split_bf16(float p0, float p1, uint32_t* hi, uint32_t* lo) {
    const uint16_t h0 = f32_to_bf16_bits(p0), h1 = f32_to_bf16_bits(p1);
    *hi = (uint32_t)h0 | ((uint32_t)h1 << 16);
    *lo = pack_bf16(p0 - __uint_as_float((uint32_t)h0 << 16), p1 - __uint_as_float((uint32_t)h1 << 16));
}


__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// 16 bytes global -> shared without passing through registers; bytes = 0 writes zeros and reads nothing
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// kExact: dk = 16 * kMmaDkSteps and dv = 8 * kMmaDvTiles exactly — the loops over fragments then have no run-time bounds, and the compiler
// is free to interleave independent products (the common head widths are instantiated so).
template <int kMmaDkSteps, int kMmaDvTiles, bool kExact>   // dk <= 16 * kMmaDkSteps (multiple of 16), dv <= 8 * kMmaDvTiles (multiple of 8)
__global__ void __launch_bounds__(128) seq_attention_mma_kernel(AttnArgs p) {
    extern __shared__ __align__(16) uint16_t smh[];
    const int dk = p.dk, dv = p.dv, ldk = dk + 8, ldvr = p.v_in_k ? ldk : dv + 8;
    const int stage_elems = p.v_in_k ? kBK * ldk : kBK * (ldk + ldvr);   // one stage: K rows [kBK][ldk], then V rows [kBK][ldvr] unless the key rows hold them
    const sllm_seq_batch& b = p.b;
    const int qt = blockIdx.x, split = blockIdx.z;
    const int seg = b.qt_seg[qt], off = b.qt_off[qt];
    const int nq = min(kBQ, b.seg_len[seg] - off), t0 = b.seg_start[seg] + off, pos0 = b.seg_pos0[seg] + off, slot = b.seg_slot[seg];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    // two warps (16 queries each) per head; a CTA of four warps serves two query heads of the same kv head from one staged tile
    const int hpc = blockDim.x >> 6, h = blockIdx.y * hpc + (warp >> 1), wq = warp & 1;
    const int hq = h % p.q_heads;                      // the query head behind result h
    const int gkv = hq / (p.q_heads / p.kv_heads);
    const int gvv = p.cross ? h / p.q_heads : gkv;     // value head
    const int dks = kExact ? kMmaDkSteps : dk / 16, dvt = kExact ? kMmaDvTiles : dv / 8;
    const uint16_t* kp = reinterpret_cast<const uint16_t*>(p.k_pool);
    const uint16_t* vp = reinterpret_cast<const uint16_t*>(p.v_pool);
    const int r0 = wq * 16 + g, r1 = r0 + 8;           // this thread's two query rows inside the tile
    const bool ok0 = r0 < nq, ok1 = r1 < nq;
    const int last_pos = pos0 + nq - 1;
    const TileList tiles(pos0, last_pos, p.window, p.keep_first, kBK);
    const float slope = p.slopes ? p.slopes[hq] : 0.0f;
    const float ld1 = p.logdist ? p.logdist[hq] : 0.0f, ld2 = p.logdist ? p.logdist[p.q_heads + hq] : 0.0f;

    // tile kt of the sequence -> stage `st` of shared memory, asynchronously (rows beyond the last position are zero-filled)
    auto issue = [&](int kt, int st) {
        const int j0 = kt * kBK;
        const int page = b.block_table[(size_t)slot * b.max_pages + j0 / b.page_len], in_page = j0 % b.page_len;
        const int valid = min(kBK, last_pos + 1 - j0);
        const uint16_t* ksrc = kp + seq_pool_row(page, p.kv_heads, gkv, b.page_len, in_page, dk);
        const uint16_t* vsrc = vp + seq_pool_row(page, p.kv_heads, gvv, b.page_len, in_page, dv);
        uint16_t* sK = smh + st * stage_elems;
        uint16_t* sV = sK + kBK * ldk;
        for (int i = threadIdx.x; i < kBK * (dk / 8); i += blockDim.x) {
            const int r = i / (dk / 8), cc = (i % (dk / 8)) * 8;
            cp_async16(sK + r * ldk + cc, r < valid ? ksrc + (size_t)r * dk + cc : ksrc, r < valid ? 16 : 0);
        }
        for (int i = threadIdx.x; i < (p.v_in_k ? 0 : kBK * (dv / 8)); i += blockDim.x) {
            const int r = i / (dv / 8), cc = (i % (dv / 8)) * 8;
            cp_async16(sV + r * ldvr + cc, r < valid ? vsrc + (size_t)r * dv + cc : vsrc, r < valid ? 16 : 0);
        }
        cp_async_commit();
    };
    if (split < tiles.n) issue(tiles.tile_of(split), 0);

    uint32_t qf[kMmaDkSteps][4];
#pragma unroll
    for (int ks = 0; ks < kMmaDkSteps; ++ks) {
        if (ks < dks) {
            const float* q0 = p.q + (size_t)(t0 + r0) * p.ldq + (size_t)hq * dk + ks * 16 + 2 * c;
            const float* q1 = p.q + (size_t)(t0 + r1) * p.ldq + (size_t)hq * dk + ks * 16 + 2 * c;
            qf[ks][0] = ok0 ? pack_bf16(q0[0], q0[1]) : 0u;
            qf[ks][1] = ok1 ? pack_bf16(q1[0], q1[1]) : 0u;
            qf[ks][2] = ok0 ? pack_bf16(q0[8], q0[9]) : 0u;
            qf[ks][3] = ok1 ? pack_bf16(q1[8], q1[9]) : 0u;
        } else {
            qf[ks][0] = qf[ks][1] = qf[ks][2] = qf[ks][3] = 0u;
        }
    }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;   // l: this thread's share of the row sums (added over the quad at the end)
    float o[kMmaDvTiles][4];
#pragma unroll
    for (int nt = 0; nt < kMmaDvTiles; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f;
    const int warp_last = pos0 + min(nq - 1, wq * 16 + 15);
    const bool warp_live = wq * 16 < nq;
    int it = 0;
    for (int idx = split; idx < tiles.n; idx += p.nsplit, ++it) {
        const int j0 = tiles.tile_of(idx) * kBK, st = it & 1;
        if (idx + p.nsplit < tiles.n) {     // the next tile travels while this one is multiplied
            issue(tiles.tile_of(idx + p.nsplit), st ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint16_t* sK = smh + st * stage_elems;
        const uint16_t* sV = p.v_in_k ? sK : sK + kBK * ldk;
        if (warp_live && j0 <= warp_last) {
        float s[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < kMmaDkSteps; ++ks) {
            if (ks < dks) {
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const uint16_t* kr = sK + (nt * 8 + g) * ldk + ks * 16 + 2 * c;
                    mma_bf16_16816(s[nt], qf[ks], *reinterpret_cast<const uint32_t*>(kr), *reinterpret_cast<const uint32_t*>(kr + 8));
                }
            }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = j0 + nt * 8 + 2 * c + (e & 1);
                const int qpos = pos0 + ((e < 2) ? r0 : r1);
                const bool see = ((e < 2) ? ok0 : ok1) && seq_sees(qpos, key, p.window, p.keep_first);
                s[nt][e] = see ? seq_score(s[nt][e], p.scale, p.softcap, slope, ld1, ld2, qpos, key) : -INFINITY;
            }
            mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
            mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float corr0 = (mn0 == -INFINITY) ? 1.0f : expf(m0 - mn0), corr1 = (mn1 == -INFINITY) ? 1.0f : expf(m1 - mn1);
        m0 = mn0;
        m1 = mn1;
        l0 *= corr0;
        l1 *= corr1;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            s[nt][0] = s[nt][0] == -INFINITY ? 0.0f : expf(s[nt][0] - mn0);
            s[nt][1] = s[nt][1] == -INFINITY ? 0.0f : expf(s[nt][1] - mn0);
            s[nt][2] = s[nt][2] == -INFINITY ? 0.0f : expf(s[nt][2] - mn1);
            s[nt][3] = s[nt][3] == -INFINITY ? 0.0f : expf(s[nt][3] - mn1);
            l0 += s[nt][0] + s[nt][1];
            l1 += s[nt][2] + s[nt][3];
        }
#pragma unroll
        for (int nt = 0; nt < kMmaDvTiles; ++nt) {
            o[nt][0] *= corr0;
            o[nt][1] *= corr0;
            o[nt][2] *= corr1;
            o[nt][3] *= corr1;
        }
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {           // 32 keys = two k-steps of 16; S tiles 2ks and 2ks+1 are the A fragment's halves
            uint32_t ah[4], al[4];
            split_bf16(s[2 * ks][0], s[2 * ks][1], &ah[0], &al[0]);
            split_bf16(s[2 * ks][2], s[2 * ks][3], &ah[1], &al[1]);
            split_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1], &ah[2], &al[2]);
            split_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3], &ah[3], &al[3]);
            const uint32_t vrow = smem_u32(sV + (ks * 16 + (lane & 15)) * ldvr);   // row-major values: ldmatrix.trans hands out the B fragments
#pragma unroll
            for (int n0 = 0; n0 < kMmaDvTiles; n0 += 4) {   // four value tiles at a time: no product waits for the one issued just before it
                uint32_t b0[4], b1[4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (n0 + i < kMmaDvTiles && n0 + i < dvt)
                        asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0[i]), "=r"(b1[i]) : "r"(vrow + (n0 + i) * 16));
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (n0 + i < kMmaDvTiles && n0 + i < dvt) mma_bf16_16816(o[n0 + i], ah, b0[i], b1[i]);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (n0 + i < kMmaDvTiles && n0 + i < dvt) mma_bf16_16816(o[n0 + i], al, b0[i], b1[i]);
            }
        }
        }
        __syncthreads();   // everyone is done with this stage before the tile after next lands in it
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = half ? r1 : r0;
        if (r >= nq) continue;
        float* rec = p.ws + (((size_t)(t0 + r) * p.heads + h) * p.nsplit + split) * (dv + 2);
        if (c == 0) {
            rec[0] = half ? m1 : m0;
            rec[1] = half ? l1 : l0;
        }
#pragma unroll
        for (int nt = 0; nt < kMmaDvTiles; ++nt) {
            if (nt < dvt) {
                rec[2 + nt * 8 + 2 * c] = o[nt][2 * half];
                rec[2 + nt * 8 + 2 * c + 1] = o[nt][2 * half + 1];
            }
        }
    }
}

// one CTA per (token, head), one thread per value column: merge the shares, normalise, turn back by the token's position, gate.
// Warp 0 turns the shares' (max, sum) into one weight per share (exp(m_s - max) / total, zero for a share that saw no key); every thread
// then adds its column over the shares with coalesced loads; pairs meet through shared memory for the rotation.
__global__ void seq_attention_finish_kernel(sllm_seq_batch b, const float* __restrict__ ws, int nsplit, int heads, int dv, const double* __restrict__ vfreq,
                                            int layout, const float* __restrict__ gate, int ldg, const float* __restrict__ sink, float* __restrict__ out, int ldo) {
    extern __shared__ float fsm[];
    float* s_w = fsm;            // [nsplit]
    float* s_o = fsm + nsplit;   // [dv]
    const int t = blockIdx.x / heads, h = blockIdx.x % heads, lane = threadIdx.x & 31;
    const float* rec = ws + ((size_t)t * heads + h) * nsplit * (dv + 2);
    if (threadIdx.x < 32) {
        float mx = -INFINITY;
        for (int s = lane; s < nsplit; s += 32) mx = fmaxf(mx, rec[(size_t)s * (dv + 2)]);
        mx = warp_max(mx);
        if (sink) mx = fmaxf(mx, sink[h]);   // the sink is one more term of the denominator: no key, no value
        float den = 0.0f;
        for (int s = lane; s < nsplit; s += 32) {
            const float ms = rec[(size_t)s * (dv + 2)];
            const float w = ms == -INFINITY ? 0.0f : expf(ms - mx);
            s_w[s] = w;
            den = fmaf(rec[(size_t)s * (dv + 2) + 1], w, den);
        }
        den = warp_sum(den);
        if (sink) den += expf(sink[h] - mx);
        const float inv_den = 1.0f / den;
        for (int s = lane; s < nsplit; s += 32) s_w[s] *= inv_den;
    }
    __syncthreads();
    const int col = threadIdx.x;
    if (col < dv) {
        float v = 0.0f;
#pragma unroll 4
        for (int s = 0; s < nsplit; ++s) v = fmaf(s_w[s], rec[(size_t)s * (dv + 2) + 2 + col], v);
        s_o[col] = v;
    }
    __syncthreads();
    const float gv = gate ? seq_sigmoid(gate[(size_t)t * ldg + h]) : 1.0f;
    float* orow = out + (size_t)t * ldo + (size_t)h * dv;
    if (!vfreq) {
        if (col < dv) orow[col] = s_o[col] * gv;
        return;
    }
    const int half = dv / 2, mi = threadIdx.x;
    if (mi < half) {
        const int ia = layout == 0 ? 2 * mi : mi, ib = layout == 0 ? 2 * mi + 1 : mi + half;
        const float u = s_o[ia], v = s_o[ib];
        float sn, cs;
        seq_angle(b.tok_pos[t], vfreq[mi], &sn, &cs);
        orow[ia] = (u * cs + v * sn) * gv;    // rotation by the negative angle
        orow[ib] = (v * cs - u * sn) * gv;
    }
}

// one CTA per token: rotate q in place, rotate k and v and store them into the pools
template <typename KV>
__global__ void seq_rotary_kv_kernel(sllm_seq_batch b, float* __restrict__ q, int ldq, int heads, int dk, const float* __restrict__ k, int ldk, int kv_heads,
                                     const float* __restrict__ v, int ldv, int dv, const double* __restrict__ freq, int n_freq, float magnitude,
                                     const double* __restrict__ vfreq, int layout, KV* __restrict__ k_pool, KV* __restrict__ v_pool) {
    const int t = blockIdx.x, posi = b.tok_pos[t], slot = b.tok_slot[t];
    const int pos = posi;
    // gridDim.y CTAs share a token: CTA y takes the work items y, y + gridDim.y, ... of each of the three loops (single tokens would
    // otherwise leave one CTA with every head's sines and cosines)
    const int tid = blockIdx.y * blockDim.x + threadIdx.x, nthr = gridDim.y * blockDim.x;
    const int page = b.block_table[(size_t)slot * b.max_pages + posi / b.page_len], in_page = posi % b.page_len;
    const int rd = 2 * n_freq, rhalf = n_freq;
    // q: heads * (dk/2 rounded up) work items; pairs beyond the rotary dimensions pass unchanged (they stay in place)
    for (int i = tid; i < heads * n_freq; i += nthr) {
        const int h = i / n_freq, mi = i % n_freq;
        const int ia = layout == 0 ? 2 * mi : mi, ib = layout == 0 ? 2 * mi + 1 : mi + rhalf;
        float sn, cs;
        seq_angle(pos, freq[mi], &sn, &cs);
        sn *= magnitude;
        cs *= magnitude;
        float* qh = q + (size_t)t * ldq + (size_t)h * dk;
        const float u = qh[ia], w = qh[ib];
        qh[ia] = u * cs - w * sn;
        qh[ib] = w * cs + u * sn;
    }
    for (int i = tid; i < kv_heads * dk; i += nthr) {
        const int g = i / dk, c = i % dk;
        const float* kh = k + (size_t)t * ldk + (size_t)g * dk;
        float val = kh[c];
        if (c < rd) {
            int mi, first;
            if (layout == 0) { mi = c >> 1; first = !(c & 1); } else { mi = c < rhalf ? c : c - rhalf; first = c < rhalf; }
            const int partner = layout == 0 ? (c ^ 1) : (first ? c + rhalf : c - rhalf);
            float sn, cs;
            seq_angle(pos, freq[mi], &sn, &cs);
            sn *= magnitude;
            cs *= magnitude;
            val = first ? kh[c] * cs - kh[partner] * sn : kh[c] * cs + kh[partner] * sn;
        }
        seq_st(k_pool, seq_pool_row(page, kv_heads, g, b.page_len, in_page, dk) + c, val);
    }
    const int vhalf = dv / 2;
    for (int i = tid; i < kv_heads * dv; i += nthr) {
        const int g = i / dv, c = i % dv;
        const float* vh = v + (size_t)t * ldv + (size_t)g * dv;
        float val = vh[c];
        if (vfreq) {
            int mi, first;
            if (layout == 0) { mi = c >> 1; first = !(c & 1); } else { mi = c < vhalf ? c : c - vhalf; first = c < vhalf; }
            const int partner = layout == 0 ? (c ^ 1) : (first ? c + vhalf : c - vhalf);
            float sn, cs;
            seq_angle(pos, vfreq[mi], &sn, &cs);
            val = first ? vh[c] * cs - vh[partner] * sn : vh[c] * cs + vh[partner] * sn;
        }
        seq_st(v_pool, seq_pool_row(page, kv_heads, g, b.page_len, in_page, dv) + c, val);
    }
}

}  // namespace sllm

using namespace sllm;

static int check_batch(const sllm_seq_batch* b, const char* who) {
    SLLM_REQUIRE(b && b->T > 0 && b->nseg > 0 && b->tok_slot && b->tok_pos && b->seg_start && b->seg_len && b->seg_slot && b->seg_pos0, SLLM_EINVAL,
                 "%s: incomplete batch description", who);
    return SLLM_OK;
}

extern "C" {

int sllm_seq_rotary_kv(const sllm_seq_batch* b, float* q, int32_t ldq, int32_t heads, int32_t dk, const float* k, int32_t ldk, int32_t kv_heads,
                       const float* v, int32_t ldv, int32_t dv, const double* freq, int32_t n_freq, float magnitude, const double* vfreq, int32_t layout,
                       void* k_pool, void* v_pool, int32_t kv_dtype, sllm_stream_t stream) {
    if (int rc = check_batch(b, "seq_rotary_kv")) return rc;
    SLLM_REQUIRE(q && k && v && k_pool && v_pool && b->block_table && heads > 0 && kv_heads > 0 && dk > 0 && dv > 0, SLLM_EINVAL, "seq_rotary_kv: bad argument");
    SLLM_REQUIRE(n_freq >= 0 && 2 * n_freq <= dk && (n_freq == 0 || freq), SLLM_EINVAL, "seq_rotary_kv: %d rotary pairs do not fit %d dimensions", n_freq, dk);
    SLLM_REQUIRE(!vfreq || dv % 2 == 0, SLLM_EINVAL, "seq_rotary_kv: rotated values need an even width");
    SLLM_REQUIRE(layout == 0 || layout == 1, SLLM_EINVAL, "seq_rotary_kv: layout 0 (interleaved) or 1 (halves)");
    SLLM_REQUIRE(kv_dtype == SLLM_F32 || kv_dtype == SLLM_BF16, SLLM_ENOTSUP, "seq_rotary_kv: fp32 or bf16 pools");
    // enough CTAs per token that a step of few tokens still spreads its sines and cosines over the machine
    const int work = std::max(heads * n_freq, kv_heads * std::max(dk, dv));
    const dim3 rgrid(b->T, std::max(1, std::min((work + 127) / 128, b->T >= 64 ? 1 : 16)));
    if (kv_dtype == SLLM_F32)
        seq_rotary_kv_kernel<float><<<rgrid, 128, 0, as_stream(stream)>>>(*b, q, ldq, heads, dk, k, ldk, kv_heads, v, ldv, dv, freq, n_freq, magnitude, vfreq,
                                                                         layout, (float*)k_pool, (float*)v_pool);
    else
        seq_rotary_kv_kernel<uint16_t><<<rgrid, 128, 0, as_stream(stream)>>>(*b, q, ldq, heads, dk, k, ldk, kv_heads, v, ldv, dv, freq, n_freq, magnitude,
                                                                            vfreq, layout, (uint16_t*)k_pool, (uint16_t*)v_pool);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_attention(const sllm_seq_batch* b, const float* q, int32_t ldq, int32_t heads, int32_t kv_heads, int32_t dk, int32_t dv, float scale,
                       const void* k_pool, const void* v_pool, int32_t kv_dtype, int32_t nsplit, float* ws, const sllm_seq_attn_opts* opts,
                       sllm_stream_t stream) {
    if (int rc = check_batch(b, "seq_attention")) return rc;
    const int v_in_k = opts && opts->values_in_keys;
    SLLM_REQUIRE(q && k_pool && (v_pool || v_in_k) && ws && b->block_table && b->qt_seg && b->qt_off && b->n_qtiles > 0, SLLM_EINVAL, "seq_attention: bad argument");
    SLLM_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dk > 0, SLLM_EINVAL, "seq_attention: %d query heads over %d kv heads", heads, kv_heads);
    SLLM_REQUIRE(dv > 0 && dv <= 512, SLLM_ENOTSUP, "seq_attention: value width %d beyond 512", dv);
    SLLM_REQUIRE(!v_in_k || dv <= dk, SLLM_EINVAL, "seq_attention: %d value columns inside key rows of %d", dv, dk);
    SLLM_REQUIRE(!opts || (opts->window >= 0 && opts->keep_first >= 0 && opts->softcap >= 0.0f), SLLM_EINVAL, "seq_attention: bad options");
    SLLM_REQUIRE(b->page_len % kBK == 0, SLLM_ENOTSUP, "seq_attention: pages of a multiple of %d positions", kBK);
    SLLM_REQUIRE(nsplit >= 1 && nsplit <= 65535, SLLM_EINVAL, "seq_attention: nsplit");
    SLLM_REQUIRE(kv_dtype == SLLM_F32 || kv_dtype == SLLM_BF16, SLLM_ENOTSUP, "seq_attention: fp32 or bf16 pools");
    const int dkp = ((dk + 3) & ~3) + 4;
    const size_t smem = ((size_t)(kBQ + kBK) * dkp + (v_in_k ? 0 : (size_t)kBK * dv)) * sizeof(float);
    SLLM_REQUIRE(smem <= (size_t)smem_optin_bytes(), SLLM_ENOTSUP, "seq_attention: heads of %d + %d floats need %zu bytes of shared memory", dk, dv, smem);
    AttnArgs p{*b, q, ldq, heads, kv_heads, dk, dv, scale, k_pool, v_pool, nsplit, ws, 0, INT_MAX, 0, 0.0f, nullptr, 0, nullptr, heads, 0};
    if (opts && opts->cross_values) {
        SLLM_REQUIRE(!v_in_k, SLLM_EINVAL, "seq_attention: values of every head need a value pool");
        p.cross = 1;
        p.heads = heads * kv_heads;        // results; ws holds that many records per token
    }
    if (opts) {
        p.window = opts->window > 0 ? opts->window : INT_MAX;
        p.keep_first = opts->window > 0 ? opts->keep_first : 0;
        p.softcap = opts->softcap;
        p.slopes = opts->slopes;
        p.v_in_k = v_in_k;
        p.logdist = opts->logdist;
    }
    dim3 grid(b->n_qtiles, p.heads, nsplit);
    // steps that hold a portion of a prompt, bf16 pools, head widths the fragments take: the tensor-core body
    if (kv_dtype == SLLM_BF16 && b->T > b->nseg && dk % 16 == 0 && dk <= 192 && dv % 8 == 0 && dv <= 128 && g_tune_seq_attn_mma) {
        const size_t smem_mma = 2 * (size_t)kBK * (dk + 8 + (v_in_k ? 0 : dv + 8)) * sizeof(uint16_t);
        const int hpc = (heads / kv_heads) % 2 == 0 ? 2 : 1;   // query heads per CTA
        grid.y = p.heads / hpc;
        const dim3 block(64 * hpc);
        cudaStream_t st = as_stream(stream);
        if (dk == 128 && dv == 128) seq_attention_mma_kernel<8, 16, true><<<grid, block, smem_mma, st>>>(p);
        else if (dk == 192 && dv == 128) seq_attention_mma_kernel<12, 16, true><<<grid, block, smem_mma, st>>>(p);
        else if (dk == 64 && dv == 64) seq_attention_mma_kernel<4, 8, true><<<grid, block, smem_mma, st>>>(p);
        else if (dk <= 128) seq_attention_mma_kernel<8, 16, false><<<grid, block, smem_mma, st>>>(p);
        else seq_attention_mma_kernel<12, 16, false><<<grid, block, smem_mma, st>>>(p);
        ++g_launches;
        SLLM_LAUNCH_CHECK();
        return SLLM_OK;
    }
    if (b->T == b->nseg && heads / kv_heads <= kBQ) {   // single tokens only: the query heads of a kv head share one CTA and its tiles
        p.by_head = 1;
        grid.y = p.cross ? kv_heads * kv_heads : kv_heads;   // with cross values: per value head too
    }
    const int chunks = dv <= 128 ? 4 : (dv <= 256 ? 8 : 16);
#define SLLM_ATTN_LAUNCH(KV, NC)                                                                                                              \
    do {                                                                                                                                      \
        if (smem > 48 * 1024) SLLM_CUDA(cudaFuncSetAttribute(seq_attention_kernel<KV, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        seq_attention_kernel<KV, NC><<<grid, 256, smem, as_stream(stream)>>>(p);                                                              \
    } while (0)
    if (kv_dtype == SLLM_F32) {
        if (chunks == 4) SLLM_ATTN_LAUNCH(float, 4); else if (chunks == 8) SLLM_ATTN_LAUNCH(float, 8); else SLLM_ATTN_LAUNCH(float, 16);
    } else {
        if (chunks == 4) SLLM_ATTN_LAUNCH(uint16_t, 4); else if (chunks == 8) SLLM_ATTN_LAUNCH(uint16_t, 8); else SLLM_ATTN_LAUNCH(uint16_t, 16);
    }
#undef SLLM_ATTN_LAUNCH
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

int sllm_seq_attention_finish(const sllm_seq_batch* b, const float* ws, int32_t nsplit, int32_t heads, int32_t dv, const double* vfreq, int32_t layout,
                              const float* gate, int32_t ldg, const float* sink, float* out, int32_t ldo, sllm_stream_t stream) {
    if (int rc = check_batch(b, "seq_attention_finish")) return rc;
    SLLM_REQUIRE(ws && out && nsplit >= 1 && heads > 0 && dv > 0 && (!vfreq || dv % 2 == 0), SLLM_EINVAL, "seq_attention_finish: bad argument");
    SLLM_REQUIRE(dv <= 1024 && nsplit <= 8192, SLLM_ENOTSUP, "seq_attention_finish: value width %d / %d shares beyond what one CTA merges", dv, nsplit);
    const int threads = std::max(32, (dv + 31) / 32 * 32);
    seq_attention_finish_kernel<<<b->T * heads, threads, (size_t)(nsplit + dv) * sizeof(float), as_stream(stream)>>>(*b, ws, nsplit, heads, dv, vfreq, layout, gate,
                                                                                                                  ldg, sink, out, ldo);
    ++g_launches;
    SLLM_LAUNCH_CHECK();
    return SLLM_OK;
}

}  // extern "C"
