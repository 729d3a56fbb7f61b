/* include/sllm_b200.h — the drop-in boundary: C ABI of libsllm_b200.so.
 *
 * B200-native (sm_100a) replacement for the transformer forward hot path of Boundwhd/SimpleLLMInference.
 * Plain pointers and sizes only: no C++ types, no torch types, no CUDA headers needed to include this file.
 * The reference has no FFI of its own (it is one C++ program); its hot-path boundary is the set of free
 * functions kernel::<op>_kernel_cuda (include/kernel/cuda/<op>_kernel.cuh) that the op layers call (source/op/<op>.cpp) plus
 * model::LlamaModel::forward (source/model/model.cpp:40-140). Each entry point below names the reference
 * interface it replaces. The C++ host mirror in simplellminference_b200/host/ (mem::Tensor, op::*Layer,
 * kernel::*_cuda, model::LlamaModel) is a thin layer over exactly these functions; INTEGRATION.md shows the
 * binding a maintainer of the reference would add.
 *
 * Conventions
 *  - every pointer named *_dev / every tensor argument is DEVICE memory of the current CUDA device unless the
 *    name ends in _host; `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *  - launchers never allocate, never synchronise, never throw; they enqueue on `stream` and return;
 *  - return value: 0 = SLLM_OK; >0 = a cudaError_t; <0 = an SLLM_E* code; sllm_last_error() gives the text
 *    (thread-local). The C++ shims turn non-zero into the reference's convention: LOG(...) prints
 *    "file: .. line: .. - msg" and std::exit(EXIT_FAILURE) (include/base/base.h:6-10);
 *  - `token` and `pos` may be read from device memory (token_dev / pos_dev non-NULL) so that the launch
 *    sequence is CUDA-graph capturable — a deliberate deviation from the reference, which reads them on the
 *    host (emb_kernel.cu:15, rope_kernel.cu:49). With the *_dev pointer NULL the by-value argument is used;
 *  - activations, RoPE tables and accumulators are fp32. Matrix weights are stored as fp32, bf16 or
 *    int8-with-group-scales (SLLM_F32 / SLLM_BF16 / SLLM_INT8); the KV cache as fp32 or bf16.
 *  - there is NO CPU fallback anywhere behind this header;
 *  - threading: the model of the reference (source/model/model.cpp drives one model from one host thread) and of the
 *    tensor-parallel runtime here — ONE process per GPU, one host thread driving an engine / batch at a time. The library keeps
 *    per-process caches of device facts and of per-kernel shared-memory attributes for the device that was current at first use, and
 *    the development knobs of sllm_tune are process-wide: do not drive two devices, or one engine from two threads, in one process.
 *    Pure-arithmetic entry points (sllm_*_plan, sllm_mega_tile_geometry, sllm_batch_arena_bytes, sllm_kvpages_*) touch no device.
 */
#ifndef SLLM_B200_H
#define SLLM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SLLM_OK 0
#define SLLM_EINVAL (-1)   /* bad argument (null pointer, size, alignment, divisibility) */
#define SLLM_ENOTSUP (-2)  /* shape or type combination not supported by the kernels */
#define SLLM_ENOMEM (-3)   /* device allocation failed */
#define SLLM_ESTATE (-4)   /* call sequence error (e.g. decode before weights are loaded) */
#define SLLM_ECOMM (-5)    /* NCCL / peer-memory error */

enum { SLLM_F32 = 0, SLLM_BF16 = 1, SLLM_INT8 = 2 };

typedef void* sllm_stream_t;

const char* sllm_last_error(void);
int sllm_abi_version(void);
/* development knobs (not part of the drop-in surface): key 0 = GEMV CTAs per SM (0 = built-in choice); prefill GEMM: key 1 = force
 * the N extent of a tile (multiple of 32, 0 = cost model), key 2 = two-SM tiles (1 / 0 force / forbid, -1 = by T), key 3 = programmatic
 * dependent launch (1 default), key 4 = K split of the residual-epilogue GEMMs (0 never, n up to n ranges, -1 cost model); batched decode:
 * key 5 = replay one CUDA graph per live-slot count instead of the launch sequence, key 6 = GEMV body with four weight rows per warp at
 * a time when 3 or more sequences share a launch, key 7 (with key 6) = down projection with K cut in two over grid.y when more sequences
 * are live than whole rows fit shared memory, so that Wdown is read once (all 0 by default: experimental until measured); key 8 = decode
 * megakernel MEASUREMENT aid, results are garbage: bit 0 = skip the grid barriers, bit 1 = skip the dot products (tools/mega_debug.py),
 * bit 4 = tensor-parallel prefill without its peer-memory exchanges (the GEMM / attention time alone); key 9 = ragged-batch attention
 * (sllm_seq_attention): 1 (default) tensor-core body for bf16 pools on steps that hold a prompt portion, 0 = always the fp32 body */
int sllm_tune(int32_t key, int32_t value);
/* device facts the host side sizes things by: sm count, max opt-in shared memory per block, total/free HBM */
int sllm_device_info(int32_t* sm_count, int32_t* smem_optin_bytes, size_t* hbm_total, size_t* hbm_free);

/* ------------------------------------------------------------------------------------------------------
 * Op launchers — one per reference CUDA kernel entry point.
 * ---------------------------------------------------------------------------------------------------- */

/* replaces kernel::add_kernel_cuda (include/kernel/cuda/add_kernel.cuh:6): out[i] = a[i] + b[i] */
int sllm_add_f32(const float* a, const float* b, float* out, int32_t n, sllm_stream_t stream);

/* replaces kernel::emb_kernel_cuda (emb_kernel.cuh:6-7): out[0..d) = table[token][:], dequantised to fp32.
 * scales: [vocab][d/group] fp32, only for SLLM_INT8. Fails with SLLM_EINVAL if the by-value token is outside
 * [0, vocab) (the reference's guard is `token > vocab`, off by one: emb_kernel.cu:16); a device-side token
 * outside the range is clamped into it. */
int sllm_embedding(const int32_t* token_dev, int32_t token, const void* table, int32_t w_dtype,
                   const float* scales, int32_t group, float* out, int32_t vocab, int32_t d,
                   sllm_stream_t stream);

/* replaces kernel::rmsnorm_kernel_cuda (rms_kernel.cuh:6-7): y = (x * 1/sqrt(mean(x^2)+eps)) * w */
int sllm_rmsnorm_f32(const float* x, const float* w, float* y, int32_t d, float eps, sllm_stream_t stream);

/* replaces kernel::matmul_kernel_cuda (matmul_kernel.cuh:6-7): y[r] = (sum_j x[j] * W[r][j]) * scale,
 * W row-major [rows][cols]. Unlike the reference's CUDA kernel, `scale` is honoured (matmul_kernel.cu:41-55
 * drops it; the CPU kernel applies it, matmul_kernel.cpp:26). cols must be a multiple of 16 bytes' worth of
 * elements (4 / 8 / 16 for f32 / bf16 / int8), W 16-byte aligned, and for SLLM_INT8 cols % group == 0,
 * group % 16 == 0, scales = [rows][cols/group] fp32. */
int sllm_gemv(const float* x, const void* W, int32_t w_dtype, const float* scales, int32_t group, float* y,
              int32_t rows, int32_t cols, float scale, sllm_stream_t stream);

/* replaces kernel::rope_cache_cal_cuda (rope_kernel.cuh:5): sin/cos tables [max_len][head_dim/2]. Computed
 * on the HOST with the same libm calls the reference CPU path makes (rope_kernel.cpp:8-17) and uploaded, so
 * the tables are bit-identical to the oracle's (GPU powf/sinf/cosf differ by ulps). Synchronous. */
int sllm_rope_tables(int32_t head_dim, int32_t max_len, float theta, float* sin_dev, float* cos_dev,
                     sllm_stream_t stream);

/* replaces kernel::rope_kernel_cuda (rope_kernel.cuh:7-8): rotate-half RoPE in place on q[0..q_dim) and
 * k[0..k_dim). The reference rotates k over q_dim too (GQA over-run); here k_dim is
 * explicit. k may be fp32 only (it is a row of an fp32 cache or a scratch vector). */
int sllm_rope_f32(float* q, float* k, const int32_t* pos_dev, int32_t pos, const float* sin_tab,
                  const float* cos_tab, int32_t q_dim, int32_t k_dim, int32_t head_dim, sllm_stream_t stream);

/* replaces kernel::mha_kernel_cuda (mha_kernel.cuh:6-21): single-query attention over cache rows 0..pos of
 * `layer`, caches laid out [layers][max_len][kv_heads*head_dim] (fp32 or bf16). Split-KV flash decoding with
 * an in-kernel combine; the reference's `score` scratch is not needed. workspace: device scratch of at least
 * sllm_mha_workspace_bytes(heads, head_dim, max_len) bytes, 16-byte aligned, zero-initialised once (the
 * kernel leaves it zeroed). head_dim must be a multiple of 8 and <= 256. */
size_t sllm_mha_workspace_bytes(int32_t heads, int32_t head_dim, int32_t max_len);
int sllm_mha_decode(const float* q, const void* key_cache, const void* value_cache, int32_t kv_dtype,
                    float* out, void* workspace, int32_t layer, const int32_t* pos_dev, int32_t pos,
                    int32_t max_len, int32_t head_dim, int32_t heads, int32_t kv_heads, sllm_stream_t stream);

/* replaces kernel::swiglu_kernel_cuda (swiglu_kernel.cuh:5): out = sigmoid(gate) * up  (sic: not SiLU,
 * swiglu_kernel.cpp:12-13) */
int sllm_swiglu_f32(const float* up, const float* gate, float* out, int32_t n, sllm_stream_t stream);

/* device version of op::argmaxLayer::forward (source/op/argmax.cpp:7-17; CPU-only in the reference): index of
 * the FIRST maximum of logits[0..n). idx_dev receives the int32 index. */
int sllm_argmax_f32(const float* logits, int32_t n, int32_t* idx_dev, sllm_stream_t stream);

/* KV-row store used by the op-by-op path when the cache is bf16: cache_row[i] = bf16(src[i]) */
int sllm_store_kv_row(const float* src, void* cache_row, int32_t kv_dtype, int32_t n, sllm_stream_t stream);

/* Sampling beyond arg-max (additive: the reference only has argmaxLayer; LayerType::kLayerSoftmax is declared but unused,
 * include/op/layer.h:17). One draw from softmax(logits / temperature) restricted to the top_k largest logits (0 = all; ties at
 * the k-th value are kept) and then to the smallest set of largest logits whose mass reaches top_p (0 or 1 = all). The draw is a
 * pure function of (logits, parameters, seed, step): u = hash(seed, step), first index whose running kept mass exceeds u * mass.
 * temperature <= 0 = arg-max (first maximum). idx_dev: device int32. */
int sllm_sample_f32(const float* logits, int32_t n, float temperature, int32_t top_k, float top_p, uint64_t seed,
                    uint64_t step, int32_t* idx_dev, sllm_stream_t stream);

/* ------------------------------------------------------------------------------------------------------
 * Synthetic weights (device side of oracle/synth_weights.h: same integer hash, bit-identical values).
 * Fills `count` elements [first, first+count) of blob segment `segment` (0 E, 1 norms, 2 wq, 3 wk, 4 wv,
 * 5 wo, 6 up, 7 gate, 8 down) of the given shape into dst in w_dtype; int8 also writes count/group scales.
 * row_len/row_stride_* let a tensor-parallel shard be cut out of the full matrix: the destination is
 * [n_rows][row_len] taken from source rows of length src_row_len starting at column src_col0.
 * ---------------------------------------------------------------------------------------------------- */
typedef struct {
    int32_t vocab, head_dim, hidden, kv_hidden, inter, max_len, layers, heads, kv_heads;
    float eps, theta;
} sllm_shape;

int sllm_synth_fill(const sllm_shape* shape, uint64_t seed, int32_t segment, int64_t src_first_row,
                    int64_t n_rows, int64_t src_row_len, int64_t src_col0, int64_t row_len, void* dst,
                    int32_t w_dtype, float* scales, int32_t group, sllm_stream_t stream);

/* fp32 -> storage type conversion of an uploaded fp32 matrix [rows][cols] (the path real checkpoints take) */
int sllm_convert_weights(const float* src_f32_dev, void* dst, int32_t w_dtype, float* scales, int32_t group,
                         int64_t rows, int64_t cols, sllm_stream_t stream);

/* ------------------------------------------------------------------------------------------------------
 * Engine — replaces model::LlamaModel::{init_mem, create_param_layers, forward} and the greedy loop of
 * predict (source/model/model.cpp:40-187, 247-469) with a static device arena, a KV cache and a
 * CUDA-graph-captured, fused decode step. One engine per GPU; tensor parallelism = one process per GPU.
 * ---------------------------------------------------------------------------------------------------- */
typedef struct {
    sllm_shape shape;
    int32_t w_dtype;   /* SLLM_F32 / SLLM_BF16 / SLLM_INT8 */
    int32_t kv_dtype;  /* SLLM_F32 / SLLM_BF16 */
    int32_t group;     /* int8 group size along the input dimension */
    int32_t tp_rank, tp_size;
    int32_t flags;     /* SLLM_ENGINE_* */
} sllm_engine_config;

#define SLLM_ENGINE_UNFUSED 1u   /* run the 13-ops-per-layer sequence of the reference instead of fused kernels */
#define SLLM_ENGINE_NO_GRAPH 2u  /* launch kernels directly instead of replaying a CUDA graph */
#define SLLM_ENGINE_PDL 4u       /* programmatic dependent launch between the kernels of a step (measured slower
                                    inside a CUDA graph on B200 than plain graph edges: off by default) */
#define SLLM_ENGINE_MEGAKERNEL 16u /* whole decode step as ONE persistent cooperative kernel whose TMA weight rings
                                    keep streaming across phases (single GPU; shapes it cannot take fall back to the
                                    per-kernel fused path — sllm_engine_mode() tells which one runs) */
#define SLLM_ENGINE_MEGA_LL 32u   /* with MEGAKERNEL on one GPU: the barrier-free {value, epoch}-word version
                                    (megakernel_ll.cu) instead of the grid-barrier one (megakernel.cu, faster on one GPU).
                                    Under tensor parallelism (MEGAKERNEL | P2P_ALLREDUCE) the word version is the only
                                    one: it carries the all-reduce inside the kernel */
#define SLLM_ENGINE_MEGA_FUSE_DOWN 64u /* experimental, with MEGAKERNEL on one GPU (fp32 / bf16 weights, hidden size = 2^k x 512 bytes per
                                    row <= 8 KB): the down projection runs inside the gate_up phase as a K-split over the values each
                                    CTA produced, partial outputs added to the residual stream with red.global.add — four grid barriers
                                    per layer instead of five, but a summation order that is not fixed (logits vary in the last bits
                                    from run to run). Costs a second, transposed copy of the down matrices. Off until measured;
                                    sllm_engine_mode() says "megakernel(fused-down)" when it is in effect */
#define SLLM_ENGINE_MEGA_V2 128u /* with MEGAKERNEL on one GPU (fp32 / bf16 weights): the megakernel with two grid-wide dependency points
                                   * per layer instead of five (csrc/megakernel2.cu): qkv -> attention -> wo chained through per-kv-head
                                   * counters, wo as a K split by kv head group adding into h with red.global.add.f32. With
                                   * MEGA_FUSE_DOWN the down projection is fused into the gate_up phase as well. Summation order of wo
                                   * (and of a fused down) is not fixed: logits differ in the last bits from run to run (inside the
                                   * decode tolerance). Shapes it cannot take fall back to the grid-barrier kernel (sllm_engine_mode). */
#define SLLM_ENGINE_P2P_ALLREDUCE 8u /* TP: one-shot all-reduce over NVLink peer memory instead of NCCL */

typedef struct sllm_engine sllm_engine;

/* stream: the stream every engine operation is enqueued on; NULL = the engine creates and owns a
 * non-blocking stream (the legacy default stream cannot be captured into a CUDA graph). */
int sllm_engine_create(const sllm_engine_config* cfg, sllm_stream_t stream, sllm_engine** out);
void sllm_engine_destroy(sllm_engine* e);

/* weights: generated on the device (synthetic), or taken from a HOST fp32 blob in the reference's order
 * (source/model/model.cpp:340-468), converted to w_dtype and cut to this rank's tensor-parallel shard. */
int sllm_engine_load_synthetic(sllm_engine* e, uint64_t seed);
int sllm_engine_load_blob_f32(sllm_engine* e, const float* blob_host, int64_t n_floats);

/* tensor-parallel communicator: id_bytes = 128-byte ncclUniqueId produced by sllm_comm_unique_id on rank 0
 * and distributed by the caller (torch.distributed / MPI / a file — plumbing is the host's business). */
int sllm_comm_unique_id(void* id_bytes_128);
int sllm_engine_init_comm(sllm_engine* e, const void* id_bytes_128);
/* peer-memory exchange for SLLM_ENGINE_P2P_ALLREDUCE: each rank exports a 64-byte IPC handle, the caller
 * all-gathers them, every rank imports all of them. */
int sllm_engine_p2p_export(sllm_engine* e, void* handle_bytes_64);
int sllm_engine_p2p_import(sllm_engine* e, const void* all_handles /* tp_size * 64 bytes */);
/* Batched prefill under tensor parallelism without a collective library: every rank exports the CUDA-IPC handle of its prefill exchange
   block and imports everybody's (same messenger protocol as above). From then on sllm_engine_prefill sums the row-parallel partial
   matrices, adds the residual, normalises and distributes the rows in one kernel over NVLink peer memory (csrc/prefill_tp.cu).
   SLLM_ENOTSUP: the engine has no such block (one rank, no SLLM_ENGINE_P2P_ALLREDUCE, shape not taken by the batched prefill) — prefill
   then needs the NCCL communicator. Every rank must issue the same sequence of sllm_engine_prefill calls (the exchange kernels wait for each
   other's epoch flags; a wait that is never answered traps after ~20 s instead of hanging the GPU): a prefill that failed on one rank only leaves
   the ranks out of step — destroy the engines. Replaces nothing in the reference (it has neither prefill nor a working multi-GPU build). */
int sllm_engine_prefill_p2p_export(sllm_engine* e, void* handle_bytes_64);
int sllm_engine_prefill_p2p_import(sllm_engine* e, const void* all_handles /* tp_size * 64 bytes */);

/* One token, one position: the semantics of LlamaModel::forward(). token/pos by value (host), synchronous.
 * logits_host (vocab floats, may be NULL) receives model_pred; next_token_host (may be NULL) the greedy
 * argmax (first maximum). */
int sllm_engine_forward(sllm_engine* e, int32_t token, int32_t pos, float* logits_host,
                        int32_t* next_token_host);

/* Greedy loop of LlamaModel::predict without tokenizer/printing: feeds prompt[0..n_prompt) one token at a
 * time, then feeds back the argmax; writes the n_total-1 tokens that follow prompt[0] to tokens_out_host.
 * Runs entirely on the device (token and position live in device memory, one graph replay per token);
 * asynchronous until the final copy of the token list. */
int sllm_engine_greedy(sllm_engine* e, const int32_t* prompt_host, int32_t n_prompt, int32_t n_total,
                       int32_t* tokens_out_host);

/* Device-resident stepping for benchmarks: set state, enqueue n steps (no host sync), read results. */
int sllm_engine_set_state(sllm_engine* e, int32_t token, int32_t pos);
int sllm_engine_enqueue_steps(sllm_engine* e, int32_t n_steps);
int sllm_engine_read_tokens(sllm_engine* e, int32_t* tokens_out_host, int32_t n);

/* Batched prefill of prompt[0..n) at positions start_pos..: the layer loop of LlamaModel::forward
 * (source/model/model.cpp:50-128) for all prompt rows at once — dense contractions as tcgen05/TMEM tensor-core
 * GEMMs fed by TMA (bf16 operands, fp32 accumulators), causal attention over the block — instead of the
 * reference's one forward() per prompt token (model.cpp:157-166). Fills the KV cache for start_pos..start_pos+n-1,
 * leaves the LAST prompt token's logits in model_pred, its arg-max as the current token and the position at
 * start_pos+n, exactly as the token-by-token loop would (the last row's classifier is a T = 1 GEMM + arg-max).
 * Needs SLLM_ENGINE_MEGAKERNEL, bf16 weights and head_dim 64/128: otherwise SLLM_ENOTSUP (feed the prompt through
 * sllm_engine_greedy / sllm_engine_forward, which is what the reference does); sllm_engine_prefill_supported
 * returns 1/0 (0: reason in sllm_last_error). Tensor parallel: also needs sllm_engine_init_comm (NCCL all-reduce of
 * the row-parallel partial sums, one per wo/down GEMM). */
int sllm_engine_prefill(sllm_engine* e, const int32_t* prompt_host, int32_t n, int32_t start_pos);
int sllm_engine_prefill_supported(const sllm_engine* e);

/* How the persistent decode megakernel (SLLM_ENGINE_MEGAKERNEL; replaces the layer loop of LlamaModel::forward,
 * source/model/model.cpp:48-139, by one launch per token) would run a shape — host arithmetic only, no launch, and no device
 * either when the two device facts are passed in (sm_count_or_0 / smem_optin_or_0 > 0; 0 = ask the current device):
 * *ok = 1 and grid (= CTAs = SMs), dynamic shared memory per CTA, KV splits per head of the attention phase; or *ok = 0 with the
 * reason in sllm_last_error (the engine then runs the per-kernel fused path: sllm_engine_mode()). word_based = 0: the grid-barrier kernel
 * (one GPU); 1: the barrier-free {value, epoch}-word kernel (SLLM_ENGINE_MEGA_LL; the one that runs under tensor parallelism,
 * tp_size > 1 plans one rank's shard; its grid may be smaller than the SM count: every CTA must own a tile row of every phase). */
int sllm_mega_plan(const sllm_shape* shape, int32_t w_dtype, int32_t group, int32_t kv_dtype, int32_t tp_size, int32_t word_based,
                   int32_t sm_count_or_0, int32_t smem_optin_or_0, int32_t* ok, int32_t* grid, int64_t* smem_bytes, int32_t* nsplit);
/* The tiled weight layout of that kernel for one [rows][cols] matrix (kind: 0 qkv, 1 wo, 2 [up; gate], 3 down, 4 classifier):
 * tiles of r physical rows x sc 16-byte chunks, ks K slices per row, tile_rows tile rows, one tile = tile_bytes contiguous bytes
 * (= one TMA bulk copy = one ring slot), the matrix = tile_rows * ks * tile_bytes = matrix_bytes (zero padding included). */
int sllm_mega_tile_geometry(int32_t rows, int32_t cols, int32_t kind, int32_t w_dtype, int32_t* ks, int32_t* sc, int32_t* r,
                            int32_t* tile_rows, int32_t* tile_bytes, int64_t* matrix_bytes);

/* Development aid for the experimental SLLM_ENGINE_MEGA_FUSE_DOWN kernel: its transposed, stripe-major copy of a row-major
 * [d][inter] down matrix (device pointers; fp32 / bf16; d * element size = 2^k * 512 bytes <= 8 KB, inter % 4 == 0). Element e of lane
 * `lane`, input jj of tile row g, output stripe ks — at index (((ks * (inter/4) + g) * 4 + jj) * 32 + lane) * E + e, E = 16 bytes of
 * elements — is W[(ks * 32 + lane) * E + e][g * 4 + jj]. */
int sllm_mega_repack_down_t(const void* src_rowmajor, void* dst, int32_t d, int32_t inter, int32_t w_dtype, sllm_stream_t stream);

/* The two prefill kernels on their own (device pointers), for op-level parity tests:
 * C[T][N] (fp32) = A[T][K] (bf16) . W[N][K]^T (bf16, row-major) on tcgen05; bn = 0 (auto), 128 or 256 = N tile. */
int sllm_prefill_gemm_bf16(const void* A, const void* W, float* C, int32_t T, int32_t N, int32_t K, int32_t bn,
                           sllm_stream_t stream);
/* How sllm_prefill_gemm_bf16 / the engine would run a [T][K] x [N][K]^T GEMM (host arithmetic only, no launch): two_sm = 1 when SM
 * pairs share 256-row tiles (tcgen05 cta_group::2), bn = N extent of a tile, ksplit = K ranges per tile (> 1 only with the
 * residual epilogue, whose partial sums are added with red.global.add), work_units = tiles x ksplit. */
int sllm_prefill_gemm_plan(int32_t T, int32_t N, int32_t K, int32_t residual_epilogue, int32_t* two_sm, int32_t* bn,
                           int32_t* ksplit, int32_t* work_units);
/* causal attention of T queries (bf16 [T][heads*head_dim]) at positions pos0.. over a HEAD-MAJOR cache
 * [kv_heads][max_len][head_dim] (kv_dtype f32 or bf16), rows 0..pos0+T-1 valid; out bf16 like q. */
int sllm_prefill_attention(const void* q, const void* key_cache, const void* value_cache, int32_t kv_dtype, void* out,
                           int32_t T, int32_t pos0, int32_t max_len, int32_t head_dim, int32_t heads, int32_t kv_heads,
                           sllm_stream_t stream);

/* ------------------------------------------------------------------------------------------------------
 * Batched multi-sequence decode over a paged KV cache (additive: the reference decodes one sequence at a time,
 * include/model/model.h:15-18 input_token{1} / position{1}, source/model/model.cpp:148-185). Up to 64 sequences,
 * each at its own position, advance one token per step and share ONE pass over the weights (the HBM traffic of a
 * decode step); every sequence follows the semantics of sllm_engine_greedy (prompt tokens fed verbatim, then the
 * first-max arg-max fed back, no EOS stop). Activations stay fp32: the decode parity contract holds per sequence.
 * ---------------------------------------------------------------------------------------------------- */

/* Page bookkeeping of the paged cache — host arithmetic only (no device, no CUDA call): a stack of free pages and, per
 * sequence, the list of pages that hold its positions [i*page_len, (i+1)*page_len). sllm_batch uses one internally; it
 * is exported so that a scheduler can plan admissions with the same rules. */
typedef struct sllm_kvpages sllm_kvpages;
sllm_kvpages* sllm_kvpages_create(int32_t n_pages, int32_t page_len, int32_t max_seqs, int32_t max_pages_per_seq);
void sllm_kvpages_destroy(sllm_kvpages* kp);
/* grow `seq` so that positions [0, n_positions) are covered; all or nothing. Returns the number of pages newly taken
 * (>= 0), SLLM_ENOMEM when the free pages do not suffice (nothing changes), SLLM_EINVAL beyond max_pages_per_seq. */
int32_t sllm_kvpages_reserve(sllm_kvpages* kp, int32_t seq, int32_t n_positions);
int sllm_kvpages_release(sllm_kvpages* kp, int32_t seq);   /* all pages of seq return to the free stack */
int32_t sllm_kvpages_free_count(const sllm_kvpages* kp);
int32_t sllm_kvpages_held(const sllm_kvpages* kp, int32_t seq);
const int32_t* sllm_kvpages_table(const sllm_kvpages* kp); /* [max_seqs][max_pages_per_seq] page ids, -1 = none */

typedef struct sllm_batch sllm_batch;
/* A batch borrows the weights, RoPE tables and stream of `e`, which must outlive it: one GPU, weights loaded, created
 * WITHOUT SLLM_ENGINE_MEGAKERNEL (the batched kernels read row-major matrices). It owns the paged cache: two pools of
 * n_pages pages of page_len positions, [pages][layers][kv_heads][page_len][head_dim] in kv_dtype, plus per-slot
 * activations. A sequence may grow to the engine's max_len (the RoPE tables' extent). */
int sllm_batch_create(sllm_engine* e, int32_t max_seqs, int32_t page_len, int32_t n_pages, int32_t kv_dtype, sllm_batch** out);
void sllm_batch_destroy(sllm_batch* b);
/* admit a sequence into the lowest free slot at position 0 (pages are taken when it steps); slot_out = its handle */
int sllm_batch_add(sllm_batch* b, const int32_t* prompt_host, int32_t n_prompt, int32_t* slot_out);
/* retire a sequence: its slot and pages are free for the next sllm_batch_add at once (stream order protects them) */
int sllm_batch_remove(sllm_batch* b, int32_t slot);
/* Sampling instead of arg-max for one sequence (additive, like sllm_sample_f32; not part of the parity contract): from now on the token
 * that follows position p of this slot is sllm_sample_f32(logits_p, temperature, top_k, top_p, seed, step = p) — a pure function of the
 * sequence, whatever its neighbours. temperature <= 0 switches back to arg-max. Prompt tokens are still fed verbatim. Retiring the
 * sequence clears the setting. */
int sllm_batch_set_sampling(sllm_batch* b, int32_t slot, float temperature, int32_t top_k, float top_p, uint64_t seed);
/* n_steps tokens for EVERY live sequence, asynchronous. Takes the pages the steps will write first, for all sequences
 * or none: SLLM_ENOMEM (nothing enqueued) when the pool is short, SLLM_EINVAL when a sequence would pass max_len. */
int sllm_batch_step(sllm_batch* b, int32_t n_steps);
/* Opt-in (on != 0): the steps of this batch run their five projection groups as tcgen05 GEMMs over the live sequences' rows (the prefill GEMM
 * kernel of csrc/prefill_gemm.cu) instead of batched GEMVs, so that every weight byte is read once per step however many sequences are live —
 * the batched GEMVs stop scaling at ~4 sequences. GEMM operands are bf16 (activations rounded after RMSNorm / attention / SwiGLU, fp32
 * accumulation): a sequence's results then agree with the reference within the bf16-operand tolerance of the prefill, not bit for bit.
 * bf16 weights only (SLLM_ENOTSUP otherwise). The reference has no batched decode (model.h:15-18: one token, one position). */
int sllm_batch_set_tensor_cores(sllm_batch* b, int32_t on);
/* the tokens that followed positions 0.. of the slot's sequence (prompt tokens included, as sllm_engine_greedy
 * reports them), at most max_tokens; *n_out = how many. Synchronises the stream. */
int sllm_batch_read(sllm_batch* b, int32_t slot, int32_t* tokens_out_host, int32_t max_tokens, int32_t* n_out);
/* logits (vocab floats) of the slot's latest step. Synchronises the stream. */
int sllm_batch_logits(sllm_batch* b, int32_t slot, float* logits_host);
/* Introspection for parity tests: per-slot buffers under the reference's ModelBufferType numbers (include/model/model.h:14-34),
 * each [max_seqs][...] fp32: 4 emb_output (the residual stream) [d], 6 query [q], 8 mha_output [q], 10 ffn_input [d], 14 swi_output
 * [I], 16 model_pred [vocab]; 2 / 3 = the key / value page pools in kv_dtype. Synchronises the stream. */
int sllm_batch_buffer(sllm_batch* b, int32_t buffer_id, void** dev_ptr, int64_t* n_elems, int32_t* dtype);
int32_t sllm_batch_free_pages(const sllm_batch* b);
int32_t sllm_batch_position(const sllm_batch* b, int32_t slot);   /* position of the slot's next step; -1 = free slot */
/* algorithmic HBM bytes of the NEXT step: every weight once, plus per live sequence its embedding row, the K/V rows
 * 0..pos it reads and the row it writes (SURVEY.md 8d B(p) with the weight term shared) */
int64_t sllm_batch_step_bytes(const sllm_batch* b);
int64_t sllm_batch_total_launches(const sllm_batch* b);
/* Device bytes sllm_batch_create(max_seqs, page_len, n_pages, kv_dtype) takes on an engine of this shape (the two page pools
 * [n_pages][layers][kv_heads][page_len][head_dim], per-slot activations and logits, attention workspace; rounded up to 1 MiB) —
 * host arithmetic only, so that a host sizes n_pages against sllm_device_info's free HBM first; -1 = bad argument. */
int64_t sllm_batch_arena_bytes(const sllm_shape* shape, int32_t max_seqs, int32_t page_len, int32_t n_pages, int32_t kv_dtype);

/* Calibrated partition of the persistent decode kernels (SLLM_ENGINE_MEGAKERNEL, one GPU, not MEGA_LL). The SMs of a B200 do not all
 * stream from HBM at the same rate (a stable pattern of about +-5 % per GPU) and every phase of the kernel ends with its slowest CTA.
 * This call runs `rounds` x 9 decode steps from (token 1, position 0) with the kernel's timeline on, measures every CTA's time per
 * byte over the big weight phases, and from then on gives each CTA a share of every phase's tile rows in inverse proportion. It
 * changes WHICH CTA computes a row, never how a row is computed: results are unchanged (bit for bit in the deterministic kernel).
 * Call it after loading weights and before use: it overwrites the first positions of the KV cache and resets the step state to
 * (token 0, position 0). sllm_engine_calibration(cta) = the measured relative time per byte (1.0 = mean, 0 = never calibrated). */
int sllm_engine_calibrate(sllm_engine* e, int32_t rounds);
float sllm_engine_calibration(const sllm_engine* e, int32_t cta);
/* Introspection for parity tests and the roofline: named buffers follow the reference's ModelBufferType
 * numbering (include/model/model.h:14-34); returns a device pointer and its element count/dtype. */
int sllm_engine_buffer(sllm_engine* e, int32_t buffer_id, void** dev_ptr, int64_t* n_elems, int32_t* dtype);
/* algorithmic HBM bytes one decode step at position pos must move on this rank */
int64_t sllm_engine_step_bytes(const sllm_engine* e, int32_t pos);
/* Enqueue ONE fused kernel of the decode step for `layer` at the current device-side position, for per-kernel
 * timing and profiling. kind: 0 embedding, 1 qkv (RMSNorm+QKV GEMV+RoPE+cache write), 2 mha (flash decoding),
 * 3 wo (+residual), 4 gate_up (RMSNorm+GEMV+sigmoid*up), 5 down (+residual), 6 classifier (+argmax; the step
 * state is left untouched). sllm_engine_kernel_bytes = the algorithmic HBM bytes of that launch (its share of
 * B(p): weights it streams, norm vector, KV rows read/written). */
int sllm_engine_enqueue_kernel(sllm_engine* e, int32_t kind, int32_t layer);
int64_t sllm_engine_kernel_bytes(const sllm_engine* e, int32_t kind, int32_t pos);
/* layout of the key_cache / value_cache buffers: 0 = [layers][max_len][kv_heads*head_dim] (the reference's,
 * model.cpp:264-265), 1 = head-major [layers][kv_heads][max_len][head_dim] (megakernel mode: a tile of positions
 * of one head is one contiguous TMA copy). Weight matrices of a megakernel engine are stored tiled (buffer ids
 * 100-105 are then opaque). */
int32_t sllm_engine_kv_layout(const sllm_engine* e);
/* which decode path this engine runs: "megakernel", "fused+graph", "fused", "unfused", ... (static string) */
const char* sllm_engine_mode(const sllm_engine* e);
/* number of kernel launches (graph kernel nodes) one decode step issues on this rank */
int32_t sllm_engine_step_launches(const sllm_engine* e);
/* total launches issued by this engine since creation */
int64_t sllm_engine_total_launches(const sllm_engine* e);

/* ------------------------------------------------------------------------------------------------------
 * Ragged token batches (sllm_seq_*): building blocks for models that mix softmax attention over a paged cache with
 * recurrent layers (additive: the reference has one Llama forward, source/model/model.cpp:40-140). A step brings T tokens
 * that belong to nseg segments; a segment is a run of consecutive positions of ONE sequence (a portion of a prompt, or
 * one decoded token) and its tokens are adjacent in the batch. Activations are fp32 [T][ld]; every matrix argument
 * comes with its row stride so that the columns of one wide projection can feed several consumers. Weights are fp32 or
 * bf16 (SLLM_F32 / SLLM_BF16). Per-sequence state (recurrent state, convolution tail) lives in slot-indexed fp32 arrays
 * owned by the caller; the softmax attention's keys and values live in page pools [pages][kv_heads][page_len][width]
 * (fp32 or bf16) addressed through a block table. All launchers enqueue on `stream`, allocate nothing and do not synchronise.
 * ---------------------------------------------------------------------------------------------------- */
typedef struct {
    int32_t T, nseg;             /* tokens and segments of this step */
    const int32_t* tok_slot;     /* [T]    state slot (= row of the block table) of each token's sequence */
    const int32_t* tok_pos;      /* [T]    position of each token in its sequence */
    const int32_t* seg_start;    /* [nseg] first token of the segment in the batch */
    const int32_t* seg_len;      /* [nseg] */
    const int32_t* seg_slot;     /* [nseg] */
    const int32_t* seg_pos0;     /* [nseg] position of the segment's first token */
    const int32_t* block_table;  /* [slots][max_pages] page of positions i*page_len.., -1 = none */
    int32_t max_pages, page_len; /* page_len: a multiple of 32 */
    int32_t n_qtiles;            /* attention work list: tiles of up to 32 consecutive queries of one segment */
    const int32_t* qt_seg;       /* [n_qtiles] segment of the tile */
    const int32_t* qt_off;       /* [n_qtiles] offset of its first query inside the segment */
    const int32_t* seg_tile0;    /* [nseg] running count of tiles of the segments before this one (tile ids in segment order) */
} sllm_seq_batch;

/* out[s][t][:] = table[ids[t]][:] * scale for every stream s (a model with one residual stream passes streams = 1) */
int sllm_seq_embed(const int32_t* ids, const void* table, int32_t w_dtype, int32_t vocab, int32_t d, int32_t streams, float scale,
                   float* out, int32_t T, sllm_stream_t stream);
/* u = sum_s coef[s] * x[s] (coef NULL = all ones), then, if norm_w is given, the RMS norm in `groups` equal consecutive parts:
 * every part divided by sqrt(mean(part^2) + eps), the whole multiplied by norm_w. x: [streams][T][d], y: [T][d]. */
int sllm_seq_hyper_read(const float* x, int32_t streams, int32_t T, int32_t d, const float* coef, const float* norm_w, int32_t groups,
                        float eps, float* y, sllm_stream_t stream);
/* all streams at once from the old ones: x[t] <- sum_s mix[s][t] * x[s] + outc[t] * y (mix NULL = identity, outc NULL = ones) */
int sllm_seq_hyper_write(float* x, int32_t streams, int32_t T, int32_t d, const float* mix, const float* outc, const float* y,
                         sllm_stream_t stream);
/* sllm_seq_hyper_write (mix, outc, y_in) followed by sllm_seq_hyper_read (coef, norm_w, groups, eps -> y_out) of the next sublayer, as one
 * pass over the streams; y_in and y_out must differ. */
int sllm_seq_hyper_write_read(float* x, int32_t streams, int32_t T, int32_t d, const float* mix, const float* outc, const float* y_in,
                              const float* coef, const float* norm_w, int32_t groups, float eps, float* y_out, sllm_stream_t stream);
/* C[b] = alpha * (A[b] . W[b]^T + bias[b]) (+ C[b] if accumulate): A fp32 [T][lda] (rounded to bf16 on load if round_a), W [N][ldw]
 * row-major in w_dtype, bias fp32 [N] or NULL, C fp32 [T][ldc]; `batch` independent products whose operands lie *_bs elements apart
 * (block-diagonal matrices). Any T, N, K. With a16 (scratch of T*K bf16 values) given, bf16 weights and a shape its tiles take, the
 * product runs on the tensor cores (tcgen05); otherwise on fp32 FMAs. a16_ready != 0: the kernel that produced A has already left
 * its rows in a16 as dense bf16 [T][K] (sllm_seq_depth_average, sllm_seq_layernorm and sllm_seq_clamped_glu can), so that the copy is
 * skipped; only meaningful when sllm_seq_linear_on_tensor_cores says the product goes there. rows_dev (device memory or NULL): a row
 * count an earlier kernel left; rows from *rows_dev on (of the T the call names) are not computed and their outputs stay as they are
 * (steps of more than 8 tokens; smaller steps compute all T rows). */
int sllm_seq_linear(const float* A, int32_t lda, const void* W, int32_t w_dtype, int32_t ldw, const float* bias, float* C, int32_t ldc,
                    int32_t T, int32_t N, int32_t K, float alpha, int32_t accumulate, int32_t round_a, int32_t batch, int64_t a_bs,
                    int64_t w_bs, int64_t bias_bs, int64_t c_bs, void* a16, int32_t a16_ready, const int32_t* rows_dev, sllm_stream_t stream);
/* `batch` products of ONE activation row each, every one with a matrix chosen on the device: C[b] = A[b / a_div] . W[w_index[b]]^T,
 * matrices w_bs elements apart in W, rows a_bs / c_bs apart in A / C; w_index[b] < 0 = no matrix (C[b] = 0). The weight-streaming body
 * of sllm_seq_linear: each product reads only its own matrix (a mixture of experts at decode sizes). */
int sllm_seq_linear_indexed(const float* A, int32_t lda, int64_t a_bs, int32_t a_div, const void* W, int32_t w_dtype, int32_t ldw, int64_t w_bs,
                            const int32_t* w_index, float* C, int32_t ldc, int64_t c_bs, int32_t batch, int32_t N, int32_t K, int32_t round_a,
                            sllm_stream_t stream);
/* 1 when sllm_seq_linear with a bf16 scratch sends this shape to the tensor cores (the weights must also be 16-byte aligned) */
int sllm_seq_linear_on_tensor_cores(int32_t T, int32_t N, int32_t K, int32_t w_dtype, int32_t ldw, int32_t batch, int32_t round_a);
/* PolyNorm: out = c0*N(z) + c1*N(z^2) + c2*N(z^3) + c3, powers element-wise, N(v) = v / sqrt(mean(v^2) + eps) over a row; coef: 4 floats */
int sllm_seq_polynorm(const float* z, int32_t ldz, const float* coef, float eps, float* out, int32_t ldo, int32_t T, int32_t n,
                      sllm_stream_t stream);
/* out[i][:] = x[rows[i]][:] (n rows of d floats) */
int sllm_seq_gather_rows(const float* x, int32_t ldx, const int32_t* rows, int32_t n, int32_t d, float* out, sllm_stream_t stream);
/* Rotary positions on q (in place) and k, rotated values, and the cache write: the first 2*n_freq dimensions of every q / k head turn
 * by pos * freq[i] with cos and sin multiplied by `magnitude`; every value head turns over all its dv dimensions by pos * vfreq[m]
 * (vfreq NULL = values are stored as they are); freq and vfreq are DOUBLE arrays and the angle is formed in double, so that its error does not
 * grow with the position. layout 0 pairs dimension 2i with 2i+1, layout 1 pairs i with i + half. k and v go to
 * their pools at (page of pos, kv head, pos % page_len). */
int sllm_seq_rotary_kv(const sllm_seq_batch* b, float* q, int32_t ldq, int32_t heads, int32_t dk, const float* k, int32_t ldk,
                       int32_t kv_heads, const float* v, int32_t ldv, int32_t dv, const double* freq, int32_t n_freq, float magnitude,
                       const double* vfreq, int32_t layout, void* k_pool, void* v_pool, int32_t kv_dtype, sllm_stream_t stream);
/* What an attention launch may ask for beyond plain causal softmax (NULL = none of it). */
typedef struct {
    int32_t window;          /* > 0: query i sees key j <= i only when i - j < window or j < keep_first; 0 = every key before it */
    int32_t keep_first;      /* the first positions of a sequence stay visible behind the window, at their true positions */
    float softcap;           /* > 0: score <- softcap * tanh(score / softcap), after the scale */
    const float* slopes;     /* [heads] or NULL: score <- score - slopes[h] * (i - j), after the cap */
    int32_t values_in_keys;  /* != 0: a value row is the first dv columns of the key row (one pool; v_pool is not read) */
    const float* logdist;    /* [2][heads] or NULL: score <- score - r1[h] * ln(1 + r2[h] * (i - j)) with r1 = row 0, r2 = row 1 */
    int32_t cross_values;    /* != 0: every query head's weights are applied to the values of EVERY key/value head (the keys it reads stay
                              * those of its own): ws holds kv_heads * heads records per token, record (value head * heads + query head) */
} sllm_seq_attn_opts;
/* Causal softmax attention of every token over positions 0..pos of its own sequence: score = (q . k) * scale, query head h reads
 * key/value head h / (heads / kv_heads). Keys are visited in tiles of 32, cut into nsplit interleaved shares; the partial results
 * (running maximum, sum, unnormalised output) go to ws: [T][heads][nsplit][dv + 2] floats. Tiles that a window hides from all queries
 * of a work item are not loaded. */
int sllm_seq_attention(const sllm_seq_batch* b, const float* q, int32_t ldq, int32_t heads, int32_t kv_heads, int32_t dk, int32_t dv,
                       float scale, const void* k_pool, const void* v_pool, int32_t kv_dtype, int32_t nsplit, float* ws,
                       const sllm_seq_attn_opts* opts, sllm_stream_t stream);
/* Merges the shares, normalises (sink [heads] or NULL: the denominator of head h also holds exp(sink[h]), a term without key or value),
 * turns every head's output back by -pos * vfreq[m] (vfreq NULL = not), multiplies head h by sigmoid(gate[t][h]) (gate NULL = not) and
 * stores out[t][h*dv ..]. */
int sllm_seq_attention_finish(const sllm_seq_batch* b, const float* ws, int32_t nsplit, int32_t heads, int32_t dv, const double* vfreq,
                              int32_t layout, const float* gate, int32_t ldg, const float* sink, float* out, int32_t ldo,
                              sllm_stream_t stream);
/* Heads scaled to unit root mean square and the cache write, for mixers without rotation: bit 0 of `unit` = every query head of q (in
 * place), bit 1 = every key head, bit 2 = every value head is divided by sqrt(mean(head^2) + eps). share 1: the values (after the
 * division) are also kept in v_shared [T][kv_heads*dv]; share 2: v <- (1 - lambda) * v + lambda * v_shared (what an earlier layer kept
 * for the same tokens). k and v go to their pools at (page of pos, kv head, pos % page_len). q_temp_every > 0: every query is also
 * multiplied by 1 + q_temp_coef * ln(floor((pos + 1) / q_temp_every) + 1), a temperature that grows with the position. */
int sllm_seq_unit_kv(const sllm_seq_batch* b, float* q, int32_t ldq, int32_t heads, int32_t dk, const float* k, int32_t ldk,
                     int32_t kv_heads, const float* v, int32_t ldv, int32_t dv, float eps, int32_t unit, float* v_shared, int32_t share,
                     float lambda, void* k_pool, void* v_pool, int32_t kv_dtype, float q_temp_coef, int32_t q_temp_every, sllm_stream_t stream);
/* Latent attention's cache write: low [T][rank + dr] is one token's low-rank row; its first `rank` entries, RMS-normed with norm_w, and
 * its last dr entries, the first 2*n_freq of them rotated by pos * freq[i] (interleaved pairs, angles in double), form the pool row
 * [pages][1][page_len][rank + dr]. q [T][heads][dn + dr]: the dr-part of every head is rotated the same way and stored at
 * q_out[t][h][rank ..] (q_out rows of heads * (rank + dr); the first `rank` columns of a head belong to the absorbed query). cos and sin
 * are multiplied by `magnitude`. low NULL: nothing is cached (the layer attends over another layer's rows), only the queries turn. */
int sllm_seq_latent_kv(const sllm_seq_batch* b, const float* q, int32_t ldq, int32_t heads, int32_t dn, int32_t dr, const float* low,
                       int32_t ldlow, int32_t rank, const float* norm_w, float eps, const double* freq, int32_t n_freq, float* q_out,
                       int32_t ldqo, void* pool, int32_t kv_dtype, float magnitude, sllm_stream_t stream);
/* ---- blocks of models whose sublayers sit between scalar RMS norms and read through a short convolution; the gated delta rule; a
 * mixture of experts ---- */
/* out[t] = table[ids[t]] + pairs[row], row = (prev_ids[t] * mul_prev + ids[t] * mul_cur) mod buckets, or row `buckets` (the last of the
 * buckets + 1 rows) when prev_ids[t] < 0: the sequence's first token */
int sllm_seq_embed_pair(const int32_t* ids, const int32_t* prev_ids, const void* table, const void* pairs, int32_t w_dtype, int32_t vocab,
                        int32_t d, int32_t buckets, int64_t mul_prev, int64_t mul_cur, float* out, int32_t T, sllm_stream_t stream);
/* y = x / sqrt(mean(x^2) + eps) * w per row of n floats (w NULL = no weight) */
int sllm_seq_rmsnorm_rows(const float* x, int32_t ldx, const float* w, float eps, float* y, int32_t ldy, int32_t T, int32_t n,
                          sllm_stream_t stream);
/* out = act(gate) * up (act 0 = silu); out fp32 [T][ldo] and / or out16 dense bf16 [T][n] (the operand of a tensor-core product) */
int sllm_seq_gated_act(const float* gate, int32_t ldg, const float* up, int32_t ldu, int32_t act, float* out, int32_t ldo, void* out16,
                       int32_t T, int32_t n, sllm_stream_t stream);
/* x <- cap * tanh(x / cap) over n floats */
int sllm_seq_softcap(float* x, int64_t n, float cap, sllm_stream_t stream);
/* The seam between two sublayers, one kernel: (1) if y: x_out = x_in + post_g * y / rms(y) (x_out != x_in); (2) if has_pre:
 * n = pre_g * x / rms(x), h = n + conv(n) with conv_w [d][taps] (last column = the current token; NULL = h = n) reaching back into
 * the step's rows and, before a portion, into ring [slots][taps-1][d] (position p at row p % (taps-1)); h16 (or NULL) = h as dense
 * bf16 rows; (3) the normed rows of every portion's last taps-1 tokens go to stash [T][d]; a later call with flush_ring (the ring this
 * call read) moves them there. rms(v) = sqrt(mean(v^2) + eps). scales (or NULL): T floats of scratch; with it, steps of 64 tokens and
 * more run as two launches (sum and per-row scale, then the convolution element-wise) so that no row is normed more than once.
 * post_norm 0: the sum takes y as it is, x_out = x_in + y (a pre-norm layer). pre_w (or NULL) [d]: a weight per channel on the normed
 * row, stored as its distance from pre_w_offset: n[c] = pre_g * (pre_w_offset + pre_w[c]) * x[c] / rms(x). */
int sllm_seq_seam(const sllm_seq_batch* b, const float* x_in, float* x_out, const float* y, float post_g, int32_t has_pre, float pre_g,
                  float eps, const float* conv_w, int32_t taps, const float* ring, float* h, void* h16, float* stash, float* flush_ring,
                  int32_t flush_taps, int32_t d, float* scales, int32_t post_norm, const float* pre_w, float pre_w_offset, sllm_stream_t stream);
/* out[t][c] = act(cb[c] + sum_j w[c][j] * x[t - taps + 1 + j][c]) (cb NULL = no bias; act 0 = none, 1 = silu), zeros before a sequence's
 * start; inputs before a portion come from ring [slots][taps-1][channels] (position p at row p % (taps-1)), which is NOT updated here
 * (sllm_seq_delta_rule, sllm_seq_ssd_scan, sllm_seq_selective_scan and sllm_seq_ring_store do that, after the convolution has run) */
int sllm_seq_conv_ring(const sllm_seq_batch* b, const float* x, int32_t ldx, int32_t channels, int32_t taps, const float* w, const float* cb,
                       const float* ring, int32_t act, float* out, int32_t ldo, sllm_stream_t stream);
/* ring[slot][p % (taps-1)][:] <- x[t][0 .. channels) for the last taps-1 tokens of every portion (p = the token's position) */
int sllm_seq_ring_store(const sllm_seq_batch* b, const float* x, int32_t ldx, int32_t channels, int32_t taps, float* ring, sllm_stream_t stream);
/* Gated delta rule per head h over each sequence, state [slots][heads][dk][dv] fp32: S <- g S; u = beta (v - S^T k); S <- S + k u^T;
 * o = S^T q, with q, k (of key head h / (heads / kv_heads)) divided by sqrt(sum(x^2) + unit_eps), q times qscale,
 * beta = sigmoid(beta_logit), g = exp(-exp(A_log[h]) * softplus(step_logit + dt_bias[h])). ring (or NULL): the last taps-1 rows of
 * conv_x [T][channels] of every portion are stored there for the convolution of the next step. */
int sllm_seq_delta_rule(const sllm_seq_batch* b, const float* q, int32_t ldq, const float* k, int32_t ldk, const float* v, int32_t ldv,
                        const float* beta_logit, int32_t ldb, const float* step_logit, int32_t lda, const float* A_log, const float* dt_bias,
                        int32_t heads, int32_t kv_heads, int32_t dk, int32_t dv, float unit_eps, float qscale, float* state, float* o,
                        int32_t ldo, const float* conv_x, int32_t ldx, int32_t channels, int32_t taps, float* ring, sllm_stream_t stream);
/* State-space duality (Mamba-2) per head h over each sequence, state [slots][heads][n_state][dv] fp32: dt = softplus(step_logit + dt_bias[h]),
 * S <- exp(-exp(A_log[h]) dt) S + dt B x^T, y = S^T C + skip[h] x (skip NULL = no such term); x [T][heads * dv], B and C
 * [T][groups * n_state], head h reads group h / (heads / groups). The kernel of sllm_seq_delta_rule without its correction term; ring as there.
 * scratch (NULL = always token by token): (n_qtiles / 4 + nseg + 1) * heads * (n_state * dv + 1) floats; with it, steps that hold a portion
 * longer than 128 tokens run as three passes over ranges of 128 tokens (every range from zero, a carry per state element, every range again
 * from its start state). */
int sllm_seq_ssd_scan(const sllm_seq_batch* b, const float* x, int32_t ldx, const float* B, int32_t ldb, const float* C, int32_t ldc,
                      const float* step_logit, int32_t lda, const float* A_log, const float* dt_bias, const float* skip, int32_t heads, int32_t groups,
                      int32_t n_state, int32_t dv, float* state, float* y, int32_t ldy, const float* conv_x, int32_t ld_conv, int32_t channels,
                      int32_t taps, float* ring, float* scratch, sllm_stream_t stream);
/* Selective scan (Mamba) per channel c over each sequence, state [slots][inner][n_state] fp32: dt = softplus(step_logit[c]),
 * S[c][n] <- exp(-dt exp(A_log[c][n])) S[c][n] + dt x[c] B[n], y[c] = sum_n S[c][n] C[n] + D[c] x[c], out = y * silu(z); B and C [T][n_state]
 * are shared by the channels. out fp32 [T][ldo] and / or out16 dense bf16 [T][inner]. ring (or NULL): the last taps-1 rows of conv_x
 * [T][inner] of every portion are stored there for the convolution of the next step. n_state <= 256. scratch (NULL = always token by token):
 * n_qtiles * inner * (n_state + 1) floats; with it, steps that hold a portion longer than 128 tokens run as three passes over ranges of 128
 * tokens (every range from zero, a carry per state element, every range again from its start state). */
int sllm_seq_selective_scan(const sllm_seq_batch* b, const float* x, int32_t ldx, const float* step_logit, int32_t lddt, const float* B, int32_t ldb,
                            const float* C, int32_t ldc, const float* z, int32_t ldz, const float* A_log, const float* D, int32_t inner,
                            int32_t n_state, float* state, float* out, int32_t ldo, void* out16, const float* conv_x, int32_t ld_conv, int32_t taps,
                            float* ring, float* scratch, sllm_stream_t stream);
/* Query and key heads RMS-normed over their dk dimensions with a weight [dk] shared by the heads (q_norm_w / k_norm_w, NULL = that kind
 * is not normed), then their first 2*n_freq dimensions turned by pos * freq[i] (layout and angles as in sllm_seq_rotary_kv); q in place,
 * k to its pool; v [T][kv_heads * dv] goes to its pool as it is (it may be k itself: values that are the keys before norm and rotation). */
int sllm_seq_normed_rotary_kv(const sllm_seq_batch* b, float* q, int32_t ldq, int32_t heads, int32_t dk, const float* k, int32_t ldk,
                              int32_t kv_heads, const float* v, int32_t ldv, int32_t dv, const float* q_norm_w, const float* k_norm_w, float eps,
                              const double* freq, int32_t n_freq, int32_t layout, void* k_pool, void* v_pool, int32_t kv_dtype,
                              sllm_stream_t stream);
/* Heads mixed after the attention: in [T][kv_heads * heads * dv] as sllm_seq_attention_finish leaves it for cross_values (record = value
 * head * heads + query head); out[t][h] = sum_g mix[h][g] * in[t][(h / (heads / kv_heads)) * heads + g]: head h's mixed weights on the
 * values of its own key/value head. out fp32 [T][ldo] and / or out16 dense bf16 [T][heads * dv]. */
int sllm_seq_head_mix(const float* in, int32_t ldi, const float* mix, int32_t heads, int32_t kv_heads, int32_t dv, float* out, int32_t ldo,
                      void* out16, int32_t T, sllm_stream_t stream);
/* Bits of the `act` argument of the mixture-of-experts calls beside the activation (bits 0-1): scores = sigmoid of each router output by
 * itself instead of the softmax over all; gated experts, whose `up` columns are [gate ff | up ff] and which compute act(gate) * up; the
 * score multiplies what the expert reads instead of what it returns. */
#define SLLM_MOE_GATED 4
#define SLLM_MOE_SCALE_INPUT 8
#define SLLM_MOE_SIGMOID 16
/* Routing and activation of a mixture of experts, per token: s = softmax(logits[0..n_route)); the `top` largest s + correction are
 * chosen (correction NULL = none; the lower index wins a tie); out / out16 [T][experts * ff] = act(up) * s for chosen experts with
 * weights (the first `experts` router outputs), zeros for the others; y [T][d] = (sum of s over chosen router outputs >= experts) * h:
 * those are experts whose output is their input. act 0 = exact gelu, 1 = tanh gelu, 2 = silu. route_w (or NULL) [T][n_route] = the
 * weights, zero where not chosen. */
int sllm_seq_moe_act(const float* logits, int32_t ldl, int32_t n_route, int32_t experts, int32_t top, const float* correction, const float* up,
                     int32_t ldu, int32_t ff, int32_t act, const float* h, int32_t ldh, int32_t d, float* out, void* out16, float* y,
                     int32_t ldy, float* route_w, int32_t T, sllm_stream_t stream);
/* The same layer with the tokens gathered per expert, for steps of many tokens. sllm_seq_moe_route: routing as above; every (token,
 * chosen expert with weights) pair takes the next free row of that expert's buffer (counts [experts] int32, zeroed before the call;
 * buffers of cap >= T rows) and the token's input row h is copied there as bf16 (rows16 [experts][cap][d]) and / or fp32 (rows32);
 * sel_e / sel_pos / sel_w [T][top] = expert (-1: none), row and score of each choice, ident [T] = the sum of the chosen identity scores.
 * Which row a pair gets depends on timing; the numbers in it do not. sllm_seq_moe_expert_act: act over the rows in use of
 * up [experts][cap][ff]. sllm_seq_moe_combine: y[t] = ident[t] * h[t] + sum_k sel_w * down[sel_e][sel_pos] (down [experts][cap][d]). */
int sllm_seq_moe_route(const float* logits, int32_t ldl, int32_t n_route, int32_t experts, int32_t top, const float* correction, const float* h,
                       int32_t ldh, int32_t d, int32_t* counts, int32_t cap, int32_t* sel_e, int32_t* sel_pos, float* sel_w, float* ident,
                       void* rows16, float* rows32, int32_t T, int32_t act, sllm_stream_t stream);
int sllm_seq_moe_expert_act(const float* up, const int32_t* counts, int32_t experts, int32_t cap, int32_t ff, int32_t act, void* out16,
                            float* out32, sllm_stream_t stream);
/* For experts chosen on the device (rows in the order of the (token, choice) pairs, sel_w the pairs' scores as sllm_seq_moe_route leaves them
 * WITHOUT SLLM_MOE_SCALE_INPUT): out [pairs][ff] = act(s * up) or, gated, act(s * gate) * (s * up) over up [pairs][ff or 2 ff], s = the score
 * when `act` has SLLM_MOE_SCALE_INPUT and 1 otherwise; w_out [pairs] = the weight sllm_seq_moe_combine has to use (1, or the score). */
int sllm_seq_moe_pair_act(const float* up, const float* sel_w, int32_t pairs, int32_t ff, int32_t act, float* out, float* w_out, sllm_stream_t stream);
int sllm_seq_moe_combine(const float* down, const int32_t* sel_e, const int32_t* sel_pos, const float* sel_w, int32_t top, const float* ident,
                         const float* h, int32_t ldh, int32_t cap, int32_t d, float* y, int32_t ldy, int32_t T, sllm_stream_t stream);
/* x <- act(x) over n floats (act as in sllm_seq_moe_act). With counts, rows16 and rows32 all NULL sllm_seq_moe_route only routes: nothing is
 * gathered and sel_pos of pair (t, k) is t * top + k. */
int sllm_seq_act(float* x, int64_t n, int32_t act, sllm_stream_t stream);
/* n_bytes of zeros at p, in stream order */
int sllm_seq_zero(void* p, int64_t n_bytes, sllm_stream_t stream);
/* y = (x - mean) / sqrt(mean((x - mean)^2) + eps) * w + bias per row (bias NULL = none); y16 (or NULL): the same rows once more, rounded
 * to bf16, dense [T][d] — the operand copy of a tensor-core product that follows */
int sllm_seq_layernorm(const float* x, int32_t ldx, const float* w, const float* bias, float eps, float* y, int32_t ldy, void* y16,
                       int32_t T, int32_t d, sllm_stream_t stream);
/* Depth-weighted average: hist [n_prev + 1 ..][T][d] holds the embedding output and every earlier layer's own result. Stores this
 * layer's result hist[n_prev] = x + y, replaces x by sum_{j <= n_prev} coef[j] * hist[j], and, with norm_w, writes the layer norm
 * (norm_w, norm_b, eps) of the new x to h, and to h16 (if given) as dense bf16 rows. */
int sllm_seq_depth_average(float* x, const float* y, float* hist, int32_t n_prev, const float* coef, const float* norm_w,
                           const float* norm_b, float eps, float* h, void* h16, int32_t T, int32_t d, sllm_stream_t stream);
/* out = g * sigmoid(alpha * g) * (u + 1), g = min(gate, limit), u = clamp(up, -limit, limit), element-wise over [T][n]; out16 (or NULL):
 * the result also as dense bf16 [T][n] (then out may be NULL) */
int sllm_seq_clamped_glu(const float* gate, int32_t ldg, const float* up, int32_t ldu, float limit, float alpha, float* out, int32_t ldo,
                         void* out16, int32_t T, int32_t n, sllm_stream_t stream);
/* Causal convolution per channel over each sequence: u[t][c] = cb[c] + sum_k w[c][k] * x[t - (taps-1-k)][c]; inputs before the segment
 * come from tail[slot][taps-1][channels] (zeros for a new sequence). The tail is NOT updated here (sllm_seq_rglru_scan does it). */
int sllm_seq_conv(const sllm_seq_batch* b, const float* x, int32_t ldx, int32_t channels, int32_t taps, const float* w, const float* cb,
                  const float* tail, float* u, int32_t ldu, sllm_stream_t stream);
/* Real-gated linear recurrent unit: r = sigmoid(lr), i = sigmoid(li), log a = -c * r * softplus(lam), S <- a*S + sqrt(1 - a^2) * i * u,
 * out = S * gelu_tanh(ypre). state: [slots][channels] fp32, read and written. Also moves the convolution tail on: tail[slot] <- the
 * last taps-1 rows of (tail[slot] ++ xconv rows of the segment) (xconv NULL = no tail). scratch (NULL = always token by token): 2 * n_qtiles *
 * channels doubles; with it, steps that hold a portion longer than 32 tokens run as three passes over tiles (tile summaries, carry, outputs). */
int sllm_seq_rglru_scan(const sllm_seq_batch* b, const float* u, int32_t ldu, const float* lr, const float* li, int32_t ldg,
                        const float* ypre, int32_t ldy, const float* lam, float c, int32_t channels, float* state, const float* xconv,
                        int32_t ldx, int32_t taps, float* tail, float* out, int32_t ldo, void* scratch, sllm_stream_t stream);
/* Gated linear attention, token by token per head: alpha = sigmoid(z)^(1/tau) per key channel, S <- diag(alpha) S + k v^T (S: dk x dv),
 * o = S^T (q * qscale). state: [slots][heads][dk][dv] fp32, read and written. dk/32 (rounded up) * dv (rounded up to 32) <= 1024.
 * scratch (NULL = always token by token): n_qtiles * heads * dk (rounded up to 64) + n_qtiles * heads * dk * dv floats, for the
 * three-pass form of steps that hold a portion longer than 32 tokens. */
int sllm_seq_gla_scan(const sllm_seq_batch* b, const float* q, int32_t ldq, const float* k, int32_t ldk, const float* v, int32_t ldv,
                      const float* z, int32_t ldz, int32_t heads, int32_t dk, int32_t dv, float qscale, float tau, float* state, float* o,
                      int32_t ldo, void* scratch, sllm_stream_t stream);
/* out[t][h*dv + j] = o[t][h*dv + j] / sqrt(mean_j(o^2) + eps) * w[j] * silu(g[t][h*dv + j]). mode bit 0: the gate comes first,
 * u = o * silu(g), out = u / sqrt(mean_j(u^2) + eps) * w; bit 1: w has heads * dv entries (one per channel of the row) instead of dv.
 * out fp32 and / or out16 dense bf16 [T][heads * dv]. */
int sllm_seq_headnorm_gate(const float* o, int32_t ldo, const float* g, int32_t ldg, const float* w, int32_t heads, int32_t dv, float eps,
                           float* out, int32_t ldout, void* out16, int32_t T, int32_t mode, sllm_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* SLLM_B200_H */
