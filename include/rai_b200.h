/* rai_b200 — C ABI of the B200 (sm_100a) execution backend for the decoder hot path of cksac/rai.
 *
 * This header is what a rai-side FFI binding (Rust `extern "C"`, or the ctypes binding shipped in
 * rai_b200/_lib.py) binds.  Each entry point names the reference interface it stands in for, as
 * `path:line` inside the rai source tree.
 *
 * Conventions
 *   - every function returns an int32 status (RB_OK == 0, negative on failure); the text of the last
 *     failure of the calling thread is available through rb_last_error().  rai's Eval rules have no
 *     error channel and unwrap (rai-core/src/backend/candle.rs, every rule), so a binding is
 *     expected to panic on a non-zero status.
 *   - pointers named *_dev are device pointers on the context's GPU; the library never takes
 *     ownership of caller memory.
 *   - all work is enqueued on the context's stream and is asynchronous unless stated otherwise.
 *   - the library never aborts the process, never traps the device and never blocks without bound:
 *     device-side waits give up after about a second and report through rb_status_word().
 */
#ifndef RAI_B200_H_
#define RAI_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library is built with hidden visibility; these are its exports */
#endif

/* ---- status codes (rai-core/src/error.rs:5-51 is the error convention of the reference) ---- */
enum {
  RB_OK = 0,
  RB_ERR_INVALID = -1,       /* bad argument */
  RB_ERR_SHAPE = -2,         /* OpError::IncompatibleShape */
  RB_ERR_DTYPE = -3,         /* unsupported dtype for this entry point */
  RB_ERR_OOM = -4,
  RB_ERR_CUDA = -5,
  RB_ERR_TIMEOUT = -6,       /* a device-side wait gave up, see rb_status_word */
  RB_ERR_UNIMPLEMENTED = -7, /* Error::Unimplemented{op,device}, rai-core/src/eval.rs:40-43 */
  RB_ERR_PARAM = -8          /* Error::ParamNotFound, rai-core/src/nn.rs:192-205 */
};

/* ---- dtype tags, same set and order as rai-core/src/dtype.rs:198-524 ---- */
enum { RB_U8 = 0, RB_U32 = 1, RB_I64 = 2, RB_F16 = 3, RB_BF16 = 4, RB_F32 = 5, RB_F64 = 6 };

/* ---- activations, rai-nn/src/activations.rs:5-30 and rai-core/src/hlops/activations.rs:5-32 ---- */
enum { RB_ACT_NONE = 0, RB_ACT_SILU = 1, RB_ACT_GELU_TANH = 2, RB_ACT_GELU_ERF = 3, RB_ACT_RELU = 4 };

/* ---- norm kinds ---- */
enum {
  RB_NORM_RMS = 0,          /* rai-nn/src/rms_norm.rs:18-22 */
  RB_NORM_RMS_ONE_PLUS = 1, /* rai-models/src/llm/gemma.rs:42-54 */
  RB_NORM_LAYER = 2         /* rai-nn/src/layer_norm.rs:32-42 */
};

/* ---- decoder families, rai-models/src/llm/{qwen2,phi2,phi3,gemma}.rs ---- */
enum { RB_ARCH_QWEN2 = 0, RB_ARCH_PHI2 = 1, RB_ARCH_PHI3 = 2, RB_ARCH_GEMMA = 3 };

/* ---- elementwise / reduce op tags of the primitive set (rai-core/src/dispatch.rs:41-157) ---- */
enum {
  RB_UN_NEG = 0, RB_UN_EXP, RB_UN_SQRT, RB_UN_RSQRT, RB_UN_SQUARE, RB_UN_TANH, RB_UN_ERF, RB_UN_SIN,
  RB_UN_COS, RB_UN_POWF, RB_UN_SILU, RB_UN_GELU_TANH, RB_UN_GELU_ERF, RB_UN_RELU, RB_UN_LOG, RB_UN_ABS,
  RB_UN_RECIP, RB_UN_ADD_SCALAR, RB_UN_MUL_SCALAR, RB_UN_SIGN, RB_UN_LOG2, RB_UN_LOG10
};
enum { RB_CMP_EQ = 0, RB_CMP_NE, RB_CMP_GT, RB_CMP_GE, RB_CMP_LT, RB_CMP_LE };
enum { RB_BIN_ADD = 0, RB_BIN_SUB, RB_BIN_MUL, RB_BIN_DIV, RB_BIN_MAXIMUM, RB_BIN_MINIMUM };
enum { RB_RED_SUM = 0, RB_RED_MAX, RB_RED_MIN };

typedef struct rb_ctx rb_ctx;
typedef struct rb_kv_cache rb_kv_cache;
typedef struct rb_model rb_model;
typedef struct rb_safetensors rb_safetensors;

/* ======================================================================================
 * Context — one per (process, GPU).  Stands in for the device cache of the reference backend
 * (rai-core/src/backend/candle.rs:139-195) and for `Cuda::new(id)` (rai-core/src/device.rs:161-196).
 * Not thread-safe per context.
 * ====================================================================================== */
int32_t rb_init(int32_t device, rb_ctx** out);
int32_t rb_destroy(rb_ctx* ctx);
/* Enqueue on an existing cudaStream_t (for instance the host framework's current stream) instead of
 * the stream the context created for itself; NULL selects CUDA's default stream. */
int32_t rb_set_stream(rb_ctx* ctx, void* cuda_stream);
/* Blocks until the stream is idle, then reports device-side give-ups (RB_ERR_TIMEOUT). */
int32_t rb_sync(rb_ctx* ctx);
const char* rb_last_error(void);
/* Copies the 4-word device status record {code, where, detail0, detail1} to `out4` (synchronises). */
int32_t rb_status_word(rb_ctx* ctx, uint32_t* out4);
int32_t rb_sm_count(rb_ctx* ctx);
/* How long a device-side wait for a tensor-parallel peer may last before the kernel gives up, reports
 * RB_ERR_TIMEOUT through the status word and returns; waits inside one kernel (on a copy, a tensor-core result, a
 * sibling block) get four times as long, so that a missing peer is reported by the exchange that waited for it and
 * not by a kernel queued behind it.  Default: about one second.
 * Stands in for nothing in the reference, whose only device code is candle's; it is the knob behind the
 * "never blocks without bound" convention above.  Applies to launches made after the call. */
int32_t rb_set_wait_budget_us(rb_ctx* ctx, int64_t microseconds);
/* Self-test of the give-up path, for test suites: runs a kernel whose wait can never be satisfied (`which` 0: an
 * mbarrier nothing arrives on, waited for with the library's own helper; 1: the tensor-parallel exchange of a
 * two-member group whose second member, zeroed memory of this GPU, never raises its flag; 2: the same exchange
 * in its flag-inside-the-data form, whose second member's words never show the exchange number; 3: that form over
 * two hops, where one row waits for the other member's share and the other row for its finished sum), with the given
 * budget.  The kernel returns when the budget runs out; RB_OK means the give-up was recorded as designed
 * (RB_ERR_TIMEOUT with the kernel's tag, outputs untouched), and the status word is clear again on return.
 * Nothing faults, traps or spins without bound.  No counterpart in the reference. */
int32_t rb_selftest_wait_gives_up(rb_ctx* ctx, int32_t which, int64_t budget_us);

/* Device memory owned by the library (`TensorLike` storage, rai-core/src/tensor.rs:19-26). */
int32_t rb_malloc(rb_ctx* ctx, size_t bytes, void** out_dev);
int32_t rb_free(rb_ctx* ctx, void* dev);
/* The same pair, stream-ordered and pooled (cudaMallocAsync / cudaFreeAsync on the context's stream): what a
 * binding uses for the output of every primitive, where the reference's rules let candle allocate
 * (candle.rs:197-1004) and drop storage with the last Rc (tensor.rs:34).  Neither call synchronises; a block
 * freed here may be handed out again by a later rb_malloc_async and is safe to reuse in stream order.  Not
 * for memory that is shared between processes (use rb_malloc). */
int32_t rb_malloc_async(rb_ctx* ctx, size_t bytes, void** out_dev);
int32_t rb_free_async(rb_ctx* ctx, void* dev);
/* ToDevice<Cuda> on Cpu data / ToDevice<Cpu> on Cuda data (rai-core/src/backend/candle.rs:776-790).
 * rb_download synchronises the stream. */
int32_t rb_upload(rb_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
int32_t rb_download(rb_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes);

/* ======================================================================================
 * Fused decoder kernels.  `dtype` is RB_BF16 (tensor-core path) or RB_F32 (plain fp32 path).
 * ====================================================================================== */

/* Embedding::fwd, rai-nn/src/embedding.rs:25-30 (+ the `* sqrt(H)` of gemma.rs:379 when scale != 1).
 * out[i, :] = table[ids[i], :] * scale.  With scale == 1 the rows are copied bit for bit. */
int32_t rb_embed_gather(rb_ctx* ctx, const void* table_dev, int32_t dtype, int64_t vocab, int64_t hidden,
                        const uint32_t* ids_dev, int64_t n_ids, float scale, void* out_dev);

/* RmsNorm::fwd / gemma RmsNorm::fwd / LayerNorm::fwd (see RB_NORM_*), fused with the residual add of
 * DecoderLayer::fwd (rai-models/src/llm/qwen2.rs:262,265) and with the reduction of split-K GEMM
 * partials:  v = x + add + sum_s acc[s] + acc_bias ;  sum_out = v ;  out = norm(v).
 * x, add, acc (float32, n_acc slabs of rows*hidden), acc_bias, bias, sum_out and out may each be NULL
 * (at least one of x/add/acc must be given; out and sum_out may alias x or add). */
int32_t rb_norm(rb_ctx* ctx, int32_t kind, const void* x_dev, const void* add_dev, const float* acc_dev,
                int32_t n_acc, const void* acc_bias_dev, const void* weight_dev, const void* bias_dev, float eps,
                int64_t rows, int64_t hidden, void* out_dev, void* sum_out_dev, int32_t dtype);

/* Linear::fwd, rai-nn/src/linear.rs:59-69, as ONE [M,K]x[N,K]^T GEMM with the bias add, the
 * activation (rai-nn/src/activations.rs:19-30) and the residual add fused into the epilogue:
 *   out = act(x . W^T + bias) + residual.   bias / residual may be NULL.  W is [N, K] row-major. */
int32_t rb_linear(rb_ctx* ctx, const void* x_dev, const void* w_dev, const void* bias_dev, const void* residual_dev,
                  void* out_dev, int64_t m, int64_t n, int64_t k, int32_t act, int32_t dtype);

/* MLP::fwd gate/up half, rai-models/src/llm/qwen2.rs:100-103, gemma.rs:131-134, phi3.rs:101-105:
 *   out = act(x . Wg^T) * (x . Wu^T).   Wg and Wu are [N, K]. */
int32_t rb_gated_linear(rb_ctx* ctx, const void* x_dev, const void* wg_dev, const void* wu_dev, void* out_dev,
                        int64_t m, int64_t n, int64_t k, int32_t act, int32_t dtype);

/* Split-K form of rb_linear for skinny M (decode): writes `n_split` float32 partial products
 * part[s][m][n]; the consumer (rb_norm / rb_rope_kv_append) sums them in a fixed order, so results
 * are deterministic.  bf16 only.  Needs n_split * m * n * 4 bytes at part_dev (scratch memory). */
int32_t rb_linear_partials(rb_ctx* ctx, const void* x_dev, const void* w_dev, float* part_dev, int64_t m, int64_t n,
                           int64_t k, int32_t n_split);
/* The split count the library would pick for this shape on this GPU (>= 1). */
int32_t rb_linear_pick_splits(rb_ctx* ctx, int64_t m, int64_t n, int64_t k);

/* Paged KV cache.  Replaces the `kv_cache: RefCell<Option<(Tensor,Tensor)>>` of Attention and its
 * growth by Tensor::cat (rai-models/src/llm/qwen2.rs:127,193-204; phi2.rs:225-243; phi3.rs:186-197;
 * gemma.rs:226-237).  Pages hold 64 tokens of one KV head: [layer][page][kv_head][64][head_dim]. */
int32_t rb_kv_cache_create(rb_ctx* ctx, int32_t layers, int32_t kv_heads, int32_t head_dim, int32_t max_batch,
                           int32_t max_seq, int32_t dtype, rb_kv_cache** out);
int32_t rb_kv_cache_destroy(rb_kv_cache* c);
/* clear_kv_cache, rai-models/src/llm/qwen2.rs:361-365: every sequence length back to 0. */
int32_t rb_kv_cache_reset(rb_kv_cache* c);
/* The sliding-window term of qwen2's mask (rai-models/src/llm/qwen2.rs:316-334): attention over this cache hides
 * key j from query i when both belong to the tokens of the same call and j + window < i (the reference's mask
 * leaves the cached prefix visible, and builds no mask for a single-token call).  Default: no window. */
int32_t rb_kv_cache_set_window(rb_kv_cache* c, int32_t window);
/* Host-side bookkeeping of Model::fwd's seqlen_offset: sequences 0..batch-1 now hold pos+s_new tokens. */
int32_t rb_kv_cache_set_len(rb_kv_cache* c, int32_t batch, int32_t len);
/* Test hook: copies K and V of tokens [t0, t0+n) of (layer, seq, kv_head) to host as [n, head_dim]. */
int32_t rb_kv_cache_read(rb_kv_cache* c, int32_t layer, int32_t seq, int32_t kv_head, int32_t t0, int32_t n,
                         void* k_host, void* v_host);

/* RotaryEmbedding::new, rai-models/src/llm/qwen2.rs:40-60 (recipe 0, also gemma.rs:71-91),
 * phi2.rs:44-64 (recipe 1), phi3.rs:40-61 (recipe 2): float32 cos/sin tables [max_pos, rot_dim/2]. */
int32_t rb_rope_tables(rb_ctx* ctx, int32_t recipe, int32_t rot_dim, int32_t max_pos, double theta, float* cos_dev,
                       float* sin_dev);

/* Head split + RotaryEmbedding::fwd + KV-cache append (rai-models/src/llm/qwen2.rs:180-204,62-71;
 * phi2.rs:66-77; phi3.rs:63-74) in one pass over the fused qkv projection.
 *   v = qkv + sum_s acc[s] + bias  (qkv or acc may be NULL), columns = [q heads | k heads | v heads];
 *   q_out[m, h*d + i] = rope(q);  K/V of token m go to position (len[b] - s_new + m % s_new) of
 *   sequence b = m / s_new, where len[] are the cache's device-side sequence lengths. */
int32_t rb_rope_kv_append(rb_ctx* ctx, const void* qkv_dev, const float* acc_dev, int32_t n_acc, const void* bias_dev,
                          const float* cos_dev, const float* sin_dev, int32_t rot_dim, int32_t batch, int32_t s_new,
                          int32_t q_heads, rb_kv_cache* cache, int32_t layer, void* q_out_dev, int32_t dtype);

/* Attention core, rai-models/src/llm/qwen2.rs:205-216 (repeat_kv + QK^T*scale + mask + softmax + PV),
 * phi2.rs:245-261, phi3.rs:199-209, gemma.rs:238-249, without materialising scores, masks or
 * repeated KV heads.  q is [batch*s_new, q_heads*head_dim]; out has the same layout (the
 * transpose(1,2).reshape of qwen2.rs:217-219 is implicit).  Causal: query s attends to keys
 * [0, len - s_new + s].  Reads K/V from the cache (rb_rope_kv_append must have run). */
int32_t rb_attention(rb_ctx* ctx, const void* q_dev, rb_kv_cache* cache, int32_t layer, int32_t batch, int32_t s_new,
                     int32_t q_heads, float scale, void* out_dev, int32_t dtype);

/* No counterpart in the reference.  Single-token (decode) attention like rb_attention with s_new = 1,
 * bf16 only, for callers that must not trigger a device allocation: rb_attention grows its split-KV
 * scratch with cudaMalloc when a larger shape arrives, which is off limits to a host runtime that owns
 * all device memory through its own pool, and unwelcome in a serving loop because an allocation can
 * synchronise the whole device.  This variant keeps that scratch in a 2 MiB array built into the
 * library (held by every GPU that loads it, until exit) and calls neither cudaMalloc nor cudaFree nor any
 * allocating library routine.  (The CUDA runtime itself may still load a kernel's code the first time that
 * kernel is launched: make the first call per head size before the host's pool takes the remaining memory.)
 *   - limit: batch * q_heads * splits * (head_dim + 2) floats must fit in 512 Ki floats; larger shapes are
 *     rejected with RB_ERR_INVALID and a message naming the sizes (use rb_attention for those);
 *   - the first call on a device looks up the array's device address (one cudaGetSymbolAddress, the
 *     context's device must be current; the look-up is guarded by a lock, so first calls from several threads are
 *     safe); make that first call before any stream capture;
 *   - all calls share the one array: two calls whose kernels overlap on the GPU (different streams or
 *     contexts of one process) race on it; calls on one stream are safe.  Nothing in it needs to start at
 *     zero: every slot a call reads was written by that call. */
int32_t rb_attention_decode_static(rb_ctx* ctx, const void* q_dev, rb_kv_cache* cache, int32_t layer, int32_t batch,
                                   int32_t q_heads, float scale, void* out_dev);

/* rb_rope_kv_append followed by rb_attention for a single new token per sequence (s_new == 1), the step a
 * KV-cached decode repeats (qwen2.rs:176-216 with seq_len 1): same inputs, same results bit for bit.  For bf16
 * caches with head_dim 64, 80, 96, 128 or 256 and a rotary width that is a multiple of 16 both run as ONE kernel: the
 * attention kernel rotates q and k itself, appends k/v to the cache, and can start fetching old K/V pages
 * before the projection that feeds it has finished; q_scratch_dev ([batch, q_heads, head_dim]) is then not
 * touched.  Every other case runs the two calls one after the other, through q_scratch_dev. */
int32_t rb_rope_attention_decode(rb_ctx* ctx, const void* qkv_dev, const float* acc_dev, int32_t n_acc, const void* bias_dev,
                                 const float* cos_dev, const float* sin_dev, int32_t rot, int32_t batch, int32_t q_heads,
                                 rb_kv_cache* cache, int32_t layer, float scale, void* q_scratch_dev, void* out_dev,
                                 int32_t dtype);

/* sample_argmax, examples/qwen2/src/main.rs:32-40: per row, the index of the maximum under f32
 * total order, the LAST index among equal maxima.  Bit-exact by construction. */
int32_t rb_argmax_rows(rb_ctx* ctx, const void* logits_dev, int32_t dtype, int64_t rows, int64_t cols,
                       uint32_t* out_dev);
/* The sampling the examples' loops actually run (examples/qwen2/src/main.rs:42-53,84-93): when
 * penalty >= 1, every token id present in the row's context window (a set: a repeated id counts once) has
 * its float32 logit divided by the penalty when >= 0, multiplied by it otherwise; then sample_argmax.
 * context_dev is [rows, context_stride] (stride <= 256), of which the first
 * min(context_count_dev[row], context_stride) slots are valid, in any order.  With eos_token >= 0 and
 * finished_dev != NULL ([rows] bytes, zero to start), a row that has produced eos_token is marked and
 * produces it from then on (the example leaves its loop there).  The logits are not modified.  Bit-exact. */
int32_t rb_sample_greedy(rb_ctx* ctx, const void* logits_dev, int32_t dtype, int64_t rows, int64_t cols, float penalty,
                         const int32_t* context_dev, int32_t context_stride, const int32_t* context_count_dev,
                         int32_t eos_token, uint8_t* finished_dev, uint32_t* out_dev);

/* ======================================================================================
 * Primitive set — the Eval rules of rai-core/src/backend/candle.rs:197-1004 that the decoders'
 * unfused graphs use.  Dense row-major operands unless strides are given (in elements).
 * ====================================================================================== */
/* candle.rs:445-473,525-553,618-626,947-978 (+ scalar operands, ops/mod.rs:203-296, as `scalar`). */
int32_t rb_unary(rb_ctx* ctx, int32_t op, const void* x_dev, void* out_dev, int64_t n, float scalar, int32_t dtype);
/* candle.rs:275-325 with the Broadcast node (candle.rs:575-583) folded in: up to 4-D, stride 0 = broadcast. */
int32_t rb_binary(rb_ctx* ctx, int32_t op, const void* a_dev, const int64_t* a_strides, const void* b_dev,
                  const int64_t* b_strides, void* out_dev, int32_t rank, const int64_t* shape, int32_t dtype);
/* candle.rs:792-803: softmax over the last dimension of [rows, cols]. */
int32_t rb_softmax_rows(rb_ctx* ctx, const void* x_dev, void* out_dev, int64_t rows, int64_t cols, int32_t dtype);
/* candle.rs:475-523: reduce over the last dimension of [rows, cols] -> [rows]. */
int32_t rb_reduce_rows(rb_ctx* ctx, int32_t op, const void* x_dev, void* out_dev, int64_t rows, int64_t cols,
                       int32_t dtype);
/* candle.rs:980-988 (ToContiguous), 555-593/891-899 (views made dense), 880-889 (Concatenate writes each
 * input with an output offset): out (dense, `shape`) = strided view of x.  Up to 6-D. */
int32_t rb_copy_strided(rb_ctx* ctx, const void* x_dev, const int64_t* x_strides, int64_t x_offset, void* out_dev,
                        const int64_t* out_strides, int64_t out_offset, int32_t rank, const int64_t* shape,
                        int32_t elem_size);
/* candle.rs:762-774 (ToDType). */
int32_t rb_cast(rb_ctx* ctx, const void* x_dev, int32_t src_dtype, void* out_dev, int32_t dst_dtype, int64_t n);
/* candle.rs:867-878 (IndexSelect along dim of [outer, dim, inner]); bit-exact row copies. */
int32_t rb_index_select(rb_ctx* ctx, const void* x_dev, int64_t outer, int64_t dim, int64_t inner,
                        const uint32_t* idx_dev, int64_t n_idx, void* out_dev, int32_t elem_size);
/* candle.rs:838-849 (Gather along the last dim of [rows, cols] with idx [rows, k]). */
int32_t rb_gather_last(rb_ctx* ctx, const void* x_dev, int64_t rows, int64_t cols, const uint32_t* idx_dev, int64_t k,
                       void* out_dev, int32_t elem_size);
/* candle.rs:901-915 (Where; cond is u8, inputs ordered on_true, on_false as in ops/where.rs:42-43). */
int32_t rb_where(rb_ctx* ctx, const uint8_t* cond_dev, const void* on_true_dev, const void* on_false_dev,
                 void* out_dev, int64_t n, int32_t dtype);
/* candle.rs:197-209 (Full) and 241-273 (Arange). */
int32_t rb_fill(rb_ctx* ctx, void* out_dev, int64_t n, double value, int32_t dtype);
int32_t rb_arange(rb_ctx* ctx, void* out_dev, int64_t n, double start, double step, int32_t dtype);
/* candle.rs:401-443 (MatMul): batched C[b] = A[b] . B[b], row-major [m,k] x [k,n]; strides in elements,
 * batch stride 0 = broadcast; trans_b != 0 means B[b] is stored [n,k] (the `.t()` of Linear). */
int32_t rb_matmul(rb_ctx* ctx, const void* a_dev, const void* b_dev, void* c_dev, int64_t batch, int64_t m, int64_t n,
                  int64_t k, int64_t a_batch_stride, int64_t b_batch_stride, int32_t trans_b, int32_t dtype);

/* ---- the rest of the rule set of rai-core/src/dispatch.rs:41-157, for graphs beyond the decoders (vision models,
 * training examples).  Correctness-first kernels: one thread per output element. ---- */
/* Equal / NotEqual / Greater / GreaterEqual / Less / LessEqual (candle.rs:327-399): u8 result; operands as rb_binary. */
int32_t rb_compare(rb_ctx* ctx, int32_t op, const void* a_dev, const int64_t* a_strides, const void* b_dev,
                   const int64_t* b_strides, uint8_t* out_dev, int32_t rank, const int64_t* shape, int32_t dtype);
/* LogSoftmax over the last dimension of [rows, cols] (candle.rs:805-836). */
int32_t rb_log_softmax_rows(rb_ctx* ctx, const void* x_dev, void* out_dev, int64_t rows, int64_t cols, int32_t dtype);
/* ArgMin over the last dimension (candle.rs:933-945 family): first index among equal minima. */
int32_t rb_argmin_rows(rb_ctx* ctx, const void* x_dev, int32_t dtype, int64_t rows, int64_t cols, uint32_t* out_dev);
/* ScatterAdd (candle.rs:990-1004; inputs x, updates, indices) and, with index_is_1d != 0, IndexAdd (candle.rs:851-865;
 * inputs x, source, index): tensors viewed as [outer, dim, inner]; out = x, then out[o, idx, i] += src[o, j, i] with
 * idx = index[o, j, i] (or index[j]).  out may be x itself.  An index beyond dim_out is skipped and reported. */
int32_t rb_scatter_add(rb_ctx* ctx, const void* x_dev, const void* src_dev, const uint32_t* idx_dev, void* out_dev,
                       int64_t outer, int64_t dim_out, int64_t dim_src, int64_t inner, int32_t index_is_1d, int32_t dtype);
/* Conv2d (candle.rs:628-663; ops/conv2d.rs:5-9) on NCHW input [N, Cin, H, W] and weight [Cout, Cin, KH, KW]; Conv1d
 * (ops/conv1d.rs:5-9) is the H = KH = 1 case.  out_shape4 (optional) receives [N, Cout, OH, OW]; with out_dev == NULL
 * the call only reports the shape. */
int32_t rb_conv2d(rb_ctx* ctx, const void* x_dev, const int32_t* x_shape4, const void* w_dev, const int32_t* w_shape4,
                  const int32_t* padding2, const int32_t* stride2, const int32_t* dilation2, void* out_dev,
                  int32_t* out_shape4, int32_t dtype);
/* ConvTranspose2d / 1d (candle.rs:702-760; ops/conv_transpose2d.rs:5-10): weight [Cin, Cout, KH, KW]. */
int32_t rb_conv_transpose2d(rb_ctx* ctx, const void* x_dev, const int32_t* x_shape4, const void* w_dev,
                            const int32_t* w_shape4, const int32_t* padding2, const int32_t* out_padding2,
                            const int32_t* stride2, const int32_t* dilation2, void* out_dev, int32_t* out_shape4,
                            int32_t dtype);
/* MaxPool2d / AvgPool2d and their 1-D forms (ops/max_pool2d.rs:6-11, ops/avg_pool2d.rs:9-13): is_max != 0 takes the
 * maximum over the part of the window inside the input, else the sum over it divided by the full window size. */
int32_t rb_pool2d(rb_ctx* ctx, int32_t is_max, const void* x_dev, const int32_t* x_shape4, const int32_t* kernel2,
                  const int32_t* stride2, const int32_t* padding2, const int32_t* dilation2, void* out_dev,
                  int32_t* out_shape4, int32_t dtype);
/* UpsampleNearest2d / 1d (ops/upsample_nearest2d.rs:6-8): [N, C, H, W] -> [N, C, out_h, out_w]. */
int32_t rb_upsample_nearest2d(rb_ctx* ctx, const void* x_dev, const int32_t* x_shape4, int32_t out_h, int32_t out_w,
                              void* out_dev, int32_t dtype);

/* ======================================================================================
 * Decoder driver — Model::new / Module::update_by_safetensors / Model::fwd / clear_kv_cache of
 * rai-models/src/llm/{qwen2,phi2,phi3,gemma}.rs and the generation step of examples/qwen2/src/main.rs:78-91.
 * ====================================================================================== */
typedef struct rb_model_config {
  int32_t arch;                    /* RB_ARCH_* */
  int32_t dtype;                   /* RB_BF16 or RB_F32 */
  int32_t vocab_size;
  int32_t hidden_size;
  int32_t intermediate_size;
  int32_t num_hidden_layers;
  int32_t num_attention_heads;
  int32_t num_key_value_heads;
  int32_t max_position_embeddings;
  int32_t rotary_dim;              /* head_dim, or partial_rotary_factor * head_dim (phi2.rs:47) */
  int32_t hidden_act;              /* RB_ACT_* */
  int32_t tie_word_embeddings;     /* lm_head shares model.embed_tokens.weight (gemma.rs:330) */
  int32_t max_batch;               /* KV-cache capacity: sequences */
  int32_t max_seq;                 /* KV-cache capacity: tokens per sequence */
  int32_t max_tokens;              /* largest batch*seq of one forward call (workspace size) */
  int32_t tp_rank;                 /* tensor-parallel rank / size (1 = single GPU) */
  int32_t tp_size;
  int32_t sliding_window;          /* Config::sliding_window (qwen2.rs:24,316-334): among the tokens of one forward call,
                                      key j is masked for query i when j + sliding_window < i; cached tokens stay
                                      visible and a single-token call has no mask, exactly as the reference builds it.
                                      Honoured for RB_ARCH_QWEN2 (the one family whose mask has the term); 0 = none */
  int32_t reserved0;               /* keeps the doubles 8-byte aligned; set to 0 */
  double rope_theta;
  double norm_eps;
} rb_model_config;

int32_t rb_model_create(rb_ctx* ctx, const rb_model_config* cfg, rb_model** out);
int32_t rb_model_destroy(rb_model* m);
/* Tensor::update_by_name, rai-core/src/nn.rs:192-205: copies (and casts to the model dtype) one named
 * parameter; names follow the derive rule of rai-core/src/nn.rs:256-269, e.g.
 * "model.layers.3.self_attn.q_proj.weight".  With tensor parallelism the FULL tensor is passed and
 * the library keeps this rank's shard.  src_dtype is RB_F32, RB_BF16, RB_F16 or RB_F64 (the float
 * types Tensor::from_safetensor accepts, rai-core/src/hlops/from_safetensor.rs:51-91). */
int32_t rb_model_load_param(rb_model* m, const char* name, const void* data, int32_t on_device, int32_t src_dtype,
                            int32_t rank, const int64_t* shape);
/* The way back, for Module::to_safetensors / named_params (rai-core/src/nn.rs:31-37,57-75): copies one named
 * parameter to the host in the MODEL dtype and the parameter's full shape (dst_bytes must be exactly that).  A
 * tensor-parallel rank returns the rectangle it keeps and zeros elsewhere.  Synchronises the stream. */
int32_t rb_model_read_param(rb_model* m, const char* name, void* dst_host, size_t dst_bytes);
/* Module::update_by_safetensors, rai-core/src/nn.rs:39-55: every parameter of the model is looked up by
 * name in the given files (names absent from the model are ignored; a later file wins over an earlier
 * one, like the reference's map insert) and cast to the model dtype; a parameter found in no file fails
 * with RB_ERR_PARAM, the reference's Error::ParamNotFound.  The files are mapped, not read: each tensor
 * goes mapping -> pinned staging -> device in chunks, the host copy of one chunk overlapping the upload
 * of the previous one, and with tensor parallelism only the rows this rank keeps are uploaded.
 * Replaces the two whole-tensor host copies of the reference's path (std::fs::read + convert_slice).
 * Finalises the model on success. */
int32_t rb_model_load_safetensors(rb_model* m, const char* const* paths, int32_t n_paths);

/* The file reader underneath, usable on its own (host only, no GPU): maps a .safetensors file and
 * validates its header the way safetensors::SafeTensors::deserialize does (header length, JSON shape,
 * data_offsets inside the file and equal to numel x element size).  Entries are listed in file order.
 * rb_safetensors_entry: dtype is an RB_* tag or -1 for a type this library has no tag for; shape8 receives
 * `rank` extents; data points into the mapping and stays valid until rb_safetensors_close. */
int32_t rb_safetensors_open(const char* path, rb_safetensors** out);
int32_t rb_safetensors_close(rb_safetensors* st);
int32_t rb_safetensors_count(const rb_safetensors* st);
int32_t rb_safetensors_entry(const rb_safetensors* st, int32_t index, const char** name, int32_t* dtype, int32_t* rank,
                             int64_t* shape8, const void** data, uint64_t* bytes);
/* Fails with RB_ERR_PARAM naming the first parameter that was never loaded. */
int32_t rb_model_finalize(rb_model* m);
/* Number of parameter names the architecture expects, and the i-th name. */
int32_t rb_model_param_count(rb_model* m);
const char* rb_model_param_name(rb_model* m, int32_t i);
/* Joins the ranks of a tensor-parallel group: `nccl_id` is the 128-byte ncclUniqueId made by rank 0. */
int32_t rb_model_tp_init(rb_model* m, const void* nccl_id, int32_t id_bytes);
/* Fills 128 bytes with a fresh ncclUniqueId (rank 0 calls this and shares the bytes). */
int32_t rb_tp_unique_id(void* out128);

/* Model::fwd (qwen2.rs:338-359 etc.): tokens [batch, seq] u32 on the device, positions start at
 * `pos` (must equal the cached length), logits [batch, vocab] in the model dtype for the LAST
 * position only.  logits_dev may be NULL. */
int32_t rb_model_forward(rb_model* m, const uint32_t* tokens_dev, int32_t batch, int32_t seq, int32_t pos,
                         void* logits_dev);
/* Model::fwd for a right-padded batch: sequence b has lens_host[b] (1..seq) valid tokens, then padding.
 * Logits come from each sequence's last valid position and the cache keeps lens_host[b] tokens of
 * sequence b, so later single-token calls continue every sequence at its own length.  The reference has
 * no counterpart: its batches are rectangular (qwen2.rs:340-351 builds one mask for all rows) and its
 * examples run one sequence; a server batching prompts of different lengths needs this. */
int32_t rb_model_forward_ragged(rb_model* m, const uint32_t* tokens_dev, int32_t batch, int32_t seq, int32_t pos,
                                const int32_t* lens_host, void* logits_dev);
/* rb_model_generate_step for the prompts of a right-padded batch, from an empty cache: host tokens
 * [batch, seq] and lens_host in, one sampled token per sequence out.  Synchronous.  Continue with
 * rb_model_generate_step / rb_model_decode_loop passing pos = -1 ("each sequence at its own length"). */
int32_t rb_model_generate_ragged(rb_model* m, const uint32_t* tokens_host, int32_t batch, int32_t seq,
                                 const int32_t* lens_host, uint32_t* next_host);
/* One iteration of the generation loop (examples/qwen2/src/main.rs:78-91) with greedy sampling:
 * host tokens in (pinned memory recommended) -> H2D -> forward -> on-device argmax -> D2H of
 * batch u32 token ids.  Synchronous.  pos is the reference's seqlen_offset and must equal the cached
 * length; pos = -1 with seq == 1 continues every sequence at its own cached length. */
int32_t rb_model_generate_step(rb_model* m, const uint32_t* tokens_host, int32_t batch, int32_t seq, int32_t pos,
                               uint32_t* next_host);
/* Decode loop kept on the device: `steps` greedy single-token steps starting from tokens_dev
 * [batch] at position pos (or -1: each sequence at its own cached length); writes out_dev [steps, batch].
 * Asynchronous. */
int32_t rb_model_decode_loop(rb_model* m, const uint32_t* tokens_dev, int32_t batch, int32_t pos, int32_t steps,
                             uint32_t* out_dev);
/* Sampling used by rb_model_generate_step and rb_model_decode_loop, as in the examples' loops
 * (examples/qwen2/src/main.rs:74-76,84-96: repeat_penalty 1.10 over repeat_last_n 64, stop at the
 * end-of-text token).  The library keeps, per sequence, the last repeat_last_n (<= 256) tokens fed to
 * those two entry points (prompt and generated alike) and applies rb_sample_greedy's rule; a penalty < 1
 * or repeat_last_n == 0 means plain argmax, eos_token < 0 means no stop rule.  A sequence that produced
 * eos_token keeps producing it (the batch stays rectangular); rb_model_finished reports which have.
 * The history restarts when a call passes pos == 0 and on rb_model_clear_kv_cache.  Default: plain argmax,
 * which is what "greedy" means in the benchmark configurations. */
int32_t rb_model_set_sampling(rb_model* m, float repeat_penalty, int32_t repeat_last_n, int32_t eos_token);
/* flags_host[b] = 1 when sequence b has produced the end-of-sequence token.  Synchronous. */
int32_t rb_model_finished(rb_model* m, int32_t batch, uint8_t* flags_host);
/* 1 when single-token steps (rb_model_decode_loop, rb_model_generate_step with seq == 1) currently replay
 * a captured CUDA graph, 0 when they are issued launch by launch.  No counterpart in the reference. */
int32_t rb_model_decode_graph_active(rb_model* m);
int32_t rb_model_clear_kv_cache(rb_model* m);
rb_kv_cache* rb_model_kv_cache(rb_model* m);
/* Number of kernels the library launched on this context since creation (self-reported count). */
int64_t rb_launch_count(rb_ctx* ctx);
/* Per-launch timing for benchmarks (no counterpart in the reference, which has no tracing call
 * sites): between rb_profile_start and rb_profile_read every kernel launch of the library is
 * bracketed by CUDA events on the context's stream.  rb_profile_read synchronises, stops profiling
 * and fills out4 = {launches, total milliseconds, algorithmic bytes, floating-point operations} for
 * one kernel class (RB_PROF_*). */
enum { RB_PROF_GEMM = 0, RB_PROF_ATTENTION = 1, RB_PROF_NORM = 2, RB_PROF_ROPE_KV = 3, RB_PROF_EMBED = 4,
       RB_PROF_ARGMAX = 5, RB_PROF_OTHER = 6, RB_PROF_CLASSES = 7 };
int32_t rb_profile_start(rb_ctx* ctx);
int32_t rb_profile_read(rb_ctx* ctx, int32_t kernel_class, double* out4);
/* Bytes of device memory the model holds for parameters (after sharding). */
int64_t rb_model_param_bytes(rb_model* m);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* RAI_B200_H_ */
