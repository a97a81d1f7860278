// Decoder driver: the host side of Model::new / update_by_safetensors / Model::fwd / clear_kv_cache of
// rai-models/src/llm/{qwen2,phi2,phi3,gemma}.rs, issuing the fused kernel sequence per layer:
//
//   norm(+pending residual sum)  ->  qkv GEMM  ->  RoPE + head split + KV append  ->  attention
//   ->  o_proj GEMM (+residual)  ->  norm  ->  gate/up GEMM (+act*mul)  ->  down GEMM (+residual)
//
// Residual adds never run as kernels of their own: a GEMM either adds the residual stream in its
// epilogue (large M) or leaves float32 split-K partials / a tensor-parallel partial sum "pending",
// and the next norm kernel folds the pending terms into the residual stream while it normalises.
//
// Tensor parallelism is Megatron style: q/k/v, gate/up and lm_head are split by output rows
// (heads, intermediate units, vocabulary), o_proj/down by input columns, with one allreduce after
// each row-parallel GEMM (NCCL over NVLink, loaded lazily so that single-GPU use needs no NCCL).
#include <dlfcn.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <string>
#include <vector>

#include "ctx.h"

using namespace rb;

namespace {

// ---- the handful of NCCL entry points the driver needs, resolved at rb_model_tp_init
struct UniqueId { char bytes[128]; };  // same layout as ncclUniqueId, which NCCL takes by value
struct Nccl {
  void* lib = nullptr;
  int (*GetUniqueId)(void*) = nullptr;
  int (*CommInitRank)(void**, int, UniqueId, int) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
  int (*CommDestroy)(void*) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
};
constexpr int kNcclFloat32 = 7, kNcclBfloat16 = 9, kNcclSum = 0, kNcclUint8 = 1;

Nccl& nccl() {
  static Nccl n;
  return n;
}

int nccl_load() {
  Nccl& n = nccl();
  if (n.lib) return RB_OK;
  void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) return fail(RB_ERR_UNIMPLEMENTED, "tensor parallelism needs libnccl.so.2: %s", dlerror());
  n.GetUniqueId = (int (*)(void*))dlsym(lib, "ncclGetUniqueId");
  n.CommInitRank = (int (*)(void**, int, UniqueId, int))dlsym(lib, "ncclCommInitRank");
  n.AllReduce = (int (*)(const void*, void*, size_t, int, int, void*, cudaStream_t))dlsym(lib, "ncclAllReduce");
  n.AllGather = (int (*)(const void*, void*, size_t, int, void*, cudaStream_t))dlsym(lib, "ncclAllGather");
  n.CommDestroy = (int (*)(void*))dlsym(lib, "ncclCommDestroy");
  n.GetErrorString = (const char* (*)(int))dlsym(lib, "ncclGetErrorString");
  if (!n.GetUniqueId || !n.CommInitRank || !n.AllReduce || !n.AllGather || !n.CommDestroy || !n.GetErrorString)
    return fail(RB_ERR_UNIMPLEMENTED, "libnccl.so.2 lacks an expected symbol");
  n.lib = lib;
  return RB_OK;
}

#define RB_NCCL(expr)                                                                                   \
  do {                                                                                                  \
    int _r = (expr);                                                                                    \
    if (_r != 0) return fail(RB_ERR_CUDA, "%s failed: %s", #expr, nccl().GetErrorString(_r));           \
  } while (0)

// One rectangular piece of a reference parameter and where it lands in this rank's buffers.
struct Piece {
  int64_t src_row0, rows, src_col0, cols;
  void* dst;
  int64_t dst_ld;  // elements
};
struct ParamSpec {
  int64_t rows, cols;  // full shape of the reference parameter (cols = 1 for vectors)
  int rank;            // 1 or 2
  std::vector<Piece> pieces;
  bool loaded = false;
};

struct LayerW {
  void *qkv = nullptr, *qkv_b = nullptr;
  void *o = nullptr, *o_b = nullptr;
  void *gate = nullptr, *up = nullptr, *fc1_b = nullptr;  // phi2: gate = fc1
  void *down = nullptr, *down_b = nullptr;                // phi2: down = fc2
  void *ln1_w = nullptr, *ln1_b = nullptr, *ln2_w = nullptr;
};

template <typename S, typename T>
__global__ void copy_cast_2d_kernel(const S* __restrict__ src, int64_t src_ld, T* __restrict__ dst, int64_t dst_ld,
                                    int64_t rows, int64_t cols) {
  const int64_t n = rows * cols;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / cols, c = i % cols;
    dst[r * dst_ld + c] = Cvt<T>::from_f(Cvt<S>::to_f(src[r * src_ld + c]));
  }
}

__global__ void set_lens_kernel(int32_t* lens, int n, int len) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) lens[i] = len;
}

// lens[i] += delta: the device-side form of "seqlen_offset grows by the tokens just fed", so that a
// captured decode step can be replayed without new kernel arguments.
__global__ void advance_lens_kernel(int32_t* lens, int n, int delta) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) lens[i] += delta;
}

// The `tokens` vector of the examples' loop (examples/qwen2/src/main.rs:66,92), of which only the last `cap`
// entries per sequence are ever read (`tokens[start_at..]`, main.rs:86-87): a ring per sequence, written at
// (count + s) % cap.  Membership is all the penalty needs, so the order inside the ring is irrelevant.
__global__ void history_push_kernel(const uint32_t* __restrict__ ids, int batch, int seq, int32_t* __restrict__ hist,
                                    int32_t* __restrict__ count, int cap, const int32_t* __restrict__ last_rows) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  const int c = count[b];
  const int valid = last_rows ? last_rows[b] - b * seq + 1 : seq;  // right-padded batch: pads are not part of the text
  for (int s = max(0, valid - cap); s < valid; ++s) hist[(size_t)b * cap + (c + s) % cap] = (int32_t)ids[(size_t)b * seq + s];
  int n = c + valid;
  if (n >= 2 * cap) n = cap + n % cap;  // same slot arithmetic, still "full", and bounded
  count[b] = n;
}

// dst[b, :] = src[rows[b], :]  (16-byte pieces; the last valid position of every sequence of a ragged batch)
__global__ void gather_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ rows, uint4* __restrict__ dst,
                                   int pieces_per_row) {
  const int b = blockIdx.x;
  const size_t r = (size_t)rows[b];
  for (int i = threadIdx.x; i < pieces_per_row; i += blockDim.x) dst[(size_t)b * pieces_per_row + i] = src[r * pieces_per_row + i];
}

// out[b, r*vl + j] = gathered[r, b, j]  (vocabulary shards back into rows of logits)
template <typename T>
__global__ void unshard_logits_kernel(const T* __restrict__ g, T* __restrict__ out, int tp, int batch, int vl) {
  const int64_t n = (int64_t)tp * batch * vl;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int j = (int)(i % vl);
    const int b = (int)((i / vl) % batch);
    const int r = (int)(i / ((int64_t)vl * batch));
    out[((int64_t)b * tp + r) * vl + j] = g[i];
  }
}

struct Pending {  // terms still to be added to the residual stream
  const float* acc = nullptr;
  int n_acc = 0;
  const void* acc_bias = nullptr;
  const void* add = nullptr;
  bool exchange = false;  // the term is one rank's share: the norm point sums it over the tensor-parallel group
  bool any() const { return (acc && n_acc > 0) || add || exchange; }
};

}  // namespace

struct rb_model {
  rb_ctx* ctx = nullptr;
  rb_model_config cfg{};
  int d = 0, nq_l = 0, nkv_l = 0, nqkv_l = 0, inter_l = 0, vocab_l = 0;
  std::vector<int> q_head_src;  // global q head of local head j, or -1 for padding
  int kv_head0 = 0;             // first global kv head of this rank
  size_t es = 2;
  std::vector<LayerW> layers;
  void *embed = nullptr, *norm_w = nullptr, *norm_b = nullptr, *lm_head = nullptr, *lm_head_b = nullptr;
  float *rope_cos = nullptr, *rope_sin = nullptr;
  rb_kv_cache* cache = nullptr;
  std::vector<void*> owned;
  std::vector<std::string> names;
  std::map<std::string, ParamSpec> params;
  int64_t param_bytes = 0;
  // workspace
  uint32_t* ids = nullptr;
  void *h = nullptr, *xn = nullptr, *tmp = nullptr, *qkv = nullptr, *q = nullptr, *attn = nullptr, *act = nullptr;
  void *last_h = nullptr, *logits = nullptr, *logits_g = nullptr;
  uint32_t* next_ids = nullptr;
  int32_t* last_rows = nullptr;           // ragged prefill: row of each sequence's last valid token
  std::vector<int32_t> last_rows_host;    // outlives the asynchronous upload
  float* scratch = nullptr;  // split-K partials
  size_t scratch_floats = 0;
  void* comm = nullptr;
  // peer-memory exchange for decode-sized allreduces (see TpPeers); xchg_base is this rank's region
  TpPeers peers{};
  void* xchg_base = nullptr;
  int xchg_index = 0;  // exchanges launched so far in this forward pass (an even number per pass: two per layer)
  void* peer_base[kTpMaxRanks] = {};
  bool use_exchange = false;
  // RAI_B200_TP_FUSED_GATE=1: a sharded gate/up GEMM sums its split-K slabs and applies activation and gating in its
  // own epilogue.  Off by default: measured slower than split-K partials plus the small finishing kernel, whose many
  // blocks read the slabs with far more parallelism.
  bool fused_gate = false;
  // Developer builds only (-DRB_DEBUG_AIDS, a library file of its own): RAI_B200_SHARD_ONLY=1 runs one rank's shard
  // without its peers to time the per-rank kernels; its outputs are not the model's.  Always false otherwise.
  bool shard_only = false;
  // One decode step (advance lengths, forward of the tokens in `ids`, argmax back into `ids`)
  // captured as a CUDA graph and replayed; re-captured when the batch or the launch plan changes.
  cudaGraphExec_t step_graph = nullptr;
  int graph_batch = 0, graph_plan = 0;
  int eager_warm_batch = 0, eager_warm_plan = 0;
  int64_t graph_launches = 0;
  bool use_graph = true;
  cudaEvent_t ev_in = nullptr, ev_out = nullptr;
  // sampling of the generation entry points (rb_model_set_sampling): repeat penalty over a ring of the
  // last `rep_last_n` tokens fed per sequence, and the end-of-sequence rule
  float rep_penalty = 0.f;
  int rep_last_n = 0;
  int32_t eos = -1;
  int32_t *hist = nullptr, *hist_count = nullptr;
  uint8_t* finished = nullptr;
};

namespace {

int dev_alloc(rb_model* m, size_t bytes, void** out, bool zero) {
  RB_TRY(rb_malloc(m->ctx, bytes, out));
  m->owned.push_back(*out);
  if (zero && bytes) RB_CUDA(cudaMemsetAsync(*out, 0, bytes, m->ctx->stream));
  return RB_OK;
}

int weight_alloc(rb_model* m, int64_t elems, void** out) {
  m->param_bytes += elems * (int64_t)m->es;
  return dev_alloc(m, (size_t)elems * m->es, out, true);
}

void add_param(rb_model* m, const std::string& name, int64_t rows, int64_t cols, int rank, std::vector<Piece> pieces) {
  ParamSpec s;
  s.rows = rows; s.cols = cols; s.rank = rank; s.pieces = std::move(pieces);
  m->names.push_back(name);
  m->params[name] = std::move(s);
}

// The exchange is used only when every one of the `tp` ranks voted 1 (the votes arrive summed).
bool exchange_agreed(float vote_sum, int tp) { return vote_sum > (float)tp - 0.5f; }

int norm_kind(const rb_model* m) {
  return m->cfg.arch == RB_ARCH_PHI2 ? RB_NORM_LAYER : m->cfg.arch == RB_ARCH_GEMMA ? RB_NORM_RMS_ONE_PLUS : RB_NORM_RMS;
}

int allreduce(rb_model* m, void* buf, size_t count) {
  if (m->shard_only) return RB_OK;  // one rank of a group run alone (profiling aid): the sum is just its own term
  RB_NCCL(nccl().AllReduce(buf, buf, count, m->cfg.dtype == RB_BF16 ? kNcclBfloat16 : kNcclFloat32, kNcclSum, m->comm,
                           m->ctx->stream));
  return RB_OK;
}

// v = h + pending ; h = v ; out = norm(v)   (out may be NULL: only fold the pending terms)
int norm_point(rb_model* m, Pending& pend, const void* w, const void* b, int64_t rows, void* out) {
  if (!out && !pend.any()) return RB_OK;
  if (pend.exchange) {  // the term is this rank's share of a sum over the group: exchange, fold and normalise at once
    RB_TRY(exchange_norm(m->ctx, m->peers, m->xchg_index++ & 1, norm_kind(m), m->h, pend.acc, pend.n_acc, pend.acc_bias,
                         pend.add, w, b, (float)m->cfg.norm_eps, rows, m->cfg.hidden_size, out, m->h));
    pend = Pending();
    return RB_OK;
  }
  RB_TRY(rb_norm(m->ctx, norm_kind(m), m->h, pend.add, pend.acc, pend.n_acc, pend.acc_bias, w, b,
                 (float)m->cfg.norm_eps, rows, m->cfg.hidden_size, out, pend.any() ? m->h : nullptr, m->cfg.dtype));
  pend = Pending();
  return RB_OK;
}

// Rows few enough for the GEMM form that sums its split-K slabs inside the kernel and applies the whole epilogue
// there (used where something must follow the sum at once: the gating product of a sharded gate/up).
bool reduce_rows(const rb_model* m, int64_t rows) {
  return m->fused_gate && m->cfg.dtype == RB_BF16 && rows <= 64 && m->ctx->gemm_reduce && !m->ctx->debug_simple_gemm;
}

bool use_partials(rb_model* m, int64_t rows, int64_t n, int64_t k, int* splits) {
  if (m->cfg.dtype != RB_BF16 || rows > 256) return false;
  const int s = rb_linear_pick_splits(m->ctx, rows, n, k);
  if (s <= 1 || (size_t)s * rows * n > m->scratch_floats) return false;
  *splits = s;
  return true;
}

// h += x . W^T + bias, either at once (epilogue residual) or left pending for the next norm_point.
int linear_into_residual(rb_model* m, Pending& pend, const void* x, const void* w, const void* bias, int64_t rows,
                         int64_t n, int64_t k) {
  if (pend.any()) RB_TRY(norm_point(m, pend, nullptr, nullptr, rows, nullptr));
  const void* b = (m->cfg.tp_rank == 0) ? bias : nullptr;  // a row-parallel bias is added once
  int s = 1;
  if (m->cfg.tp_size > 1) {
    // this rank's partial product -> tmp, summed over ranks, folded into the residual by the next norm
    if (m->use_exchange && rows <= kTpMaxRows && n == m->cfg.hidden_size) {
      // decode-sized: the next norm point pushes the partial product into the peers' exchange buffers, waits for
      // theirs and sums them as it reads
      if (use_partials(m, rows, n, k, &s)) {
        RB_TRY(rb_linear_partials(m->ctx, x, w, m->scratch, rows, n, k, s));
        pend.acc = m->scratch; pend.n_acc = s; pend.acc_bias = b;
      } else {
        RB_TRY(rb_linear(m->ctx, x, w, b, nullptr, m->tmp, rows, n, k, RB_ACT_NONE, m->cfg.dtype));
        pend.add = m->tmp;
      }
      pend.exchange = true;
      return RB_OK;
    }
    if (use_partials(m, rows, n, k, &s)) {
      RB_TRY(rb_linear_partials(m->ctx, x, w, m->scratch, rows, n, k, s));
      RB_TRY(rb_norm(m->ctx, RB_NORM_RMS, nullptr, nullptr, m->scratch, s, b, nullptr, nullptr, 0.f, rows, n, nullptr,
                     m->tmp, m->cfg.dtype));
    } else {
      RB_TRY(rb_linear(m->ctx, x, w, b, nullptr, m->tmp, rows, n, k, RB_ACT_NONE, m->cfg.dtype));
    }
    RB_TRY(allreduce(m, m->tmp, (size_t)rows * n));
    pend.add = m->tmp;
    return RB_OK;
  }
  if (use_partials(m, rows, n, k, &s)) {
    RB_TRY(rb_linear_partials(m->ctx, x, w, m->scratch, rows, n, k, s));
    pend.acc = m->scratch; pend.n_acc = s; pend.acc_bias = b;
    return RB_OK;
  }
  return rb_linear(m->ctx, x, w, b, m->h, m->h, rows, n, k, RB_ACT_NONE, m->cfg.dtype);
}

int forward_body(rb_model* m, const uint32_t* tokens, int batch, int seq, void* logits_out, const int32_t* last_rows = nullptr);

// act = activation(x . W1^T [+ b1]) [* (x . Wup^T)]  -- the first half of MLP::fwd.  When the fused kernel
// would leave most SMs idle (decode-sized rows and few 128-row weight tiles, i.e. small or sharded
// intermediate sizes) the product is computed as split-K partials over [gate; up] and a small kernel
// applies bias, activation and gating.
int mlp_up(rb_model* m, const LayerW& w, int64_t rows) {
  const rb_model_config& c = m->cfg;
  rb_ctx* ctx = m->ctx;
  const bool gated = c.arch != RB_ARCH_PHI2;
  const int H = c.hidden_size;
  const int64_t n_all = gated ? 2 * (int64_t)m->inter_l : m->inter_l;
  const int64_t fused_items = (m->inter_l + 127) / 128;
  int s = 1;
  if (c.dtype == RB_BF16 && !ctx->debug_simple && rows <= 256 && fused_items * 4 < (int64_t)ctx->sm_count * 3) {
    if (reduce_rows(m, rows) && (m->inter_l % 8) == 0) {
      // few weight tiles (a sharded or small intermediate size): split K, sum inside the kernel, activation and
      // gating product in the same epilogue - one launch where split-K partials plus a finishing kernel took two
      GemmArgs a;
      a.x = m->xn; a.w = w.gate; a.w2 = gated ? w.up : nullptr; a.bias = gated ? nullptr : w.fc1_b; a.out = m->act;
      a.m = rows; a.n = m->inter_l; a.k = H; a.act = c.hidden_act; a.reduce = true;
      ProfScope prof(ctx, RB_PROF_GEMM, 2.0 * ((gated ? 2.0 : 1.0) * m->inter_l * H + (double)rows * H + (double)rows * m->inter_l),
                     (gated ? 4.0 : 2.0) * rows * m->inter_l * H);
      return gemm_tc_bf16(ctx, a);
    }
    s = rb_linear_pick_splits(ctx, rows, n_all, H);
    if ((size_t)s * rows * n_all <= m->scratch_floats) {
      RB_TRY(rb_linear_partials(ctx, m->xn, w.gate, m->scratch, rows, n_all, H, s));
      return act_from_partials(ctx, m->scratch, s, rows, n_all, m->inter_l, gated, w.fc1_b, c.hidden_act, m->act);
    }
  }
  if (gated) return rb_gated_linear(ctx, m->xn, w.gate, w.up, m->act, rows, m->inter_l, H, c.hidden_act, c.dtype);
  return rb_linear(ctx, m->xn, w.gate, w.fc1_b, nullptr, m->act, rows, m->inter_l, H, c.hidden_act, c.dtype);
}

int forward_impl(rb_model* m, const uint32_t* tokens, int batch, int seq, int pos, void* logits_out) {
  const rb_model_config& c = m->cfg;
  rb_ctx* ctx = m->ctx;
  const int64_t rows = (int64_t)batch * seq;
  RB_REQUIRE(batch > 0 && batch <= c.max_batch, "forward: batch %d exceeds max_batch %d", batch, c.max_batch);
  RB_REQUIRE(seq > 0 && rows <= c.max_tokens, "forward: %lld tokens exceed max_tokens %d", (long long)rows, c.max_tokens);
  RB_REQUIRE(pos >= 0 && pos + seq <= m->cache->max_seq && pos + seq <= c.max_position_embeddings,
             "forward: position %d + %d exceeds the cache / rotary table capacity", pos, seq);
  for (int b = 0; b < batch; ++b)
    RB_REQUIRE(m->cache->host_lens[b] == pos, "forward: seqlen_offset %d differs from the cached length %d of sequence %d",
               pos, m->cache->host_lens[b], b);
  // device-side lengths after this call's tokens are appended
  set_lens_kernel<<<(batch + 127) / 128, 128, 0, ctx->stream>>>(m->cache->seq_lens, batch, pos + seq);
  ctx->launches++;
  for (int b = 0; b < batch; ++b) m->cache->host_lens[b] = pos + seq;
  return forward_body(m, tokens, batch, seq, logits_out);
}

// The launches of one forward pass.  Everything position-dependent is read from device memory (the
// cache's sequence lengths), so the same sequence of launches serves every decode step.
int forward_body(rb_model* m, const uint32_t* tokens, int batch, int seq, void* logits_out, const int32_t* last_rows) {
  const rb_model_config& c = m->cfg;
  rb_ctx* ctx = m->ctx;
  RB_REQUIRE(c.tp_size == 1 || m->comm || m->shard_only,
             "forward: this is rank %d of a %d-way tensor-parallel model and rb_model_tp_init has not run", c.tp_rank, c.tp_size);
  const int64_t rows = (int64_t)batch * seq;
  const int H = c.hidden_size, d = m->d;
  m->xchg_index = 0;

  const float emb_scale = c.arch == RB_ARCH_GEMMA ? sqrtf((float)H) : 1.0f;  // gemma.rs:379
  RB_TRY(rb_embed_gather(ctx, m->embed, c.dtype, c.vocab_size, H, tokens, rows, emb_scale, m->h));

  const float scale = 1.0f / sqrtf((float)d);
  const int L = c.num_hidden_layers;
  Pending pend;
  for (int l = 0; l < L; ++l) {
    const LayerW& w = m->layers[l];
    // input_layernorm, folding what the previous layer left pending
    RB_TRY(norm_point(m, pend, w.ln1_w, w.ln1_b, rows, m->xn));
    // q/k/v projection -> rope -> cache
    int s = 1;
    if (use_partials(m, rows, m->nqkv_l, H, &s)) {
      RB_TRY(rb_linear_partials(ctx, m->xn, w.qkv, m->scratch, rows, m->nqkv_l, H, s));
      if (seq == 1) {  // single-token step: RoPE and the cache append ride in the attention kernel when they can
        RB_TRY(rb_rope_attention_decode(ctx, nullptr, m->scratch, s, w.qkv_b, m->rope_cos, m->rope_sin, c.rotary_dim, batch,
                                        m->nq_l, m->cache, l, scale, m->q, m->attn, c.dtype));
      } else {
        RB_TRY(rb_rope_kv_append(ctx, nullptr, m->scratch, s, w.qkv_b, m->rope_cos, m->rope_sin, c.rotary_dim, batch, seq,
                                 m->nq_l, m->cache, l, m->q, c.dtype));
        RB_TRY(rb_attention(ctx, m->q, m->cache, l, batch, seq, m->nq_l, scale, m->attn, c.dtype));
      }
    } else {
      RB_TRY(rb_linear(ctx, m->xn, w.qkv, w.qkv_b, nullptr, m->qkv, rows, m->nqkv_l, H, RB_ACT_NONE, c.dtype));
      if (seq == 1) {
        RB_TRY(rb_rope_attention_decode(ctx, m->qkv, nullptr, 0, nullptr, m->rope_cos, m->rope_sin, c.rotary_dim, batch,
                                        m->nq_l, m->cache, l, scale, m->q, m->attn, c.dtype));
      } else {
        RB_TRY(rb_rope_kv_append(ctx, m->qkv, nullptr, 0, nullptr, m->rope_cos, m->rope_sin, c.rotary_dim, batch, seq,
                                 m->nq_l, m->cache, l, m->q, c.dtype));
        RB_TRY(rb_attention(ctx, m->q, m->cache, l, batch, seq, m->nq_l, scale, m->attn, c.dtype));
      }
    }
    RB_TRY(linear_into_residual(m, pend, m->attn, w.o, w.o_b, rows, H, (int64_t)m->nq_l * d));
    if (c.arch == RB_ARCH_PHI2) {
      // parallel block (phi2.rs:293-299): the MLP reads the same normed input as the attention.
      // The attention output may still sit in the split-K scratch that the MLP is about to reuse: fold it first.
      if (pend.acc) RB_TRY(norm_point(m, pend, nullptr, nullptr, rows, nullptr));
      RB_TRY(mlp_up(m, w, rows));
    } else {
      RB_TRY(norm_point(m, pend, w.ln2_w, nullptr, rows, m->xn));  // post_attention_layernorm
      RB_TRY(mlp_up(m, w, rows));
    }
    RB_TRY(linear_into_residual(m, pend, m->act, w.down, w.down_b, rows, H, m->inter_l));
  }
  RB_TRY(norm_point(m, pend, nullptr, nullptr, rows, nullptr));  // fold the last layer's output

  // logits for the last position only (qwen2.rs:356-358; phi2.rs:345-346 normalises every row first,
  // which is the same thing for a row-wise norm)
  const void* last = m->h;
  if (seq > 1 && last_rows) {
    RB_REQUIRE(((size_t)H * m->es) % 16 == 0, "ragged forward: hidden rows must be multiples of 16 bytes");
    gather_rows_kernel<<<batch, 128, 0, ctx->stream>>>((const uint4*)m->h, last_rows, (uint4*)m->last_h, (int)((size_t)H * m->es / 16));
    RB_CUDA(cudaGetLastError());
    ctx->launches++;
    last = m->last_h;
  } else if (seq > 1) {
    RB_CUDA(cudaMemcpy2DAsync(m->last_h, (size_t)H * m->es, (const char*)m->h + (size_t)(seq - 1) * H * m->es,
                              (size_t)seq * H * m->es, (size_t)H * m->es, batch, cudaMemcpyDeviceToDevice, ctx->stream));
    last = m->last_h;
  }
  RB_TRY(rb_norm(ctx, norm_kind(m), last, nullptr, nullptr, 0, nullptr, m->norm_w, m->norm_b, (float)c.norm_eps, batch, H,
                 m->xn, nullptr, c.dtype));
  void* head_w = m->lm_head ? m->lm_head : m->embed;
  if (c.tp_size == 1) {
    RB_TRY(rb_linear(ctx, m->xn, head_w, m->lm_head_b, nullptr, m->logits, batch, m->vocab_l, H, RB_ACT_NONE, c.dtype));
  } else {
    RB_TRY(rb_linear(ctx, m->xn, head_w, m->lm_head_b, nullptr, m->logits_g, batch, m->vocab_l, H, RB_ACT_NONE, c.dtype));
    void* gathered = (char*)m->logits_g + (size_t)batch * m->vocab_l * m->es;
    const size_t shard_bytes = (size_t)batch * m->vocab_l * m->es;
    if (!m->shard_only) {
      RB_NCCL(nccl().AllGather(m->logits_g, gathered, shard_bytes, kNcclUint8, m->comm, ctx->stream));
    } else {
      // a rank run without its peers: its own vocabulary shard in place, zeros where the others' would be
      RB_CUDA(cudaMemsetAsync(gathered, 0, shard_bytes * c.tp_size, ctx->stream));
      RB_CUDA(cudaMemcpyAsync((char*)gathered + shard_bytes * c.tp_rank, m->logits_g, shard_bytes, cudaMemcpyDeviceToDevice,
                              ctx->stream));
    }
    const int64_t n = (int64_t)c.tp_size * batch * m->vocab_l;
    const int blocks = (int)std::min<int64_t>((n + 255) / 256, 4096);
    if (c.dtype == RB_BF16)
      unshard_logits_kernel<__nv_bfloat16><<<blocks, 256, 0, ctx->stream>>>((const __nv_bfloat16*)gathered,
                                                                           (__nv_bfloat16*)m->logits, c.tp_size, batch,
                                                                           m->vocab_l);
    else
      unshard_logits_kernel<float><<<blocks, 256, 0, ctx->stream>>>((const float*)gathered, (float*)m->logits, c.tp_size,
                                                                   batch, m->vocab_l);
    ctx->launches++;
  }
  if (logits_out && logits_out != m->logits)
    RB_CUDA(cudaMemcpyAsync(logits_out, m->logits, (size_t)batch * c.vocab_size * m->es, cudaMemcpyDeviceToDevice,
                            ctx->stream));
  return RB_OK;
}

}  // namespace

extern "C" int32_t rb_tp_unique_id(void* out128) {
  RB_REQUIRE(out128, "rb_tp_unique_id: null output");
  RB_TRY(nccl_load());
  RB_NCCL(nccl().GetUniqueId(out128));
  return RB_OK;
}

extern "C" int32_t rb_model_tp_init(rb_model* m, const void* id, int32_t id_bytes) {
  RB_REQUIRE(m && id && id_bytes == 128, "rb_model_tp_init: expects a 128-byte ncclUniqueId");
  if (m->cfg.tp_size <= 1) return RB_OK;
  if (m->shard_only) return RB_OK;
  RB_TRY(nccl_load());
  UniqueId u;
  memcpy(u.bytes, id, 128);
  RB_CUDA(cudaSetDevice(m->ctx->device));
  RB_NCCL(nccl().CommInitRank(&m->comm, m->cfg.tp_size, u, m->cfg.tp_rank));
  const char* xe = getenv("RAI_B200_TP_EXCHANGE");  // RAI_B200_TP_EXCHANGE=0: NCCL allreduce for every size
  if (m->cfg.dtype != RB_BF16 || m->cfg.tp_size > kTpMaxRanks || (xe && xe[0] == '0') || (m->cfg.hidden_size % 8)) return RB_OK;
  // ---- peer-memory exchange: one region per rank = [flags: 2 slots x 8 source ranks x 256 rows | 2 data slots]
  rb_ctx* ctx = m->ctx;
  const int tp = m->cfg.tp_size, rank = m->cfg.tp_rank;
  const size_t slot_elems = (size_t)kTpMaxRows * m->cfg.hidden_size;
  // How the exchange signals arrival (see exchange_norm_kernel): 0 = a flag array beside the data; 1 = the flag inside
  // every 8-byte word, sent straight to every peer (a group of two); 2 = the same words over two hops through the
  // row's owner (wider groups).  RAI_B200_TP_EXCHANGE_FORM=0/1/2 overrides (the same on every rank).
  int mode = tp <= kTpDirectRanks ? kTpInDataDirect : tp <= kTpTwoHopRanks ? kTpInDataTwoHop : kTpFlagArray;
  if (const char* fd = getenv("RAI_B200_TP_EXCHANGE_FORM")) {
    const int want = atoi(fd);
    if (want == kTpFlagArray || want == kTpInDataTwoHop || (want == kTpInDataDirect && tp <= kTpDirectRanks)) mode = want;
  }
  // flags, then [2 slots][tp sources][rows x hidden] bf16 (4 bytes per element instead of 2 with the flag in the data;
  // the two-hop form adds [2 slots][rows x hidden] for the finished rows)
  const size_t bytes = kTpFlagBytes + (mode == kTpFlagArray ? 2 * (size_t)tp * slot_elems * 2
                                                  : (2 * (size_t)tp + (mode == kTpInDataTwoHop ? 2 : 0)) * slot_elems * 4);
  RB_TRY(rb_malloc(ctx, bytes, &m->xchg_base));
  m->owned.push_back(m->xchg_base);
  RB_CUDA(cudaMemsetAsync(m->xchg_base, 0, bytes, ctx->stream));
  cudaIpcMemHandle_t mine;
  RB_CUDA(cudaIpcGetMemHandle(&mine, m->xchg_base));
  // all-gather the handles with NCCL itself (device staging), then open every peer's region
  char* stage = nullptr;
  RB_CUDA(cudaMalloc(&stage, sizeof(mine) * (size_t)(tp + 1)));
  RB_CUDA(cudaMemcpyAsync(stage, &mine, sizeof(mine), cudaMemcpyHostToDevice, ctx->stream));
  RB_NCCL(nccl().AllGather(stage, stage + sizeof(mine), sizeof(mine), kNcclUint8, m->comm, ctx->stream));
  std::vector<cudaIpcMemHandle_t> all(tp);
  RB_CUDA(cudaMemcpyAsync(all.data(), stage + sizeof(mine), sizeof(mine) * (size_t)tp, cudaMemcpyDeviceToHost, ctx->stream));
  RB_CUDA(cudaStreamSynchronize(ctx->stream));
  cudaFree(stage);
  bool opened = true;
  for (int r = 0; r < tp && opened; ++r) {
    if (r == rank) { m->peer_base[r] = m->xchg_base; continue; }
    cudaError_t e = cudaIpcOpenMemHandle(&m->peer_base[r], all[r], cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) { cudaGetLastError(); m->peer_base[r] = nullptr; opened = false; }
  }
  // The ranks decide together: every rank, whether it could map its peers or not, joins ONE sum of "ok" votes, and
  // the exchange is used only if all voted yes.  (A rank that dropped out on its own would leave the others in a
  // collective it never joins, and the two sides would then run different protocols.)
  {
    float* vote = nullptr;
    RB_CUDA(cudaMalloc(&vote, sizeof(float)));
    const float mine_ok = opened ? 1.0f : 0.0f;
    RB_CUDA(cudaMemcpyAsync(vote, &mine_ok, sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    int nst = nccl().AllReduce(vote, vote, 1, kNcclFloat32, kNcclSum, m->comm, ctx->stream);
    float total = 0.f;
    cudaError_t ce = cudaMemcpyAsync(&total, vote, sizeof(float), cudaMemcpyDeviceToHost, ctx->stream);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(ctx->stream);
    cudaFree(vote);
    if (nst != 0) return fail(RB_ERR_CUDA, "tensor-parallel set-up: the agreement allreduce failed: %s", nccl().GetErrorString(nst));
    RB_CUDA(ce);
    if (!exchange_agreed(total, tp)) {
      // at least one rank has no peer access: every rank closes what it opened and stays on NCCL
      for (int q = 0; q < tp; ++q)
        if (q != rank && m->peer_base[q]) { cudaIpcCloseMemHandle(m->peer_base[q]); m->peer_base[q] = nullptr; }
      return RB_OK;
    }
  }
  TpPeers& p = m->peers;
  for (int r = 0; r < tp; ++r) {
    p.flags[r] = (uint32_t*)m->peer_base[r];
    p.xbuf[r] = (const char*)m->peer_base[r] + kTpFlagBytes;
  }
  // the two exchange counters are touched by this GPU only: keep them off the lines the peers write
  void* local = nullptr;
  RB_TRY(rb_malloc(ctx, 256, &local));
  m->owned.push_back(local);
  RB_CUDA(cudaMemsetAsync(local, 0, 256, ctx->stream));
  p.seq = (uint32_t*)local;
  p.rank = rank; p.size = tp; p.slot_elems = (int64_t)slot_elems;
  p.form = mode;
  // (the vote above was also the meeting point: no rank publishes before every rank has zeroed its region and
  // opened its peers)
  RB_CUDA(cudaStreamSynchronize(ctx->stream));
  m->use_exchange = true;
  return RB_OK;
}

extern "C" int32_t rb_model_create(rb_ctx* ctx, const rb_model_config* cfg, rb_model** out) {
  RB_REQUIRE(ctx && cfg && out, "rb_model_create: null argument");
  const rb_model_config& c = *cfg;
  RB_REQUIRE(c.arch >= RB_ARCH_QWEN2 && c.arch <= RB_ARCH_GEMMA, "rb_model_create: unknown arch %d", c.arch);
  RB_REQUIRE(c.dtype == RB_BF16 || c.dtype == RB_F32, "rb_model_create: dtype %d unsupported", c.dtype);
  RB_REQUIRE(c.hidden_size > 0 && c.num_attention_heads > 0 && c.hidden_size % c.num_attention_heads == 0,
             "rb_model_create: hidden_size must divide by num_attention_heads");
  RB_REQUIRE(c.num_key_value_heads > 0 && c.num_attention_heads % c.num_key_value_heads == 0,
             "rb_model_create: num_attention_heads must divide by num_key_value_heads");
  RB_REQUIRE(c.tp_size >= 1 && c.tp_rank >= 0 && c.tp_rank < c.tp_size, "rb_model_create: bad tensor-parallel rank");
  RB_REQUIRE(c.max_batch > 0 && c.max_seq > 0 && c.max_tokens >= c.max_batch, "rb_model_create: bad capacities");
  RB_REQUIRE(c.sliding_window >= 0, "rb_model_create: negative sliding_window");
  const int tp = c.tp_size, rank = c.tp_rank;
  const int nq = c.num_attention_heads, nkv = c.num_key_value_heads, G = nq / nkv;
  RB_REQUIRE(c.intermediate_size % tp == 0 && c.vocab_size % tp == 0,
             "rb_model_create: intermediate_size and vocab_size must divide by tp_size");
  RB_REQUIRE((tp <= nkv && nkv % tp == 0) || (tp > nkv && tp % nkv == 0),
             "rb_model_create: tp_size %d and %d KV heads do not divide either way", tp, nkv);

  rb_model* m = new rb_model();
  m->ctx = ctx;
  m->cfg = c;
  {
    const char* g = getenv("RAI_B200_GRAPH");  // RAI_B200_GRAPH=0: plain launches for every decode step
    m->use_graph = !(g && g[0] == '0');
    const char* fp = getenv("RAI_B200_TP_FUSED_GATE");
    m->fused_gate = fp && fp[0] == '1';
  }
  m->d = c.hidden_size / nq;
  m->es = dtype_size(c.dtype);
  const int d = m->d, H = c.hidden_size;
  // ---- head assignment
  if (tp <= nkv) {
    m->nkv_l = nkv / tp;
    m->kv_head0 = rank * m->nkv_l;
    m->nq_l = m->nkv_l * G;
    for (int j = 0; j < m->nq_l; ++j) m->q_head_src.push_back(m->kv_head0 * G + j);
  } else {
    // more ranks than KV heads: `rpk` ranks share one KV head, each takes ceil(G / rpk) of its query
    // heads; the last of them may carry zero-weight padding heads (their o_proj columns are zero)
    const int rpk = tp / nkv, qpr = (G + rpk - 1) / rpk;
    m->nkv_l = 1;
    m->kv_head0 = rank / rpk;
    m->nq_l = qpr;
    const int sub = rank % rpk;
    for (int j = 0; j < qpr; ++j) {
      const int within = sub * qpr + j;
      m->q_head_src.push_back(within < G ? m->kv_head0 * G + within : -1);
    }
  }
  m->nqkv_l = (m->nq_l + 2 * m->nkv_l) * d;
  m->inter_l = c.intermediate_size / tp;
  m->vocab_l = c.vocab_size / tp;
  const int I = c.intermediate_size, Il = m->inter_l, V = c.vocab_size, Vl = m->vocab_l;
  const bool phi2 = c.arch == RB_ARCH_PHI2, phi3 = c.arch == RB_ARCH_PHI3;
  const bool qkv_bias = c.arch == RB_ARCH_QWEN2 || phi2;

  int st = RB_OK;
  auto A = [&](int64_t elems, void** p) { if (st == RB_OK) st = weight_alloc(m, elems, p); };
  auto P = [&](void* base, int64_t elem_off) { return (void*)((char*)base + elem_off * (int64_t)m->es); };

  A((int64_t)V * H, &m->embed);
  A(H, &m->norm_w);
  if (phi2) A(H, &m->norm_b);
  const bool own_head = !(c.arch == RB_ARCH_GEMMA || c.tie_word_embeddings);
  if (own_head || tp > 1) A((int64_t)Vl * H, &m->lm_head);
  if (phi2) A(Vl, &m->lm_head_b);
  m->layers.resize(c.num_hidden_layers);
  for (auto& w : m->layers) {
    A((int64_t)m->nqkv_l * H, &w.qkv);
    if (qkv_bias) A(m->nqkv_l, &w.qkv_b);
    A((int64_t)H * m->nq_l * d, &w.o);
    if (phi2) A(H, &w.o_b);
    if (!phi2) {  // gate and up in one buffer, gate rows first: one skinny GEMM can then cover both
      A((int64_t)2 * Il * H, &w.gate);
      w.up = st == RB_OK ? (void*)((char*)w.gate + (size_t)Il * H * m->es) : nullptr;
    } else {
      A((int64_t)Il * H, &w.gate);
      A(Il, &w.fc1_b);
    }
    A((int64_t)H * Il, &w.down);
    if (phi2) A(H, &w.down_b);
    A(H, &w.ln1_w);
    if (phi2) A(H, &w.ln1_b); else A(H, &w.ln2_w);
  }
  if (st != RB_OK) { rb_model_destroy(m); return st; }

  // ---- parameter registry (names per the derive rule, rai-core/src/nn.rs:256-269)
  {
    std::vector<Piece> pe{{0, V, 0, H, m->embed, H}};
    if (!own_head && tp > 1) pe.push_back({(int64_t)rank * Vl, Vl, 0, H, m->lm_head, H});  // tied head, vocab shard
    add_param(m, "model.embed_tokens.weight", V, H, 2, pe);
  }
  const std::string fnorm = phi2 ? "model.final_layernorm" : "model.norm";
  add_param(m, fnorm + ".weight", H, 1, 1, {{0, H, 0, 1, m->norm_w, 1}});
  if (phi2) add_param(m, fnorm + ".bias", H, 1, 1, {{0, H, 0, 1, m->norm_b, 1}});
  if (own_head) {
    add_param(m, "lm_head.weight", V, H, 2, {{(int64_t)rank * Vl, Vl, 0, H, m->lm_head, H}});
    if (phi2) add_param(m, "lm_head.bias", V, 1, 1, {{(int64_t)rank * Vl, Vl, 0, 1, m->lm_head_b, 1}});
  }
  for (int l = 0; l < c.num_hidden_layers; ++l) {
    LayerW& w = m->layers[l];
    const std::string pre = "model.layers." + std::to_string(l) + ".";
    // fused qkv rows: [local q heads | local k heads | local v heads]
    auto head_pieces = [&](int64_t src_head_row0, bool is_q, int64_t dst_row0, void* dst, int64_t cols, int64_t ld) {
      std::vector<Piece> ps;
      if (is_q) {
        for (int j = 0; j < m->nq_l; ++j)
          if (m->q_head_src[j] >= 0)
            ps.push_back({src_head_row0 + (int64_t)m->q_head_src[j] * d, d, 0, cols, P(dst, (dst_row0 + (int64_t)j * d) * ld), ld});
      } else {
        ps.push_back({src_head_row0 + (int64_t)m->kv_head0 * d, (int64_t)m->nkv_l * d, 0, cols, P(dst, dst_row0 * ld), ld});
      }
      return ps;
    };
    const int64_t kq = (int64_t)m->nq_l * d, kk = (int64_t)m->nkv_l * d;
    if (phi3) {
      std::vector<Piece> ps = head_pieces(0, true, 0, w.qkv, H, H);
      auto pk = head_pieces((int64_t)nq * d, false, kq, w.qkv, H, H);
      auto pv = head_pieces((int64_t)(nq + nkv) * d, false, kq + kk, w.qkv, H, H);
      ps.insert(ps.end(), pk.begin(), pk.end());
      ps.insert(ps.end(), pv.begin(), pv.end());
      add_param(m, pre + "self_attn.qkv_proj.weight", (int64_t)(nq + 2 * nkv) * d, H, 2, ps);
    } else {
      add_param(m, pre + "self_attn.q_proj.weight", (int64_t)nq * d, H, 2, head_pieces(0, true, 0, w.qkv, H, H));
      add_param(m, pre + "self_attn.k_proj.weight", (int64_t)nkv * d, H, 2, head_pieces(0, false, kq, w.qkv, H, H));
      add_param(m, pre + "self_attn.v_proj.weight", (int64_t)nkv * d, H, 2, head_pieces(0, false, kq + kk, w.qkv, H, H));
      if (qkv_bias) {
        add_param(m, pre + "self_attn.q_proj.bias", (int64_t)nq * d, 1, 1, head_pieces(0, true, 0, w.qkv_b, 1, 1));
        add_param(m, pre + "self_attn.k_proj.bias", (int64_t)nkv * d, 1, 1, head_pieces(0, false, kq, w.qkv_b, 1, 1));
        add_param(m, pre + "self_attn.v_proj.bias", (int64_t)nkv * d, 1, 1, head_pieces(0, false, kq + kk, w.qkv_b, 1, 1));
      }
    }
    {  // o_proj / dense: input columns follow the local query heads
      std::vector<Piece> ps;
      for (int j = 0; j < m->nq_l; ++j)
        if (m->q_head_src[j] >= 0)
          ps.push_back({0, H, (int64_t)m->q_head_src[j] * d, d, P(w.o, (int64_t)j * d), kq});
      add_param(m, pre + (phi2 ? "self_attn.dense.weight" : "self_attn.o_proj.weight"), H, (int64_t)nq * d, 2, ps);
      if (phi2) add_param(m, pre + "self_attn.dense.bias", H, 1, 1, {{0, H, 0, 1, w.o_b, 1}});
    }
    if (phi3) {
      add_param(m, pre + "mlp.gate_up_proj.weight", 2 * (int64_t)I, H, 2,
                {{(int64_t)rank * Il, Il, 0, H, w.gate, H}, {(int64_t)I + (int64_t)rank * Il, Il, 0, H, w.up, H}});
      add_param(m, pre + "mlp.down_proj.weight", H, I, 2, {{0, H, (int64_t)rank * Il, Il, w.down, Il}});
    } else if (phi2) {
      add_param(m, pre + "mlp.fc1.weight", I, H, 2, {{(int64_t)rank * Il, Il, 0, H, w.gate, H}});
      add_param(m, pre + "mlp.fc1.bias", I, 1, 1, {{(int64_t)rank * Il, Il, 0, 1, w.fc1_b, 1}});
      add_param(m, pre + "mlp.fc2.weight", H, I, 2, {{0, H, (int64_t)rank * Il, Il, w.down, Il}});
      add_param(m, pre + "mlp.fc2.bias", H, 1, 1, {{0, H, 0, 1, w.down_b, 1}});
    } else {
      add_param(m, pre + "mlp.gate_proj.weight", I, H, 2, {{(int64_t)rank * Il, Il, 0, H, w.gate, H}});
      add_param(m, pre + "mlp.up_proj.weight", I, H, 2, {{(int64_t)rank * Il, Il, 0, H, w.up, H}});
      add_param(m, pre + "mlp.down_proj.weight", H, I, 2, {{0, H, (int64_t)rank * Il, Il, w.down, Il}});
    }
    add_param(m, pre + "input_layernorm.weight", H, 1, 1, {{0, H, 0, 1, w.ln1_w, 1}});
    if (phi2) add_param(m, pre + "input_layernorm.bias", H, 1, 1, {{0, H, 0, 1, w.ln1_b, 1}});
    else add_param(m, pre + "post_attention_layernorm.weight", H, 1, 1, {{0, H, 0, 1, w.ln2_w, 1}});
  }

  // ---- rotary tables, cache, workspace
  const int half = c.rotary_dim / 2;
  const int recipe = phi2 ? 1 : phi3 ? 2 : 0;
  auto W = [&](size_t bytes, void** p) { if (st == RB_OK) st = dev_alloc(m, bytes, p, false); };
  W((size_t)c.max_position_embeddings * half * sizeof(float), (void**)&m->rope_cos);
  W((size_t)c.max_position_embeddings * half * sizeof(float), (void**)&m->rope_sin);
  if (st == RB_OK) st = rb_rope_tables(ctx, recipe, c.rotary_dim, c.max_position_embeddings, c.rope_theta, m->rope_cos, m->rope_sin);
  if (st == RB_OK) st = rb_kv_cache_create(ctx, c.num_hidden_layers, m->nkv_l, d, c.max_batch, c.max_seq, c.dtype, &m->cache);
  if (st == RB_OK && c.arch == RB_ARCH_QWEN2 && c.sliding_window > 0) st = rb_kv_cache_set_window(m->cache, c.sliding_window);
  // split-KV scratch for the worst case (every sequence, 32 splits): a generation then never allocates
  if (st == RB_OK && c.dtype == RB_BF16)
    st = attention_reserve_scratch(ctx, (size_t)c.max_batch * m->nq_l * 32 * (d + 2) * sizeof(float));
  if (st == RB_OK && c.dtype == RB_BF16)  // slabs of the GEMMs that reduce split-K in the kernel: 8 splits, 64 rows, two sets when gated
    st = gemm_reserve_scratch(ctx, (size_t)2 * 8 * 64 * std::max(m->inter_l, H) * sizeof(float));
  const size_t MT = c.max_tokens;
  W(MT * sizeof(uint32_t), (void**)&m->ids);
  W(MT * H * m->es, &m->h);
  W(MT * H * m->es, &m->xn);
  if (tp > 1) W(MT * H * m->es, &m->tmp);
  W(MT * m->nqkv_l * m->es, &m->qkv);
  W(MT * m->nq_l * d * m->es, &m->q);
  W(MT * m->nq_l * d * m->es, &m->attn);
  W(MT * Il * m->es, &m->act);
  W((size_t)c.max_batch * H * m->es, &m->last_h);
  W((size_t)c.max_batch * V * m->es, &m->logits);
  if (tp > 1) W((size_t)c.max_batch * Vl * m->es * (tp + 1), &m->logits_g);
  W((size_t)c.max_batch * sizeof(uint32_t), (void**)&m->next_ids);
  W((size_t)c.max_batch * sizeof(int32_t), (void**)&m->last_rows);
  if (c.dtype == RB_BF16) {
    // split-K scratch: up to 16 slabs of min(max_tokens, 256) rows of the widest split-K output
    const size_t rows = std::min<size_t>(MT, 256);
    m->scratch_floats = (size_t)16 * rows * std::max(m->nqkv_l, H);
    W(m->scratch_floats * sizeof(float), (void**)&m->scratch);
  }
  if (st != RB_OK) { rb_model_destroy(m); return st; }
#ifdef RB_DEBUG_AIDS
  {
    const char* so = getenv("RAI_B200_SHARD_ONLY");
    m->shard_only = tp > 1 && so && so[0] == '1';
    if (m->shard_only && c.dtype == RB_BF16 && (H % 8) == 0) {
      // the exchange kernels still run, against a group of one (this rank's own region)
      const size_t slot_elems = (size_t)kTpMaxRows * H;
      st = dev_alloc(m, kTpFlagBytes + 512 + 2 * slot_elems * 2, &m->xchg_base, true);
      if (st != RB_OK) { rb_model_destroy(m); return st; }
      TpPeers& p = m->peers;
      p.flags[0] = (uint32_t*)m->xchg_base;
      p.seq = (uint32_t*)((char*)m->xchg_base + kTpFlagBytes);
      p.xbuf[0] = (const char*)m->xchg_base + kTpFlagBytes + 512;
      p.rank = 0; p.size = 1; p.slot_elems = (int64_t)slot_elems; p.form = kTpFlagArray;
      m->peer_base[0] = m->xchg_base;
      m->use_exchange = true;
    }
  }
#endif
  RB_CUDA(cudaStreamSynchronize(ctx->stream));
  *out = m;
  return RB_OK;
}

extern "C" int32_t rb_model_destroy(rb_model* m) {
  if (!m) return RB_OK;
  cudaStreamSynchronize(m->ctx->stream);
  if (m->step_graph) cudaGraphExecDestroy(m->step_graph);
  if (m->ev_in) cudaEventDestroy(m->ev_in);
  if (m->ev_out) cudaEventDestroy(m->ev_out);
  for (int r = 0; r < kTpMaxRanks; ++r)
    if (m->peer_base[r] && m->peer_base[r] != m->xchg_base) cudaIpcCloseMemHandle(m->peer_base[r]);
  if (m->comm && nccl().CommDestroy) nccl().CommDestroy(m->comm);
  if (m->cache) rb_kv_cache_destroy(m->cache);
  for (void* p : m->owned) rb_free(m->ctx, p);
  delete m;
  return RB_OK;
}

extern "C" int32_t rb_model_param_count(rb_model* m) { return m ? (int32_t)m->names.size() : 0; }
extern "C" const char* rb_model_param_name(rb_model* m, int32_t i) {
  return (m && i >= 0 && i < (int32_t)m->names.size()) ? m->names[i].c_str() : nullptr;
}
extern "C" int64_t rb_model_param_bytes(rb_model* m) { return m ? m->param_bytes : 0; }
extern "C" rb_kv_cache* rb_model_kv_cache(rb_model* m) { return m ? m->cache : nullptr; }

template <typename S>
static int copy_pieces(rb_model* m, const ParamSpec& sp, const S* src_dev) {
  for (const Piece& pc : sp.pieces) {
    const int64_t n = pc.rows * pc.cols;
    if (n == 0) continue;
    const int blocks = (int)std::min<int64_t>((n + 255) / 256, 8192);
    const S* src = src_dev + pc.src_row0 * sp.cols + pc.src_col0;
    if (m->cfg.dtype == RB_BF16)
      copy_cast_2d_kernel<S, __nv_bfloat16><<<blocks, 256, 0, m->ctx->stream>>>(src, sp.cols, (__nv_bfloat16*)pc.dst,
                                                                                pc.dst_ld, pc.rows, pc.cols);
    else
      copy_cast_2d_kernel<S, float><<<blocks, 256, 0, m->ctx->stream>>>(src, sp.cols, (float*)pc.dst, pc.dst_ld, pc.rows,
                                                                        pc.cols);
    m->ctx->launches++;
    RB_TRY(launch_status("copy_cast_2d"));
  }
  return RB_OK;
}

static int copy_pieces_any(rb_model* m, const ParamSpec& sp, const void* src_dev, int32_t src_dtype) {
  switch (src_dtype) {
    case RB_F32: return copy_pieces<float>(m, sp, (const float*)src_dev);
    case RB_BF16: return copy_pieces<__nv_bfloat16>(m, sp, (const __nv_bfloat16*)src_dev);
    case RB_F16: return copy_pieces<__half>(m, sp, (const __half*)src_dev);
    case RB_F64: return copy_pieces<double>(m, sp, (const double*)src_dev);
  }
  return fail(RB_ERR_DTYPE, "parameter source dtype %d unsupported (F32, BF16, F16, F64)", src_dtype);
}

static int check_param_shape(const char* name, const ParamSpec& sp, int32_t rank, const int64_t* shape) {
  const int64_t rows = rank >= 1 ? shape[0] : 1, cols = rank >= 2 ? shape[1] : 1;
  if (rank != sp.rank || rows != sp.rows || cols != sp.cols)
    return fail(RB_ERR_SHAPE, "parameter '%s': got shape [%lld, %lld] (rank %d), expected [%lld, %lld] (rank %d)", name,
                (long long)rows, (long long)cols, rank, (long long)sp.rows, (long long)sp.cols, sp.rank);
  return RB_OK;
}

extern "C" int32_t rb_model_load_param(rb_model* m, const char* name, const void* data, int32_t on_device,
                                       int32_t src_dtype, int32_t rank, const int64_t* shape) {
  RB_REQUIRE(m && name && data && shape, "rb_model_load_param: null argument");
  auto it = m->params.find(name);
  if (it == m->params.end()) return fail(RB_ERR_PARAM, "parameter '%s' is not part of this model", name);
  ParamSpec& sp = it->second;
  RB_REQUIRE(src_dtype == RB_F32 || src_dtype == RB_BF16 || src_dtype == RB_F16 || src_dtype == RB_F64,
             "rb_model_load_param: source dtype %d unsupported", src_dtype);
  RB_TRY(check_param_shape(name, sp, rank, shape));
  const size_t bytes = (size_t)sp.rows * sp.cols * dtype_size(src_dtype);
  const void* src = data;
  void* staging = nullptr;
  if (!on_device) {
    RB_TRY(rb_malloc(m->ctx, bytes, &staging));
    int st = rb_upload(m->ctx, staging, data, bytes);
    if (st != RB_OK) { rb_free(m->ctx, staging); return st; }
    src = staging;
  }
  int st = copy_pieces_any(m, sp, src, src_dtype);
  if (staging) {
    cudaStreamSynchronize(m->ctx->stream);
    cudaFree(staging);
  }
  if (st == RB_OK) sp.loaded = true;
  return st;
}

namespace {

// Streams host bytes to the device through two pinned buffers: while chunk k is in flight to the GPU the
// host copies chunk k+1 out of the file mapping (which is where the page faults, i.e. the disk reads, happen).
struct PinnedPipe {
  static constexpr size_t kChunk = 32u << 20;
  void* buf[2] = {nullptr, nullptr};
  cudaEvent_t done[2] = {nullptr, nullptr};
  int next = 0;
  int init() {
    for (int i = 0; i < 2; ++i) {
      RB_CUDA(cudaHostAlloc(&buf[i], kChunk, cudaHostAllocDefault));
      RB_CUDA(cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming));
    }
    return RB_OK;
  }
  int send(void* dst_dev, const void* src_host, size_t bytes, cudaStream_t stream) {
    for (size_t off = 0; off < bytes; off += kChunk) {
      const size_t n = std::min(kChunk, bytes - off);
      RB_CUDA(cudaEventSynchronize(done[next]));  // the buffer's previous upload has left it
      memcpy(buf[next], (const char*)src_host + off, n);
      RB_CUDA(cudaMemcpyAsync((char*)dst_dev + off, buf[next], n, cudaMemcpyHostToDevice, stream));
      RB_CUDA(cudaEventRecord(done[next], stream));
      next ^= 1;
    }
    return RB_OK;
  }
  ~PinnedPipe() {
    for (int i = 0; i < 2; ++i) {
      if (done[i]) { cudaEventSynchronize(done[i]); cudaEventDestroy(done[i]); }
      if (buf[i]) cudaFreeHost(buf[i]);
    }
  }
};

}  // namespace

extern "C" int32_t rb_model_load_safetensors(rb_model* m, const char* const* paths, int32_t n_paths) {
  RB_REQUIRE(m && paths && n_paths > 0, "rb_model_load_safetensors: null or empty argument");
  struct Files {
    std::vector<rb_safetensors*> v;
    ~Files() { for (rb_safetensors* s : v) rb_safetensors_close(s); }
  } files;
  // last file wins for a name that appears in several (the reference inserts into one map, file by file)
  std::map<std::string, std::pair<int, int>> where;
  size_t staging_bytes = 0;
  for (int f = 0; f < n_paths; ++f) {
    RB_REQUIRE(paths[f], "rb_model_load_safetensors: path %d is null", f);
    rb_safetensors* st = nullptr;
    RB_TRY(rb_safetensors_open(paths[f], &st));
    files.v.push_back(st);
    for (int i = 0; i < rb_safetensors_count(st); ++i) {
      const char* name;
      RB_TRY(rb_safetensors_entry(st, i, &name, nullptr, nullptr, nullptr, nullptr, nullptr));
      if (m->params.count(name)) where[name] = {f, i};
    }
  }
  for (const std::string& n : m->names)
    if (!where.count(n) && !m->params[n].loaded)
      return fail(RB_ERR_PARAM, "parameter '%s' was found in none of the %d safetensors file(s)", n.c_str(), n_paths);

  // rows of the source this rank keeps (all of them without tensor parallelism)
  struct Job { std::string name; int file, index; int64_t row0, row1; };
  std::vector<Job> jobs;
  for (auto& kv : where) {
    const ParamSpec& sp = m->params[kv.first];
    int64_t r0 = sp.rows, r1 = 0;
    for (const Piece& pc : sp.pieces)
      if (pc.rows > 0 && pc.cols > 0) { r0 = std::min(r0, pc.src_row0); r1 = std::max(r1, pc.src_row0 + pc.rows); }
    if (r1 <= r0) { r0 = 0; r1 = 0; }
    jobs.push_back({kv.first, kv.second.first, kv.second.second, r0, r1});
  }
  // file order, so that the mapping is read front to back
  std::sort(jobs.begin(), jobs.end(), [](const Job& a, const Job& b) { return a.file != b.file ? a.file < b.file : a.index < b.index; });
  for (const Job& j : jobs) {
    int32_t dtype, rank;
    int64_t shape[8];
    const char* name;
    RB_TRY(rb_safetensors_entry(files.v[j.file], j.index, &name, &dtype, &rank, shape, nullptr, nullptr));
    const ParamSpec& sp = m->params[j.name];
    RB_REQUIRE(dtype == RB_F32 || dtype == RB_BF16 || dtype == RB_F16 || dtype == RB_F64,
               "parameter '%s' is stored as a non-floating type", name);
    RB_TRY(check_param_shape(name, sp, rank, shape));
    staging_bytes = std::max(staging_bytes, (size_t)(j.row1 - j.row0) * sp.cols * dtype_size(dtype));
  }

  rb_ctx* ctx = m->ctx;
  PinnedPipe pipe;
  RB_TRY(pipe.init());
  void* staging = nullptr;
  if (staging_bytes) RB_TRY(rb_malloc(ctx, staging_bytes, &staging));
  int st = RB_OK;
  for (const Job& j : jobs) {
    int32_t dtype;
    const void* data;
    st = rb_safetensors_entry(files.v[j.file], j.index, nullptr, &dtype, nullptr, nullptr, &data, nullptr);
    if (st != RB_OK) break;
    ParamSpec& sp = m->params[j.name];
    const size_t es = dtype_size(dtype), row_bytes = (size_t)sp.cols * es;
    if (j.row1 > j.row0) {
      st = pipe.send(staging, (const char*)data + (size_t)j.row0 * row_bytes, (size_t)(j.row1 - j.row0) * row_bytes, ctx->stream);
      if (st != RB_OK) break;
      // copy_pieces indexes rows of the whole tensor: hand it the address row 0 would have
      st = copy_pieces_any(m, sp, (const char*)staging - (size_t)j.row0 * row_bytes, dtype);
      if (st != RB_OK) break;
    }
    sp.loaded = true;
  }
  cudaStreamSynchronize(ctx->stream);
  if (staging) rb_free(ctx, staging);
  RB_TRY(st);
  return rb_model_finalize(m);
}

extern "C" int32_t rb_model_read_param(rb_model* m, const char* name, void* dst_host, size_t dst_bytes) {
  RB_REQUIRE(m && name && dst_host, "rb_model_read_param: null argument");
  auto it = m->params.find(name);
  if (it == m->params.end()) return fail(RB_ERR_PARAM, "parameter '%s' is not part of this model", name);
  const ParamSpec& sp = it->second;
  const size_t row_bytes = (size_t)sp.cols * m->es, need = (size_t)sp.rows * row_bytes;
  RB_REQUIRE(dst_bytes == need, "rb_model_read_param: '%s' is %zu bytes in the model dtype, the buffer holds %zu", name, need,
             dst_bytes);
  RB_CUDA(cudaStreamSynchronize(m->ctx->stream));
  memset(dst_host, 0, need);  // what a tensor-parallel rank does not keep reads as zero
  for (const Piece& pc : sp.pieces) {
    if (pc.rows == 0 || pc.cols == 0) continue;
    char* dst = (char*)dst_host + (size_t)pc.src_row0 * row_bytes + (size_t)pc.src_col0 * m->es;
    RB_CUDA(cudaMemcpy2D(dst, row_bytes, pc.dst, (size_t)pc.dst_ld * m->es, (size_t)pc.cols * m->es, (size_t)pc.rows,
                         cudaMemcpyDeviceToHost));
  }
  return RB_OK;
}

extern "C" int32_t rb_model_finalize(rb_model* m) {
  RB_REQUIRE(m, "rb_model_finalize: null model");
  for (const std::string& n : m->names)
    if (!m->params[n].loaded) return fail(RB_ERR_PARAM, "parameter '%s' was never loaded", n.c_str());
  RB_CUDA(cudaStreamSynchronize(m->ctx->stream));
  return RB_OK;
}

extern "C" int32_t rb_model_clear_kv_cache(rb_model* m) {
  RB_REQUIRE(m, "rb_model_clear_kv_cache: null model");
  if (m->hist_count) {
    RB_CUDA(cudaMemsetAsync(m->hist_count, 0, (size_t)m->cfg.max_batch * sizeof(int32_t), m->ctx->stream));
    RB_CUDA(cudaMemsetAsync(m->finished, 0, (size_t)m->cfg.max_batch, m->ctx->stream));
  }
  return rb_kv_cache_reset(m->cache);
}

extern "C" int32_t rb_model_set_sampling(rb_model* m, float repeat_penalty, int32_t repeat_last_n, int32_t eos_token) {
  RB_REQUIRE(m, "rb_model_set_sampling: null model");
  RB_REQUIRE(repeat_last_n >= 0 && repeat_last_n <= 256, "rb_model_set_sampling: repeat_last_n %d outside [0, 256]", repeat_last_n);
  RB_REQUIRE(eos_token < m->cfg.vocab_size, "rb_model_set_sampling: eos token %d outside the vocabulary", eos_token);
  RB_REQUIRE(!(repeat_penalty != repeat_penalty), "rb_model_set_sampling: the penalty is NaN");
  RB_CUDA(cudaStreamSynchronize(m->ctx->stream));
  // a captured decode step has the old sampler baked in
  if (m->step_graph) { cudaGraphExecDestroy(m->step_graph); m->step_graph = nullptr; }
  m->eager_warm_batch = m->eager_warm_plan = 0;
  if (!m->hist_count) {
    RB_TRY(dev_alloc(m, (size_t)m->cfg.max_batch * 256 * sizeof(int32_t), (void**)&m->hist, true));
    RB_TRY(dev_alloc(m, (size_t)m->cfg.max_batch * sizeof(int32_t), (void**)&m->hist_count, true));
    RB_TRY(dev_alloc(m, (size_t)m->cfg.max_batch, (void**)&m->finished, true));
  }
  m->rep_penalty = repeat_penalty;
  m->rep_last_n = repeat_last_n;
  m->eos = eos_token < 0 ? -1 : eos_token;
  RB_CUDA(cudaMemsetAsync(m->hist_count, 0, (size_t)m->cfg.max_batch * sizeof(int32_t), m->ctx->stream));
  RB_CUDA(cudaMemsetAsync(m->finished, 0, (size_t)m->cfg.max_batch, m->ctx->stream));
  return RB_OK;
}

extern "C" int32_t rb_model_finished(rb_model* m, int32_t batch, uint8_t* flags_host) {
  RB_REQUIRE(m && flags_host, "rb_model_finished: null argument");
  RB_REQUIRE(batch >= 0 && batch <= m->cfg.max_batch, "rb_model_finished: batch %d exceeds max_batch", batch);
  if (!m->finished) { memset(flags_host, 0, (size_t)batch); return RB_OK; }
  RB_CUDA(cudaMemcpyAsync(flags_host, m->finished, (size_t)batch, cudaMemcpyDeviceToHost, m->ctx->stream));
  RB_CUDA(cudaStreamSynchronize(m->ctx->stream));
  return RB_OK;
}

// Right-padded batch: sequence b has lens[b] valid tokens followed by padding.  The rectangle runs as usual
// (under the causal mask a pad can only influence later pads), the logits come from each sequence's last
// valid row, and the cache keeps lens[b] tokens of sequence b: the pads' K/V rows lie beyond that length,
// are never read, and are overwritten by the tokens decoded next.
static int forward_ragged(rb_model* m, const uint32_t* tokens, int batch, int seq, int pos, const int32_t* lens, void* logits_out) {
  rb_ctx* ctx = m->ctx;
  rb_kv_cache* kc = m->cache;
  for (int b = 0; b < batch; ++b)
    RB_REQUIRE(lens[b] >= 1 && lens[b] <= seq, "ragged forward: sequence %d has %d valid tokens of %d", b, lens[b], seq);
  m->last_rows_host.assign((size_t)batch, 0);
  for (int b = 0; b < batch; ++b) m->last_rows_host[b] = b * seq + lens[b] - 1;
  RB_CUDA(cudaMemcpyAsync(m->last_rows, m->last_rows_host.data(), (size_t)batch * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
  const rb_model_config& c = m->cfg;
  const int64_t rows = (int64_t)batch * seq;
  RB_REQUIRE(batch > 0 && batch <= c.max_batch, "forward: batch %d exceeds max_batch %d", batch, c.max_batch);
  RB_REQUIRE(seq > 0 && rows <= c.max_tokens, "forward: %lld tokens exceed max_tokens %d", (long long)rows, c.max_tokens);
  RB_REQUIRE(pos >= 0 && pos + seq <= kc->max_seq && pos + seq <= c.max_position_embeddings,
             "forward: position %d + %d exceeds the cache / rotary table capacity", pos, seq);
  for (int b = 0; b < batch; ++b)
    RB_REQUIRE(kc->host_lens[b] == pos, "forward: seqlen_offset %d differs from the cached length %d of sequence %d", pos,
               kc->host_lens[b], b);
  set_lens_kernel<<<(batch + 127) / 128, 128, 0, ctx->stream>>>(kc->seq_lens, batch, pos + seq);
  ctx->launches++;
  for (int b = 0; b < batch; ++b) kc->host_lens[b] = pos + seq;
  RB_TRY(forward_body(m, tokens, batch, seq, logits_out, seq > 1 ? m->last_rows : nullptr));
  for (int b = 0; b < batch; ++b) kc->host_lens[b] = pos + lens[b];
  RB_CUDA(cudaMemcpyAsync(kc->seq_lens, kc->host_lens.data(), (size_t)batch * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
  return RB_OK;
}

extern "C" int32_t rb_model_forward_ragged(rb_model* m, const uint32_t* tokens_dev, int32_t batch, int32_t seq, int32_t pos,
                                           const int32_t* lens_host, void* logits_dev) {
  RB_REQUIRE(m && tokens_dev && lens_host, "rb_model_forward_ragged: null argument");
  return forward_ragged(m, tokens_dev, batch, seq, pos, lens_host, logits_dev);
}

extern "C" int32_t rb_model_forward(rb_model* m, const uint32_t* tokens_dev, int32_t batch, int32_t seq, int32_t pos,
                                    void* logits_dev) {
  RB_REQUIRE(m && tokens_dev, "rb_model_forward: null argument");
  return forward_impl(m, tokens_dev, batch, seq, pos, logits_dev);
}

namespace {

bool sampling_on(const rb_model* m) { return (m->rep_penalty >= 1.0f && m->rep_last_n > 0) || m->eos >= 0; }

// Forget the tokens seen and the finished marks: a new generation starts (position 0 or a cleared cache).
int sampling_reset(rb_model* m) {
  if (!m->hist_count) return RB_OK;
  RB_CUDA(cudaMemsetAsync(m->hist_count, 0, (size_t)m->cfg.max_batch * sizeof(int32_t), m->ctx->stream));
  RB_CUDA(cudaMemsetAsync(m->finished, 0, (size_t)m->cfg.max_batch, m->ctx->stream));
  return RB_OK;
}

// The tokens about to be fed join the history BEFORE the sampling that follows their forward pass: at
// that point the examples' `tokens` holds the prompt and every token generated so far (main.rs:84-92).
int history_push(rb_model* m, const uint32_t* ids, int batch, int seq, const int32_t* last_rows = nullptr) {
  if (!(m->rep_penalty >= 1.0f && m->rep_last_n > 0)) return RB_OK;
  history_push_kernel<<<(batch + 127) / 128, 128, 0, m->ctx->stream>>>(ids, batch, seq, m->hist, m->hist_count, m->rep_last_n,
                                                                      last_rows);
  RB_CUDA(cudaGetLastError());
  m->ctx->launches++;
  return RB_OK;
}

int sample_tokens(rb_model* m, int batch, uint32_t* out) {
  if (!sampling_on(m)) return rb_argmax_rows(m->ctx, m->logits, m->cfg.dtype, batch, m->cfg.vocab_size, out);
  return rb_sample_greedy(m->ctx, m->logits, m->cfg.dtype, batch, m->cfg.vocab_size, m->rep_penalty, m->hist, m->rep_last_n,
                          m->hist_count, m->eos, m->finished, out);
}

// Whatever host-side state shapes the launches of a decode step: a captured step is reused only
// while this stays the same (today: how many KV splits the attention uses).
int decode_plan(rb_model* m, int batch) {
  int max_len = 0;
  for (int b = 0; b < batch; ++b) max_len = std::max(max_len, m->cache->host_lens[b]);
  return attention_decode_splits(m->ctx, batch, m->nkv_l, max_len, m->d);
}

int decode_step_launches(rb_model* m, int batch) {
  rb_ctx* ctx = m->ctx;
  advance_lens_kernel<<<(batch + 127) / 128, 128, 0, ctx->stream>>>(m->cache->seq_lens, batch, 1);
  ctx->launches++;
  RB_TRY(history_push(m, m->ids, batch, 1));
  RB_TRY(forward_body(m, m->ids, batch, 1, nullptr));
  // the sampled token goes straight back into `ids`, the input of the next step
  return sample_tokens(m, batch, m->ids);
}

// One greedy decode step on the tokens in m->ids (result left in m->ids), on the context's current
// stream, replaying a captured CUDA graph when one fits.  The first step of a new (batch, plan) runs
// eagerly (it may allocate scratch and set kernel attributes), the second is captured, later ones replay.
int decode_step(rb_model* m, int batch) {
  rb_ctx* ctx = m->ctx;
  rb_kv_cache* c = m->cache;
  RB_REQUIRE(batch > 0 && batch <= m->cfg.max_batch, "decode: batch %d exceeds max_batch %d", batch, m->cfg.max_batch);
  // every sequence continues at its own cached length (they differ after a ragged prefill)
  for (int b = 0; b < batch; ++b)
    RB_REQUIRE(c->host_lens[b] + 1 <= c->max_seq && c->host_lens[b] + 1 <= m->cfg.max_position_embeddings,
               "decode: position %d of sequence %d exceeds the cache / rotary table capacity", c->host_lens[b], b);
  for (int b = 0; b < batch; ++b) c->host_lens[b] += 1;
  const int plan = decode_plan(m, batch);
  const bool graphable = m->use_graph && !ctx->profiling && !ctx->debug_simple;
  if (graphable && m->step_graph && m->graph_batch == batch && m->graph_plan == plan) {
    RB_CUDA(cudaGraphLaunch(m->step_graph, ctx->stream));
    ctx->launches += m->graph_launches;
    return RB_OK;
  }
  if (graphable && m->eager_warm_batch == batch && m->eager_warm_plan == plan) {
    // capture on the library's own stream (the default stream cannot be captured), ordered with the
    // caller's stream by events on both sides
    cudaStream_t user = ctx->stream;
    if (m->step_graph) { cudaGraphExecDestroy(m->step_graph); m->step_graph = nullptr; }
    cudaGraph_t graph = nullptr;
    const int64_t launches0 = ctx->launches;
    int st = RB_OK;
    cudaError_t ce = cudaStreamBeginCapture(ctx->own_stream, cudaStreamCaptureModeRelaxed);
    if (ce == cudaSuccess) {
      ctx->stream = ctx->own_stream;
      st = decode_step_launches(m, batch);
      ctx->stream = user;
      ce = cudaStreamEndCapture(ctx->own_stream, &graph);
      if (st == RB_OK && ce == cudaSuccess) ce = cudaGraphInstantiate(&m->step_graph, graph, 0);
      if (graph) cudaGraphDestroy(graph);
    }
    if (st != RB_OK || ce != cudaSuccess || !m->step_graph) {
      // capture is an optimisation: fall back to plain launches for the rest of this model's life
      if (getenv("RAI_B200_VERBOSE"))
        fprintf(stderr, "rai_b200: decode-step capture failed (status %d: %s; cuda: %s); using plain launches\n", st,
                st != RB_OK ? rb_last_error() : "-", cudaGetErrorString(ce));
      cudaGetLastError();
      m->step_graph = nullptr;
      m->use_graph = false;
      ctx->launches = launches0;
      return decode_step_launches(m, batch);
    }
    m->graph_launches = ctx->launches - launches0;
    ctx->launches = launches0;
    m->graph_batch = batch;
    m->graph_plan = plan;
    RB_CUDA(cudaGraphLaunch(m->step_graph, ctx->stream));
    ctx->launches += m->graph_launches;
    return RB_OK;
  }
  m->eager_warm_batch = batch;
  m->eager_warm_plan = plan;
  return decode_step_launches(m, batch);
}

// Runs `fn` with the context's stream switched to the library's own (capturable) stream, ordered
// after the caller's stream on entry and before it on exit.
template <typename F>
int on_own_stream(rb_model* m, F fn) {
  rb_ctx* ctx = m->ctx;
  cudaStream_t user = ctx->stream;
  if (user == ctx->own_stream) return fn();
  if (!m->ev_in) {
    RB_CUDA(cudaEventCreateWithFlags(&m->ev_in, cudaEventDisableTiming));
    RB_CUDA(cudaEventCreateWithFlags(&m->ev_out, cudaEventDisableTiming));
  }
  RB_CUDA(cudaEventRecord(m->ev_in, user));
  RB_CUDA(cudaStreamWaitEvent(ctx->own_stream, m->ev_in, 0));
  ctx->stream = ctx->own_stream;
  const int st = fn();
  ctx->stream = user;
  RB_CUDA(cudaEventRecord(m->ev_out, ctx->own_stream));
  RB_CUDA(cudaStreamWaitEvent(user, m->ev_out, 0));
  return st;
}

}  // namespace

extern "C" int32_t rb_model_decode_graph_active(rb_model* m) { return (m && m->step_graph) ? 1 : 0; }

extern "C" int32_t rb_model_generate_step(rb_model* m, const uint32_t* tokens_host, int32_t batch, int32_t seq,
                                          int32_t pos, uint32_t* next_host) {
  RB_REQUIRE(m && tokens_host && next_host, "rb_model_generate_step: null argument");
  RB_REQUIRE(batch > 0 && seq > 0 && (int64_t)batch * seq <= m->cfg.max_tokens, "rb_model_generate_step: bad sizes");
  rb_ctx* ctx = m->ctx;
  const bool single = seq == 1 && !ctx->profiling;
  RB_REQUIRE(pos >= 0 || seq == 1, "generate_step: a negative seqlen_offset (own lengths) needs single-token steps");
  if (single && pos >= 0)
    for (int b = 0; b < batch; ++b)
      RB_REQUIRE(m->cache->host_lens[b] == pos, "generate_step: seqlen_offset %d differs from the cached length %d", pos,
                 m->cache->host_lens[b]);
  const int st = on_own_stream(m, [&]() -> int {
    RB_CUDA(cudaMemcpyAsync(m->ids, tokens_host, (size_t)batch * seq * sizeof(uint32_t), cudaMemcpyHostToDevice, ctx->stream));
    const uint32_t* result = m->ids;
    if (pos == 0) RB_TRY(sampling_reset(m));
    if (single) {
      RB_TRY(decode_step(m, batch));
    } else {
      int at = pos;
      if (at < 0) {  // own lengths, plain launches (profiling): they must agree for a rectangular forward
        at = m->cache->host_lens[0];
        for (int b = 0; b < batch; ++b)
          RB_REQUIRE(m->cache->host_lens[b] == at, "generate_step: sequences of different lengths cannot be profiled launch by launch");
      }
      RB_TRY(history_push(m, m->ids, batch, seq));
      RB_TRY(forward_impl(m, m->ids, batch, seq, at, nullptr));
      RB_TRY(sample_tokens(m, batch, m->next_ids));
      result = m->next_ids;
    }
    RB_CUDA(cudaMemcpyAsync(next_host, result, (size_t)batch * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
    return RB_OK;
  });
  RB_TRY(st);
  RB_CUDA(cudaStreamSynchronize(ctx->own_stream));
  return rb_sync(ctx);
}

extern "C" int32_t rb_model_generate_ragged(rb_model* m, const uint32_t* tokens_host, int32_t batch, int32_t seq,
                                            const int32_t* lens_host, uint32_t* next_host) {
  RB_REQUIRE(m && tokens_host && lens_host && next_host, "rb_model_generate_ragged: null argument");
  RB_REQUIRE(batch > 0 && seq > 0 && (int64_t)batch * seq <= m->cfg.max_tokens, "rb_model_generate_ragged: bad sizes");
  rb_ctx* ctx = m->ctx;
  const int st = on_own_stream(m, [&]() -> int {
    RB_CUDA(cudaMemcpyAsync(m->ids, tokens_host, (size_t)batch * seq * sizeof(uint32_t), cudaMemcpyHostToDevice, ctx->stream));
    RB_TRY(sampling_reset(m));
    RB_TRY(forward_ragged(m, m->ids, batch, seq, 0, lens_host, nullptr));
    // the history takes each sequence's valid tokens only (last_rows was uploaded by forward_ragged)
    RB_TRY(history_push(m, m->ids, batch, seq, seq > 1 ? m->last_rows : nullptr));
    RB_TRY(sample_tokens(m, batch, m->next_ids));
    RB_CUDA(cudaMemcpyAsync(next_host, m->next_ids, (size_t)batch * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
    return RB_OK;
  });
  RB_TRY(st);
  RB_CUDA(cudaStreamSynchronize(ctx->own_stream));
  return rb_sync(ctx);
}

extern "C" int32_t rb_model_decode_loop(rb_model* m, const uint32_t* tokens_dev, int32_t batch, int32_t pos,
                                        int32_t steps, uint32_t* out_dev) {
  RB_REQUIRE(m && tokens_dev && out_dev, "rb_model_decode_loop: null argument");
  RB_REQUIRE(batch > 0 && batch <= m->cfg.max_batch && steps >= 0, "rb_model_decode_loop: bad sizes");
  if (pos >= 0)
    for (int b = 0; b < batch; ++b)
      RB_REQUIRE(m->cache->host_lens[b] == pos, "decode_loop: seqlen_offset %d differs from the cached length %d", pos,
                 m->cache->host_lens[b]);
  rb_ctx* ctx = m->ctx;
  auto body = [&]() -> int {
    RB_CUDA(cudaMemcpyAsync(m->ids, tokens_dev, (size_t)batch * sizeof(uint32_t), cudaMemcpyDeviceToDevice, ctx->stream));
    if (pos == 0) RB_TRY(sampling_reset(m));
    for (int i = 0; i < steps; ++i) {
      RB_TRY(decode_step(m, batch));
      RB_CUDA(cudaMemcpyAsync(out_dev + (size_t)i * batch, m->ids, (size_t)batch * sizeof(uint32_t),
                              cudaMemcpyDeviceToDevice, ctx->stream));
    }
    return RB_OK;
  };
  if (ctx->profiling) return body();  // per-launch event timing needs plain launches on the caller's stream
  return on_own_stream(m, body);
}
