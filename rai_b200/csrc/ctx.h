// Internal definition of the context and the KV cache behind the opaque handles of the C ABI.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <map>
#include <tuple>
#include <vector>

#include "common.cuh"

struct rb_ctx {
  int device = 0;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;
  int sm_count = 148;
  uint32_t* status_dev = nullptr;  // 4 words, see rb_status_word
  int64_t launches = 0;
  // Tensor maps are keyed by (base pointer, rows, cols, row stride in elements, box rows).
  std::map<std::tuple<const void*, int64_t, int64_t, int64_t, int>, CUtensorMap> tmaps;
  bool pdl = true;            // RAI_B200_PDL=0 turns programmatic dependent launch off (debugging aid)
  // shared memory a decode-sized GEMM spends on its operand ring (RAI_B200_GEMM_RING_KB overrides)
  size_t gemm_ring_bytes = 200 * 1024;
  bool attn_tc = true;        // RAI_B200_ATTN_TC=0: prefill attention on the mma.sync kernel for every head size (debugging aid)
  bool gemm_reduce = true;    // RAI_B200_GEMM_REDUCE=0: rb_linear / rb_gated_linear never split K inside the kernel (debugging aid)
  float* gemm_scratch = nullptr;   // float32 slabs of the GEMMs that reduce split-K inside the kernel; grow-only
  size_t gemm_scratch_bytes = 0;
  uint32_t* gemm_tile_count = nullptr;  // [2][kGemmMaxReduceTiles] arrival / done counters of those GEMMs, self-resetting
  long long wait_budget_cycles = 2000000000LL;  // give-up time of a device-side wait for ANOTHER GPU (rb_set_wait_budget_us)
  // Waits inside one kernel (operand rings, accumulators, sibling blocks) may begin before the kernel's predecessor
  // has finished, and that predecessor may itself be waiting for a peer: they get four times the budget, so that
  // when a peer never arrives it is the exchange that reports it, not a bystander further down the stream.
  long long local_wait_cycles() const { return wait_budget_cycles > (1LL << 60) ? wait_budget_cycles : 4 * wait_budget_cycles; }
  int tmap_cache_limit = 4096;  // tensor maps kept before the cache is emptied
  // argmax across blocks: running best (key << 32 | index) and arrival count per row; self-resetting
  unsigned long long* argmax_best = nullptr;
  unsigned int* argmax_count = nullptr;
  // split-KV partials of the decode attention: grown on demand, owned by the context (one stream at a time)
  bool pool_ready = false;  // the device's default memory pool has been told to keep freed blocks
  float* attn_scratch = nullptr;
  size_t attn_scratch_bytes = 0;
  std::vector<void*> retired;  // outgrown scratch buffers, kept until rb_destroy (captured graphs may still name them)
  std::vector<struct rb_kv_cache*> caches;  // live caches, for the clean-up after a device-side give-up
  double cycles_per_us = 1965.0;  // SM clock, to turn a wait budget in microseconds into cycles
  bool debug_simple = false;
  bool debug_no_fuse = false;  // RAI_B200_FUSE_ROPE=0
  bool debug_simple_gemm = false, debug_simple_attn = false;  // RAI_B200_SIMPLE_GEMM / _ATTN: one kernel family only  // RAI_B200_SIMPLE=1: route bf16 through the plain kernels (debugging aid)
  // Optional per-launch timing (rb_profile_start / rb_profile_read): an event pair around each launch.
  struct ProfRec { int cls; cudaEvent_t a, b; double bytes, flops; };
  bool profiling = false;
  std::vector<ProfRec> prof;
};

// Pages of 64 tokens.  K and V each: [layer][page][kv_head][64][head_dim] in the cache dtype.
struct rb_kv_cache {
  rb_ctx* ctx = nullptr;
  int layers = 0, kv_heads = 0, head_dim = 0, max_batch = 0, max_seq = 0, dtype = RB_BF16;
  int pages_per_seq = 0, num_pages = 0;
  int window = 1 << 30;  // sliding-window width of the attention mask (rb_kv_cache_set_window); 2^30 = none
  void* k = nullptr;
  void* v = nullptr;
  int32_t* block_table = nullptr;  // device [max_batch][pages_per_seq]
  int32_t* seq_lens = nullptr;     // device [max_batch]
  uint32_t* split_count = nullptr;  // device [max_batch][kv_heads]: arrivals of a split decode attention; self-resetting
  std::vector<int32_t> host_lens;
  size_t layer_stride_elems() const { return (size_t)num_pages * kv_heads * 64 * head_dim; }
};

// Peer-memory exchange of a tensor-parallel group for decode-sized allreduces (exchange_norm_kernel, one block per
// row).  Flag-array form: every rank stores its partial row into its own place in every PEER's exchange buffer (posted
// stores over NVLink), raises the flag of (source rank, row) in every peer's flag array with a system-scope release,
// waits (bounded) for that row's flag from every peer - not for the other rows - and sums the copies in its own memory
// and its own row in rank order, the same on every rank.  The two flag-in-data forms need no flag array: every
// 8-byte word carries 4 bytes of payload and the exchange number (see the kernel).  Two slots, chosen by the parity
// of an exchange number kept on the device, so replayed CUDA graphs need no new arguments: launches alternate
// between two local counters (a launch reads one and sets the other for its successor), so no kernel changes a word
// its own blocks are still reading.  Slot n & 1 is free again when exchange n + 2 starts: a rank gets there only
// after every rank has delivered its rows of exchange n + 1, which a rank does only after its own exchange n has
// completed.
constexpr int kGemmMaxReduceTiles = 256;

constexpr int kTpMaxRanks = 8;
constexpr int kTpMaxRows = 256;
// Forms of the exchange (see exchange_norm_kernel): how arrival is signalled and which way the rows travel.
enum TpForm : int { kTpFlagArray = 0, kTpInDataDirect = 1, kTpInDataTwoHop = 2 };
constexpr int kTpDirectRanks = 2;      // widest group that sends flag-in-data words straight to every peer
constexpr int kTpTwoHopRanks = 8;      // widest group that takes the two-hop form of them by default
constexpr size_t kTpFlagBytes = (size_t)2 * kTpMaxRanks * kTpMaxRows * sizeof(uint32_t);  // [2 slots][source rank][row]
struct TpPeers {
  const void* xbuf[kTpMaxRanks];   // every rank's exchange buffer (own included), [2 slots][size sources][kTpMaxRows][hidden]
                                   // (flag-in-data form: the same shape in 8-byte words of 2 elements + the exchange number)
  uint32_t* flags[kTpMaxRanks];    // every rank's flag array, [2][kTpMaxRanks][kTpMaxRows]
  uint32_t* seq;                   // local: two exchange counters 128 bytes apart, seq[0] for even launches, seq[32] for odd
  int rank, size;
  int form;                        // a TpForm
  int64_t slot_elems;              // kTpMaxRows * hidden
};

namespace rb {
constexpr int kPageTokens = 64;
constexpr int kArgmaxRows = 4096;  // rows one argmax launch can reduce across blocks

// Brackets one kernel launch with CUDA events when profiling is on; `bytes` / `flops` are the
// algorithmic (not measured) HBM bytes and floating-point operations of the launch.
struct ProfScope {
  rb_ctx* ctx;
  size_t idx = 0;
  bool on;
  ProfScope(rb_ctx* c, int cls, double bytes, double flops) : ctx(c), on(c->profiling) {
    if (!on) return;
    rb_ctx::ProfRec r{cls, nullptr, nullptr, bytes, flops};
    if (cudaEventCreate(&r.a) != cudaSuccess || cudaEventCreate(&r.b) != cudaSuccess) { on = false; return; }
    cudaEventRecord(r.a, c->stream);
    idx = c->prof.size();
    c->prof.push_back(r);
  }
  ~ProfScope() {
    if (on) cudaEventRecord(ctx->prof[idx].b, ctx->stream);
  }
};

// Internal launchers shared between api.cu and model.cu (defined next to their kernels).
int tmap_2d_bf16(rb_ctx* ctx, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows, CUtensorMap* out);

struct GemmArgs {
  const void* x = nullptr;      // [M, K]
  const void* w = nullptr;      // [N, K]
  const void* w2 = nullptr;     // gated: up weights [N, K]
  const void* bias = nullptr;   // [N]
  const void* residual = nullptr;  // [M, N]
  void* out = nullptr;          // [M, N] (model dtype) or float partials [n_split][M][N]
  int64_t m = 0, n = 0, k = 0;
  int act = RB_ACT_NONE;
  int n_split = 1;              // > 1: write float partials, no epilogue
  bool partials = false;
  bool reduce = false;            // M <= 64: if K is split, sum the splits inside the kernel and apply the epilogue
};
int gemm_tc_bf16(rb_ctx* ctx, const GemmArgs& a);
int gemm_tc_pick_splits(rb_ctx* ctx, int64_t m, int64_t n, int64_t k);
int gemm_reserve_scratch(rb_ctx* ctx, size_t bytes);
int gemm_simple(rb_ctx* ctx, const GemmArgs& a, int dtype);

int attention_mma_bf16(rb_ctx* ctx, const void* q, rb_kv_cache* c, int layer, int batch, int s_new, int q_heads,
                       float scale, void* out);
// decoder_kernels.cu: the tensor-parallel sum of a row-parallel product (split-K slabs + bias, or a finished bf16
// tensor `part`) over the exchange buffers, the residual add and the following norm, in one kernel.
// sum_out = h + sum over ranks; out = norm(sum_out) (out may be NULL).  `parity` alternates 0,1,0,1.. launch by launch.
int exchange_norm(rb_ctx* ctx, const TpPeers& tp, int parity, int kind, const void* h, const float* acc, int n_acc,
                  const void* acc_bias, const void* part, const void* w, const void* b, float eps, int64_t rows,
                  int64_t hidden, void* out, void* sum_out);
// decoder_kernels.cu: out[r, j] = act(sum_s part[s][r][j] + bias[j]) (* sum_s part[s][r][j + n_out] when gated)
int act_from_partials(rb_ctx* ctx, const float* part, int n_split, int64_t rows, int64_t n_all, int64_t n_out, bool gated,
                      const void* bias, int act, void* out);
// Single-token step with the RoPE / KV-append work folded into the decode attention kernel (bf16 caches,
// head sizes that are multiples of 64).  `attention_can_fuse_rope` says whether the shapes and pointers allow it.
bool attention_can_fuse_rope(const rb_kv_cache* c, int q_heads, int rot, const void* qkv, const float* acc, int n_acc,
                             const void* bias, const float* cos_t, const float* sin_t, int batch);
int attention_decode_fused_rope(rb_ctx* ctx, const void* qkv, const float* acc, int n_acc, const void* bias,
                                const float* cos_t, const float* sin_t, int rot, rb_kv_cache* c, int layer, int batch,
                                int q_heads, float scale, void* out);
int attention_decode_splits(rb_ctx* ctx, int batch, int kv_heads, int max_len, int head_dim);
int attention_reserve_scratch(rb_ctx* ctx, size_t bytes);
// attention_tc.cu: causal prefill attention on tcgen05 (head sizes 64 and 128, query length >= 128)
bool attention_prefill_tc_supported(const rb_kv_cache* c, int s_new, int q_heads, const void* q, const void* out);
int attention_prefill_tc(rb_ctx* ctx, const void* q, rb_kv_cache* c, int layer, int batch, int s_new, int q_heads, float scale,
                         void* out);
int attention_simple(rb_ctx* ctx, const void* q, rb_kv_cache* c, int layer, int batch, int s_new, int q_heads,
                     float scale, void* out, int dtype);
}  // namespace rb
