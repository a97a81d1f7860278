// Context, memory, KV-cache management and the dispatch of the fused entry points to their kernels.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <string>

#include "ctx.h"

namespace rb {

static thread_local std::string g_last_error;

void set_error(const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
}

int fail(int code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

}  // namespace rb

using namespace rb;

static void prof_clear(rb_ctx* ctx) {
  for (auto& r : ctx->prof) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
  ctx->prof.clear();
}

extern "C" const char* rb_last_error(void) { return g_last_error.c_str(); }

extern "C" int32_t rb_init(int32_t device, rb_ctx** out) {
  RB_REQUIRE(out, "rb_init: null output");
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return fail(RB_ERR_CUDA, "rb_init: no CUDA device available (%s); this library has no CPU path",
                e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
  RB_REQUIRE(device >= 0 && device < count, "rb_init: device %d out of range (0..%d)", device, count - 1);
  RB_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  RB_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(RB_ERR_UNIMPLEMENTED, "rb_init: device %d is sm_%d%d; this library is built for sm_100a only", device,
                prop.major, prop.minor);
  rb_ctx* c = new rb_ctx();
  c->device = device;
  c->sm_count = prop.multiProcessorCount;
  {
    int khz = 0;
    if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device) == cudaSuccess && khz > 0) c->cycles_per_us = khz / 1000.0;
    else cudaGetLastError();
  }
  RB_CUDA(cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking));
  c->stream = c->own_stream;
  RB_CUDA(cudaMalloc(&c->status_dev, 4 * sizeof(uint32_t)));
  RB_CUDA(cudaMemset(c->status_dev, 0, 4 * sizeof(uint32_t)));
  RB_CUDA(cudaMalloc(&c->argmax_best, kArgmaxRows * sizeof(unsigned long long)));
  RB_CUDA(cudaMalloc(&c->argmax_count, kArgmaxRows * sizeof(unsigned int)));
  RB_CUDA(cudaMemset(c->argmax_best, 0, kArgmaxRows * sizeof(unsigned long long)));
  RB_CUDA(cudaMemset(c->argmax_count, 0, kArgmaxRows * sizeof(unsigned int)));
  RB_CUDA(cudaMalloc(&c->gemm_tile_count, 2 * kGemmMaxReduceTiles * sizeof(uint32_t)));
  RB_CUDA(cudaMemset(c->gemm_tile_count, 0, 2 * kGemmMaxReduceTiles * sizeof(uint32_t)));
  const char* dbg = getenv("RAI_B200_SIMPLE");
  c->debug_simple = dbg && dbg[0] == '1';
  const char* dg = getenv("RAI_B200_SIMPLE_GEMM");
  const char* da = getenv("RAI_B200_SIMPLE_ATTN");
  c->debug_simple_gemm = c->debug_simple || (dg && dg[0] == '1');
  c->debug_simple_attn = c->debug_simple || (da && da[0] == '1');
  const char* nf = getenv("RAI_B200_FUSE_ROPE");  // RAI_B200_FUSE_ROPE=0: separate RoPE/append and attention launches
  c->debug_no_fuse = nf && nf[0] == '0';
  const char* pdl = getenv("RAI_B200_PDL");
  c->pdl = !(pdl && pdl[0] == '0');
  if (const char* at = getenv("RAI_B200_ATTN_TC")) c->attn_tc = at[0] != '0';
  if (const char* gr = getenv("RAI_B200_GEMM_REDUCE")) c->gemm_reduce = gr[0] != '0';
  if (const char* rk = getenv("RAI_B200_GEMM_RING_KB")) {
    const long kb = atol(rk);
    if (kb >= 32 && kb <= 200) c->gemm_ring_bytes = (size_t)kb * 1024;
  }
  *out = c;
  return RB_OK;
}

extern "C" int32_t rb_destroy(rb_ctx* ctx) {
  if (!ctx) return RB_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  prof_clear(ctx);
  if (ctx->status_dev) cudaFree(ctx->status_dev);
  if (ctx->argmax_best) cudaFree(ctx->argmax_best);
  if (ctx->argmax_count) cudaFree(ctx->argmax_count);
  if (ctx->attn_scratch) cudaFree(ctx->attn_scratch);
  for (void* r : ctx->retired) cudaFree(r);
  if (ctx->gemm_scratch) cudaFree(ctx->gemm_scratch);
  if (ctx->gemm_tile_count) cudaFree(ctx->gemm_tile_count);
  if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
  delete ctx;
  return RB_OK;
}

extern "C" int32_t rb_set_stream(rb_ctx* ctx, void* s) {
  RB_REQUIRE(ctx, "rb_set_stream: null context");
  ctx->stream = (cudaStream_t)s;  // NULL is CUDA's default stream, which torch uses unless told otherwise
  return RB_OK;
}

extern "C" int32_t rb_status_word(rb_ctx* ctx, uint32_t* out4) {
  RB_REQUIRE(ctx && out4, "rb_status_word: null argument");
  RB_CUDA(cudaStreamSynchronize(ctx->stream));
  RB_CUDA(cudaMemcpy(out4, ctx->status_dev, 4 * sizeof(uint32_t), cudaMemcpyDeviceToHost));
  return RB_OK;
}

extern "C" int32_t rb_sync(rb_ctx* ctx) {
  RB_REQUIRE(ctx, "rb_sync: null context");
  uint32_t w[4];
  RB_TRY(rb_status_word(ctx, w));
  if (w[0] != 0) {
    RB_CUDA(cudaMemset(ctx->status_dev, 0, 4 * sizeof(uint32_t)));
    const int code = -(int)w[0];
    if (code == RB_ERR_TIMEOUT) {
      // blocks that gave up returned before they were counted: re-arm the self-resetting arrival counters
      for (rb_kv_cache* kc : ctx->caches)
        RB_CUDA(cudaMemset(kc->split_count, 0, (size_t)kc->max_batch * kc->kv_heads * sizeof(uint32_t)));
      RB_CUDA(cudaMemset(ctx->argmax_best, 0, kArgmaxRows * sizeof(unsigned long long)));
      RB_CUDA(cudaMemset(ctx->argmax_count, 0, kArgmaxRows * sizeof(unsigned int)));
      RB_CUDA(cudaMemset(ctx->gemm_tile_count, 0, 2 * kGemmMaxReduceTiles * sizeof(uint32_t)));
    }
    return fail(code, "device-side check failed: code %d at 0x%x (detail %u, %u)", code, w[1], w[2], w[3]);
  }
  return RB_OK;
}

extern "C" int32_t rb_set_wait_budget_us(rb_ctx* ctx, int64_t microseconds) {
  RB_REQUIRE(ctx, "rb_set_wait_budget_us: null context");
  RB_REQUIRE(microseconds >= 1 && microseconds <= 60000000, "rb_set_wait_budget_us: %lld us outside [1, 60 000 000]",
             (long long)microseconds);
  ctx->wait_budget_cycles = (long long)((double)microseconds * ctx->cycles_per_us);
  return RB_OK;
}

extern "C" int32_t rb_profile_start(rb_ctx* ctx) {
  RB_REQUIRE(ctx, "rb_profile_start: null context");
  RB_CUDA(cudaStreamSynchronize(ctx->stream));
  prof_clear(ctx);
  ctx->profiling = true;
  return RB_OK;
}

extern "C" int32_t rb_profile_read(rb_ctx* ctx, int32_t cls, double* out4) {
  RB_REQUIRE(ctx && out4, "rb_profile_read: null argument");
  RB_REQUIRE(cls >= 0 && cls < RB_PROF_CLASSES, "rb_profile_read: unknown kernel class %d", cls);
  ctx->profiling = false;
  RB_CUDA(cudaStreamSynchronize(ctx->stream));
  out4[0] = out4[1] = out4[2] = out4[3] = 0.0;
  for (auto& r : ctx->prof) {
    if (r.cls != cls) continue;
    float ms = 0.f;
    RB_CUDA(cudaEventElapsedTime(&ms, r.a, r.b));
    out4[0] += 1.0; out4[1] += ms; out4[2] += r.bytes; out4[3] += r.flops;
  }
  return RB_OK;
}

extern "C" int32_t rb_sm_count(rb_ctx* ctx) { return ctx ? ctx->sm_count : 0; }
extern "C" int64_t rb_launch_count(rb_ctx* ctx) { return ctx ? ctx->launches : 0; }

extern "C" int32_t rb_malloc(rb_ctx* ctx, size_t bytes, void** out) {
  RB_REQUIRE(ctx && out, "rb_malloc: null argument");
  *out = nullptr;
  if (bytes == 0) return RB_OK;
  cudaError_t e = cudaMalloc(out, bytes);
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();
    return fail(RB_ERR_OOM, "rb_malloc: out of device memory asking for %zu bytes", bytes);
  }
  RB_CUDA(e);
  return RB_OK;
}

// Stream-ordered allocation from the device's memory pool, for bindings that allocate a fresh output per
// primitive (every Eval rule of the reference does, candle.rs:197-1004): no device synchronisation on either
// side, freed blocks are reused by later allocations on the same stream.
extern "C" int32_t rb_malloc_async(rb_ctx* ctx, size_t bytes, void** out) {
  RB_REQUIRE(ctx && out, "rb_malloc_async: null argument");
  *out = nullptr;
  if (bytes == 0) return RB_OK;
  if (!ctx->pool_ready) {
    cudaMemPool_t pool = nullptr;
    RB_CUDA(cudaDeviceGetDefaultMemPool(&pool, ctx->device));
    unsigned long long keep = ~0ull;  // keep freed memory in the pool instead of returning it to the driver
    RB_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
    ctx->pool_ready = true;
  }
  cudaError_t e = cudaMallocAsync(out, bytes, ctx->stream);
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();
    return fail(RB_ERR_OOM, "rb_malloc_async: out of device memory asking for %zu bytes", bytes);
  }
  RB_CUDA(e);
  return RB_OK;
}

extern "C" int32_t rb_free_async(rb_ctx* ctx, void* dev) {
  RB_REQUIRE(ctx, "rb_free_async: null context");
  if (!dev) return RB_OK;
  // ordered after everything already issued on the context's stream; tensor maps keyed by this address stay
  // valid for a later allocation of the same address and shape, and are dropped wholesale when the table fills
  RB_CUDA(cudaFreeAsync(dev, ctx->stream));
  return RB_OK;
}

extern "C" int32_t rb_free(rb_ctx* ctx, void* dev) {
  RB_REQUIRE(ctx, "rb_free: null context");
  if (!dev) return RB_OK;
  RB_CUDA(cudaStreamSynchronize(ctx->stream));
  // tensor maps built over this allocation must not outlive it
  for (auto it = ctx->tmaps.begin(); it != ctx->tmaps.end();)
    it = (std::get<0>(it->first) == dev) ? ctx->tmaps.erase(it) : std::next(it);
  RB_CUDA(cudaFree(dev));
  return RB_OK;
}

extern "C" int32_t rb_upload(rb_ctx* ctx, void* dst, const void* src, size_t bytes) {
  RB_REQUIRE(ctx && (bytes == 0 || (dst && src)), "rb_upload: null argument");
  if (bytes) RB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  return RB_OK;
}

extern "C" int32_t rb_download(rb_ctx* ctx, void* dst, const void* src, size_t bytes) {
  RB_REQUIRE(ctx && (bytes == 0 || (dst && src)), "rb_download: null argument");
  if (bytes) RB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  RB_CUDA(cudaStreamSynchronize(ctx->stream));
  return RB_OK;
}

// ------------------------------------------------------------------------------------------ KV cache
extern "C" int32_t rb_kv_cache_create(rb_ctx* ctx, int32_t layers, int32_t kv_heads, int32_t head_dim,
                                      int32_t max_batch, int32_t max_seq, int32_t dtype, rb_kv_cache** out) {
  RB_REQUIRE(ctx && out, "rb_kv_cache_create: null argument");
  RB_REQUIRE(layers > 0 && kv_heads > 0 && head_dim > 0 && max_batch > 0 && max_seq > 0, "rb_kv_cache_create: bad sizes");
  RB_REQUIRE(dtype == RB_BF16 || dtype == RB_F32, "rb_kv_cache_create: dtype %d unsupported", dtype);
  RB_REQUIRE(head_dim % 8 == 0 && head_dim <= 256, "rb_kv_cache_create: head_dim %d unsupported", head_dim);
  rb_kv_cache* c = new rb_kv_cache();
  c->ctx = ctx;
  c->layers = layers; c->kv_heads = kv_heads; c->head_dim = head_dim;
  c->max_batch = max_batch; c->dtype = dtype;
  c->pages_per_seq = (max_seq + kPageTokens - 1) / kPageTokens;
  c->max_seq = c->pages_per_seq * kPageTokens;
  c->num_pages = c->pages_per_seq * max_batch;
  const size_t bytes = (size_t)layers * c->layer_stride_elems() * dtype_size(dtype);
  int st = rb_malloc(ctx, bytes, &c->k);
  if (st == RB_OK) st = rb_malloc(ctx, bytes, &c->v);
  if (st == RB_OK) st = rb_malloc(ctx, (size_t)c->num_pages * sizeof(int32_t), (void**)&c->block_table);
  if (st == RB_OK) st = rb_malloc(ctx, (size_t)max_batch * sizeof(int32_t), (void**)&c->seq_lens);
  if (st == RB_OK) st = rb_malloc(ctx, (size_t)max_batch * kv_heads * sizeof(uint32_t), (void**)&c->split_count);
  if (st != RB_OK) { rb_kv_cache_destroy(c); return st; }
  // Zero the pages: the tail of a sequence's last page is read (and masked) by the attention
  // kernels, so it must hold finite values.
  RB_CUDA(cudaMemsetAsync(c->k, 0, bytes, ctx->stream));
  RB_CUDA(cudaMemsetAsync(c->v, 0, bytes, ctx->stream));
  std::vector<int32_t> bt(c->num_pages);
  for (int i = 0; i < c->num_pages; ++i) bt[i] = i;  // sequence b owns pages [b*pages_per_seq, ...)
  RB_CUDA(cudaMemcpyAsync(c->block_table, bt.data(), bt.size() * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
  RB_CUDA(cudaMemsetAsync(c->seq_lens, 0, (size_t)max_batch * sizeof(int32_t), ctx->stream));
  RB_CUDA(cudaMemsetAsync(c->split_count, 0, (size_t)max_batch * kv_heads * sizeof(uint32_t), ctx->stream));
  RB_CUDA(cudaStreamSynchronize(ctx->stream));
  c->host_lens.assign(max_batch, 0);
  ctx->caches.push_back(c);
  *out = c;
  return RB_OK;
}

extern "C" int32_t rb_kv_cache_destroy(rb_kv_cache* c) {
  if (!c) return RB_OK;
  cudaStreamSynchronize(c->ctx->stream);
  for (auto it = c->ctx->caches.begin(); it != c->ctx->caches.end(); ++it)
    if (*it == c) { c->ctx->caches.erase(it); break; }
  if (c->k) cudaFree(c->k);
  if (c->v) cudaFree(c->v);
  if (c->block_table) cudaFree(c->block_table);
  if (c->seq_lens) cudaFree(c->seq_lens);
  if (c->split_count) cudaFree(c->split_count);
  delete c;
  return RB_OK;
}

extern "C" int32_t rb_kv_cache_reset(rb_kv_cache* c) {
  RB_REQUIRE(c, "rb_kv_cache_reset: null cache");
  RB_CUDA(cudaMemsetAsync(c->seq_lens, 0, (size_t)c->max_batch * sizeof(int32_t), c->ctx->stream));
  c->host_lens.assign(c->max_batch, 0);
  return RB_OK;
}

extern "C" int32_t rb_kv_cache_set_window(rb_kv_cache* c, int32_t window) {
  RB_REQUIRE(c, "rb_kv_cache_set_window: null cache");
  RB_REQUIRE(window >= 0, "rb_kv_cache_set_window: negative window %d", window);
  c->window = window > (1 << 30) ? (1 << 30) : window;   // key + window must not overflow an int
  return RB_OK;
}

extern "C" int32_t rb_kv_cache_set_len(rb_kv_cache* c, int32_t batch, int32_t len) {
  RB_REQUIRE(c, "rb_kv_cache_set_len: null cache");
  RB_REQUIRE(batch > 0 && batch <= c->max_batch, "rb_kv_cache_set_len: batch %d exceeds capacity %d", batch, c->max_batch);
  RB_REQUIRE(len >= 0 && len <= c->max_seq, "rb_kv_cache_set_len: length %d exceeds capacity %d", len, c->max_seq);
  for (int b = 0; b < batch; ++b) c->host_lens[b] = len;
  // host_lens is a std::vector that outlives the copy; pageable source: the copy is staged by the runtime
  RB_CUDA(cudaMemcpyAsync(c->seq_lens, c->host_lens.data(), (size_t)batch * sizeof(int32_t), cudaMemcpyHostToDevice,
                          c->ctx->stream));
  return RB_OK;
}

extern "C" int32_t rb_kv_cache_read(rb_kv_cache* c, int32_t layer, int32_t seq, int32_t kv_head, int32_t t0, int32_t n,
                                    void* k_host, void* v_host) {
  RB_REQUIRE(c && k_host && v_host, "rb_kv_cache_read: null argument");
  RB_REQUIRE(layer >= 0 && layer < c->layers && seq >= 0 && seq < c->max_batch && kv_head >= 0 && kv_head < c->kv_heads,
             "rb_kv_cache_read: index out of range");
  RB_REQUIRE(t0 >= 0 && n >= 0 && t0 + n <= c->max_seq, "rb_kv_cache_read: token range out of capacity");
  const size_t es = dtype_size(c->dtype), row = (size_t)c->head_dim * es;
  RB_CUDA(cudaStreamSynchronize(c->ctx->stream));
  for (int i = 0; i < n; ++i) {
    const int t = t0 + i;
    const int page = seq * c->pages_per_seq + t / kPageTokens;  // identity block table
    const size_t off = ((size_t)layer * c->layer_stride_elems() +
                        (((size_t)page * c->kv_heads + kv_head) * kPageTokens + t % kPageTokens) * c->head_dim) * es;
    RB_CUDA(cudaMemcpy((char*)k_host + i * row, (char*)c->k + off, row, cudaMemcpyDeviceToHost));
    RB_CUDA(cudaMemcpy((char*)v_host + i * row, (char*)c->v + off, row, cudaMemcpyDeviceToHost));
  }
  return RB_OK;
}

// ------------------------------------------------------------------------------------------ fused ops
extern "C" int32_t rb_linear(rb_ctx* ctx, const void* x, const void* w, const void* bias, const void* residual,
                             void* out, int64_t m, int64_t n, int64_t k, int32_t act, int32_t dtype) {
  RB_REQUIRE(ctx && x && w && out, "rb_linear: null argument");
  RB_REQUIRE(m >= 0 && n > 0 && k > 0, "rb_linear: bad sizes");
  GemmArgs a;
  a.x = x; a.w = w; a.bias = bias; a.residual = residual; a.out = out;
  a.m = m; a.n = n; a.k = k; a.act = act;
  a.reduce = ctx->gemm_reduce;  // decode-sized with few weight tiles: split K over idle SMs, summed inside the kernel
  const double es = (double)dtype_size(dtype);
  ProfScope prof(ctx, RB_PROF_GEMM, es * ((double)n * k + (double)m * k + (double)m * n * (residual ? 2 : 1) + (bias ? n : 0)),
                 2.0 * m * n * k);
  if (dtype == RB_BF16 && !ctx->debug_simple_gemm) return gemm_tc_bf16(ctx, a);
  return gemm_simple(ctx, a, dtype);
}

extern "C" int32_t rb_gated_linear(rb_ctx* ctx, const void* x, const void* wg, const void* wu, void* out, int64_t m,
                                   int64_t n, int64_t k, int32_t act, int32_t dtype) {
  RB_REQUIRE(ctx && x && wg && wu && out, "rb_gated_linear: null argument");
  RB_REQUIRE(m >= 0 && n > 0 && k > 0, "rb_gated_linear: bad sizes");
  GemmArgs a;
  a.x = x; a.w = wg; a.w2 = wu; a.out = out;
  a.m = m; a.n = n; a.k = k; a.act = act;
  a.reduce = ctx->gemm_reduce;
  const double es = (double)dtype_size(dtype);
  ProfScope prof(ctx, RB_PROF_GEMM, es * (2.0 * n * k + (double)m * k + (double)m * n), 4.0 * m * n * k);
  if (dtype == RB_BF16 && !ctx->debug_simple_gemm) return gemm_tc_bf16(ctx, a);
  return gemm_simple(ctx, a, dtype);
}

extern "C" int32_t rb_linear_partials(rb_ctx* ctx, const void* x, const void* w, float* part, int64_t m, int64_t n,
                                      int64_t k, int32_t n_split) {
  RB_REQUIRE(ctx && x && w && part, "rb_linear_partials: null argument");
  RB_REQUIRE(m > 0 && m <= 256 && n > 0 && k > 0 && n_split >= 1, "rb_linear_partials: bad sizes (M must be <= 256)");
  GemmArgs a;
  a.x = x; a.w = w; a.out = part;
  a.m = m; a.n = n; a.k = k;
  a.n_split = n_split; a.partials = true;
  ProfScope prof(ctx, RB_PROF_GEMM, 2.0 * ((double)n * k + (double)m * k) + 4.0 * n_split * m * n, 2.0 * m * n * k);
  if (!ctx->debug_simple_gemm) return gemm_tc_bf16(ctx, a);
  return gemm_simple(ctx, a, RB_BF16);
}

extern "C" int32_t rb_linear_pick_splits(rb_ctx* ctx, int64_t m, int64_t n, int64_t k) {
  if (!ctx || m <= 0 || n <= 0 || k <= 0) return 1;
  return gemm_tc_pick_splits(ctx, m, n, k);
}

extern "C" int32_t rb_rope_attention_decode(rb_ctx* ctx, const void* qkv, const float* acc, int32_t n_acc, const void* bias,
                                            const float* cos_t, const float* sin_t, int32_t rot, int32_t batch,
                                            int32_t q_heads, rb_kv_cache* c, int32_t layer, float scale, void* q_scratch,
                                            void* out, int32_t dtype) {
  RB_REQUIRE(ctx && c && out && cos_t && sin_t && q_scratch, "rb_rope_attention_decode: null argument");
  RB_REQUIRE(qkv || (acc && n_acc > 0), "rb_rope_attention_decode: no input given");
  RB_REQUIRE(dtype == c->dtype, "rb_rope_attention_decode: cache dtype differs");
  RB_REQUIRE(layer >= 0 && layer < c->layers, "rb_rope_attention_decode: layer %d out of range", layer);
  RB_REQUIRE(batch > 0 && batch <= c->max_batch, "rb_rope_attention_decode: bad batch");
  RB_REQUIRE(q_heads > 0 && q_heads % c->kv_heads == 0, "rb_rope_attention_decode: %d query heads over %d KV heads", q_heads,
             c->kv_heads);
  RB_REQUIRE(rot >= 0 && rot <= c->head_dim && (rot % 2) == 0, "rb_rope_attention_decode: bad rotary dim %d", rot);
  for (int b = 0; b < batch; ++b)
    RB_REQUIRE(c->host_lens[b] >= 1, "rb_rope_attention_decode: sequence %d is empty (its length must already count the new token)", b);
  if (!acc) n_acc = 0;
  const bool fused = dtype == RB_BF16 && !ctx->debug_simple_attn && !ctx->debug_no_fuse &&
                     attention_can_fuse_rope(c, q_heads, rot, qkv, acc, n_acc, bias, cos_t, sin_t, batch);
  if (!fused) {
    RB_TRY(rb_rope_kv_append(ctx, qkv, acc, n_acc, bias, cos_t, sin_t, rot, batch, 1, q_heads, c, layer, q_scratch, dtype));
    return rb_attention(ctx, q_scratch, c, layer, batch, 1, q_heads, scale, out, dtype);
  }
  double kv_tokens = 0.0;
  for (int b = 0; b < batch; ++b) kv_tokens += c->host_lens[b];
  const double d = c->head_dim, ncol = (double)(q_heads + 2 * c->kv_heads) * d;
  ProfScope prof(ctx, RB_PROF_ATTENTION,
                 2.0 * (2.0 * kv_tokens * c->kv_heads * d + batch * q_heads * d) + batch * ncol * ((qkv ? 2.0 : 0.0) + 4.0 * n_acc) +
                     2.0 * batch * 2.0 * c->kv_heads * d,
                 4.0 * kv_tokens * q_heads * d);
  return attention_decode_fused_rope(ctx, qkv, acc, n_acc, bias, cos_t, sin_t, rot, c, layer, batch, q_heads, scale, out);
}

extern "C" int32_t rb_attention(rb_ctx* ctx, const void* q, rb_kv_cache* c, int32_t layer, int32_t batch, int32_t s_new,
                                int32_t q_heads, float scale, void* out, int32_t dtype) {
  RB_REQUIRE(ctx && q && c && out, "rb_attention: null argument");
  RB_REQUIRE(dtype == c->dtype, "rb_attention: cache dtype differs");
  RB_REQUIRE(layer >= 0 && layer < c->layers, "rb_attention: layer %d out of range", layer);
  RB_REQUIRE(batch > 0 && batch <= c->max_batch && s_new > 0, "rb_attention: bad batch/seq");
  RB_REQUIRE(q_heads > 0 && q_heads % c->kv_heads == 0, "rb_attention: %d query heads over %d KV heads", q_heads,
             c->kv_heads);
  for (int b = 0; b < batch; ++b)
    RB_REQUIRE(c->host_lens[b] >= s_new, "rb_attention: sequence %d holds %d tokens, fewer than the %d new ones", b,
               c->host_lens[b], s_new);
  double kv_tokens = 0.0, pairs = 0.0;  // keys read; (query, key) pairs under the causal mask
  for (int b = 0; b < batch; ++b) {
    const double len = c->host_lens[b];
    kv_tokens += len;
    pairs += (double)s_new * (len - s_new) + 0.5 * s_new * (s_new + 1.0);
  }
  const double es = (double)dtype_size(dtype), d = c->head_dim;
  ProfScope prof(ctx, RB_PROF_ATTENTION,
                 es * (2.0 * kv_tokens * c->kv_heads * d + 2.0 * batch * s_new * q_heads * d), 4.0 * pairs * q_heads * d);
  if (dtype == RB_BF16 && !ctx->debug_simple_attn) return attention_mma_bf16(ctx, q, c, layer, batch, s_new, q_heads, scale, out);
  return attention_simple(ctx, q, c, layer, batch, s_new, q_heads, scale, out, dtype);
}
