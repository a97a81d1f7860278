// HBM-bound kernels of the decoder layer: embedding gather, fused norm (+residual, +split-K
// reduction), RoPE + head split + paged KV append, vocabulary argmax.  Each is one pass over its
// data with float32 arithmetic inside, whatever the storage dtype.
#include <math.h>

#include <vector>

#include "ctx.h"

namespace rb {

// ------------------------------------------------------------------------------------------
// Embedding::fwd — rai-nn/src/embedding.rs:25-30.  One block per id; 16-byte copies when the row
// allows it.  Algorithmic bytes per row: 2 * hidden * elem (read + write).
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const uint32_t* __restrict__ ids, int64_t vocab,
                                    int hidden, float scale, T* __restrict__ out, uint32_t* status) {
  const int64_t i = blockIdx.x;
  uint32_t id = ids[i];
  if (id >= (uint64_t)vocab) {  // record and clamp: never read out of bounds, never trap
    if (threadIdx.x == 0) { status[0] = (uint32_t)(-RB_ERR_INVALID); status[1] = 0xE3BEDu; status[2] = id; }
    id = (uint32_t)(vocab - 1);
  }
  const T* src = table + (size_t)id * hidden;
  T* dst = out + (size_t)i * hidden;
  if (scale == 1.0f) {
    const size_t bytes = (size_t)hidden * sizeof(T);
    if ((bytes & 15) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
      const uint4* s4 = reinterpret_cast<const uint4*>(src);
      uint4* d4 = reinterpret_cast<uint4*>(dst);
      for (int j = threadIdx.x; j < (int)(bytes >> 4); j += blockDim.x) d4[j] = s4[j];
    } else {
      for (int j = threadIdx.x; j < hidden; j += blockDim.x) dst[j] = src[j];
    }
  } else {
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) dst[j] = Cvt<T>::from_f(Cvt<T>::to_f(src[j]) * scale);
  }
}

// ------------------------------------------------------------------------------------------
// Fused norm.  One block per row; the row lives in shared memory as float32 between the
// statistics pass and the scaling pass, so HBM sees one read of each input and one write of each
// output.  kind: RB_NORM_RMS (rai-nn/src/rms_norm.rs:18-22), RB_NORM_RMS_ONE_PLUS (gemma.rs:42-54),
// RB_NORM_LAYER (rai-nn/src/layer_norm.rs:32-42, population variance per hlops/var.rs:33-38).
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void norm_kernel(int kind, const T* __restrict__ x, const T* __restrict__ add,
                            const float* __restrict__ acc, int n_acc, size_t acc_stride,
                            const T* __restrict__ acc_bias, const T* __restrict__ w, const T* __restrict__ b,
                            float eps, int hidden, T* __restrict__ out, T* __restrict__ sum_out) {
  extern __shared__ float row_f[];
  __shared__ float red[32];
  const size_t base = (size_t)blockIdx.x * hidden;
  float s = 0.f;
  const float inv_sqrt_h = 1.0f / sqrtf((float)hidden);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = 0.f;
    if (x) v += Cvt<T>::to_f(x[base + i]);
    if (add) v += Cvt<T>::to_f(add[base + i]);
    for (int k = 0; k < n_acc; ++k) v += acc[(size_t)k * acc_stride + base + i];
    if (acc_bias) v += Cvt<T>::to_f(acc_bias[i]);
    const T vt = Cvt<T>::from_f(v);  // the residual stream is stored in the model dtype
    v = Cvt<T>::to_f(vt);
    if (sum_out) sum_out[base + i] = vt;
    row_f[i] = v;
    if (kind == RB_NORM_LAYER) s += v;
    else if (kind == RB_NORM_RMS) { const float t = v * inv_sqrt_h; s += t * t; }
    else s += v * v;
  }
  if (!out) return;
  s = block_sum(s, red);
  if (kind == RB_NORM_LAYER) {
    const float mean = s / (float)hidden;
    float q = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) { const float d = row_f[i] - mean; q += d * d; }
    q = block_sum(q, red);
    const float r = 1.0f / sqrtf(q / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float y = (row_f[i] - mean) * r;
      if (w) y = Cvt<T>::to_f(w[i]) * y + (b ? Cvt<T>::to_f(b[i]) : 0.f);
      out[base + i] = Cvt<T>::from_f(y);
    }
  } else if (kind == RB_NORM_RMS) {
    const float r = 1.0f / sqrtf(s + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
      out[base + i] = Cvt<T>::from_f(Cvt<T>::to_f(w[i]) * row_f[i] * r);
  } else {
    const float r = 1.0f / sqrtf(s / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
      out[base + i] = Cvt<T>::from_f(row_f[i] * r * (Cvt<T>::to_f(w[i]) + 1.0f));
  }
}

// ------------------------------------------------------------------------------------------
// Head split + RoPE + paged KV append.  One block per token.  Pairing is (i, i + rot/2) within the
// first `rot` lanes of each head ("rotate_half", qwen2.rs:33-38); lanes >= rot pass through
// (phi2.rs:66-77).  The rotation runs in float32 and the result is rounded once at the store.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_append_kernel(const T* __restrict__ qkv, const float* __restrict__ acc, int n_acc,
                                      size_t acc_stride, const T* __restrict__ bias,
                                      const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
                                      int s_new, int q_heads, int kv_heads, int d, T* __restrict__ q_out,
                                      T* __restrict__ k_cache, T* __restrict__ v_cache,
                                      const int32_t* __restrict__ block_table, const int32_t* __restrict__ seq_lens,
                                      int pages_per_seq, int max_seq, uint32_t* status) {
  extern __shared__ float vals[];  // all (q + 2 kv) * d columns of this token
  const int m = blockIdx.x;
  const int b = m / s_new, s = m % s_new;
  const int ncol = (q_heads + 2 * kv_heads) * d;
  const int pos = seq_lens[b] - s_new + s;
  if (pos < 0 || pos >= max_seq) {
    if (threadIdx.x == 0) { status[0] = (uint32_t)(-RB_ERR_INVALID); status[1] = 0x20BEu; status[2] = (uint32_t)pos; }
    return;
  }
  for (int c = threadIdx.x; c < ncol; c += blockDim.x) {
    float v = 0.f;
    if (qkv) v += Cvt<T>::to_f(qkv[(size_t)m * ncol + c]);
    for (int k = 0; k < n_acc; ++k) v += acc[(size_t)k * acc_stride + (size_t)m * ncol + c];
    if (bias) v += Cvt<T>::to_f(bias[c]);
    vals[c] = v;
  }
  __syncthreads();
  const int half = rot >> 1;
  const int page = block_table[(size_t)b * pages_per_seq + pos / kPageTokens];
  const int slot = pos % kPageTokens;
  for (int c = threadIdx.x; c < ncol; c += blockDim.x) {
    const int head = c / d, i = c % d;
    float y = vals[c];
    const bool is_v = head >= q_heads + kv_heads;
    if (!is_v && i < rot) {
      const int j = (i < half) ? i : i - half;
      const float cs = cos_t[(size_t)pos * half + j], sn = sin_t[(size_t)pos * half + j];
      const float partner = (i < half) ? -vals[c + half] : vals[c - half];
      y = y * cs + partner * sn;  // float32 inside, one rounding at the store
    }
    const T yt = Cvt<T>::from_f(y);
    if (head < q_heads) {
      q_out[(size_t)m * q_heads * d + c] = yt;
    } else {
      const int kvh = is_v ? head - q_heads - kv_heads : head - q_heads;
      const size_t off = (((size_t)page * kv_heads + kvh) * kPageTokens + slot) * d + i;
      (is_v ? v_cache : k_cache)[off] = yt;
    }
  }
}

// ------------------------------------------------------------------------------------------
// Vocabulary argmax under f32 total order, last index among equals
// (examples/qwen2/src/main.rs:32-40: `max_by(total_cmp)`).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t total_order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

template <typename T>
__global__ void argmax_rows_kernel(const T* __restrict__ x, int64_t cols, uint32_t* __restrict__ out) {
  __shared__ unsigned long long best[32];
  const T* row = x + (size_t)blockIdx.x * cols;
  unsigned long long loc = 0;  // (key << 32) | index: larger index wins among equal keys
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) {
    const unsigned long long cand = ((unsigned long long)total_order_key(Cvt<T>::to_f(row[i])) << 32) | (uint32_t)i;
    loc = cand > loc ? cand : loc;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, loc, o);
    loc = other > loc ? other : loc;
  }
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) best[wid] = loc;
  __syncthreads();
  if (wid == 0) {
    loc = (lane < (int)((blockDim.x + 31) >> 5)) ? best[lane] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, loc, o);
      loc = other > loc ? other : loc;
    }
    if (lane == 0) out[blockIdx.x] = (uint32_t)(loc & 0xffffffffull);
  }
}

}  // namespace rb

using namespace rb;

extern "C" int32_t rb_embed_gather(rb_ctx* ctx, const void* table, int32_t dtype, int64_t vocab, int64_t hidden,
                                   const uint32_t* ids, int64_t n_ids, float scale, void* out) {
  RB_REQUIRE(ctx && table && ids && out, "rb_embed_gather: null argument");
  RB_REQUIRE(vocab > 0 && hidden > 0 && n_ids >= 0, "rb_embed_gather: bad sizes");
  if (n_ids == 0) return RB_OK;
  ProfScope prof(ctx, RB_PROF_EMBED, 2.0 * n_ids * hidden * dtype_size(dtype), 0.0);
  const int threads = 128;
  if (dtype == RB_BF16)
    embed_gather_kernel<__nv_bfloat16><<<(unsigned)n_ids, threads, 0, ctx->stream>>>(
        (const __nv_bfloat16*)table, ids, vocab, (int)hidden, scale, (__nv_bfloat16*)out, ctx->status_dev);
  else if (dtype == RB_F32)
    embed_gather_kernel<float><<<(unsigned)n_ids, threads, 0, ctx->stream>>>((const float*)table, ids, vocab,
                                                                            (int)hidden, scale, (float*)out,
                                                                            ctx->status_dev);
  else
    return fail(RB_ERR_DTYPE, "rb_embed_gather: dtype %d unsupported", dtype);
  ctx->launches++;
  return launch_status("embed_gather");
}

extern "C" int32_t rb_norm(rb_ctx* ctx, int32_t kind, const void* x, const void* add, const float* acc, int32_t n_acc,
                           const void* acc_bias, const void* w, const void* b, float eps, int64_t rows, int64_t hidden,
                           void* out, void* sum_out, int32_t dtype) {
  RB_REQUIRE(ctx, "rb_norm: null context");
  RB_REQUIRE(x || add || (acc && n_acc > 0), "rb_norm: no input given");
  RB_REQUIRE(out || sum_out, "rb_norm: no output given");
  RB_REQUIRE(kind >= RB_NORM_RMS && kind <= RB_NORM_LAYER, "rb_norm: bad kind %d", kind);
  RB_REQUIRE(!out || w || kind == RB_NORM_LAYER, "rb_norm: weight required");
  RB_REQUIRE(rows >= 0 && hidden > 0 && hidden <= 49152 / 4 * 4, "rb_norm: hidden %lld out of range", (long long)hidden);
  if (rows == 0) return RB_OK;
  if (!acc) n_acc = 0;
  const size_t smem = (size_t)hidden * sizeof(float);
  const int threads = hidden >= 2048 ? 512 : 256;
  const size_t acc_stride = (size_t)rows * hidden;
  ProfScope prof(ctx, RB_PROF_NORM,
                 (double)rows * hidden * (dtype_size(dtype) * ((x ? 1 : 0) + (add ? 1 : 0) + (out ? 1 : 0) + (sum_out ? 1 : 0)) + 4.0 * n_acc),
                 0.0);
  if (dtype == RB_BF16) {
    auto kern = norm_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024) RB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<(unsigned)rows, threads, smem, ctx->stream>>>(kind, (const __nv_bfloat16*)x, (const __nv_bfloat16*)add, acc,
                                                         n_acc, acc_stride, (const __nv_bfloat16*)acc_bias,
                                                         (const __nv_bfloat16*)w, (const __nv_bfloat16*)b, eps,
                                                         (int)hidden, (__nv_bfloat16*)out, (__nv_bfloat16*)sum_out);
  } else if (dtype == RB_F32) {
    auto kern = norm_kernel<float>;
    if (smem > 48 * 1024) RB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<(unsigned)rows, threads, smem, ctx->stream>>>(kind, (const float*)x, (const float*)add, acc, n_acc,
                                                         acc_stride, (const float*)acc_bias, (const float*)w,
                                                         (const float*)b, eps, (int)hidden, (float*)out,
                                                         (float*)sum_out);
  } else {
    return fail(RB_ERR_DTYPE, "rb_norm: dtype %d unsupported", dtype);
  }
  ctx->launches++;
  return launch_status("norm");
}

extern "C" int32_t rb_rope_tables(rb_ctx* ctx, int32_t recipe, int32_t rot_dim, int32_t max_pos, double theta,
                                  float* cos_dev, float* sin_dev) {
  RB_REQUIRE(ctx && cos_dev && sin_dev, "rb_rope_tables: null argument");
  RB_REQUIRE(rot_dim > 0 && (rot_dim % 2) == 0 && max_pos > 0, "rb_rope_tables: bad sizes");
  const int half = rot_dim / 2;
  std::vector<float> inv(half), c((size_t)max_pos * half), s((size_t)max_pos * half);
  for (int j = 0; j < half; ++j) {
    const int i = 2 * j;
    if (recipe == 0) {         // qwen2.rs:45-48, gemma.rs:76-79: f64 pow, cast to f32, f32 reciprocal
      inv[j] = 1.0f / (float)pow(theta, (double)i / (double)rot_dim);
    } else if (recipe == 1) {  // phi2.rs:48-51: everything in f32
      inv[j] = 1.0f / powf((float)theta, (float)i / (float)rot_dim);
    } else {                   // phi3.rs:45-48: f64 throughout, cast with the table
      inv[j] = (float)(1.0 / pow(theta, (double)i / (double)rot_dim));
    }
  }
  for (int p = 0; p < max_pos; ++p)
    for (int j = 0; j < half; ++j) {
      const float f = (float)p * inv[j];
      c[(size_t)p * half + j] = cosf(f);
      s[(size_t)p * half + j] = sinf(f);
    }
  RB_CUDA(cudaMemcpyAsync(cos_dev, c.data(), c.size() * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  RB_CUDA(cudaMemcpyAsync(sin_dev, s.data(), s.size() * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  RB_CUDA(cudaStreamSynchronize(ctx->stream));  // the staging vectors die with this frame
  return RB_OK;
}

extern "C" int32_t rb_rope_kv_append(rb_ctx* ctx, const void* qkv, const float* acc, int32_t n_acc, const void* bias,
                                     const float* cos_t, const float* sin_t, int32_t rot, int32_t batch, int32_t s_new,
                                     int32_t q_heads, rb_kv_cache* c, int32_t layer, void* q_out, int32_t dtype) {
  RB_REQUIRE(ctx && c && q_out && cos_t && sin_t, "rb_rope_kv_append: null argument");
  RB_REQUIRE(qkv || (acc && n_acc > 0), "rb_rope_kv_append: no input given");
  RB_REQUIRE(dtype == c->dtype, "rb_rope_kv_append: cache dtype differs");
  RB_REQUIRE(layer >= 0 && layer < c->layers, "rb_rope_kv_append: layer %d out of range", layer);
  RB_REQUIRE(batch > 0 && batch <= c->max_batch && s_new > 0, "rb_rope_kv_append: bad batch/seq");
  RB_REQUIRE(rot >= 0 && rot <= c->head_dim && (rot % 2) == 0, "rb_rope_kv_append: bad rotary dim %d", rot);
  if (!acc) n_acc = 0;
  const int d = c->head_dim, ncol = (q_heads + 2 * c->kv_heads) * d;
  const size_t smem = (size_t)ncol * sizeof(float);
  const size_t acc_stride = (size_t)batch * s_new * ncol;
  const size_t loff = (size_t)layer * c->layer_stride_elems();
  const int threads = 256;
  ProfScope prof(ctx, RB_PROF_ROPE_KV, (double)batch * s_new * ncol * (dtype_size(dtype) * (qkv ? 2.0 : 1.0) + 4.0 * n_acc), 0.0);
  if (dtype == RB_BF16) {
    auto kern = rope_kv_append_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024) RB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<batch * s_new, threads, smem, ctx->stream>>>(
        (const __nv_bfloat16*)qkv, acc, n_acc, acc_stride, (const __nv_bfloat16*)bias, cos_t, sin_t, rot, s_new,
        q_heads, c->kv_heads, d, (__nv_bfloat16*)q_out, (__nv_bfloat16*)c->k + loff, (__nv_bfloat16*)c->v + loff,
        c->block_table, c->seq_lens, c->pages_per_seq, c->max_seq, ctx->status_dev);
  } else if (dtype == RB_F32) {
    auto kern = rope_kv_append_kernel<float>;
    if (smem > 48 * 1024) RB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<batch * s_new, threads, smem, ctx->stream>>>((const float*)qkv, acc, n_acc, acc_stride, (const float*)bias,
                                                        cos_t, sin_t, rot, s_new, q_heads, c->kv_heads, d,
                                                        (float*)q_out, (float*)c->k + loff, (float*)c->v + loff,
                                                        c->block_table, c->seq_lens, c->pages_per_seq, c->max_seq,
                                                        ctx->status_dev);
  } else {
    return fail(RB_ERR_DTYPE, "rb_rope_kv_append: dtype %d unsupported", dtype);
  }
  ctx->launches++;
  return launch_status("rope_kv_append");
}

extern "C" int32_t rb_argmax_rows(rb_ctx* ctx, const void* logits, int32_t dtype, int64_t rows, int64_t cols,
                                  uint32_t* out) {
  RB_REQUIRE(ctx && logits && out, "rb_argmax_rows: null argument");
  RB_REQUIRE(rows >= 0 && cols > 0 && cols <= 0xffffffffLL, "rb_argmax_rows: bad sizes");
  if (rows == 0) return RB_OK;
  ProfScope prof(ctx, RB_PROF_ARGMAX, (double)rows * cols * dtype_size(dtype), 0.0);
  if (dtype == RB_BF16)
    argmax_rows_kernel<__nv_bfloat16><<<(unsigned)rows, 1024, 0, ctx->stream>>>((const __nv_bfloat16*)logits, cols, out);
  else if (dtype == RB_F32)
    argmax_rows_kernel<float><<<(unsigned)rows, 1024, 0, ctx->stream>>>((const float*)logits, cols, out);
  else
    return fail(RB_ERR_DTYPE, "rb_argmax_rows: dtype %d unsupported", dtype);
  ctx->launches++;
  return launch_status("argmax_rows");
}
