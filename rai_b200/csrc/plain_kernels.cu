// Plain CUDA-core kernels: the float32 data path (rai's F32 models), and a bf16 cross-check of the
// tensor-core kernels that a developer can select with RAI_B200_SIMPLE=1.  Straightforward
// shared-memory tiling, float32 accumulation, no tensor cores.
#include "ctx.h"

namespace rb {

// C[m, n] = sum_k X[m, k] * W[n, k]   (both operands K-major), epilogue as in rb_linear /
// rb_gated_linear.  64 x 64 output tile, 16-wide K slices, 256 threads with a 4 x 4 micro-tile.
template <typename T, bool GATED>
__global__ void gemm_plain_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ w2,
                                  const T* __restrict__ bias, const T* __restrict__ residual, T* __restrict__ out,
                                  float* __restrict__ part, int m, int n, int k, int act, int k_per_split) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float xs[BK][BM + 1];
  __shared__ float ws[BK][BN + 1];
  __shared__ float ws2[GATED ? BK : 1][BN + 1];
  const int tm = blockIdx.y * BM, tn = blockIdx.x * BN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int k0 = blockIdx.z * k_per_split, k1 = min(k, k0 + k_per_split);
  float acc[4][4] = {}, acc2[4][4] = {};
  for (int kk = k0; kk < k1; kk += BK) {
    for (int i = threadIdx.x; i < BM * BK; i += blockDim.x) {
      const int r = i / BK, c = i % BK;
      xs[c][r] = (tm + r < m && kk + c < k1) ? Cvt<T>::to_f(x[(size_t)(tm + r) * k + kk + c]) : 0.f;
      const bool ok = tn + r < n && kk + c < k1;
      ws[c][r] = ok ? Cvt<T>::to_f(w[(size_t)(tn + r) * k + kk + c]) : 0.f;
      if (GATED) ws2[c][r] = ok ? Cvt<T>::to_f(w2[(size_t)(tn + r) * k + kk + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < BK; ++c) {
      float a[4], b[4], b2[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[c][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) { b[j] = ws[c][tx * 4 + j]; if (GATED) b2[j] = ws2[c][tx * 4 + j]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (GATED) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = tm + ty * 4 + i, c = tn + tx * 4 + j;
      if (r >= m || c >= n) continue;
      if (part) { part[((size_t)blockIdx.z * m + r) * n + c] = acc[i][j]; continue; }
      float v = acc[i][j];
      if (GATED) {
        // gate and up are tensors of the model dtype before the product (qwen2.rs:101-103)
        v = act_apply(act, v) * acc2[i][j];
      } else {
        if (bias) v += Cvt<T>::to_f(bias[c]);
        v = act_apply(act, v);
        if (residual) v += Cvt<T>::to_f(residual[(size_t)r * n + c]);
      }
      out[(size_t)r * n + c] = Cvt<T>::from_f(v);
    }
}

// Decode-sized float32 Linear (M <= 8 rows; the reference's examples generate with batch 1 in float32,
// examples/qwen2/src/main.rs:58).  One warp per output feature: its weight row is read once with 16-byte loads
// and all M dot products ride along, so the kernel is bound by the weight stream like its bf16 counterpart.
template <bool GATED>
__global__ void __launch_bounds__(256) gemv_f32_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                       const float* __restrict__ w2, const float* __restrict__ bias,
                                                       const float* __restrict__ residual, float* __restrict__ out, int m,
                                                       int n, int k, int act, int vec) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.x * 8 + warp;
  if (col >= n) return;
  const float* wr = w + (size_t)col * k;
  const float* wr2 = GATED ? w2 + (size_t)col * k : nullptr;
  float acc[8], acc2[8];
#pragma unroll
  for (int r = 0; r < 8; ++r) { acc[r] = 0.f; acc2[r] = 0.f; }
  if (vec) {
    for (int i = lane * 4; i < k; i += 128) {
      const float4 a = *reinterpret_cast<const float4*>(wr + i);
      float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
      if (GATED) b = *reinterpret_cast<const float4*>(wr2 + i);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r >= m) break;
        const float4 xv = *reinterpret_cast<const float4*>(x + (size_t)r * k + i);
        acc[r] = fmaf(a.w, xv.w, fmaf(a.z, xv.z, fmaf(a.y, xv.y, fmaf(a.x, xv.x, acc[r]))));
        if (GATED) acc2[r] = fmaf(b.w, xv.w, fmaf(b.z, xv.z, fmaf(b.y, xv.y, fmaf(b.x, xv.x, acc2[r]))));
      }
    }
  } else {
    for (int i = lane; i < k; i += 32) {
      const float a = wr[i], b = GATED ? wr2[i] : 0.f;
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r >= m) break;
        const float xv = x[(size_t)r * k + i];
        acc[r] = fmaf(a, xv, acc[r]);
        if (GATED) acc2[r] = fmaf(b, xv, acc2[r]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    if (r >= m) break;
    float v = warp_sum(acc[r]);
    const float v2 = GATED ? warp_sum(acc2[r]) : 0.f;
    if (lane != 0) continue;
    if (GATED) {
      v = act_apply(act, v) * v2;
    } else {
      if (bias) v += bias[col];
      v = act_apply(act, v);
      if (residual) v += residual[(size_t)r * n + col];
    }
    out[(size_t)r * n + col] = v;
  }
}

// One block per (token, query head): its 8 warps take every 8th key of the paged cache, each with an online
// softmax of its own (lanes split head_dim), and their (max, sum, O) states are merged through shared memory.
// float32 throughout.  Correct for any head_dim <= 256.
constexpr int kPlainAttnWarps = 8;
template <typename T>
__global__ void __launch_bounds__(kPlainAttnWarps * 32)
attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                       const int32_t* __restrict__ block_table, const int32_t* __restrict__ seq_lens, int pages_per_seq,
                       int s_new, int q_heads, int kv_heads, int d, float scale, int window, T* __restrict__ out) {
  __shared__ float sm_m[kPlainAttnWarps], sm_l[kPlainAttnWarps], sm_o[kPlainAttnWarps][256];
  const int m = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = m / s_new, s = m % s_new;
  const int limit = seq_lens[b] - s_new + s;  // last visible key
  const int kvh = h / (q_heads / kv_heads);
  float qv[8], o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int i = lane + 32 * j;
    qv[j] = i < d ? Cvt<T>::to_f(q[((size_t)m * q_heads + h) * d + i]) : 0.f;
    o[j] = 0.f;
  }
  float mx = -INFINITY, l = 0.f;
  const int call_base = seq_lens[b] - s_new;  // first token of this call
  for (int t = warp; t <= limit; t += kPlainAttnWarps) {
    // sliding window (qwen2.rs:316-334): it acts among the tokens of one call only, the cached prefix stays visible
    if (t >= call_base && t + window < limit) continue;
    const int page = block_table[(size_t)b * pages_per_seq + t / kPageTokens];
    const size_t off = (((size_t)page * kv_heads + kvh) * kPageTokens + (t % kPageTokens)) * d;
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = lane + 32 * j;
      if (i < d) dot += qv[j] * Cvt<T>::to_f(k_cache[off + i]);
    }
    dot = warp_sum(dot) * scale;
    const float mn = fmaxf(mx, dot);
    const float corr = expf(mx - mn), p = expf(dot - mn);
    l = l * corr + p;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = lane + 32 * j;
      if (i < d) o[j] = o[j] * corr + p * Cvt<T>::to_f(v_cache[off + i]);
    }
    mx = mn;
  }
  if (lane == 0) { sm_m[warp] = mx; sm_l[warp] = l; }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int i = lane + 32 * j;
    if (i < d) sm_o[warp][i] = o[j];
  }
  __syncthreads();
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < kPlainAttnWarps; ++w) M = fmaxf(M, sm_m[w]);
  float L = 0.f;
#pragma unroll
  for (int w = 0; w < kPlainAttnWarps; ++w) L += (sm_m[w] == -INFINITY) ? 0.f : sm_l[w] * expf(sm_m[w] - M);
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float O = 0.f;
#pragma unroll
    for (int w = 0; w < kPlainAttnWarps; ++w) O += (sm_m[w] == -INFINITY) ? 0.f : sm_o[w][i] * expf(sm_m[w] - M);
    out[((size_t)m * q_heads + h) * d + i] = Cvt<T>::from_f(O / L);
  }
}

static bool gemv_f32_launch(rb_ctx* ctx, const GemmArgs& a) {
  if (a.partials || a.m > 8) return false;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const int vec = (a.k % 4 == 0) && al16(a.x) && al16(a.w) && (!a.w2 || al16(a.w2));
  const dim3 grid((unsigned)((a.n + 7) / 8));
  if (a.w2)
    gemv_f32_kernel<true><<<grid, 256, 0, ctx->stream>>>((const float*)a.x, (const float*)a.w, (const float*)a.w2, nullptr, nullptr,
                                                         (float*)a.out, (int)a.m, (int)a.n, (int)a.k, a.act, vec);
  else
    gemv_f32_kernel<false><<<grid, 256, 0, ctx->stream>>>((const float*)a.x, (const float*)a.w, nullptr, (const float*)a.bias,
                                                          (const float*)a.residual, (float*)a.out, (int)a.m, (int)a.n, (int)a.k,
                                                          a.act, vec);
  ctx->launches++;
  return true;
}

template <typename T>
static int gemm_plain_launch(rb_ctx* ctx, const GemmArgs& a) {
  const int splits = a.partials ? a.n_split : 1;
  dim3 grid((unsigned)((a.n + 63) / 64), (unsigned)((a.m + 63) / 64), (unsigned)splits);
  int kps = (int)a.k;
  if (splits > 1) kps = (int)(((a.k + splits - 1) / splits + 15) / 16 * 16);
  if (a.w2)
    gemm_plain_kernel<T, true><<<grid, 256, 0, ctx->stream>>>((const T*)a.x, (const T*)a.w, (const T*)a.w2, nullptr,
                                                             nullptr, (T*)a.out, nullptr, (int)a.m, (int)a.n, (int)a.k,
                                                             a.act, kps);
  else
    gemm_plain_kernel<T, false><<<grid, 256, 0, ctx->stream>>>(
        (const T*)a.x, (const T*)a.w, nullptr, (const T*)a.bias, (const T*)a.residual, a.partials ? nullptr : (T*)a.out,
        a.partials ? (float*)a.out : nullptr, (int)a.m, (int)a.n, (int)a.k, a.act, kps);
  ctx->launches++;
  return launch_status("gemm_plain");
}

int gemm_simple(rb_ctx* ctx, const GemmArgs& a, int dtype) {
  if (a.m == 0 || a.n == 0) return RB_OK;
  if (dtype == RB_F32) {
    if (gemv_f32_launch(ctx, a)) return launch_status("gemv_f32");
    return gemm_plain_launch<float>(ctx, a);
  }
  if (dtype == RB_BF16) return gemm_plain_launch<__nv_bfloat16>(ctx, a);
  return fail(RB_ERR_DTYPE, "gemm: dtype %d unsupported", dtype);
}

int attention_simple(rb_ctx* ctx, const void* q, rb_kv_cache* c, int layer, int batch, int s_new, int q_heads,
                     float scale, void* out, int dtype) {
  const size_t loff = (size_t)layer * c->layer_stride_elems();
  const int warps = kPlainAttnWarps;
  dim3 grid((unsigned)(batch * s_new), (unsigned)q_heads);
  if (dtype == RB_F32)
    attention_plain_kernel<float><<<grid, warps * 32, 0, ctx->stream>>>(
        (const float*)q, (const float*)c->k + loff, (const float*)c->v + loff, c->block_table, c->seq_lens,
        c->pages_per_seq, s_new, q_heads, c->kv_heads, c->head_dim, scale, c->window, (float*)out);
  else if (dtype == RB_BF16)
    attention_plain_kernel<__nv_bfloat16><<<grid, warps * 32, 0, ctx->stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)c->k + loff, (const __nv_bfloat16*)c->v + loff, c->block_table,
        c->seq_lens, c->pages_per_seq, s_new, q_heads, c->kv_heads, c->head_dim, scale, c->window, (__nv_bfloat16*)out);
  else
    return fail(RB_ERR_DTYPE, "attention: dtype %d unsupported", dtype);
  ctx->launches++;
  return launch_status("attention_plain");
}

}  // namespace rb
