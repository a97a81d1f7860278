// The primitive set: one kernel per Eval rule of rai-core/src/backend/candle.rs that the decoders'
// unfused graphs reach (elementwise, broadcast binary, softmax, reductions, strided copies, casts,
// index_select / gather, where, fill / arange, batched matmul).  These keep `Tensor::...(&Cuda)`
// working for arbitrary graphs; the decoder driver itself uses the fused kernels instead.
#include <math.h>

#include "ctx.h"

namespace rb {

template <typename T>
__global__ void unary_kernel(int op, const T* __restrict__ x, T* __restrict__ out, int64_t n, float sc) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = Cvt<T>::to_f(x[i]);
    float y;
    switch (op) {
      case RB_UN_NEG: y = -v; break;
      case RB_UN_EXP: y = expf(v); break;
      case RB_UN_SQRT: y = sqrtf(v); break;
      case RB_UN_RSQRT: y = 1.0f / sqrtf(v); break;  // candle.rs:545-553: sqrt then recip
      case RB_UN_SQUARE: y = v * v; break;
      case RB_UN_TANH: y = tanhf(v); break;
      case RB_UN_ERF: y = erff(v); break;
      case RB_UN_SIN: y = sinf(v); break;
      case RB_UN_COS: y = cosf(v); break;
      case RB_UN_POWF: y = powf(v, sc); break;
      case RB_UN_SILU: y = act_apply(RB_ACT_SILU, v); break;
      case RB_UN_GELU_TANH: y = act_apply(RB_ACT_GELU_TANH, v); break;
      case RB_UN_GELU_ERF: y = act_apply(RB_ACT_GELU_ERF, v); break;
      case RB_UN_RELU: y = fmaxf(v, 0.f); break;
      case RB_UN_LOG: y = logf(v); break;
      case RB_UN_ABS: y = fabsf(v); break;
      case RB_UN_RECIP: y = 1.0f / v; break;
      case RB_UN_ADD_SCALAR: y = v + sc; break;
      case RB_UN_MUL_SCALAR: y = v * sc; break;
      case RB_UN_SIGN: y = (v > 0.f) ? 1.f : (v < 0.f ? -1.f : 0.f); break;
      case RB_UN_LOG2: y = log2f(v); break;
      case RB_UN_LOG10: y = log10f(v); break;
      default: y = v;
    }
    out[i] = Cvt<T>::from_f(y);
  }
}

struct Dims4 {
  int64_t shape[4];
  int64_t sa[4];
  int64_t sb[4];
};

template <typename T>
__global__ void binary_kernel(int op, const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, Dims4 d,
                              int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i, oa = 0, ob = 0;
#pragma unroll
    for (int k = 3; k >= 0; --k) {
      const int64_t c = r % d.shape[k];
      r /= d.shape[k];
      oa += c * d.sa[k];
      ob += c * d.sb[k];
    }
    const float x = Cvt<T>::to_f(a[oa]), y = Cvt<T>::to_f(b[ob]);
    float z;
    switch (op) {
      case RB_BIN_ADD: z = x + y; break;
      case RB_BIN_SUB: z = x - y; break;
      case RB_BIN_MUL: z = x * y; break;
      case RB_BIN_DIV: z = x / y; break;
      case RB_BIN_MAXIMUM: z = fmaxf(x, y); break;
      default: z = fminf(x, y);
    }
    out[i] = Cvt<T>::from_f(z);
  }
}

// candle.rs:792-803 — max, subtract, exp, sum, divide; one block per row, float32 inside.
template <typename T>
__global__ void softmax_rows_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t cols) {
  __shared__ float red[32];
  const T* row = x + (size_t)blockIdx.x * cols;
  T* orow = out + (size_t)blockIdx.x * cols;
  float mx = -INFINITY;
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) mx = fmaxf(mx, Cvt<T>::to_f(row[i]));
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = (threadIdx.x & 31) < ((blockDim.x + 31) >> 5) ? red[threadIdx.x & 31] : -INFINITY;
  mx = warp_max(mx);
  float s = 0.f;
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) s += expf(Cvt<T>::to_f(row[i]) - mx);
  s = block_sum(s, red);
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x)
    orow[i] = Cvt<T>::from_f(expf(Cvt<T>::to_f(row[i]) - mx) / s);
}

template <typename T>
__global__ void reduce_rows_kernel(int op, const T* __restrict__ x, T* __restrict__ out, int64_t cols) {
  __shared__ float red[32];
  const T* row = x + (size_t)blockIdx.x * cols;
  float v = op == RB_RED_SUM ? 0.f : op == RB_RED_MAX ? -INFINITY : INFINITY;
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) {
    const float e = Cvt<T>::to_f(row[i]);
    v = op == RB_RED_SUM ? v + e : op == RB_RED_MAX ? fmaxf(v, e) : fminf(v, e);
  }
  if (op == RB_RED_SUM) {
    v = block_sum(v, red);
  } else {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float u = __shfl_xor_sync(0xffffffffu, v, o);
      v = op == RB_RED_MAX ? fmaxf(v, u) : fminf(v, u);
    }
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    const float init = op == RB_RED_MAX ? -INFINITY : INFINITY;
    v = (threadIdx.x & 31) < ((blockDim.x + 31) >> 5) ? red[threadIdx.x & 31] : init;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float u = __shfl_xor_sync(0xffffffffu, v, o);
      v = op == RB_RED_MAX ? fmaxf(v, u) : fminf(v, u);
    }
  }
  if (threadIdx.x == 0) out[blockIdx.x] = Cvt<T>::from_f(v);
}

struct Dims6 {
  int64_t shape[6];
  int64_t sx[6];
  int64_t so[6];
};

template <typename E>
__global__ void copy_strided_kernel(const E* __restrict__ x, E* __restrict__ out, Dims6 d, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i, ox = 0, oo = 0;
#pragma unroll
    for (int k = 5; k >= 0; --k) {
      const int64_t c = r % d.shape[k];
      r /= d.shape[k];
      ox += c * d.sx[k];
      oo += c * d.so[k];
    }
    out[oo] = x[ox];
  }
}

template <typename S, typename D>
__device__ __forceinline__ D cast_one(S v);
#define RB_CAST(S, D, expr) \
  template <> __device__ __forceinline__ D cast_one<S, D>(S v) { return (expr); }
RB_CAST(float, float, v)
RB_CAST(float, __nv_bfloat16, __float2bfloat16_rn(v))
RB_CAST(float, uint32_t, (uint32_t)v)
RB_CAST(float, uint8_t, (uint8_t)v)
RB_CAST(__nv_bfloat16, float, __bfloat162float(v))
RB_CAST(__nv_bfloat16, __nv_bfloat16, v)
RB_CAST(__nv_bfloat16, uint32_t, (uint32_t)__bfloat162float(v))
RB_CAST(__nv_bfloat16, uint8_t, (uint8_t)__bfloat162float(v))
RB_CAST(uint32_t, float, (float)v)
RB_CAST(uint32_t, __nv_bfloat16, __float2bfloat16_rn((float)v))
RB_CAST(uint32_t, uint32_t, v)
RB_CAST(uint32_t, uint8_t, (uint8_t)v)
RB_CAST(uint8_t, float, (float)v)
RB_CAST(uint8_t, __nv_bfloat16, __float2bfloat16_rn((float)v))
RB_CAST(uint8_t, uint32_t, (uint32_t)v)
RB_CAST(uint8_t, uint8_t, v)
#undef RB_CAST

template <typename S, typename D>
__global__ void cast_kernel(const S* __restrict__ x, D* __restrict__ out, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = cast_one<S, D>(x[i]);
}

template <typename E>
__global__ void index_select_kernel(const E* __restrict__ x, int64_t dim, int64_t inner, const uint32_t* __restrict__ idx,
                                    int64_t n_idx, E* __restrict__ out, int64_t n, uint32_t* status) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t in = i % inner, j = (i / inner) % n_idx, o = i / (inner * n_idx);
    uint32_t s = idx[j];
    if (s >= (uint64_t)dim) { status[0] = (uint32_t)(-RB_ERR_INVALID); status[1] = 0x15E1u; status[2] = s; s = (uint32_t)dim - 1; }
    out[i] = x[(o * dim + s) * inner + in];
  }
}

template <typename E>
__global__ void gather_last_kernel(const E* __restrict__ x, int64_t cols, const uint32_t* __restrict__ idx, int64_t k,
                                   E* __restrict__ out, int64_t n, uint32_t* status) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / k;
    uint32_t s = idx[i];
    if (s >= (uint64_t)cols) { status[0] = (uint32_t)(-RB_ERR_INVALID); status[1] = 0x6A74u; status[2] = s; s = (uint32_t)cols - 1; }
    out[i] = x[r * cols + s];
  }
}

template <typename T>
__global__ void where_kernel(const uint8_t* __restrict__ c, const T* __restrict__ a, const T* __restrict__ b,
                             T* __restrict__ out, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = c[i] ? a[i] : b[i];
}

template <typename D>
__global__ void arange_kernel(D* __restrict__ out, int64_t n, double start, double step) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = cast_one<float, D>((float)(start + step * (double)i));
}

// Row-major B ([k, n]) matmul for the primitive: C[b] = A[b] . B[b]; plain tiling, float32 accumulate.
template <typename T>
__global__ void matmul_nn_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ c, int m, int n, int k,
                                 int64_t sa, int64_t sb) {
  __shared__ float as[16][17], bs[16][17];
  const T* ap = a + (size_t)blockIdx.z * sa;
  const T* bp = b + (size_t)blockIdx.z * sb;
  T* cp = c + (size_t)blockIdx.z * m * n;
  const int row = blockIdx.y * 16 + threadIdx.y, col = blockIdx.x * 16 + threadIdx.x;
  float acc = 0.f;
  for (int k0 = 0; k0 < k; k0 += 16) {
    as[threadIdx.y][threadIdx.x] = (row < m && k0 + threadIdx.x < k) ? Cvt<T>::to_f(ap[(size_t)row * k + k0 + threadIdx.x]) : 0.f;
    bs[threadIdx.y][threadIdx.x] = (col < n && k0 + threadIdx.y < k) ? Cvt<T>::to_f(bp[(size_t)(k0 + threadIdx.y) * n + col]) : 0.f;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 16; ++j) acc = fmaf(as[threadIdx.y][j], bs[j][threadIdx.x], acc);
    __syncthreads();
  }
  if (row < m && col < n) cp[(size_t)row * n + col] = Cvt<T>::from_f(acc);
}

inline int grid_for(int64_t n) { return (int)std::min<int64_t>((n + 255) / 256, 148 * 16); }

}  // namespace rb

using namespace rb;

#define RB_DISPATCH_FLOAT(dtype, what, ...)                                    \
  if (dtype == RB_BF16) { using T = __nv_bfloat16; __VA_ARGS__; }              \
  else if (dtype == RB_F32) { using T = float; __VA_ARGS__; }                  \
  else return fail(RB_ERR_DTYPE, what ": dtype %d unsupported", dtype);

extern "C" int32_t rb_unary(rb_ctx* ctx, int32_t op, const void* x, void* out, int64_t n, float scalar, int32_t dtype) {
  RB_REQUIRE(ctx && (n == 0 || (x && out)) && n >= 0, "rb_unary: bad argument");
  RB_REQUIRE(op >= RB_UN_NEG && op <= RB_UN_LOG10, "rb_unary: unknown op %d", op);
  if (n == 0) return RB_OK;
  RB_DISPATCH_FLOAT(dtype, "rb_unary", (unary_kernel<T><<<grid_for(n), 256, 0, ctx->stream>>>(op, (const T*)x, (T*)out, n, scalar)));
  ctx->launches++;
  return launch_status("unary");
}

extern "C" int32_t rb_binary(rb_ctx* ctx, int32_t op, const void* a, const int64_t* sa, const void* b, const int64_t* sb,
                             void* out, int32_t rank, const int64_t* shape, int32_t dtype) {
  RB_REQUIRE(ctx && a && b && out && shape, "rb_binary: null argument");
  RB_REQUIRE(rank >= 0 && rank <= 4, "rb_binary: rank %d unsupported (0..4)", rank);
  RB_REQUIRE(op >= RB_BIN_ADD && op <= RB_BIN_MINIMUM, "rb_binary: unknown op %d", op);
  Dims4 d;
  int64_t n = 1;
  for (int k = 0; k < 4; ++k) { d.shape[k] = 1; d.sa[k] = 0; d.sb[k] = 0; }
  int64_t dense = 1;
  for (int k = rank - 1; k >= 0; --k) {
    const int slot = 4 - rank + k;
    d.shape[slot] = shape[k];
    d.sa[slot] = sa ? sa[k] : dense;
    d.sb[slot] = sb ? sb[k] : dense;
    dense *= shape[k];
    n *= shape[k];
  }
  if (n == 0) return RB_OK;
  RB_DISPATCH_FLOAT(dtype, "rb_binary", (binary_kernel<T><<<grid_for(n), 256, 0, ctx->stream>>>(op, (const T*)a, (const T*)b, (T*)out, d, n)));
  ctx->launches++;
  return launch_status("binary");
}

extern "C" int32_t rb_softmax_rows(rb_ctx* ctx, const void* x, void* out, int64_t rows, int64_t cols, int32_t dtype) {
  RB_REQUIRE(ctx && x && out && rows >= 0 && cols > 0, "rb_softmax_rows: bad argument");
  if (rows == 0) return RB_OK;
  RB_DISPATCH_FLOAT(dtype, "rb_softmax_rows", (softmax_rows_kernel<T><<<(unsigned)rows, 256, 0, ctx->stream>>>((const T*)x, (T*)out, cols)));
  ctx->launches++;
  return launch_status("softmax_rows");
}

extern "C" int32_t rb_reduce_rows(rb_ctx* ctx, int32_t op, const void* x, void* out, int64_t rows, int64_t cols,
                                  int32_t dtype) {
  RB_REQUIRE(ctx && x && out && rows >= 0 && cols > 0, "rb_reduce_rows: bad argument");
  RB_REQUIRE(op >= RB_RED_SUM && op <= RB_RED_MIN, "rb_reduce_rows: unknown op %d", op);
  if (rows == 0) return RB_OK;
  RB_DISPATCH_FLOAT(dtype, "rb_reduce_rows", (reduce_rows_kernel<T><<<(unsigned)rows, 256, 0, ctx->stream>>>(op, (const T*)x, (T*)out, cols)));
  ctx->launches++;
  return launch_status("reduce_rows");
}

extern "C" int32_t rb_copy_strided(rb_ctx* ctx, const void* x, const int64_t* xs, int64_t xoff, void* out,
                                   const int64_t* os, int64_t ooff, int32_t rank, const int64_t* shape, int32_t es) {
  RB_REQUIRE(ctx && x && out && shape, "rb_copy_strided: null argument");
  RB_REQUIRE(rank >= 0 && rank <= 6, "rb_copy_strided: rank %d unsupported (0..6)", rank);
  Dims6 d;
  int64_t n = 1, dense = 1;
  for (int k = 0; k < 6; ++k) { d.shape[k] = 1; d.sx[k] = 0; d.so[k] = 0; }
  for (int k = rank - 1; k >= 0; --k) {
    const int slot = 6 - rank + k;
    d.shape[slot] = shape[k];
    d.sx[slot] = xs ? xs[k] : dense;
    d.so[slot] = os ? os[k] : dense;
    dense *= shape[k];
    n *= shape[k];
  }
  if (n == 0) return RB_OK;
  const int g = grid_for(n);
  switch (es) {
    case 1: copy_strided_kernel<uint8_t><<<g, 256, 0, ctx->stream>>>((const uint8_t*)x + xoff, (uint8_t*)out + ooff, d, n); break;
    case 2: copy_strided_kernel<uint16_t><<<g, 256, 0, ctx->stream>>>((const uint16_t*)x + xoff, (uint16_t*)out + ooff, d, n); break;
    case 4: copy_strided_kernel<uint32_t><<<g, 256, 0, ctx->stream>>>((const uint32_t*)x + xoff, (uint32_t*)out + ooff, d, n); break;
    case 8: copy_strided_kernel<uint64_t><<<g, 256, 0, ctx->stream>>>((const uint64_t*)x + xoff, (uint64_t*)out + ooff, d, n); break;
    default: return fail(RB_ERR_DTYPE, "rb_copy_strided: element size %d unsupported", es);
  }
  ctx->launches++;
  return launch_status("copy_strided");
}

template <typename S>
static int cast_from(rb_ctx* ctx, const void* x, void* out, int32_t dst, int64_t n) {
  const int g = grid_for(n);
  switch (dst) {
    case RB_F32: cast_kernel<S, float><<<g, 256, 0, ctx->stream>>>((const S*)x, (float*)out, n); break;
    case RB_BF16: cast_kernel<S, __nv_bfloat16><<<g, 256, 0, ctx->stream>>>((const S*)x, (__nv_bfloat16*)out, n); break;
    case RB_U32: cast_kernel<S, uint32_t><<<g, 256, 0, ctx->stream>>>((const S*)x, (uint32_t*)out, n); break;
    case RB_U8: cast_kernel<S, uint8_t><<<g, 256, 0, ctx->stream>>>((const S*)x, (uint8_t*)out, n); break;
    default: return fail(RB_ERR_DTYPE, "rb_cast: destination dtype %d unsupported", dst);
  }
  ctx->launches++;
  return launch_status("cast");
}

extern "C" int32_t rb_cast(rb_ctx* ctx, const void* x, int32_t src, void* out, int32_t dst, int64_t n) {
  RB_REQUIRE(ctx && (n == 0 || (x && out)) && n >= 0, "rb_cast: bad argument");
  if (n == 0) return RB_OK;
  switch (src) {
    case RB_F32: return cast_from<float>(ctx, x, out, dst, n);
    case RB_BF16: return cast_from<__nv_bfloat16>(ctx, x, out, dst, n);
    case RB_U32: return cast_from<uint32_t>(ctx, x, out, dst, n);
    case RB_U8: return cast_from<uint8_t>(ctx, x, out, dst, n);
  }
  return fail(RB_ERR_DTYPE, "rb_cast: source dtype %d unsupported", src);
}

extern "C" int32_t rb_index_select(rb_ctx* ctx, const void* x, int64_t outer, int64_t dim, int64_t inner,
                                   const uint32_t* idx, int64_t n_idx, void* out, int32_t es) {
  RB_REQUIRE(ctx && x && idx && out && outer >= 0 && dim > 0 && inner > 0 && n_idx >= 0, "rb_index_select: bad argument");
  const int64_t n = outer * n_idx * inner;
  if (n == 0) return RB_OK;
  const int g = grid_for(n);
  switch (es) {
    case 1: index_select_kernel<uint8_t><<<g, 256, 0, ctx->stream>>>((const uint8_t*)x, dim, inner, idx, n_idx, (uint8_t*)out, n, ctx->status_dev); break;
    case 2: index_select_kernel<uint16_t><<<g, 256, 0, ctx->stream>>>((const uint16_t*)x, dim, inner, idx, n_idx, (uint16_t*)out, n, ctx->status_dev); break;
    case 4: index_select_kernel<uint32_t><<<g, 256, 0, ctx->stream>>>((const uint32_t*)x, dim, inner, idx, n_idx, (uint32_t*)out, n, ctx->status_dev); break;
    case 8: index_select_kernel<uint64_t><<<g, 256, 0, ctx->stream>>>((const uint64_t*)x, dim, inner, idx, n_idx, (uint64_t*)out, n, ctx->status_dev); break;
    default: return fail(RB_ERR_DTYPE, "rb_index_select: element size %d unsupported", es);
  }
  ctx->launches++;
  return launch_status("index_select");
}

extern "C" int32_t rb_gather_last(rb_ctx* ctx, const void* x, int64_t rows, int64_t cols, const uint32_t* idx, int64_t k,
                                  void* out, int32_t es) {
  RB_REQUIRE(ctx && x && idx && out && rows >= 0 && cols > 0 && k >= 0, "rb_gather_last: bad argument");
  const int64_t n = rows * k;
  if (n == 0) return RB_OK;
  const int g = grid_for(n);
  switch (es) {
    case 2: gather_last_kernel<uint16_t><<<g, 256, 0, ctx->stream>>>((const uint16_t*)x, cols, idx, k, (uint16_t*)out, n, ctx->status_dev); break;
    case 4: gather_last_kernel<uint32_t><<<g, 256, 0, ctx->stream>>>((const uint32_t*)x, cols, idx, k, (uint32_t*)out, n, ctx->status_dev); break;
    default: return fail(RB_ERR_DTYPE, "rb_gather_last: element size %d unsupported", es);
  }
  ctx->launches++;
  return launch_status("gather_last");
}

extern "C" int32_t rb_where(rb_ctx* ctx, const uint8_t* cond, const void* a, const void* b, void* out, int64_t n,
                            int32_t dtype) {
  RB_REQUIRE(ctx && (n == 0 || (cond && a && b && out)) && n >= 0, "rb_where: bad argument");
  if (n == 0) return RB_OK;
  RB_DISPATCH_FLOAT(dtype, "rb_where", (where_kernel<T><<<grid_for(n), 256, 0, ctx->stream>>>(cond, (const T*)a, (const T*)b, (T*)out, n)));
  ctx->launches++;
  return launch_status("where");
}

extern "C" int32_t rb_arange(rb_ctx* ctx, void* out, int64_t n, double start, double step, int32_t dtype) {
  RB_REQUIRE(ctx && (n == 0 || out) && n >= 0, "rb_arange: bad argument");
  if (n == 0) return RB_OK;
  const int g = grid_for(n);
  switch (dtype) {
    case RB_F32: arange_kernel<float><<<g, 256, 0, ctx->stream>>>((float*)out, n, start, step); break;
    case RB_BF16: arange_kernel<__nv_bfloat16><<<g, 256, 0, ctx->stream>>>((__nv_bfloat16*)out, n, start, step); break;
    case RB_U32: arange_kernel<uint32_t><<<g, 256, 0, ctx->stream>>>((uint32_t*)out, n, start, step); break;
    case RB_U8: arange_kernel<uint8_t><<<g, 256, 0, ctx->stream>>>((uint8_t*)out, n, start, step); break;
    default: return fail(RB_ERR_DTYPE, "rb_arange: dtype %d unsupported", dtype);
  }
  ctx->launches++;
  return launch_status("arange");
}

extern "C" int32_t rb_fill(rb_ctx* ctx, void* out, int64_t n, double value, int32_t dtype) {
  return rb_arange(ctx, out, n, value, 0.0, dtype);
}

extern "C" int32_t rb_matmul(rb_ctx* ctx, const void* a, const void* b, void* c, int64_t batch, int64_t m, int64_t n,
                             int64_t k, int64_t sa, int64_t sb, int32_t trans_b, int32_t dtype) {
  RB_REQUIRE(ctx && a && b && c, "rb_matmul: null argument");
  RB_REQUIRE(batch >= 0 && m >= 0 && n > 0 && k > 0, "rb_matmul: bad sizes");
  RB_REQUIRE(dtype == RB_BF16 || dtype == RB_F32, "rb_matmul: dtype %d unsupported", dtype);
  if (batch == 0 || m == 0) return RB_OK;
  const size_t es = dtype_size(dtype);
  if (trans_b) {
    // B[b] is [n, k]: the Linear form.  A broadcast B over a dense batch of A is ONE GEMM of M = batch*m
    // (rai-nn/src/linear.rs:59-69 builds exactly this with a stride-0 broadcast of the weight).
    if (sb == 0 && (batch == 1 || sa == m * k))
      return rb_linear(ctx, a, b, nullptr, nullptr, c, batch * m, n, k, RB_ACT_NONE, dtype);
    for (int64_t i = 0; i < batch; ++i)
      RB_TRY(rb_linear(ctx, (const char*)a + i * sa * es, (const char*)b + i * sb * es, nullptr, nullptr,
                       (char*)c + i * m * n * es, m, n, k, RB_ACT_NONE, dtype));
    return RB_OK;
  }
  dim3 grid((unsigned)((n + 15) / 16), (unsigned)((m + 15) / 16), (unsigned)batch), block(16, 16);
  if (dtype == RB_BF16)
    matmul_nn_kernel<__nv_bfloat16><<<grid, block, 0, ctx->stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                                     (__nv_bfloat16*)c, (int)m, (int)n, (int)k, sa, sb);
  else
    matmul_nn_kernel<float><<<grid, block, 0, ctx->stream>>>((const float*)a, (const float*)b, (float*)c, (int)m, (int)n,
                                                             (int)k, sa, sb);
  ctx->launches++;
  return launch_status("matmul_nn");
}
