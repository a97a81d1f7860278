// The rest of the primitive set of rai-core/src/dispatch.rs:41-157 — what general graphs (the vision models and the
// training examples) reach beyond the decoders: comparisons, log-softmax, arg-min, scatter / index add, convolutions,
// pooling and nearest-neighbour upsampling.  One thread per output element, float32 arithmetic inside whatever the
// storage type; these are correctness-first kernels that keep `Tensor::...(&Cuda)` total, not tuned ones.
#include <math.h>

#include "ctx.h"

namespace rb {
namespace {

inline unsigned blocks_for(int64_t n) { return (unsigned)std::min<int64_t>((n + 255) / 256, 65535 * 16); }

struct Cmp4 {
  int64_t shape[4], sa[4], sb[4];
};

// Equal .. LessEqual (candle.rs:327-399): u8 result, operands with strides (stride 0 = broadcast).
template <typename T>
__global__ void compare_kernel(int op, const T* __restrict__ a, const T* __restrict__ b, uint8_t* __restrict__ out, Cmp4 d,
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
    bool v;
    switch (op) {
      case RB_CMP_EQ: v = x == y; break;
      case RB_CMP_NE: v = x != y; break;
      case RB_CMP_GT: v = x > y; break;
      case RB_CMP_GE: v = x >= y; break;
      case RB_CMP_LT: v = x < y; break;
      default: v = x <= y;
    }
    out[i] = v ? 1 : 0;
  }
}

// LogSoftmax over the last dimension (candle.rs:805-816: x - max - log(sum(exp(x - max)))).
template <typename T>
__global__ void log_softmax_rows_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t cols) {
  __shared__ float red[32];
  const T* row = x + (size_t)blockIdx.x * cols;
  T* orow = out + (size_t)blockIdx.x * cols;
  float mx = -INFINITY;
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) mx = fmaxf(mx, Cvt<T>::to_f(row[i]));
  mx = warp_max(mx);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) red[w] = mx;
  __syncthreads();
  mx = lane < nw ? red[lane] : -INFINITY;
  mx = warp_max(mx);
  __syncthreads();
  float s = 0.f;
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) s += expf(Cvt<T>::to_f(row[i]) - mx);
  s = block_sum(s, red);
  const float lse = logf(s);
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) orow[i] = Cvt<T>::from_f(Cvt<T>::to_f(row[i]) - mx - lse);
}

// ArgMin over the last dimension: first index among equal minima (candle's argmin keeps the first).
template <typename T>
__global__ void argmin_rows_kernel(const T* __restrict__ x, int64_t cols, uint32_t* __restrict__ out) {
  __shared__ float bv[32];
  __shared__ uint32_t bi[32];
  const T* row = x + (size_t)blockIdx.x * cols;
  float best = INFINITY;
  uint32_t idx = 0xffffffffu;
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) {
    const float v = Cvt<T>::to_f(row[i]);
    if (v < best || (v == best && (uint32_t)i < idx)) { best = v; idx = (uint32_t)i; }
  }
  auto fold = [&](float ov, uint32_t oi) { if (ov < best || (ov == best && oi < idx)) { best = ov; idx = oi; } };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) fold(__shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) { bv[w] = best; bi[w] = idx; }
  __syncthreads();
  if (w == 0) {
    best = lane < nw ? bv[lane] : INFINITY;
    idx = lane < nw ? bi[lane] : 0xffffffffu;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) fold(__shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
    if (lane == 0) out[blockIdx.x] = idx;
  }
}

__device__ __forceinline__ void atomic_add_t(float* p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void atomic_add_t(__nv_bfloat16* p, float v) { atomicAdd(p, __float2bfloat16_rn(v)); }

// ScatterAdd (candle.rs:990-1004): out starts as x; out[o, idx[o, j, i], i] += src[o, j, i] along `dim`, tensors viewed
// as [outer, dim, inner].  IndexAdd (candle.rs:851-865) is the same with a 1-D index: out[o, idx[j], i] += src[o, j, i].
template <typename T>
__global__ void scatter_add_kernel(T* __restrict__ out, const T* __restrict__ src, const uint32_t* __restrict__ idx,
                                   int64_t outer, int64_t dim_out, int64_t dim_src, int64_t inner, int index_is_1d,
                                   uint32_t* status) {
  const int64_t n = outer * dim_src * inner;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = e % inner, j = (e / inner) % dim_src, o = e / (inner * dim_src);
    const uint32_t t = index_is_1d ? idx[j] : idx[e];
    if ((int64_t)t >= dim_out) {  // record and skip: never write out of bounds, never trap
      status[0] = (uint32_t)(-RB_ERR_INVALID); status[1] = 0x5CA7u; status[2] = t;
      continue;
    }
    atomic_add_t(out + (o * dim_out + t) * inner + i, Cvt<T>::to_f(src[e]));
  }
}

struct ConvDims {
  int n, cin, h, w, cout, kh, kw, oh, ow;
  int pad_h, pad_w, stride_h, stride_w, dil_h, dil_w;
  int out_pad_h, out_pad_w;
};

// Conv2d / Conv1d (candle.rs:628-700): x [N, Cin, H, W], w [Cout, Cin, KH, KW], NCHW, no groups (the reference's op
// has none).  Conv1d is the H = KH = 1 case.
template <typename T>
__global__ void conv2d_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ out, ConvDims d) {
  const int64_t total = (int64_t)d.n * d.cout * d.oh * d.ow;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int ox = (int)(e % d.ow), oy = (int)((e / d.ow) % d.oh), co = (int)((e / ((int64_t)d.ow * d.oh)) % d.cout);
    const int b = (int)(e / ((int64_t)d.ow * d.oh * d.cout));
    float acc = 0.f;
    for (int ci = 0; ci < d.cin; ++ci)
      for (int ky = 0; ky < d.kh; ++ky) {
        const int iy = oy * d.stride_h - d.pad_h + ky * d.dil_h;
        if (iy < 0 || iy >= d.h) continue;
        for (int kx = 0; kx < d.kw; ++kx) {
          const int ix = ox * d.stride_w - d.pad_w + kx * d.dil_w;
          if (ix < 0 || ix >= d.w) continue;
          acc += Cvt<T>::to_f(x[(((size_t)b * d.cin + ci) * d.h + iy) * d.w + ix]) *
                 Cvt<T>::to_f(w[(((size_t)co * d.cin + ci) * d.kh + ky) * d.kw + kx]);
        }
      }
    out[e] = Cvt<T>::from_f(acc);
  }
}

// ConvTranspose2d / 1d (candle.rs:702-760): x [N, Cin, H, W], w [Cin, Cout, KH, KW]; gather form (each output element
// collects the inputs that reach it), so no atomics.
template <typename T>
__global__ void conv_transpose2d_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ out, ConvDims d) {
  const int64_t total = (int64_t)d.n * d.cout * d.oh * d.ow;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int ox = (int)(e % d.ow), oy = (int)((e / d.ow) % d.oh), co = (int)((e / ((int64_t)d.ow * d.oh)) % d.cout);
    const int b = (int)(e / ((int64_t)d.ow * d.oh * d.cout));
    float acc = 0.f;
    for (int ky = 0; ky < d.kh; ++ky) {
      const int ty = oy + d.pad_h - ky * d.dil_h;
      if (ty < 0 || ty % d.stride_h) continue;
      const int iy = ty / d.stride_h;
      if (iy >= d.h) continue;
      for (int kx = 0; kx < d.kw; ++kx) {
        const int tx = ox + d.pad_w - kx * d.dil_w;
        if (tx < 0 || tx % d.stride_w) continue;
        const int ix = tx / d.stride_w;
        if (ix >= d.w) continue;
        for (int ci = 0; ci < d.cin; ++ci)
          acc += Cvt<T>::to_f(x[(((size_t)b * d.cin + ci) * d.h + iy) * d.w + ix]) *
                 Cvt<T>::to_f(w[(((size_t)ci * d.cout + co) * d.kh + ky) * d.kw + kx]);
      }
    }
    out[e] = Cvt<T>::from_f(acc);
  }
}

// MaxPool2d / AvgPool2d (candle.rs:933-945, and their 1-D forms as H = 1): windows that would leave the input are
// clipped for max (padding contributes nothing); average divides by the full window like candle's avg_pool2d, which
// takes no padding.
template <typename T>
__global__ void pool2d_kernel(int is_max, const T* __restrict__ x, T* __restrict__ out, ConvDims d) {
  const int64_t total = (int64_t)d.n * d.cin * d.oh * d.ow;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int ox = (int)(e % d.ow), oy = (int)((e / d.ow) % d.oh);
    const int64_t plane = e / ((int64_t)d.ow * d.oh);
    const T* xp = x + (size_t)plane * d.h * d.w;
    float acc = is_max ? -INFINITY : 0.f;
    for (int ky = 0; ky < d.kh; ++ky) {
      const int iy = oy * d.stride_h - d.pad_h + ky * d.dil_h;
      if (iy < 0 || iy >= d.h) continue;
      for (int kx = 0; kx < d.kw; ++kx) {
        const int ix = ox * d.stride_w - d.pad_w + kx * d.dil_w;
        if (ix < 0 || ix >= d.w) continue;
        const float v = Cvt<T>::to_f(xp[(size_t)iy * d.w + ix]);
        acc = is_max ? fmaxf(acc, v) : acc + v;
      }
    }
    out[e] = Cvt<T>::from_f(is_max ? acc : acc / (float)(d.kh * d.kw));
  }
}

// UpsampleNearest2d / 1d (candle.rs:1006-1030): source index = floor(dst * in / out).
template <typename T>
__global__ void upsample_nearest2d_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t planes, int h, int w, int oh,
                                          int ow) {
  const int64_t total = planes * oh * ow;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int ox = (int)(e % ow), oy = (int)((e / ow) % oh);
    const int64_t plane = e / ((int64_t)ow * oh);
    const int iy = min(h - 1, (int)(((int64_t)oy * h) / oh)), ix = min(w - 1, (int)(((int64_t)ox * w) / ow));
    out[e] = x[((size_t)plane * h + iy) * w + ix];
  }
}

}  // namespace
}  // namespace rb

using namespace rb;

#define RB_FLOAT_CASES(dtype, what, ...)                                       \
  if (dtype == RB_BF16) { using T = __nv_bfloat16; __VA_ARGS__; }              \
  else if (dtype == RB_F32) { using T = float; __VA_ARGS__; }                  \
  else return fail(RB_ERR_DTYPE, what ": dtype %d unsupported", dtype);

extern "C" int32_t rb_compare(rb_ctx* ctx, int32_t op, const void* a, const int64_t* sa, const void* b, const int64_t* sb,
                              uint8_t* out, int32_t rank, const int64_t* shape, int32_t dtype) {
  RB_REQUIRE(ctx && a && b && out && shape, "rb_compare: null argument");
  RB_REQUIRE(rank >= 0 && rank <= 4, "rb_compare: rank %d unsupported (0..4)", rank);
  RB_REQUIRE(op >= RB_CMP_EQ && op <= RB_CMP_LE, "rb_compare: unknown op %d", op);
  Cmp4 d;
  int64_t n = 1, dense = 1;
  for (int k = 0; k < 4; ++k) { d.shape[k] = 1; d.sa[k] = 0; d.sb[k] = 0; }
  for (int k = rank - 1; k >= 0; --k) {
    const int slot = 4 - rank + k;
    d.shape[slot] = shape[k];
    d.sa[slot] = sa ? sa[k] : dense;
    d.sb[slot] = sb ? sb[k] : dense;
    dense *= shape[k];
    n *= shape[k];
  }
  if (n == 0) return RB_OK;
  RB_FLOAT_CASES(dtype, "rb_compare", (compare_kernel<T><<<blocks_for(n), 256, 0, ctx->stream>>>(op, (const T*)a, (const T*)b, out, d, n)));
  ctx->launches++;
  return launch_status("compare");
}

extern "C" int32_t rb_log_softmax_rows(rb_ctx* ctx, const void* x, void* out, int64_t rows, int64_t cols, int32_t dtype) {
  RB_REQUIRE(ctx && x && out && rows >= 0 && cols > 0, "rb_log_softmax_rows: bad argument");
  if (rows == 0) return RB_OK;
  RB_FLOAT_CASES(dtype, "rb_log_softmax_rows", (log_softmax_rows_kernel<T><<<(unsigned)rows, 256, 0, ctx->stream>>>((const T*)x, (T*)out, cols)));
  ctx->launches++;
  return launch_status("log_softmax_rows");
}

extern "C" int32_t rb_argmin_rows(rb_ctx* ctx, const void* x, int32_t dtype, int64_t rows, int64_t cols, uint32_t* out) {
  RB_REQUIRE(ctx && x && out && rows >= 0 && cols > 0 && cols <= 0xffffffffLL, "rb_argmin_rows: bad argument");
  if (rows == 0) return RB_OK;
  RB_FLOAT_CASES(dtype, "rb_argmin_rows", (argmin_rows_kernel<T><<<(unsigned)rows, 256, 0, ctx->stream>>>((const T*)x, cols, out)));
  ctx->launches++;
  return launch_status("argmin_rows");
}

extern "C" int32_t rb_scatter_add(rb_ctx* ctx, const void* x, const void* src, const uint32_t* idx, void* out, int64_t outer,
                                  int64_t dim_out, int64_t dim_src, int64_t inner, int32_t index_is_1d, int32_t dtype) {
  RB_REQUIRE(ctx && x && src && idx && out, "rb_scatter_add: null argument");
  RB_REQUIRE(outer >= 0 && dim_out > 0 && dim_src >= 0 && inner >= 0, "rb_scatter_add: bad sizes");
  const int64_t n_out = outer * dim_out * inner, n = outer * dim_src * inner;
  if (n_out == 0) return RB_OK;
  const size_t es = dtype_size(dtype);
  if (out != x) RB_CUDA(cudaMemcpyAsync(out, x, (size_t)n_out * es, cudaMemcpyDeviceToDevice, ctx->stream));
  if (n == 0) return RB_OK;
  RB_FLOAT_CASES(dtype, "rb_scatter_add",
                 (scatter_add_kernel<T><<<blocks_for(n), 256, 0, ctx->stream>>>((T*)out, (const T*)src, idx, outer, dim_out, dim_src,
                                                                            inner, index_is_1d, ctx->status_dev)));
  ctx->launches++;
  return launch_status("scatter_add");
}

static int conv_dims(ConvDims& d, const int32_t* xs, const int32_t* ws, bool transposed, const int32_t* padding,
                     const int32_t* stride, const int32_t* dilation, const int32_t* out_padding) {
  d.n = xs[0]; d.cin = xs[1]; d.h = xs[2]; d.w = xs[3];
  d.kh = ws[2]; d.kw = ws[3];
  d.pad_h = padding[0]; d.pad_w = padding[1];
  d.stride_h = stride[0]; d.stride_w = stride[1];
  d.dil_h = dilation[0]; d.dil_w = dilation[1];
  d.out_pad_h = out_padding ? out_padding[0] : 0; d.out_pad_w = out_padding ? out_padding[1] : 0;
  RB_REQUIRE(d.stride_h > 0 && d.stride_w > 0 && d.dil_h > 0 && d.dil_w > 0 && d.kh > 0 && d.kw > 0, "convolution: bad geometry");
  if (!transposed) {
    RB_REQUIRE(ws[1] == d.cin, "conv2d: weight has %d input channels, the input %d", ws[1], d.cin);
    d.cout = ws[0];
    d.oh = (d.h + 2 * d.pad_h - d.dil_h * (d.kh - 1) - 1) / d.stride_h + 1;
    d.ow = (d.w + 2 * d.pad_w - d.dil_w * (d.kw - 1) - 1) / d.stride_w + 1;
  } else {
    RB_REQUIRE(ws[0] == d.cin, "conv_transpose2d: weight has %d input channels, the input %d", ws[0], d.cin);
    d.cout = ws[1];
    d.oh = (d.h - 1) * d.stride_h - 2 * d.pad_h + d.dil_h * (d.kh - 1) + d.out_pad_h + 1;
    d.ow = (d.w - 1) * d.stride_w - 2 * d.pad_w + d.dil_w * (d.kw - 1) + d.out_pad_w + 1;
  }
  RB_REQUIRE(d.oh > 0 && d.ow > 0, "convolution: empty output (%d x %d)", d.oh, d.ow);
  return RB_OK;
}

extern "C" int32_t rb_conv2d(rb_ctx* ctx, const void* x, const int32_t* x_shape4, const void* w, const int32_t* w_shape4,
                             const int32_t* padding2, const int32_t* stride2, const int32_t* dilation2, void* out,
                             int32_t* out_shape4, int32_t dtype) {
  RB_REQUIRE(ctx && x && x_shape4 && w && w_shape4 && padding2 && stride2 && dilation2, "rb_conv2d: null argument");
  ConvDims d{};
  RB_TRY(conv_dims(d, x_shape4, w_shape4, false, padding2, stride2, dilation2, nullptr));
  if (out_shape4) { out_shape4[0] = d.n; out_shape4[1] = d.cout; out_shape4[2] = d.oh; out_shape4[3] = d.ow; }
  if (!out) return RB_OK;  // shape query
  const int64_t total = (int64_t)d.n * d.cout * d.oh * d.ow;
  RB_FLOAT_CASES(dtype, "rb_conv2d", (conv2d_kernel<T><<<blocks_for(total), 256, 0, ctx->stream>>>((const T*)x, (const T*)w, (T*)out, d)));
  ctx->launches++;
  return launch_status("conv2d");
}

extern "C" int32_t rb_conv_transpose2d(rb_ctx* ctx, const void* x, const int32_t* x_shape4, const void* w,
                                       const int32_t* w_shape4, const int32_t* padding2, const int32_t* out_padding2,
                                       const int32_t* stride2, const int32_t* dilation2, void* out, int32_t* out_shape4,
                                       int32_t dtype) {
  RB_REQUIRE(ctx && x && x_shape4 && w && w_shape4 && padding2 && out_padding2 && stride2 && dilation2,
             "rb_conv_transpose2d: null argument");
  ConvDims d{};
  RB_TRY(conv_dims(d, x_shape4, w_shape4, true, padding2, stride2, dilation2, out_padding2));
  if (out_shape4) { out_shape4[0] = d.n; out_shape4[1] = d.cout; out_shape4[2] = d.oh; out_shape4[3] = d.ow; }
  if (!out) return RB_OK;
  const int64_t total = (int64_t)d.n * d.cout * d.oh * d.ow;
  RB_FLOAT_CASES(dtype, "rb_conv_transpose2d",
                 (conv_transpose2d_kernel<T><<<blocks_for(total), 256, 0, ctx->stream>>>((const T*)x, (const T*)w, (T*)out, d)));
  ctx->launches++;
  return launch_status("conv_transpose2d");
}

extern "C" int32_t rb_pool2d(rb_ctx* ctx, int32_t is_max, const void* x, const int32_t* x_shape4, const int32_t* kernel2,
                             const int32_t* stride2, const int32_t* padding2, const int32_t* dilation2, void* out,
                             int32_t* out_shape4, int32_t dtype) {
  RB_REQUIRE(ctx && x && x_shape4 && kernel2 && stride2 && padding2 && dilation2, "rb_pool2d: null argument");
  ConvDims d{};
  const int32_t wshape[4] = {x_shape4[1], x_shape4[1], kernel2[0], kernel2[1]};
  RB_TRY(conv_dims(d, x_shape4, wshape, false, padding2, stride2, dilation2, nullptr));
  if (out_shape4) { out_shape4[0] = d.n; out_shape4[1] = d.cin; out_shape4[2] = d.oh; out_shape4[3] = d.ow; }
  if (!out) return RB_OK;
  const int64_t total = (int64_t)d.n * d.cin * d.oh * d.ow;
  RB_FLOAT_CASES(dtype, "rb_pool2d", (pool2d_kernel<T><<<blocks_for(total), 256, 0, ctx->stream>>>(is_max ? 1 : 0, (const T*)x, (T*)out, d)));
  ctx->launches++;
  return launch_status("pool2d");
}

extern "C" int32_t rb_upsample_nearest2d(rb_ctx* ctx, const void* x, const int32_t* x_shape4, int32_t out_h, int32_t out_w,
                                         void* out, int32_t dtype) {
  RB_REQUIRE(ctx && x && x_shape4 && out && out_h > 0 && out_w > 0, "rb_upsample_nearest2d: bad argument");
  const int64_t planes = (int64_t)x_shape4[0] * x_shape4[1];
  const int64_t total = planes * out_h * out_w;
  if (total == 0) return RB_OK;
  RB_FLOAT_CASES(dtype, "rb_upsample_nearest2d",
                 (upsample_nearest2d_kernel<T><<<blocks_for(total), 256, 0, ctx->stream>>>((const T*)x, (T*)out, planes, x_shape4[2],
                                                                                       x_shape4[3], out_h, out_w)));
  ctx->launches++;
  return launch_status("upsample_nearest2d");
}
