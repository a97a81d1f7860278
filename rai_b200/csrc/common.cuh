// Shared declarations of the rai_b200 library: status codes, dtype tags, error reporting,
// small device helpers.  Everything here is internal; the exported surface is include/rai_b200.h.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string>
#include <utility>

#include "../../include/rai_b200.h"

namespace rb {

// Last error text of the calling thread (read through rb_last_error()).
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);

#define RB_CUDA(expr)                                                                         \
  do {                                                                                        \
    cudaError_t _e = (expr);                                                                  \
    if (_e != cudaSuccess)                                                                    \
      return ::rb::fail(RB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),  \
                        __FILE__, __LINE__);                                                  \
  } while (0)

#define RB_TRY(expr)                \
  do {                              \
    int _s = (expr);                \
    if (_s != RB_OK) return _s;     \
  } while (0)

#define RB_REQUIRE(cond, ...)                                        \
  do {                                                               \
    if (!(cond)) return ::rb::fail(RB_ERR_INVALID, __VA_ARGS__);     \
  } while (0)

inline int launch_status(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(RB_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
  return RB_OK;
}

inline size_t dtype_size(int dt) {
  switch (dt) {
    case RB_U8: return 1;
    case RB_F16: case RB_BF16: return 2;
    case RB_U32: case RB_F32: return 4;
    case RB_I64: case RB_F64: return 8;
  }
  return 0;
}

// Programmatic dependent launch.  Kernels of the decoder chain are launched with the
// programmatic-stream-serialization attribute: a kernel may become resident while its predecessor
// is still running, does whatever does not depend on the predecessor (barrier set-up, TMEM
// allocation, prefetch of weights), and calls pdl_wait() before it touches anything the
// predecessor produced or may still be reading.  pdl_launch_dependents() lets the successor do the same.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Launches `kern` with the programmatic-stream-serialization attribute when `pdl` is set.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 bool pdl, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(std::forward<Args>(args))...);
}

// Device status word: kernels that wait on barriers record a give-up here instead of trapping.
// Layout: [0] = error code (0 ok), [1] = where (kernel-specific tag), [2..3] = details.
uint32_t* device_status_word();  // device pointer (per current device), zero-initialised

template <typename T> struct Cvt;
template <> struct Cvt<float> {
  __device__ __forceinline__ static float to_f(float v) { return v; }
  __device__ __forceinline__ static float from_f(float v) { return v; }
};
template <> struct Cvt<__nv_bfloat16> {
  __device__ __forceinline__ static float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ __forceinline__ static __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Cvt<__half> {
  __device__ __forceinline__ static float to_f(__half v) { return __half2float(v); }
  __device__ __forceinline__ static __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Cvt<double> {
  __device__ __forceinline__ static float to_f(double v) { return (float)v; }
  __device__ __forceinline__ static double from_f(float v) { return (double)v; }
};

// 8 consecutive elements as float32 (16-byte accesses for bf16, two for float32)
__device__ __forceinline__ void load8(const float* p, float* v) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void store8(float* p, const float* v) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* v) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

__device__ __forceinline__ uint4 pack8_bf16(const float* v) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return u;
}

// v[i] += slab_0[i] + slab_1[i] + ... in slab order (so the result does not depend on how the loads are
// scheduled), with the loads of up to G slabs issued before the first sum needs them: one memory round trip
// per group instead of one per slab.
template <int G = 8>
__device__ __forceinline__ void add_slabs(const float* __restrict__ acc, int n_acc, size_t stride, size_t off, float* v) {
  for (int k0 = 0; k0 < n_acc; k0 += G) {
    float t[G][8];
#pragma unroll
    for (int k = 0; k < G; ++k)
      if (k0 + k < n_acc) load8(acc + (size_t)(k0 + k) * stride + off, t[k]);
#pragma unroll
    for (int k = 0; k < G; ++k)
      if (k0 + k < n_acc) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += t[k][i];
      }
  }
}

// x*cos + rotate_half(x)*sin for 8 lanes of the first half (lo, partner -hi) and the 8 matching lanes of
// the second half (hi, partner lo) of a rotary block (rai-models/src/llm/qwen2.rs:33-38,63-71).  Written
// with explicit fused multiply-adds so that every kernel that rotates produces the same bits.
__device__ __forceinline__ void rope_rotate8(const float* lo, const float* hi, const float* cs, const float* sn,
                                             float* ylo, float* yhi) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    ylo[i] = __fmaf_rn(lo[i], cs[i], -__fmul_rn(hi[i], sn[i]));
    yhi[i] = __fmaf_rn(hi[i], cs[i], __fmul_rn(lo[i], sn[i]));
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum for blocks of up to 1024 threads; `red` is 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// Activation tags shared by the GEMM epilogues and the elementwise kernels
// (rai-core/src/hlops/activations.rs:20-32).
__device__ __forceinline__ float act_apply(int act, float x) {
  switch (act) {
    case RB_ACT_SILU: return x / (__expf(-x) + 1.0f);
    case RB_ACT_GELU_TANH: {
      const float c = 0.7978845608028654f;
      return 0.5f * x * (1.0f + tanhf(c * (x + 0.044715f * x * x * x)));
    }
    case RB_ACT_GELU_ERF: return x * 0.5f * (1.0f + erff(x * 0.7071067811865476f));
    case RB_ACT_RELU: return fmaxf(x, 0.f);
    default: return x;
  }
}

}  // namespace rb
