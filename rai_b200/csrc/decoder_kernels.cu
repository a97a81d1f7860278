// HBM-bound kernels of the decoder layer: embedding gather, fused norm (+residual, +split-K
// reduction), RoPE + head split + paged KV append, vocabulary argmax.  Each is one pass over its
// data with float32 arithmetic inside, whatever the storage dtype.
#include <math.h>

#include <algorithm>
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
  pdl_launch_dependents();
  pdl_wait();
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
  pdl_launch_dependents();
  pdl_wait();
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


// 8 elements per thread-chunk, at most kChunks chunks per thread held in registers: every load of
// the row (inputs, residual, all split-K slabs, bias) is in flight at once, which is what matters at
// decode where only `rows` blocks exist and the kernel is pure latency.
template <typename T>
__device__ __forceinline__ void round_to(float* v) {
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = Cvt<T>::to_f(Cvt<T>::from_f(v[i]));
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// 16 bytes of this rank's exchange buffer, which its peers write over NVLink: read at system scope so that no
// stale L1 line can serve it
__device__ __forceinline__ uint4 load16_sys(const void* p) {
  uint4 u;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(p) : "memory");
  return u;
}
// Two 8-byte words at system scope.  Each word is one scalar access of the memory model, so a reader sees a word
// either whole or not at all: what the flag-in-data form of the exchange rests on.
__device__ __forceinline__ void st_relaxed_sys_2x64(void* p, uint64_t a, uint64_t b) {
  asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void ld_relaxed_sys_2x64(const void* p, uint64_t& a, uint64_t& b) {
  asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ void add8_bf16(const uint4& u, float* v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] += f.x; v[2 * i + 1] += f.y; }
}

// kSlabs = false is the instantiation for calls without split-K partials (prefill): without the registers that keep
// eight slab loads in flight, several blocks share an SM and the kernel streams at memory speed.
template <typename T, int kChunks, bool kSlabs>
__global__ void __launch_bounds__(512) norm_vec_kernel(int kind, const T* __restrict__ x, const T* __restrict__ add,
                                const float* __restrict__ acc, int n_acc, size_t acc_stride,
                                const T* __restrict__ acc_bias, const T* __restrict__ w, const T* __restrict__ b,
                                float eps, int hidden, T* __restrict__ out, T* __restrict__ sum_out, int64_t n_rows) {
  __shared__ float red[32];
  pdl_launch_dependents();
  float wv[kChunks][8], bv[kChunks][8];
  const int nchunk = hidden >> 3;
  // weights do not depend on the previous kernel: fetch them before waiting for it
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
#pragma unroll
    for (int i = 0; i < 8; ++i) { wv[c][i] = 1.f; bv[c][i] = 0.f; }
    if (ch < nchunk && out) {
      if (w) load8(w + ch * 8, wv[c]);
      if (b) load8(b + ch * 8, bv[c]);
    }
  }
  pdl_wait();
  // One block may take several rows (prefill launches fewer blocks than rows: the weights stay in registers and the
  // block's start-up is paid once).
  auto do_row = [&](int64_t row) {
  const size_t base = (size_t)row * hidden;
  float v[kChunks][8];
  float s = 0.f;
  const float inv_sqrt_h = 1.0f / sqrtf((float)hidden);
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
#pragma unroll
    for (int i = 0; i < 8; ++i) v[c][i] = 0.f;
    if (ch >= nchunk) continue;
    float t[8];
    if (x) { load8(x + base + ch * 8, t);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[c][i] += t[i]; }
    if (add) { load8(add + base + ch * 8, t);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[c][i] += t[i]; }
    if (kSlabs) {
      add_slabs(acc, n_acc, acc_stride, base + ch * 8, v[c]);
      if (acc_bias) { load8(acc_bias + ch * 8, t);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[c][i] += t[i]; }
    }
    round_to<T>(v[c]);  // the residual stream is stored in the model dtype
    if (sum_out) store8(sum_out + base + ch * 8, v[c]);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (kind == RB_NORM_LAYER) s += v[c][i];
      else if (kind == RB_NORM_RMS) { const float t2 = v[c][i] * inv_sqrt_h; s += t2 * t2; }
      else s += v[c][i] * v[c][i];
    }
  }
  if (!out) return;
  s = block_sum(s, red);
  float mean = 0.f, r;
  if (kind == RB_NORM_LAYER) {
    mean = s / (float)hidden;
    float q = 0.f;
#pragma unroll
    for (int c = 0; c < kChunks; ++c)
      if (threadIdx.x + c * blockDim.x < nchunk) {
#pragma unroll
        for (int i = 0; i < 8; ++i) { const float d = v[c][i] - mean; q += d * d; }
      }
    q = block_sum(q, red);
    r = 1.0f / sqrtf(q / (float)hidden + eps);
  } else if (kind == RB_NORM_RMS) {
    r = 1.0f / sqrtf(s + eps);
  } else {
    r = 1.0f / sqrtf(s / (float)hidden + eps);
  }
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch >= nchunk) continue;
    float y[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (kind == RB_NORM_LAYER) { y[i] = (v[c][i] - mean) * r; if (w) y[i] = wv[c][i] * y[i] + bv[c][i]; }
      else if (kind == RB_NORM_RMS) y[i] = wv[c][i] * v[c][i] * r;
      else y[i] = v[c][i] * r * (wv[c][i] + 1.0f);
    }
    store8(out + base + ch * 8, y);
  }
  };
  for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) do_row(row);
}


// Tensor-parallel allreduce of a row-parallel product, fused with the residual add and the norm that follow it.  One
// block per row: it finishes this rank's partial row (split-K slabs + bias, or a bf16 tensor), pushes it into this
// rank's place of the next slot in every PEER's exchange buffer (posted stores over NVLink, nobody waits for a reply),
// raises that row's flag on every peer, then waits (bounded) for the same row from every peer, sums the copies that
// now sit in its OWN memory - and its own, still in registers - in rank order, the same on every rank, adds the
// residual stream and normalises.  A row waits only for that row: no block waits for another block of its own kernel.
//
// Exchange numbers live on the device so that a captured graph replays unchanged: a launch with parity q reads
// counter[q] (exchange number = counter[q] + 1) and, when done, sets counter[q ^ 1] to that number for the next
// launch, whose parity is the opposite one; no launch writes the counter its own blocks read.
//
// kTpInDataDirect, flag in the data, direct (a group of two): no flag array and no fence.  Every 8-byte word a peer receives
// carries 4 bytes of payload and the exchange number; the receiver polls the words themselves until they all show
// this exchange's number.  Twice the bytes on the wire, but the sender never waits for its stores to be acknowledged
// and the receiver has the data the moment it has the flag: shorter by one NVLink round trip.  That pays between two
// GPUs (3.43 -> 3.19-3.29 ms per decode step of the 7B model); among four the doubled bytes already cost more than
// the round trip saves (2.79-2.82 against 2.73 ms).
//
// kTpInDataTwoHop, flag in the data, two hops (wider groups): row r has an owner, rank r % size.  The other ranks send their
// partial row to the owner only; the owner sums the copies in rank order, rounds, and sends the finished row to
// everyone.  Two one-way trips instead of a push, a fence and a flag, and 2 (size - 1) / size rows per rank and
// exchange on the wire instead of size - 1 (or twice that with the flag in the data).  Every rank gets the same
// bits, since only the owner adds.  Against the flag array, per decode step of the 7B model: 2.72 -> 2.62 ms among
// four GPUs, 2.68 -> 2.57 ms among eight.
template <typename T, int kChunks, int kMode>
__global__ void __launch_bounds__(512) exchange_norm_kernel(int kind, const T* __restrict__ h, const float* __restrict__ acc, int n_acc,
                                     size_t acc_stride, const T* __restrict__ acc_bias, const T* __restrict__ part,
                                     const T* __restrict__ w, const T* __restrict__ b, float eps, int hidden,
                                     T* __restrict__ out, T* __restrict__ sum_out, const TpPeers tp, int parity,
                                     uint32_t* status, long long wait_cycles) {
  __shared__ float red[32];
  __shared__ uint32_t give_up;
  pdl_launch_dependents();
  float wv[kChunks][8], bv[kChunks][8];
  const int nchunk = hidden >> 3;
  // weights do not depend on the previous kernel: fetch them before waiting for it
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
#pragma unroll
    for (int i = 0; i < 8; ++i) { wv[c][i] = 1.f; bv[c][i] = 0.f; }
    if (ch < nchunk && out) {
      if (w) load8(w + ch * 8, wv[c]);
      if (b) load8(b + ch * 8, bv[c]);
    }
  }
  if (threadIdx.x == 0) give_up = 0u;
  pdl_wait();
  const int row = blockIdx.x;
  const size_t base = (size_t)row * hidden;
  const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(tp.seq + parity * 32) + 1u;
  const size_t slot_off = (size_t)(seq & 1u) * tp.size * tp.slot_elems;   // [2 slots][size sources][rows x hidden]
  // ---- this rank's partial row, rounded to the model dtype, into every rank's buffer
  uint4 own[kChunks];
#pragma unroll
  for (int c = 0; c < kChunks; ++c) own[c] = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch >= nchunk) continue;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, t[8];
    if (part) { load8(part + base + ch * 8, t);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += t[i]; }
    add_slabs(acc, n_acc, acc_stride, base + ch * 8, v);
    if (acc_bias) { load8(acc_bias + ch * 8, t);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += t[i]; }
    const uint4 packed = pack8_bf16(v);
    own[c] = packed;
    if (kMode == kTpInDataDirect) {
      const uint64_t tag = (uint64_t)seq << 32;
      const size_t word = (slot_off + (size_t)tp.rank * tp.slot_elems + base + ch * 8) >> 1;  // 2 elements per 8-byte word
#pragma unroll
      for (int r = 0; r < kTpDirectRanks; ++r)
        if (r < tp.size && r != tp.rank) {
          uint64_t* dst = reinterpret_cast<uint64_t*>(const_cast<void*>(tp.xbuf[r])) + word;
          st_relaxed_sys_2x64(dst, tag | packed.x, tag | packed.y);
          st_relaxed_sys_2x64(dst + 2, tag | packed.z, tag | packed.w);
        }
    } else if (kMode == kTpInDataTwoHop) {
      const int owner = row % tp.size;
      if (owner != tp.rank) {   // this rank's share of the row goes to the row's owner only
        const uint64_t tag = (uint64_t)seq << 32;
        uint64_t* dst = reinterpret_cast<uint64_t*>(const_cast<void*>(tp.xbuf[owner])) +
                        ((slot_off + (size_t)tp.rank * tp.slot_elems + base + ch * 8) >> 1);
        st_relaxed_sys_2x64(dst, tag | packed.x, tag | packed.y);
        st_relaxed_sys_2x64(dst + 2, tag | packed.z, tag | packed.w);
      }
    } else {
#pragma unroll
      for (int r = 0; r < kTpMaxRanks; ++r)
        if (r < tp.size && r != tp.rank)
          *reinterpret_cast<uint4*>(reinterpret_cast<T*>(const_cast<void*>(tp.xbuf[r])) + slot_off + (size_t)tp.rank * tp.slot_elems +
                                    base + ch * 8) = packed;
    }
  }
  float v[kChunks][8];
  if (kMode == kTpInDataTwoHop) {
    const int owner = row % tp.size;
    const uint64_t tag = (uint64_t)seq << 32;
    // finished rows live behind the 2 x size gathering slots: [2 slots][rows x hidden]
    const size_t res_off = (size_t)2 * tp.size * tp.slot_elems + (size_t)(seq & 1u) * tp.slot_elems;
    const long long t0 = clock64();
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      const int ch = threadIdx.x + c * blockDim.x;
#pragma unroll
      for (int i = 0; i < 8; ++i) v[c][i] = 0.f;
      if (ch >= nchunk) continue;
      if (owner == tp.rank) {
        // ---- the owner: every other rank's share of this row, summed in rank order with its own, sent to everyone
        uint4 pr[kTpMaxRanks];
        bool all = false;
        while (!all) {
          all = true;
#pragma unroll
          for (int r = 0; r < kTpMaxRanks; ++r)
            if (r < tp.size && r != tp.rank) {
              const uint64_t* src = reinterpret_cast<const uint64_t*>(tp.xbuf[tp.rank]) +
                                    ((slot_off + (size_t)r * tp.slot_elems + base + ch * 8) >> 1);
              uint64_t a0, a1, a2, a3;
              ld_relaxed_sys_2x64(src, a0, a1);
              ld_relaxed_sys_2x64(src + 2, a2, a3);
              all = all && (uint32_t)(a0 >> 32) == seq && (uint32_t)(a1 >> 32) == seq && (uint32_t)(a2 >> 32) == seq &&
                    (uint32_t)(a3 >> 32) == seq;
              pr[r] = make_uint4((uint32_t)a0, (uint32_t)a1, (uint32_t)a2, (uint32_t)a3);
            }
          if (!all && clock64() - t0 > wait_cycles) {
            status[0] = (uint32_t)(-RB_ERR_TIMEOUT); status[1] = 0x7A11u; status[2] = (uint32_t)tp.rank; status[3] = seq;
            give_up = 1u;
            break;
          }
        }
        if (!all) continue;
        float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < kTpMaxRanks; ++r)   // rank order
          if (r < tp.size) add8_bf16(r == tp.rank ? own[c] : pr[r], sum);
        const uint4 red = pack8_bf16(sum);  // what an allreduce in the model dtype would have delivered
        const size_t word = (res_off + base + ch * 8) >> 1;
#pragma unroll
        for (int r = 0; r < kTpMaxRanks; ++r)
          if (r < tp.size && r != tp.rank) {
            uint64_t* dst = reinterpret_cast<uint64_t*>(const_cast<void*>(tp.xbuf[r])) + word;
            st_relaxed_sys_2x64(dst, tag | red.x, tag | red.y);
            st_relaxed_sys_2x64(dst + 2, tag | red.z, tag | red.w);
          }
        add8_bf16(red, v[c]);
      } else {
        // ---- everyone else: the finished row from its owner
        const uint64_t* src = reinterpret_cast<const uint64_t*>(tp.xbuf[tp.rank]) + ((res_off + base + ch * 8) >> 1);
        uint64_t a0 = 0, a1 = 0, a2 = 0, a3 = 0;
        bool all = false;
        while (!all) {
          ld_relaxed_sys_2x64(src, a0, a1);
          ld_relaxed_sys_2x64(src + 2, a2, a3);
          all = (uint32_t)(a0 >> 32) == seq && (uint32_t)(a1 >> 32) == seq && (uint32_t)(a2 >> 32) == seq &&
                (uint32_t)(a3 >> 32) == seq;
          if (!all && clock64() - t0 > wait_cycles) {
            status[0] = (uint32_t)(-RB_ERR_TIMEOUT); status[1] = 0x7A11u; status[2] = (uint32_t)tp.rank; status[3] = seq;
            give_up = 1u;
            break;
          }
        }
        if (!all) continue;
        add8_bf16(make_uint4((uint32_t)a0, (uint32_t)a1, (uint32_t)a2, (uint32_t)a3), v[c]);
      }
    }
  } else if (kMode == kTpInDataDirect) {
    // ---- the same row from every peer: each thread polls the words it will sum (its own row is still in registers)
    const long long t0 = clock64();
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      const int ch = threadIdx.x + c * blockDim.x;
#pragma unroll
      for (int i = 0; i < 8; ++i) v[c][i] = 0.f;
      if (ch >= nchunk) continue;
      uint4 pr[kTpDirectRanks];
      bool all = false;
      while (!all) {
        all = true;
#pragma unroll
        for (int r = 0; r < kTpDirectRanks; ++r)
          if (r < tp.size && r != tp.rank) {
            const uint64_t* src = reinterpret_cast<const uint64_t*>(tp.xbuf[tp.rank]) +
                                  ((slot_off + (size_t)r * tp.slot_elems + base + ch * 8) >> 1);
            uint64_t a0, a1, a2, a3;
            ld_relaxed_sys_2x64(src, a0, a1);
            ld_relaxed_sys_2x64(src + 2, a2, a3);
            all = all && (uint32_t)(a0 >> 32) == seq && (uint32_t)(a1 >> 32) == seq && (uint32_t)(a2 >> 32) == seq &&
                  (uint32_t)(a3 >> 32) == seq;
            pr[r] = make_uint4((uint32_t)a0, (uint32_t)a1, (uint32_t)a2, (uint32_t)a3);
          }
        if (!all && clock64() - t0 > wait_cycles) {
          status[0] = (uint32_t)(-RB_ERR_TIMEOUT); status[1] = 0x7A11u; status[2] = (uint32_t)tp.rank; status[3] = seq;
          give_up = 1u;
          break;
        }
      }
#pragma unroll
      for (int r = 0; r < kTpDirectRanks; ++r)   // rank order, on every rank alike
        if (r < tp.size) add8_bf16(r == tp.rank ? own[c] : pr[r], v[c]);
    }
  } else {
  __syncthreads();  // the block's stores are ordered before the releases below (cumulativity through the barrier)
  if ((int)threadIdx.x < tp.size) {
    // a release at system scope: every store of the block that the barrier ordered before it is performed at the peer
    // before the flag can be seen there (no separate fence: the release carries one)
    if ((int)threadIdx.x != tp.rank)
      st_release_sys(tp.flags[threadIdx.x] + ((size_t)(seq & 1u) * kTpMaxRanks + tp.rank) * kTpMaxRows + row, seq);
    // ---- and the same row from every other rank: thread t waits for rank t (this rank's own row is still in registers)
    const uint32_t* flag = tp.flags[tp.rank] + ((size_t)(seq & 1u) * kTpMaxRanks + threadIdx.x) * kTpMaxRows + row;
    const long long t0 = clock64();
    while ((int)threadIdx.x != tp.rank && (int32_t)(ld_acquire_sys(flag) - seq) < 0) {
      if (clock64() - t0 > wait_cycles) {
        status[0] = (uint32_t)(-RB_ERR_TIMEOUT); status[1] = 0x7A11u; status[2] = (uint32_t)tp.rank; status[3] = seq;
        give_up = 1u;
        break;
      }
    }
  }
  }
  __syncthreads();
  // the exchange number moves on whether or not a peer arrived: the next launch must not reuse this one's slot
  if (row == 0 && threadIdx.x == 0) *reinterpret_cast<volatile uint32_t*>(tp.seq + (parity ^ 1) * 32) = seq;
  if (give_up) return;  // a peer never arrived: leave the outputs alone, the host sees the status
  // (flag array form) the pollers' acquire loads plus the barrier order every thread's (system-scope) reads below
  // behind the flags
  float s = 0.f;
  const float inv_sqrt_h = 1.0f / sqrtf((float)hidden);
  const T* mine = reinterpret_cast<const T*>(tp.xbuf[tp.rank]) + slot_off + base;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch >= nchunk) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[c][i] = 0.f;
      continue;
    }
    float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (kMode != kTpFlagArray) {
#pragma unroll
      for (int i = 0; i < 8; ++i) { sum[i] = v[c][i]; v[c][i] = 0.f; }
      if (h) load8(h + base + ch * 8, v[c]);
    } else {
      uint4 pr[kTpMaxRanks];  // all copies in flight at once, still packed
#pragma unroll
      for (int i = 0; i < 8; ++i) v[c][i] = 0.f;
#pragma unroll
      for (int r = 0; r < kTpMaxRanks; ++r)
        if (r < tp.size) pr[r] = r == tp.rank ? own[c] : load16_sys(mine + (size_t)r * tp.slot_elems + ch * 8);
      if (h) load8(h + base + ch * 8, v[c]);
#pragma unroll
      for (int r = 0; r < kTpMaxRanks; ++r)   // rank order, on every rank alike
        if (r < tp.size) add8_bf16(pr[r], sum);
    }
    round_to<T>(sum);  // what an allreduce in the model dtype would have delivered
#pragma unroll
    for (int i = 0; i < 8; ++i) v[c][i] += sum[i];
    round_to<T>(v[c]);  // the residual stream is stored in the model dtype
    if (sum_out) store8(sum_out + base + ch * 8, v[c]);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (kind == RB_NORM_LAYER) s += v[c][i];
      else if (kind == RB_NORM_RMS) { const float t2 = v[c][i] * inv_sqrt_h; s += t2 * t2; }
      else s += v[c][i] * v[c][i];
    }
  }
  if (!out) return;
  s = block_sum(s, red);
  float mean = 0.f, r;
  if (kind == RB_NORM_LAYER) {
    mean = s / (float)hidden;
    float q = 0.f;
#pragma unroll
    for (int c = 0; c < kChunks; ++c)
      if (threadIdx.x + c * blockDim.x < nchunk) {
#pragma unroll
        for (int i = 0; i < 8; ++i) { const float d = v[c][i] - mean; q += d * d; }
      }
    q = block_sum(q, red);
    r = 1.0f / sqrtf(q / (float)hidden + eps);
  } else if (kind == RB_NORM_RMS) {
    r = 1.0f / sqrtf(s + eps);
  } else {
    r = 1.0f / sqrtf(s / (float)hidden + eps);
  }
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch >= nchunk) continue;
    float y[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (kind == RB_NORM_LAYER) { y[i] = (v[c][i] - mean) * r; if (w) y[i] = wv[c][i] * y[i] + bv[c][i]; }
      else if (kind == RB_NORM_RMS) y[i] = wv[c][i] * v[c][i] * r;
      else y[i] = v[c][i] * r * (wv[c][i] + 1.0f);
    }
    store8(out + base + ch * 8, y);
  }
}


// Finishes an MLP up-projection that was computed as split-K partials over [gate; up]: sums the slabs in
// a fixed order, adds the bias, applies the activation (hlops/activations.rs:20-32) and the gating
// product (qwen2.rs:101-103).  8 outputs per thread.
__global__ void act_from_partials_kernel(const float* __restrict__ part, int n_split, size_t slab, int n_all, int n_out,
                                         int gated, const __nv_bfloat16* __restrict__ bias, int act,
                                         __nv_bfloat16* __restrict__ out, int64_t total_chunks) {
  pdl_launch_dependents();
  pdl_wait();
  const int chunks_per_row = n_out >> 3;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total_chunks; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / chunks_per_row;
    const int j = (int)(i % chunks_per_row) * 8;
    float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, u[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, t[8];
    for (int s = 0; s < n_split; ++s) {
      load8(part + (size_t)s * slab + (size_t)r * n_all + j, t);
#pragma unroll
      for (int k = 0; k < 8; ++k) g[k] += t[k];
      if (gated) {
        load8(part + (size_t)s * slab + (size_t)r * n_all + n_out + j, t);
#pragma unroll
        for (int k = 0; k < 8; ++k) u[k] += t[k];
      }
    }
    if (bias) { load8(bias + j, t);
#pragma unroll
      for (int k = 0; k < 8; ++k) g[k] += t[k]; }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      // gate and up are tensors of the model dtype before the product in the reference; round like the fused kernel does not
      const float a = act_apply(act, g[k]);
      g[k] = gated ? a * u[k] : a;
    }
    store8(out + (size_t)r * n_out + j, g);
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
  pdl_launch_dependents();
  pdl_wait();
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


// Vector form of the kernel above for head_dim % 8 == 0 and (rot/2) % 8 == 0: a work item is
// either a pair of 8-element chunks (lanes i..i+8 and i+rot/2..) of a q or k head, rotated together,
// or one pass-through chunk (lanes >= rot, and all of v).  16-byte loads and stores throughout.
template <typename T>
__global__ void rope_kv_append_vec_kernel(const T* __restrict__ qkv, const float* __restrict__ acc, int n_acc,
                                          size_t acc_stride, const T* __restrict__ bias,
                                          const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
                                          int s_new, int q_heads, int kv_heads, int d, T* __restrict__ q_out,
                                          T* __restrict__ k_cache, T* __restrict__ v_cache,
                                          const int32_t* __restrict__ block_table,
                                          const int32_t* __restrict__ seq_lens, int pages_per_seq, int max_seq,
                                          uint32_t* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int m = blockIdx.x;
  const int b = m / s_new, sq = m % s_new;
  const int ncol = (q_heads + 2 * kv_heads) * d;
  const int pos = seq_lens[b] - s_new + sq;
  if (pos < 0 || pos >= max_seq) {
    if (threadIdx.x == 0) { status[0] = (uint32_t)(-RB_ERR_INVALID); status[1] = 0x20BEu; status[2] = (uint32_t)pos; }
    return;
  }
  const int half = rot >> 1;
  const int pair_items = half >> 3, pass_items = (d - rot) >> 3;
  const int per_rot_head = pair_items + pass_items;  // items of one q or k head
  const int rot_heads = q_heads + kv_heads;
  const int v_items = d >> 3;
  const int total = rot_heads * per_rot_head + kv_heads * v_items;
  const int page = block_table[(size_t)b * pages_per_seq + pos / kPageTokens];
  const int slot = pos % kPageTokens;
  const size_t row = (size_t)m * ncol;
  auto gather = [&](int col, float* v) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
    float t[8];
    if (qkv) { load8(qkv + row + col, t);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += t[i]; }
    for (int k = 0; k < n_acc; ++k) { load8(acc + (size_t)k * acc_stride + row + col, t);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += t[i]; }
    if (bias) { load8(bias + col, t);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += t[i]; }
  };
  auto emit = [&](int head, int lane0, const float* v) {
    if (head < q_heads) {
      store8(q_out + (size_t)m * q_heads * d + head * d + lane0, v);
    } else {
      const bool is_v = head >= rot_heads;
      const int kvh = is_v ? head - rot_heads : head - q_heads;
      const size_t off = (((size_t)page * kv_heads + kvh) * kPageTokens + slot) * d + lane0;
      store8((is_v ? v_cache : k_cache) + off, v);
    }
  };
  for (int it = threadIdx.x; it < total; it += blockDim.x) {
    if (it < rot_heads * per_rot_head) {
      const int head = it / per_rot_head, j = it % per_rot_head;
      if (j < pair_items) {
        const int i0 = j * 8;
        float lo[8], hi[8], cs[8], sn[8], ylo[8], yhi[8];
        gather(head * d + i0, lo);
        gather(head * d + i0 + half, hi);
        load8(cos_t + (size_t)pos * half + i0, cs);
        load8(sin_t + (size_t)pos * half + i0, sn);
        rope_rotate8(lo, hi, cs, sn, ylo, yhi);
        emit(head, i0, ylo);
        emit(head, i0 + half, yhi);
      } else {
        const int i0 = rot + (j - pair_items) * 8;
        float v[8];
        gather(head * d + i0, v);
        emit(head, i0, v);
      }
    } else {
      const int k = it - rot_heads * per_rot_head;
      const int head = rot_heads + k / v_items, i0 = (k % v_items) * 8;
      float v[8];
      gather(head * d + i0, v);
      emit(head, i0, v);
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

// Each row is split over gridDim.x blocks; a block folds its segment into a 64-bit (key << 32 | index)
// candidate, merges it into the row's running best with atomicMax (order-independent, so the result
// is deterministic), and the last block to arrive writes the index and resets the scratch words.
//
// PEN = true adds the examples' repeat penalty (examples/qwen2/src/main.rs:42-53,84-88): the token ids in
// the row's context window form a set (a hash set in shared memory, so a repeated id is penalised once);
// a member's float32 logit is divided by the penalty when >= 0 and multiplied by it otherwise before it
// competes.  The penalised value never goes back to the logits' storage type, exactly like the host code,
// which penalises a float32 copy.  `eos`/`finished` give the loop's stop rule per row: a row that has
// produced `eos` keeps producing it.
struct SampleArgs {
  const int32_t* context = nullptr;        // [rows, context_stride] token ids
  const int32_t* context_count = nullptr;  // [rows] ids pushed so far; min(count, stride) slots are valid
  int context_stride = 0;
  float penalty = 0.f;
  int32_t eos = -1;
  uint8_t* finished = nullptr;             // [rows] or null
};
constexpr int kSampleTableSlots = 1024;    // hash slots, 4x the largest context window
constexpr int kSampleMaxContext = 256;

__device__ __forceinline__ uint32_t sample_emit(const SampleArgs& sa, int r, uint32_t idx) {
  if (sa.eos >= 0 && sa.finished) {
    if (sa.finished[r]) idx = (uint32_t)sa.eos;
    else if (idx == (uint32_t)sa.eos) sa.finished[r] = 1;
  }
  return idx;
}

template <typename T, bool PEN>
__global__ void argmax_rows_kernel(const T* __restrict__ x, int64_t cols, uint32_t* __restrict__ out,
                                   unsigned long long* __restrict__ best_g, unsigned int* __restrict__ count_g,
                                   SampleArgs sa) {
  __shared__ unsigned long long best[32];
  __shared__ int32_t table[PEN ? kSampleTableSlots : 1];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.y;
  const T* row = x + (size_t)r * cols;
  const int64_t seg = ((cols + gridDim.x - 1) / gridDim.x + 7) & ~int64_t(7);
  const int64_t c0 = (int64_t)blockIdx.x * seg, c1 = min(cols, c0 + seg);
  if (PEN) {
    for (int i = threadIdx.x; i < kSampleTableSlots; i += blockDim.x) table[i] = -1;
    __syncthreads();
    const int valid = min(sa.context_count[r], sa.context_stride);
    for (int i = threadIdx.x; i < valid; i += blockDim.x) {
      const int32_t tok = sa.context[(size_t)r * sa.context_stride + i];
      if (tok < 0) continue;
      uint32_t h = ((uint32_t)tok * 0x9E3779B1u) >> 22;
      for (int probe = 0; probe < kSampleTableSlots; ++probe) {   // at most 256 of 1024 slots ever fill
        const int32_t prev = atomicCAS(&table[h], -1, tok);
        if (prev == -1 || prev == tok) break;
        h = (h + 1) & (kSampleTableSlots - 1);
      }
    }
    __syncthreads();
  }
  unsigned long long loc = 0;
  auto consider = [&](float f, int64_t i) {
    if (PEN) {
      uint32_t h = ((uint32_t)i * 0x9E3779B1u) >> 22;
      for (int probe = 0; probe < kSampleTableSlots; ++probe) {
        const int32_t t = table[h];
        if (t == -1) break;
        if (t == (int32_t)i) { f = (f >= 0.f) ? __fdiv_rn(f, sa.penalty) : __fmul_rn(f, sa.penalty); break; }
        h = (h + 1) & (kSampleTableSlots - 1);
      }
    }
    const unsigned long long cand = ((unsigned long long)total_order_key(f) << 32) | (uint32_t)i;
    loc = cand > loc ? cand : loc;
  };
  const bool vec = ((reinterpret_cast<uintptr_t>(row) & 15) == 0) && ((cols * sizeof(T)) % 16 == 0);
  if (vec) {
    for (int64_t i = c0 + (int64_t)threadIdx.x * 8; i + 8 <= c1; i += (int64_t)blockDim.x * 8) {
      float v[8];
      load8(row + i, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) consider(v[j], i + j);
    }
    const int64_t tail = c0 + ((c1 - c0) & ~int64_t(7));
    for (int64_t i = tail + threadIdx.x; i < c1; i += blockDim.x) consider(Cvt<T>::to_f(row[i]), i);
  } else {
    for (int64_t i = c0 + threadIdx.x; i < c1; i += blockDim.x) consider(Cvt<T>::to_f(row[i]), i);
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
    if (lane == 0) {
      if (gridDim.x == 1) { out[r] = sample_emit(sa, r, (uint32_t)(loc & 0xffffffffull)); return; }
      atomicMax(&best_g[r], loc);
      __threadfence();
      const unsigned int arrived = atomicAdd(&count_g[r], 1u);
      if (arrived == gridDim.x - 1) {
        __threadfence();
        const unsigned long long fin = atomicExch(&best_g[r], 0ull);  // read and reset for the next call
        count_g[r] = 0u;
        out[r] = sample_emit(sa, r, (uint32_t)(fin & 0xffffffffull));
      }
    }
  }
}

}  // namespace rb

using namespace rb;

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
static int embed_launch(rb_ctx* ctx, const void* table, int64_t vocab, int64_t hidden, const uint32_t* ids, int64_t n_ids,
                        float scale, void* out) {
  RB_CUDA(launch_kernel(embed_gather_kernel<T>, dim3((unsigned)n_ids), dim3(128), 0, ctx->stream, ctx->pdl,
                        (const T*)table, ids, vocab, (int)hidden, scale, (T*)out, ctx->status_dev));
  return RB_OK;
}

extern "C" int32_t rb_embed_gather(rb_ctx* ctx, const void* table, int32_t dtype, int64_t vocab, int64_t hidden,
                                   const uint32_t* ids, int64_t n_ids, float scale, void* out) {
  RB_REQUIRE(ctx && table && ids && out, "rb_embed_gather: null argument");
  RB_REQUIRE(vocab > 0 && hidden > 0 && n_ids >= 0, "rb_embed_gather: bad sizes");
  if (n_ids == 0) return RB_OK;
  ProfScope prof(ctx, RB_PROF_EMBED, 2.0 * n_ids * hidden * dtype_size(dtype), 0.0);
  if (dtype == RB_BF16) RB_TRY(embed_launch<__nv_bfloat16>(ctx, table, vocab, hidden, ids, n_ids, scale, out));
  else if (dtype == RB_F32) RB_TRY(embed_launch<float>(ctx, table, vocab, hidden, ids, n_ids, scale, out));
  else return fail(RB_ERR_DTYPE, "rb_embed_gather: dtype %d unsupported", dtype);
  ctx->launches++;
  return RB_OK;
}

template <typename T>
static int norm_launch(rb_ctx* ctx, int kind, const void* x, const void* add, const float* acc, int n_acc,
                       const void* acc_bias, const void* w, const void* b, float eps, int64_t rows, int64_t hidden,
                       void* out, void* sum_out) {
  const size_t acc_stride = (size_t)rows * hidden;
  const bool vec_ok = (hidden % 8) == 0 && hidden <= 16384 && aligned16(x) && aligned16(add) && aligned16(acc) &&
                      aligned16(acc_bias) && aligned16(w) && aligned16(b) && aligned16(out) && aligned16(sum_out) &&
                      ((acc_stride * sizeof(float)) % 16) == 0;
  if (vec_ok) {
    const int nchunk = (int)(hidden / 8);
    int threads = std::min(512, (nchunk + 31) / 32 * 32);
    const int chunks = (nchunk + threads - 1) / threads;
    // decode-sized calls get a block per row (pure latency); prefill-sized ones a few blocks per SM that walk the rows
    const int64_t blocks = std::min<int64_t>(rows, (int64_t)ctx->sm_count * 8);
    auto go = [&](auto kern) {
      return launch_kernel(kern, dim3((unsigned)blocks), dim3(threads), 0, ctx->stream, ctx->pdl, kind, (const T*)x,
                           (const T*)add, acc, n_acc, acc_stride, (const T*)acc_bias, (const T*)w, (const T*)b, eps,
                           (int)hidden, (T*)out, (T*)sum_out, (int64_t)rows);
    };
    if (n_acc > 0 || acc_bias) {
      if (chunks == 1) RB_CUDA(go(norm_vec_kernel<T, 1, true>));
      else if (chunks == 2) RB_CUDA(go(norm_vec_kernel<T, 2, true>));
      else RB_CUDA(go(norm_vec_kernel<T, 4, true>));
    } else {
      if (chunks == 1) RB_CUDA(go(norm_vec_kernel<T, 1, false>));
      else if (chunks == 2) RB_CUDA(go(norm_vec_kernel<T, 2, false>));
      else RB_CUDA(go(norm_vec_kernel<T, 4, false>));
    }
    return RB_OK;
  }
  const size_t smem = (size_t)hidden * sizeof(float);
  const int threads = hidden >= 2048 ? 512 : 256;
  auto kern = norm_kernel<T>;
  if (smem > 48 * 1024) RB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  RB_CUDA(launch_kernel(kern, dim3((unsigned)rows), dim3(threads), smem, ctx->stream, ctx->pdl, kind, (const T*)x,
                        (const T*)add, acc, n_acc, acc_stride, (const T*)acc_bias, (const T*)w, (const T*)b, eps,
                        (int)hidden, (T*)out, (T*)sum_out));
  return RB_OK;
}

extern "C" int32_t rb_norm(rb_ctx* ctx, int32_t kind, const void* x, const void* add, const float* acc, int32_t n_acc,
                           const void* acc_bias, const void* w, const void* b, float eps, int64_t rows, int64_t hidden,
                           void* out, void* sum_out, int32_t dtype) {
  RB_REQUIRE(ctx, "rb_norm: null context");
  RB_REQUIRE(x || add || (acc && n_acc > 0), "rb_norm: no input given");
  RB_REQUIRE(out || sum_out, "rb_norm: no output given");
  RB_REQUIRE(kind >= RB_NORM_RMS && kind <= RB_NORM_LAYER, "rb_norm: bad kind %d", kind);
  RB_REQUIRE(!out || w || kind == RB_NORM_LAYER, "rb_norm: weight required");
  RB_REQUIRE(rows >= 0 && hidden > 0 && hidden <= 49152, "rb_norm: hidden %lld out of range", (long long)hidden);
  if (rows == 0) return RB_OK;
  if (!acc) n_acc = 0;
  if (n_acc == 0) acc = nullptr;
  ProfScope prof(ctx, RB_PROF_NORM,
                 (double)rows * hidden * (dtype_size(dtype) * ((x ? 1 : 0) + (add ? 1 : 0) + (out ? 1 : 0) + (sum_out ? 1 : 0)) + 4.0 * n_acc),
                 0.0);
  if (dtype == RB_BF16)
    RB_TRY(norm_launch<__nv_bfloat16>(ctx, kind, x, add, acc, n_acc, acc_bias, w, b, eps, rows, hidden, out, sum_out));
  else if (dtype == RB_F32)
    RB_TRY(norm_launch<float>(ctx, kind, x, add, acc, n_acc, acc_bias, w, b, eps, rows, hidden, out, sum_out));
  else
    return fail(RB_ERR_DTYPE, "rb_norm: dtype %d unsupported", dtype);
  ctx->launches++;
  return RB_OK;
}

namespace rb {

int exchange_norm(rb_ctx* ctx, const TpPeers& tp, int parity, int kind, const void* h, const float* acc, int n_acc,
                  const void* acc_bias, const void* part, const void* w, const void* b, float eps, int64_t rows,
                  int64_t hidden, void* out, void* sum_out) {
  RB_REQUIRE(rows > 0 && rows <= kTpMaxRows, "exchange_norm: %lld rows exceed the exchange buffer", (long long)rows);
  RB_REQUIRE((hidden % 8) == 0 && hidden <= 16384, "exchange_norm: hidden %lld unsupported", (long long)hidden);
  RB_REQUIRE((part != nullptr) != (acc != nullptr && n_acc > 0), "exchange_norm: exactly one form of the partial product");
  RB_REQUIRE(tp.size >= 1 && tp.size <= kTpMaxRanks && (parity == 0 || parity == 1), "exchange_norm: bad group");
  using T = __nv_bfloat16;
  const size_t acc_stride = (size_t)rows * hidden;
  RB_REQUIRE(aligned16(h) && aligned16(acc) && aligned16(acc_bias) && aligned16(part) && aligned16(w) && aligned16(b) &&
                 aligned16(out) && aligned16(sum_out) && ((acc_stride * sizeof(float)) % 16) == 0,
             "exchange_norm: operands must be 16-byte aligned");
  ProfScope prof(ctx, RB_PROF_NORM, (double)rows * hidden * (2.0 * (3 + 2 * tp.size) + 4.0 * n_acc), 0.0);
  const int nchunk = (int)(hidden / 8);
  const int threads = std::min(512, (nchunk + 31) / 32 * 32);
  const int chunks = (nchunk + threads - 1) / threads;
  auto go = [&](auto kern) {
    return launch_kernel(kern, dim3((unsigned)rows), dim3(threads), 0, ctx->stream, ctx->pdl, kind, (const T*)h, acc, n_acc,
                         acc_stride, (const T*)acc_bias, (const T*)part, (const T*)w, (const T*)b, eps, (int)hidden, (T*)out,
                         (T*)sum_out, tp, parity, ctx->status_dev, ctx->wait_budget_cycles);
  };
  if (tp.form == kTpInDataDirect) {
    RB_REQUIRE(tp.size <= kTpDirectRanks, "exchange_norm: the direct flag-in-data form takes groups of up to %d", kTpDirectRanks);
    if (chunks == 1) RB_CUDA(go(exchange_norm_kernel<T, 1, kTpInDataDirect>));
    else if (chunks == 2) RB_CUDA(go(exchange_norm_kernel<T, 2, kTpInDataDirect>));
    else RB_CUDA(go(exchange_norm_kernel<T, 4, kTpInDataDirect>));
  } else if (tp.form == kTpInDataTwoHop) {
    if (chunks == 1) RB_CUDA(go(exchange_norm_kernel<T, 1, kTpInDataTwoHop>));
    else if (chunks == 2) RB_CUDA(go(exchange_norm_kernel<T, 2, kTpInDataTwoHop>));
    else RB_CUDA(go(exchange_norm_kernel<T, 4, kTpInDataTwoHop>));
  } else {
    if (chunks == 1) RB_CUDA(go(exchange_norm_kernel<T, 1, kTpFlagArray>));
    else if (chunks == 2) RB_CUDA(go(exchange_norm_kernel<T, 2, kTpFlagArray>));
    else RB_CUDA(go(exchange_norm_kernel<T, 4, kTpFlagArray>));
  }
  ctx->launches++;
  return RB_OK;
}

int act_from_partials(rb_ctx* ctx, const float* part, int n_split, int64_t rows, int64_t n_all, int64_t n_out, bool gated,
                      const void* bias, int act, void* out) {
  RB_REQUIRE(part && out && rows > 0 && n_out > 0 && (n_out % 8) == 0 && (n_all % 4) == 0, "act_from_partials: bad shape");
  ProfScope prof(ctx, RB_PROF_OTHER, (double)rows * (4.0 * n_split * n_all + 2.0 * n_out), 0.0);
  const int64_t chunks = rows * (n_out / 8);
  const int blocks = (int)std::min<int64_t>((chunks + 127) / 128, 8 * ctx->sm_count);
  RB_CUDA(launch_kernel(act_from_partials_kernel, dim3((unsigned)blocks), dim3(128), 0, ctx->stream, ctx->pdl, part, n_split,
                        (size_t)rows * n_all, (int)n_all, (int)n_out, gated ? 1 : 0, (const __nv_bfloat16*)bias, act,
                        (__nv_bfloat16*)out, chunks));
  ctx->launches++;
  return RB_OK;
}

}  // namespace rb

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

template <typename T>
static int rope_launch(rb_ctx* ctx, const void* qkv, const float* acc, int n_acc, const void* bias, const float* cos_t,
                       const float* sin_t, int rot, int batch, int s_new, int q_heads, rb_kv_cache* c, int layer,
                       void* q_out) {
  const int d = c->head_dim, ncol = (q_heads + 2 * c->kv_heads) * d;
  const size_t acc_stride = (size_t)batch * s_new * ncol;
  const size_t loff = (size_t)layer * c->layer_stride_elems();
  T* kc = (T*)c->k + loff;
  T* vc = (T*)c->v + loff;
  const int half = rot / 2;
  const bool vec_ok = (d % 8) == 0 && (half % 8) == 0 && aligned16(qkv) && aligned16(acc) && aligned16(bias) &&
                      aligned16(q_out) && aligned16(cos_t) && aligned16(sin_t) && ((acc_stride * sizeof(float)) % 16) == 0;
  if (vec_ok) {
    const int items = (q_heads + c->kv_heads) * (half / 8 + (d - rot) / 8) + c->kv_heads * (d / 8);
    const int threads = std::min(512, (items + 31) / 32 * 32);
    RB_CUDA(launch_kernel(rope_kv_append_vec_kernel<T>, dim3((unsigned)(batch * s_new)), dim3(threads), 0, ctx->stream,
                          ctx->pdl, (const T*)qkv, acc, n_acc, acc_stride, (const T*)bias, cos_t, sin_t, rot, s_new,
                          q_heads, c->kv_heads, d, (T*)q_out, kc, vc, (const int32_t*)c->block_table,
                          (const int32_t*)c->seq_lens, c->pages_per_seq, c->max_seq, ctx->status_dev));
    return RB_OK;
  }
  const size_t smem = (size_t)ncol * sizeof(float);
  auto kern = rope_kv_append_kernel<T>;
  if (smem > 48 * 1024) RB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  RB_CUDA(launch_kernel(kern, dim3((unsigned)(batch * s_new)), dim3(256), smem, ctx->stream, ctx->pdl, (const T*)qkv, acc,
                        n_acc, acc_stride, (const T*)bias, cos_t, sin_t, rot, s_new, q_heads, c->kv_heads, d, (T*)q_out,
                        kc, vc, (const int32_t*)c->block_table, (const int32_t*)c->seq_lens, c->pages_per_seq,
                        c->max_seq, ctx->status_dev));
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
  if (n_acc == 0) acc = nullptr;
  const int ncol = (q_heads + 2 * c->kv_heads) * c->head_dim;
  ProfScope prof(ctx, RB_PROF_ROPE_KV, (double)batch * s_new * ncol * (dtype_size(dtype) * (qkv ? 2.0 : 1.0) + 4.0 * n_acc), 0.0);
  if (dtype == RB_BF16)
    RB_TRY(rope_launch<__nv_bfloat16>(ctx, qkv, acc, n_acc, bias, cos_t, sin_t, rot, batch, s_new, q_heads, c, layer, q_out));
  else if (dtype == RB_F32)
    RB_TRY(rope_launch<float>(ctx, qkv, acc, n_acc, bias, cos_t, sin_t, rot, batch, s_new, q_heads, c, layer, q_out));
  else
    return fail(RB_ERR_DTYPE, "rb_rope_kv_append: dtype %d unsupported", dtype);
  ctx->launches++;
  return RB_OK;
}

template <typename T>
static int argmax_launch(rb_ctx* ctx, const void* logits, int64_t rows, int64_t cols, uint32_t* out, SampleArgs sa) {
  // enough blocks per row to fill the GPU, at least ~2K elements each
  int per_row = (int)std::min<int64_t>(std::max<int64_t>(1, (2 * ctx->sm_count + rows - 1) / rows), (cols + 2047) / 2048);
  per_row = std::max(1, std::min(per_row, 64));
  const bool pen = sa.context != nullptr;
  for (int64_t r0 = 0; r0 < rows; r0 += kArgmaxRows) {
    const int64_t n = std::min<int64_t>(kArgmaxRows, rows - r0);
    SampleArgs part = sa;
    if (pen) { part.context += r0 * sa.context_stride; part.context_count += r0; }
    if (part.finished) part.finished += r0;
    if (pen)
      RB_CUDA(launch_kernel(argmax_rows_kernel<T, true>, dim3((unsigned)per_row, (unsigned)n), dim3(256), 0, ctx->stream,
                            ctx->pdl, (const T*)logits + r0 * cols, cols, out + r0, ctx->argmax_best, ctx->argmax_count, part));
    else
      RB_CUDA(launch_kernel(argmax_rows_kernel<T, false>, dim3((unsigned)per_row, (unsigned)n), dim3(256), 0, ctx->stream,
                            ctx->pdl, (const T*)logits + r0 * cols, cols, out + r0, ctx->argmax_best, ctx->argmax_count, part));
    ctx->launches++;
  }
  return RB_OK;
}

extern "C" int32_t rb_argmax_rows(rb_ctx* ctx, const void* logits, int32_t dtype, int64_t rows, int64_t cols,
                                  uint32_t* out) {
  RB_REQUIRE(ctx && logits && out, "rb_argmax_rows: null argument");
  RB_REQUIRE(rows >= 0 && cols > 0 && cols <= 0xffffffffLL, "rb_argmax_rows: bad sizes");
  if (rows == 0) return RB_OK;
  ProfScope prof(ctx, RB_PROF_ARGMAX, (double)rows * cols * dtype_size(dtype), 0.0);
  if (dtype == RB_BF16) return argmax_launch<__nv_bfloat16>(ctx, logits, rows, cols, out, SampleArgs{});
  if (dtype == RB_F32) return argmax_launch<float>(ctx, logits, rows, cols, out, SampleArgs{});
  return fail(RB_ERR_DTYPE, "rb_argmax_rows: dtype %d unsupported", dtype);
}

extern "C" int32_t rb_sample_greedy(rb_ctx* ctx, const void* logits, int32_t dtype, int64_t rows, int64_t cols,
                                    float penalty, const int32_t* context, int32_t context_stride,
                                    const int32_t* context_count, int32_t eos_token, uint8_t* finished, uint32_t* out) {
  RB_REQUIRE(ctx && logits && out, "rb_sample_greedy: null argument");
  RB_REQUIRE(rows >= 0 && cols > 0 && cols <= 0xffffffffLL, "rb_sample_greedy: bad sizes");
  if (rows == 0) return RB_OK;
  SampleArgs sa;
  // the examples apply the penalty only when it is >= 1 (examples/qwen2/src/main.rs:85)
  if (penalty >= 1.0f && context_stride > 0) {
    RB_REQUIRE(context && context_count, "rb_sample_greedy: a penalty needs the context window and its counts");
    RB_REQUIRE(context_stride <= kSampleMaxContext, "rb_sample_greedy: context window %d exceeds %d tokens", context_stride,
               kSampleMaxContext);
    sa.context = context;
    sa.context_count = context_count;
    sa.context_stride = context_stride;
    sa.penalty = penalty;
  }
  if (eos_token >= 0 && finished) { sa.eos = eos_token; sa.finished = finished; }
  ProfScope prof(ctx, RB_PROF_ARGMAX, (double)rows * cols * dtype_size(dtype), 0.0);
  if (dtype == RB_BF16) return argmax_launch<__nv_bfloat16>(ctx, logits, rows, cols, out, sa);
  if (dtype == RB_F32) return argmax_launch<float>(ctx, logits, rows, cols, out, sa);
  return fail(RB_ERR_DTYPE, "rb_sample_greedy: dtype %d unsupported", dtype);
}
