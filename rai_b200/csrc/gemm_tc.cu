// bf16 GEMM for Linear::fwd (rai-nn/src/linear.rs:59-69) on the 5th-generation tensor cores:
// C[M,N] = X[M,K] . W[N,K]^T with float32 accumulation in tensor memory.
//
// One persistent CTA per SM, 6 warps with fixed roles:
//   warp 0   TMA producer: streams 64-wide K slices of both operands into a ring of shared-memory
//            stages (128-byte swizzle), completion counted on an mbarrier per stage;
//   warp 1   owns the TMEM allocation; one lane issues tcgen05.mma (M=128, N=BN, K=16) four times
//            per stage and commits to the stage's "empty" barrier, then to the accumulator's
//            "full" barrier when the K loop of a work item ends;
//   warps 2-5 epilogue: tcgen05.ld the accumulator (each warp its own 32 TMEM lanes), apply bias /
//            activation / gating / residual, store.  Two accumulator stages, so the epilogue of
//            item i overlaps the K loop of item i+1.
//
// Operands are named by the TMEM axis they feed: the P operand's rows become TMEM lanes (128 per
// tile), the Q operand's rows become TMEM columns (BN per tile).
//   normal (SWAP = false): P = X, Q = W  — prefill-sized M.
//   swapped (SWAP = true):  P = W, Q = X  — decode-sized M (<= 256): the weight matrix, which is
//            all of the HBM traffic, streams through the 128-row side at full tile efficiency while
//            the few activation rows ride along as the narrow N side.  Two forms of split-K, both through
//            float32 slabs in global memory (they stay in L2): `partials` leaves the slabs to the consumer
//            kernel, which sums them in a fixed order while it reads its input anyway (the cheapest form on
//            one GPU); `reduce` (M <= 64) sums them inside this kernel - every CTA holds one (tile, split),
//            all are resident at once, the splits of a tile wait for one another (bounded) and each then
//            sums one slice of the tile's rows in split order and applies the full epilogue (bias,
//            activation, gating, residual) to it.
//            (Two variants were built, measured and removed: the splits of a tile as a thread-block cluster
//            reducing through distributed shared memory - 5 us slower per launch, a cluster is only scheduled
//            once all its SMs are free and so loses the overlap with the previous kernel's tail - and, on top of
//            `reduce`, an epilogue that pushes the finished slice straight into the tensor-parallel peers'
//            exchange buffers - 9 us per launch against 8 us for the separate publishing kernel, whose many
//            small blocks read the slabs with far more parallelism than one CTA per tile slice can.)
// GATED computes act(X.Wg^T) * (X.Wu^T) with two accumulators per stage (qwen2.rs:100-103).
//
// Every barrier wait is bounded; a give-up is recorded in the context's status word and the CTA
// drains its in-flight copies, frees its TMEM and returns.
#include <stdlib.h>

#include <algorithm>
#include <vector>

#include "ctx.h"
#include "ptx.cuh"

namespace rb {

using bf16 = __nv_bfloat16;

namespace {

constexpr int kBM = 128;        // TMEM lanes per tile
constexpr int kBK = 64;         // K elements per stage (one 128-byte swizzle row)
constexpr int kThreads = 192;
constexpr int kSmemBudget = 200 * 1024;

template <int BN, bool SWAP, bool GATED>
struct Cfg {
  static constexpr int kPTiles = (GATED && SWAP) ? 2 : 1;
  static constexpr int kQTiles = (GATED && !SWAP) ? 2 : 1;
  static constexpr int kPBytes = kBM * kBK * 2;
  static constexpr int kQBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kPTiles * kPBytes + kQTiles * kQBytes;
  static constexpr int kStagesRaw = kSmemBudget / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kAcc = GATED ? 2 : 1;
  static constexpr int kAccCols = kAcc * BN;
  static constexpr int kNeedCols = 2 * kAccCols;
  static constexpr int kTmemCols = kNeedCols <= 32 ? 32 : kNeedCols <= 64 ? 64 : kNeedCols <= 128 ? 128
                                   : kNeedCols <= 256 ? 256 : 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;  // + alignment slack
  static_assert(kNeedCols <= 512, "accumulators exceed tensor memory");
  static_assert(kStages >= 2, "stage does not fit");
  static_assert(kQBytes % 1024 == 0, "Q tile must keep 1024-byte alignment");
};

struct Params {
  int m, n, k;          // C is [m, n]
  int p_rows, q_rows;   // rows of the P / Q operands (normal: m, n; swapped: n, m)
  int n_p, n_q;         // tiles along each
  int num_kb, kb_per_split, n_split;
  int n_items;
  const bf16* bias;
  const bf16* residual;
  bf16* out;
  float* part;
  int act;
  int stages;           // ring depth of this launch, 2..Cfg::kStages
  int reduce;           // split-K reduced inside the kernel: the splits of a tile wait for one another (see the epilogue)
  uint32_t* tile_count; // reduce: arrivals per tile, and readers done per tile; both self-resetting
  uint32_t* tile_done;
  long long wait_cycles;  // give-up budget of every bounded wait
  uint32_t* status;
};

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void decode_item(const Params& p, int item, bool swap, int& pt, int& qt, int& split) {
  if (swap) {
    split = item % p.n_split;
    const int tile = item / p.n_split;
    qt = tile % p.n_q;
    pt = tile / p.n_q;
  } else {
    split = 0;
    constexpr int G = 16;  // P tiles per raster group: concurrent CTAs share operand tiles in L2
    const int per_group = G * p.n_q;
    const int group = item / per_group;
    const int first = group * G;
    const int gsz = min(p.n_p - first, G);
    const int in_group = item % per_group;
    pt = first + in_group % gsz;
    qt = in_group / gsz;
  }
}

__device__ __forceinline__ uint4 pack8(const float* v) {
  uint4 r;
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]);
  __nv_bfloat162 b = __floats2bfloat162_rn(v[2], v[3]);
  __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]);
  __nv_bfloat162 d = __floats2bfloat162_rn(v[6], v[7]);
  r.x = *reinterpret_cast<uint32_t*>(&a);
  r.y = *reinterpret_cast<uint32_t*>(&b);
  r.z = *reinterpret_cast<uint32_t*>(&c);
  r.w = *reinterpret_cast<uint32_t*>(&d);
  return r;
}
__device__ __forceinline__ void unpack8(const uint4& u, float* v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

constexpr int kEpiPitch = kBM + 8;  // elements; keeps the 16-byte row reads of the staging tile conflict-free

// Barrier among the 128 epilogue threads only (hardware barrier 1; __syncthreads is barrier 0).
__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Activation over a register array with the selector hoisted out of the element loop
// (rai-core/src/hlops/activations.rs:20-32); fast-math forms, results are rounded to bf16 anyway.
template <int N>
__device__ __forceinline__ void act_inplace(int act, float (&v)[N]) {
  if (act == RB_ACT_SILU) {
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] = __fdividef(v[i], 1.0f + __expf(-v[i]));
  } else if (act == RB_ACT_GELU_TANH) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const float x = v[i];
      v[i] = 0.5f * x * (1.0f + tanh_fast(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    }
  } else if (act == RB_ACT_GELU_ERF) {
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] = v[i] * 0.5f * (1.0f + erff(v[i] * 0.7071067811865476f));
  } else if (act == RB_ACT_RELU) {
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] = fmaxf(v[i], 0.f);
  }
}

template <int BN, bool SWAP, bool GATED>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_p, const __grid_constant__ CUtensorMap tm_p2,
               const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_q2, const Params p) {
  using C = Cfg<BN, SWAP, GATED>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[C::kStages];
  __shared__ __align__(8) uint64_t empty_bar[C::kStages];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile uint32_t abort_flag;
  __shared__ uint32_t issued_count;  // stages the producer has handed to the copy engine
  __shared__ volatile uint32_t epi_ok[4];
  __shared__ __align__(16) bf16 epi_tile[32 * kEpiPitch];  // 32 output rows x 128 columns, padded

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_stages = p.stages;
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  if (threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) { ptx::mbar_init(&full_bar[s], 1); ptx::mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { ptx::mbar_init(&acc_full[a], 1); ptx::mbar_init(&acc_empty[a], 4); }
    abort_flag = 0;
    issued_count = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::tma_prefetch_desc(&tm_p);
    ptx::tma_prefetch_desc(&tm_q);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&tmem_base_slot, C::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  pdl_launch_dependents();
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // The weight operand does not depend on the kernel before this one: its first ring of
      // stages is requested right away, and only then does the producer wait for the predecessor
      // before it requests the matching activation tiles.  On a chain of decode-sized GEMMs this
      // hides the launch, set-up and pipeline-fill latency behind the previous kernel.
      // decode-sized GEMMs read every weight byte exactly once: evict-first keeps them from pushing
      // the activations and split-K partials out of L2
      const uint64_t stream_policy = ptx::policy_evict_first();
      auto load_weights = [&](uint8_t* st, int stage, int kb, int pt, int qt) {
        if (SWAP) {
          ptx::tma_load_2d_hint(st, &tm_p, &full_bar[stage], kb * kBK, pt * kBM, stream_policy);
          if (C::kPTiles == 2)
            ptx::tma_load_2d_hint(st + C::kPBytes, &tm_p2, &full_bar[stage], kb * kBK, pt * kBM, stream_policy);
        } else {
          uint8_t* qs = st + C::kPTiles * C::kPBytes;
          ptx::tma_load_2d(qs, &tm_q, &full_bar[stage], kb * kBK, qt * BN);
          if (C::kQTiles == 2) ptx::tma_load_2d(qs + C::kQBytes, &tm_q2, &full_bar[stage], kb * kBK, qt * BN);
        }
      };
      auto load_activations = [&](uint8_t* st, int stage, int kb, int pt, int qt) {
        if (SWAP) ptx::tma_load_2d(st + C::kPTiles * C::kPBytes, &tm_q, &full_bar[stage], kb * kBK, qt * BN);
        else ptx::tma_load_2d(st, &tm_p, &full_bar[stage], kb * kBK, pt * kBM);
      };
      int n_pre = 0;
      for (int item = blockIdx.x; item < p.n_items && n_pre < n_stages; item += gridDim.x) {
        int pt, qt, split;
        decode_item(p, item, SWAP, pt, qt, split);
        const int kb0 = split * p.kb_per_split, kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1 && n_pre < n_stages; ++kb, ++n_pre) {
          ptx::mbar_expect_tx(&full_bar[n_pre], C::kStageBytes);
          load_weights(tiles + (size_t)n_pre * C::kStageBytes, n_pre, kb, pt, qt);
        }
      }
      pdl_wait();
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x) {
        int pt, qt, split;
        decode_item(p, item, SWAP, pt, qt, split);
        const int kb0 = split * p.kb_per_split, kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          uint8_t* st = tiles + (size_t)stage * C::kStageBytes;
          if ((int)issued >= n_pre) {
            if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1u, &abort_flag, p.wait_cycles)) { ok = false; break; }
            ptx::mbar_expect_tx(&full_bar[stage], C::kStageBytes);
            load_weights(st, stage, kb, pt, qt);
          }
          load_activations(st, stage, kb, pt, qt);
          ++issued;
          if (++stage == n_stages) { stage = 0; phase ^= 1u; }
        }
      }
      issued_count = issued;
      if (!ok) { p.status[0] = (uint32_t)(-RB_ERR_TIMEOUT); p.status[1] = 0x6E01u; p.status[2] = blockIdx.x; }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::umma_idesc_bf16(kBM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int as = 0;
      uint32_t aphase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x) {
        int pt, qt, split;
        decode_item(p, item, SWAP, pt, qt, split);
        const int kb0 = split * p.kb_per_split, kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        if (kb0 >= kb1) continue;  // empty split: the epilogue writes zeros on its own
        if (!ptx::mbar_wait(&acc_empty[as], aphase ^ 1u, &abort_flag, p.wait_cycles)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t d0 = tmem_base + (uint32_t)(as * C::kAccCols);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!ptx::mbar_wait(&full_bar[stage], phase, &abort_flag, p.wait_cycles)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t st = ptx::smem_u32(tiles + (size_t)stage * C::kStageBytes);
          const uint32_t p0 = st, p1 = st + (C::kPTiles == 2 ? C::kPBytes : 0);
          const uint32_t q0 = st + C::kPTiles * C::kPBytes, q1 = q0 + (C::kQTiles == 2 ? C::kQBytes : 0);
#pragma unroll
          for (int j = 0; j < kBK / 16; ++j) {
            const uint32_t acc = (kb > kb0 || j > 0) ? 1u : 0u;
            ptx::umma_bf16(d0, ptx::umma_desc_k_sw128(p0 + j * 32), ptx::umma_desc_k_sw128(q0 + j * 32), idesc, acc);
            if (GATED)
              ptx::umma_bf16(d0 + BN, ptx::umma_desc_k_sw128(p1 + j * 32), ptx::umma_desc_k_sw128(q1 + j * 32), idesc,
                             acc);
          }
          ptx::umma_commit(&empty_bar[stage]);  // the stage is free once these MMAs have read it
          if (++stage == n_stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        ptx::umma_commit(&acc_full[as]);
        if (++as == 2) { as = 0; aphase ^= 1u; }
      }
      if (!ok) { p.status[0] = (uint32_t)(-RB_ERR_TIMEOUT); p.status[1] = 0x6E02u; p.status[2] = blockIdx.x; }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    pdl_wait();  // bias/residual reads and every store below must follow the predecessor's completion
    const int quarter = warp & 3;              // the 32 TMEM lanes this warp may read
    const int lane_row = quarter * 32 + lane;  // row of the P operand inside the tile
    int as = 0;
    uint32_t aphase = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x) {
      int pt, qt, split;
      decode_item(p, item, SWAP, pt, qt, split);
      if (split * p.kb_per_split >= p.num_kb) {  // empty split (only with partials): zero slab, no accumulator
        const int gn = pt * kBM + lane_row;
        if (p.part && gn < p.n)
          for (int gm = qt * BN; gm < min(p.m, (qt + 1) * BN); ++gm) p.part[((size_t)split * p.m + gm) * p.n + gn] = 0.f;
        continue;
      }
      // The four epilogue warps meet at named barriers below, so they must agree on giving up.
      const bool mine = ptx::mbar_wait(&acc_full[as], aphase, &abort_flag, p.wait_cycles);
      if (lane == 0) epi_ok[warp - 2] = mine ? 1u : 0u;
      epi_barrier();
      const bool all_ok = (epi_ok[0] & epi_ok[1] & epi_ok[2] & epi_ok[3]) != 0u;
      epi_barrier();
      if (!all_ok) { ok = false; break; }
      ptx::tc_fence_after();
      const uint32_t t0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(as * C::kAccCols);
      constexpr int CH = BN >= 32 ? 32 : 16;  // columns per TMEM load
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += CH) {
        float v[CH], g[GATED ? CH : 1];
        {
          uint32_t r[CH];
          if (CH == 32) ptx::tmem_ld_32x32(t0 + c0, reinterpret_cast<uint32_t(&)[32]>(r));
          else ptx::tmem_ld_32x16(t0 + c0, reinterpret_cast<uint32_t(&)[16]>(r));
          ptx::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < CH; ++j) v[j] = __uint_as_float(r[j]);
          if (GATED) {
            if (CH == 32) ptx::tmem_ld_32x32(t0 + BN + c0, reinterpret_cast<uint32_t(&)[32]>(r));
            else ptx::tmem_ld_32x16(t0 + BN + c0, reinterpret_cast<uint32_t(&)[16]>(r));
            ptx::tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < CH; ++j) { g[j] = v[j]; v[j] = __uint_as_float(r[j]); }
          }
        }
        // here: GATED ? (g = gate product, v = up product) : (v = product)
        if (SWAP && p.reduce) {
          // this CTA's share of the K range as a float32 slab tile in global memory (it stays in L2); the gated
          // form keeps two sets of slabs, gate products first
          const int gn = pt * kBM + lane_row;
          if (gn < p.n) {
            const size_t set = (size_t)p.n_split * p.m * p.n;
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              const int gm = qt * BN + c0 + j;
              if (gm < p.m) {
                const size_t at = ((size_t)split * p.m + gm) * p.n + gn;
                if (GATED) { p.part[at] = g[j]; p.part[set + at] = v[j]; }
                else p.part[at] = v[j];
              }
            }
          }
        } else if (SWAP) {
          const int gn = pt * kBM + lane_row;  // output column = weight row
          if (p.part) {
            if (gn < p.n) {
#pragma unroll
              for (int j = 0; j < CH; ++j) {
                const int gm = qt * BN + c0 + j;
                if (gm < p.m) p.part[((size_t)split * p.m + gm) * p.n + gn] = v[j];
              }
            }
          } else {
            if (GATED) {
              act_inplace(p.act, g);
#pragma unroll
              for (int j = 0; j < CH; ++j) v[j] *= g[j];
            } else {
              const float bias = (p.bias && gn < p.n) ? __bfloat162float(p.bias[gn]) : 0.f;
#pragma unroll
              for (int j = 0; j < CH; ++j) v[j] += bias;
              act_inplace(p.act, v);
            }
            // The accumulator holds the tile transposed (lane = output column).  Turn it through
            // shared memory so that the global stores are 16-byte pieces of output rows.
#pragma unroll
            for (int j = 0; j < CH; ++j) epi_tile[j * kEpiPitch + lane_row] = __float2bfloat16_rn(v[j]);
            epi_barrier();
            const int et = threadIdx.x - 64;
            const bool vec_ok = (p.n % 8) == 0;
            for (int id = et; id < CH * (kBM / 8); id += 128) {
              const int j = id / (kBM / 8), c8 = (id % (kBM / 8)) * 8;
              const int gm = qt * BN + c0 + j, gn8 = pt * kBM + c8;
              if (gm >= p.m || gn8 >= p.n) continue;
              uint4 u = *reinterpret_cast<const uint4*>(epi_tile + j * kEpiPitch + c8);
              bf16* dst = p.out + (size_t)gm * p.n + gn8;
              if (vec_ok) {
                if (!GATED && p.residual) {
                  float a8[8], r8[8];
                  unpack8(u, a8);
                  unpack8(*reinterpret_cast<const uint4*>(p.residual + (size_t)gm * p.n + gn8), r8);
#pragma unroll
                  for (int i = 0; i < 8; ++i) a8[i] += r8[i];
                  u = pack8(a8);
                }
                *reinterpret_cast<uint4*>(dst) = u;
              } else {
                const bf16* e = reinterpret_cast<const bf16*>(&u);
                for (int i = 0; i < 8 && gn8 + i < p.n; ++i) {
                  float y = __bfloat162float(e[i]);
                  if (!GATED && p.residual) y += __bfloat162float(p.residual[(size_t)gm * p.n + gn8 + i]);
                  dst[i] = __float2bfloat16_rn(y);
                }
              }
            }
            epi_barrier();  // the staging tile is rewritten by the next chunk
          }
        } else {
          const int gm = pt * kBM + lane_row;
          const int gn0 = qt * BN + c0;
          if (GATED) act_inplace(p.act, g);
          if (gm < p.m) {
            const bool vec_ok = (p.n % 8) == 0;
#pragma unroll
            for (int j8 = 0; j8 < CH; j8 += 8) {
              const int gn = gn0 + j8;
              if (gn >= p.n) break;
              float y[8];
              if (GATED) {
#pragma unroll
                for (int j = 0; j < 8; ++j) y[j] = g[j8 + j] * v[j8 + j];  // g already holds act(gate)
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) y[j] = v[j8 + j];
                if (p.bias) {
                  if (vec_ok) {
                    float b8[8];
                    unpack8(*reinterpret_cast<const uint4*>(p.bias + gn), b8);
#pragma unroll
                    for (int j = 0; j < 8; ++j) y[j] += b8[j];
                  } else {
                    for (int j = 0; j < 8 && gn + j < p.n; ++j) y[j] += __bfloat162float(p.bias[gn + j]);
                  }
                }
                act_inplace(p.act, y);
                if (p.residual) {
                  if (vec_ok) {
                    float r8[8];
                    unpack8(*reinterpret_cast<const uint4*>(p.residual + (size_t)gm * p.n + gn), r8);
#pragma unroll
                    for (int j = 0; j < 8; ++j) y[j] += r8[j];
                  } else {
                    for (int j = 0; j < 8 && gn + j < p.n; ++j)
                      y[j] += __bfloat162float(p.residual[(size_t)gm * p.n + gn + j]);
                  }
                }
              }
              if (vec_ok) {
                *reinterpret_cast<uint4*>(p.out + (size_t)gm * p.n + gn) = pack8(y);
              } else {
                for (int j = 0; j < 8 && gn + j < p.n; ++j) p.out[(size_t)gm * p.n + gn + j] = __float2bfloat16_rn(y[j]);
              }
            }
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&acc_empty[as]);
      if (++as == 2) { as = 0; aphase ^= 1u; }
    }
    if (!ok && lane == 0) { p.status[0] = (uint32_t)(-RB_ERR_TIMEOUT); p.status[1] = 0x6E03u; p.status[2] = blockIdx.x; }
    if (SWAP && p.reduce) {
      // -------------------------------------------------------------- split-K reduction inside the kernel
      // Every CTA holds exactly one (tile, split) and all of them are resident at once (the grid is at most one
      // CTA per SM), so the splits of a tile can wait for one another: each counts itself in when its slab tile
      // is written, waits (bounded) until all `n_split` have, and then sums ONE slice of the tile's rows out of all
      // slabs - in split order, so the result does not depend on who finished first - and applies the full
      // epilogue to that slice.  The last one to finish reading re-arms the tile's counters for the next launch.
      const int et = threadIdx.x - 64;
      int pt, qt, split;
      decode_item(p, blockIdx.x, true, pt, qt, split);
      const int tile = pt * p.n_q + qt;
      const int ns = p.n_split;
      epi_barrier();  // the epilogue threads' slab stores precede thread 0's fence
      if (et == 0) {
        bool arrived_all = ok;
        if (ok) {
          __threadfence();
          atomicAdd(p.tile_count + tile, 1u);
          const long long t0 = clock64();
          while (ld_acquire_gpu(p.tile_count + tile) < (uint32_t)ns) {
            if (clock64() - t0 > p.wait_cycles) { arrived_all = false; break; }
          }
          if (!arrived_all) { p.status[0] = (uint32_t)(-RB_ERR_TIMEOUT); p.status[1] = 0x6E04u; p.status[2] = blockIdx.x; p.status[3] = (uint32_t)tile; }
        }
        epi_ok[0] = arrived_all ? 1u : 0u;
      }
      epi_barrier();
      if (epi_ok[0]) {
        const int m_eff = min(BN, p.m - qt * BN);
        const int per = (m_eff + ns - 1) / ns;
        const int j0 = min(m_eff, split * per), j1 = min(m_eff, j0 + per);
        const int gn = pt * kBM + lane_row;
        const bool col_ok = gn < p.n;
        const float bias = (!GATED && p.bias && col_ok) ? __bfloat162float(p.bias[gn]) : 0.f;
        const size_t slab = (size_t)p.m * p.n, set = (size_t)ns * slab;
        for (int jc = j0; jc < j1; jc += 32) {
          const int jc1 = min(j1, jc + 32);
          for (int j = jc; j < jc1; j += 4) {
            float a[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
            if (col_ok) {
              float ta[8][4], tu[GATED ? 8 : 1][4];
#pragma unroll
              for (int q = 0; q < 8; ++q)  // every load of this group is in flight before the first sum needs one
                if (q < ns) {
#pragma unroll
                  for (int i = 0; i < 4; ++i)
                    if (j + i < jc1) {
                      const size_t at = (size_t)q * slab + (size_t)(qt * BN + j + i) * p.n + gn;
                      ta[q][i] = __ldcg(p.part + at);
                      if (GATED) tu[q][i] = __ldcg(p.part + set + at);
                    }
                }
#pragma unroll
              for (int q = 0; q < 8; ++q)  // split order
                if (q < ns) {
#pragma unroll
                  for (int i = 0; i < 4; ++i)
                    if (j + i < jc1) { a[i] += ta[q][i]; if (GATED) u[i] += tu[q][i]; }
                }
            }
            if (GATED) {
              act_inplace(p.act, a);
#pragma unroll
              for (int i = 0; i < 4; ++i) a[i] *= u[i];
            } else {
#pragma unroll
              for (int i = 0; i < 4; ++i) a[i] += bias;
              act_inplace(p.act, a);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (j + i < jc1) epi_tile[(j + i - jc) * kEpiPitch + lane_row] = __float2bfloat16_rn(a[i]);
          }
          epi_barrier();
          // 16-byte pieces of output rows: residual, then the store
          for (int id = et; id < (jc1 - jc) * (kBM / 8); id += 128) {
            const int jj = id / (kBM / 8), c8 = (id % (kBM / 8)) * 8;
            const int gm = qt * BN + jc + jj, gn8 = pt * kBM + c8;
            if (gn8 >= p.n) continue;
            uint4 o = *reinterpret_cast<const uint4*>(epi_tile + jj * kEpiPitch + c8);
            const size_t at = (size_t)gm * p.n + gn8;
            if (!GATED && p.residual) {
              float a8[8], r8[8];
              unpack8(o, a8);
              unpack8(*reinterpret_cast<const uint4*>(p.residual + at), r8);
#pragma unroll
              for (int i = 0; i < 8; ++i) a8[i] += r8[i];
              o = pack8(a8);
            }
            *reinterpret_cast<uint4*>(p.out + at) = o;
          }
          epi_barrier();  // the staging rows are rewritten by the next chunk
        }
        if (et == 0) {
          // this CTA has read what it needs of the tile's slabs: the last reader re-arms the counters
          if (atomicAdd(p.tile_done + tile, 1u) == (uint32_t)ns - 1u) { p.tile_count[tile] = 0u; p.tile_done[tile] = 0u; }
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before();
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) {
    // Give copies that were already handed to the copy engine a bounded chance to land before the
    // shared memory is released: each full barrier completes when its bytes have arrived.
    volatile uint32_t never = 0;
    const uint32_t issued = issued_count;
    const uint32_t ns = (uint32_t)n_stages;
    for (uint32_t i = (issued > ns ? issued - ns : 0); i < issued; ++i)
      ptx::mbar_wait(&full_bar[i % ns], (i / ns) & 1u, &never, p.wait_cycles);
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

template <int BN, bool SWAP, bool GATED>
int launch(rb_ctx* ctx, const GemmArgs& a, Params& p, int want_split = 0) {
  using C = Cfg<BN, SWAP, GATED>;
  const void* pbase = SWAP ? a.w : a.x;
  const void* p2base = SWAP ? a.w2 : a.x;
  const void* qbase = SWAP ? a.x : a.w;
  const void* q2base = SWAP ? a.x : a.w2;
  CUtensorMap tp, tp2, tq, tq2;
  RB_TRY(tmap_2d_bf16(ctx, pbase, p.p_rows, a.k, a.k, kBM, &tp));
  RB_TRY(tmap_2d_bf16(ctx, (GATED && SWAP) ? p2base : pbase, p.p_rows, a.k, a.k, kBM, &tp2));
  RB_TRY(tmap_2d_bf16(ctx, qbase, p.q_rows, a.k, a.k, BN, &tq));
  RB_TRY(tmap_2d_bf16(ctx, (GATED && !SWAP) ? q2base : qbase, p.q_rows, a.k, a.k, BN, &tq2));
  p.n_p = (p.p_rows + kBM - 1) / kBM;
  p.n_q = (p.q_rows + BN - 1) / BN;
  auto kern = gemm_tc_kernel<BN, SWAP, GATED>;
  static bool attr_set[64] = {};  // the attribute belongs to the (kernel, device) pair
  const int dv = ctx->device & 63;
  if (!attr_set[dv]) {
    RB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    attr_set[dv] = true;
  }
  // Ring depth: as deep as the shared-memory budget allows (decode-sized launches are bound by the bytes they
  // keep in flight; a shallower ring measured slower even where it lets two kernels share an SM).
  int stages = C::kStages;
  if (SWAP) stages = std::max(2, std::min(C::kStages, (int)(ctx->gemm_ring_bytes / C::kStageBytes)));
  p.stages = stages;
  const size_t smem = (size_t)stages * C::kStageBytes + 1024;
  p.wait_cycles = ctx->local_wait_cycles();

  if (SWAP && want_split >= 1) {
    // Split-K reduced inside the kernel: one CTA per (tile, split), all resident at once.
    const int tiles = p.n_p * p.n_q;
    int s = std::min(want_split, 8);
    for (; s > 1; --s) {
      const int per = (p.num_kb + s - 1) / s;
      if ((p.num_kb + per - 1) / per == s) break;  // no split may be left without K blocks
    }
    p.n_split = s;
    p.kb_per_split = (p.num_kb + s - 1) / s;
    p.reduce = 1;
    p.n_items = tiles * s;
    if (p.n_items > ctx->sm_count || tiles > kGemmMaxReduceTiles)
      return fail(RB_ERR_INVALID, "GEMM: %d tiles x %d splits exceed one CTA per SM", tiles, s);
    RB_TRY(gemm_reserve_scratch(ctx, (size_t)(GATED ? 2 : 1) * s * p.m * p.n * sizeof(float)));
    p.part = ctx->gemm_scratch;
    p.tile_count = ctx->gemm_tile_count;
    p.tile_done = ctx->gemm_tile_count + kGemmMaxReduceTiles;
    RB_CUDA(launch_kernel(kern, dim3((unsigned)p.n_items), dim3(kThreads), smem, ctx->stream, ctx->pdl, tp, tp2, tq, tq2, p));
    ctx->launches++;
    return RB_OK;
  }
  p.n_items = p.n_p * p.n_q * p.n_split;
  const int grid = std::min(p.n_items, ctx->sm_count);
  RB_CUDA(launch_kernel(kern, dim3((unsigned)grid), dim3(kThreads), smem, ctx->stream, ctx->pdl, tp, tp2, tq, tq2, p));
  ctx->launches++;
  return RB_OK;
}

}  // namespace

// The map is copied into the caller's storage: the cache may evict entries at any call.
int tmap_2d_bf16(rb_ctx* ctx, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows, CUtensorMap* out) {
  auto key = std::make_tuple(base, rows, cols, ld, box_rows);
  auto it = ctx->tmaps.find(key);
  if (it != ctx->tmaps.end()) { *out = it->second; return RB_OK; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(RB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15))
    return fail(RB_ERR_INVALID, "GEMM operand must be 16-byte aligned with a row pitch that is a multiple of 16 bytes");
  CUtensorMap tm;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(RB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  if (ctx->tmaps.size() >= (size_t)ctx->tmap_cache_limit) ctx->tmaps.clear();
  ctx->tmaps.emplace(key, tm);
  *out = tm;
  return RB_OK;
}

// How many ways to split K for a decode-sized launch that would otherwise leave most SMs idle (1 = do not split).
int gemm_reserve_scratch(rb_ctx* ctx, size_t bytes);

int gemm_tc_pick_splits(rb_ctx* ctx, int64_t m, int64_t n, int64_t k) {
  if (m > 256) return 1;
  const int64_t bn = m <= 16 ? 16 : m <= 64 ? 64 : m <= 128 ? 128 : 256;
  const int64_t tiles = ((n + kBM - 1) / kBM) * ((m + bn - 1) / bn);
  const int64_t num_kb = (k + kBK - 1) / kBK;
  if (tiles * 4 >= (int64_t)ctx->sm_count * 3) return 1;
  int64_t s = ctx->sm_count / tiles;
  s = std::min<int64_t>(s, 16);
  s = std::min<int64_t>(s, std::max<int64_t>(1, num_kb / 4));
  if (s <= 1) return 1;
  const int64_t per = (num_kb + s - 1) / s;
  return (int)((num_kb + per - 1) / per);
}

// Splits of a launch that reduces split-K inside the kernel: enough to fill the SMs, at most 8, at least two K
// blocks each.  0 = this launch does not take that form.  On one GPU the consumer-side reduction (`partials`) is
// cheaper, so the form is used only where the caller asks for the whole epilogue in one launch (`reduce`).
static int reduce_splits(rb_ctx* ctx, const GemmArgs& a, int num_kb, bool gated) {
  if (!a.reduce || a.partials || a.m > 64 || (a.n % 8) != 0) return 0;
  const int64_t tiles = (a.n + kBM - 1) / kBM;  // M <= 64: one tile along the rows
  if (tiles > ctx->sm_count || tiles > kGemmMaxReduceTiles) return 0;
  int64_t s = std::min<int64_t>(8, ctx->sm_count / tiles);
  s = std::min<int64_t>(s, std::max<int64_t>(1, num_kb / 2));
  if (tiles * 4 >= (int64_t)ctx->sm_count * 3 || s <= 1) return 0;
  return (int)s;
}

// Float32 slab space of the in-kernel reduction, grow-only like the attention scratch (captured graphs name it).
int gemm_reserve_scratch(rb_ctx* ctx, size_t bytes) {
  if (ctx->gemm_scratch_bytes >= bytes) return RB_OK;
  float* fresh = nullptr;
  RB_CUDA(cudaMalloc(&fresh, bytes));
  if (ctx->gemm_scratch) ctx->retired.push_back(ctx->gemm_scratch);
  ctx->gemm_scratch = fresh;
  ctx->gemm_scratch_bytes = bytes;
  return RB_OK;
}

int gemm_tc_bf16(rb_ctx* ctx, const GemmArgs& a) {
  if (a.m == 0 || a.n == 0) return RB_OK;
  RB_REQUIRE(a.k > 0 && (a.k % 8) == 0, "GEMM: K = %lld must be a positive multiple of 8", (long long)a.k);
  const bool gated = a.w2 != nullptr;
  RB_REQUIRE(!(gated && a.partials), "GEMM: split-K partials are not available for the gated form");
  Params p{};
  p.m = (int)a.m; p.n = (int)a.n; p.k = (int)a.k;
  p.num_kb = (int)((a.k + kBK - 1) / kBK);
  p.n_split = 1;
  p.kb_per_split = p.num_kb;
  p.bias = (const bf16*)a.bias;
  p.residual = (const bf16*)a.residual;
  p.out = a.partials ? nullptr : (bf16*)a.out;
  p.part = a.partials ? (float*)a.out : nullptr;
  p.act = a.act;
  p.status = ctx->status_dev;
  const bool swap = a.m <= 256 && !(gated && a.m > 128);
  if (a.partials) {
    RB_REQUIRE(swap, "GEMM: split-K partials need M <= 256");
    const int s = std::max(1, a.n_split);
    p.kb_per_split = (p.num_kb + s - 1) / s;
    p.n_split = s;
  }
  const int rs = swap ? reduce_splits(ctx, a, p.num_kb, gated) : 0;
  if (swap) {
    p.p_rows = (int)a.n; p.q_rows = (int)a.m;
    if (gated) {
      if (a.m <= 16) return launch<16, true, true>(ctx, a, p, rs);
      if (a.m <= 64) return launch<64, true, true>(ctx, a, p, rs);
      return launch<128, true, true>(ctx, a, p);
    }
    if (a.m <= 16) return launch<16, true, false>(ctx, a, p, rs);
    if (a.m <= 64) return launch<64, true, false>(ctx, a, p, rs);
    if (a.m <= 128) return launch<128, true, false>(ctx, a, p);
    return launch<256, true, false>(ctx, a, p);
  }
  p.p_rows = (int)a.m; p.q_rows = (int)a.n;
  if (gated) return launch<128, false, true>(ctx, a, p);
  return launch<256, false, false>(ctx, a, p);
}

}  // namespace rb
