// Causal prefill attention on the 5th-generation tensor cores, for head sizes 64 and 128 and query lengths of at
// least one tile: softmax(Q K^T * scale + mask) V over the paged bf16 KV cache without materialising scores
// (rai-models/src/llm/qwen2.rs:205-216 and its phi3 / gemma twins; the fused op the reference itself has for this
// is ops::FlashAttention, rai-core/src/ops/flash_attention.rs:154-176).
//
// One CTA = 128 query rows of one (sequence, query head); it walks the causal range of 64-key tiles (a cache page is
// one tile).  Six warps with fixed roles, the same division of labour as the GEMM:
//   warp 0     TMA producer: the Q tile once, then K and V tiles through two 2-deep rings (K is released as soon as
//              its scores are done, V after P.V, so the next K is on its way while the softmax runs);
//   warp 1     owns the TMEM allocation; one lane issues tcgen05.mma: S = Q.K^T (M 128, N 64, K head_dim) into one of
//              two score buffers in tensor memory, and O += P.V (M 128, N head_dim, K 64) with V read straight from
//              its [keys][head_dim] tile as an MN-major operand - no transposed copy of V anywhere;
//   warps 2-5  softmax: each thread owns one query row (its TMEM lane), so row max and row sum need no shuffles.
//              tcgen05.ld the scores, scale + mask, online softmax in float32, P rounded to bf16 into shared memory in
//              the swizzled K-major layout the MMA reads.  O stays in tensor memory for the whole walk; the reference
//              point of the exponentials follows the running max lazily (it moves only when the max has grown by more
//              than 2^8), so the in-place rescaling of O (tcgen05.ld / multiply / tcgen05.st) runs a handful of times
//              per walk.  At the end O / l goes out as bf16 rows.
// The score MMA of tile j+1 is issued before the P.V MMA of tile j, so the tensor pipe computes the next scores while
// the softmax warps work on the current ones; two CTAs fit per SM (112 KB of shared memory, 256 TMEM columns
// each), which overlaps one CTA's softmax with the other's MMAs.
//
// Every wait is bounded; a give-up is recorded in the context's status word, in-flight copies are drained, the TMEM
// allocation is freed and the CTA returns without writing output.
#include <stdlib.h>

#include <algorithm>

#include "ctx.h"
#include "ptx.cuh"

namespace rb {

using bf16 = __nv_bfloat16;

namespace {

constexpr int kBM = 128;  // query rows per CTA = TMEM lanes
constexpr int kBN = 64;   // keys per tile = tokens per cache page
constexpr int kThreads = 192;
constexpr float kLog2e = 1.4426950408889634f;

template <int D>
struct TCfg {
  static constexpr int kQBytes = kBM * D * 2;   // [D/64 column blocks][128 rows][128 bytes]
  static constexpr int kKBytes = kBN * D * 2;   // [D/64][64 keys][128 bytes]
  static constexpr int kVBytes = kBN * D * 2;
  static constexpr int kPBytes = kBM * kBN * 2;  // [128 rows][128 bytes]
  static constexpr int kTileBytes = kQBytes + 2 * kKBytes + 2 * kVBytes + kPBytes;
  static constexpr int kBarBytes = 256;          // barriers and control words, after the tiles
  // at least 100 KB, so that never more than two CTAs (256 TMEM columns each) share an SM
  static constexpr int kSmemBytes = (kTileBytes + kBarBytes) > 100 * 1024 ? (kTileBytes + kBarBytes) : 100 * 1024;
  static constexpr int kTmemCols = 256;          // two score buffers of 64 columns, then O (head_dim columns)
  static constexpr uint32_t kOCol = 2 * kBN;
};

// 2^x by the special-function unit (2 ulp; -inf gives +0, which is what a masked score must contribute)
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct TParams {
  const int32_t* block_table;
  const int32_t* seq_lens;
  int pages_per_seq, s_new, q_heads, kv_heads, group, window;
  float scale_log2;
  bf16* out;
  uint32_t* status;
  long long wait_cycles;
#ifdef RB_DEBUG_AIDS
  unsigned long long* trace;  // developer build: cycles per phase of one softmax thread (see launch_tc)
#endif
};

#ifdef RB_DEBUG_AIDS
#define RB_TICK(slot) do { if (tracing) { const long long _t = clock64(); tr[slot] += (unsigned long long)(_t - t_prev); t_prev = _t; } } while (0)
#else
#define RB_TICK(slot) do { } while (0)
#endif

struct Ctrl {  // lives in dynamic shared memory behind the tiles
  uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_empty[2], p_full, o_done;
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t k_issued, v_issued;
};
static_assert(sizeof(Ctrl) <= 256, "control block exceeds its reservation");

template <int D>
__global__ void __launch_bounds__(kThreads, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                            const __grid_constant__ CUtensorMap tm_v, const TParams p) {
  using C = TCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + C::kQBytes;
  uint8_t* v_s = k_s + 2 * C::kKBytes;
  uint8_t* p_s = v_s + 2 * C::kVBytes;
  Ctrl* ctl = reinterpret_cast<Ctrl*>(p_s + C::kPBytes);
  volatile uint32_t* abort_flag = &ctl->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    ptx::mbar_init(&ctl->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&ctl->k_full[i], 1); ptx::mbar_init(&ctl->k_empty[i], 1);
      ptx::mbar_init(&ctl->v_full[i], 1); ptx::mbar_init(&ctl->v_empty[i], 1);
      ptx::mbar_init(&ctl->s_full[i], 1); ptx::mbar_init(&ctl->s_empty[i], 4);
    }
    ptx::mbar_init(&ctl->p_full, 4);
    ptx::mbar_init(&ctl->o_done, 1);
    ctl->abort_flag = 0;
    ctl->k_issued = ctl->v_issued = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::tma_prefetch_desc(&tm_q);
    ptx::tma_prefetch_desc(&tm_k);
    ptx::tma_prefetch_desc(&tm_v);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&ctl->tmem_base, C::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  pdl_launch_dependents();
  pdl_wait();  // q and the newest K/V rows come from the kernel before this one

  const int q0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * kBM;  // longest causal ranges first
  const int head = blockIdx.y, b = blockIdx.z, kvh = head / p.group;
  const int len = p.seq_lens[b];
  const int base = len - p.s_new;  // absolute position of query row 0
  // Key tiles this CTA walks.  The window term acts among the tokens of one call only (qwen2.rs:316-334), so whole
  // tiles can be skipped only when nothing is cached.
  const int tile_lo = base == 0 ? max(0, q0 - p.window) / kBN : 0;
  const int tile_hi = (min(base + q0 + kBM, len) + kBN - 1) / kBN;
  const int n = tile_hi - tile_lo;
  // The tiles must sit on a 1024-byte boundary (swizzle atoms); nothing else lives in shared memory before them.
  const bool layout_ok = (ptx::smem_u32(smem) & 1023u) == 0u && n >= 1;
  if (!layout_ok && threadIdx.x == 0) { p.status[0] = (uint32_t)(-RB_ERR_CUDA); p.status[1] = 0xA7C0u; p.status[2] = blockIdx.x; }

  if (layout_ok && warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      ptx::mbar_expect_tx(&ctl->q_full, C::kQBytes);
#pragma unroll
      for (int cb = 0; cb < D / 64; ++cb)
        ptx::tma_load_2d(q_s + cb * (kBM * 128), &tm_q, &ctl->q_full, head * D + cb * 64, b * p.s_new + q0);
      bool ok = true;
      for (int j = 0; j < n && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        const int page = p.block_table[(size_t)b * p.pages_per_seq + tile_lo + j];
        const int y = (page * p.kv_heads + kvh) * kBN;  // first row of this (page, KV head) in the layer
        if (!ptx::mbar_wait(&ctl->k_empty[st], ph ^ 1u, abort_flag, p.wait_cycles)) { ok = false; break; }
        ptx::mbar_expect_tx(&ctl->k_full[st], C::kKBytes);
#pragma unroll
        for (int cb = 0; cb < D / 64; ++cb)
          ptx::tma_load_2d(k_s + st * C::kKBytes + cb * (kBN * 128), &tm_k, &ctl->k_full[st], cb * 64, y);
        ctl->k_issued = (uint32_t)(j + 1);
        if (!ptx::mbar_wait(&ctl->v_empty[st], ph ^ 1u, abort_flag, p.wait_cycles)) { ok = false; break; }
        ptx::mbar_expect_tx(&ctl->v_full[st], C::kVBytes);
#pragma unroll
        for (int cb = 0; cb < D / 64; ++cb)
          ptx::tma_load_2d(v_s + st * C::kVBytes + cb * (kBN * 128), &tm_v, &ctl->v_full[st], cb * 64, y);
        ctl->v_issued = (uint32_t)(j + 1);
      }
      if (!ok) { p.status[0] = (uint32_t)(-RB_ERR_TIMEOUT); p.status[1] = 0xA7C1u; p.status[2] = blockIdx.x; p.status[3] = blockIdx.z; }
    }
  } else if (layout_ok && warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = ptx::umma_idesc_bf16(kBM, kBN);
      constexpr uint32_t idesc_o = ptx::umma_idesc_bf16(kBM, D, false, true);  // B = V, MN-major
      const uint32_t qa = ptx::smem_u32(q_s), ka = ptx::smem_u32(k_s), va = ptx::smem_u32(v_s), pa = ptx::smem_u32(p_s);
      bool ok = ptx::mbar_wait(&ctl->q_full, 0u, abort_flag, p.wait_cycles);
      auto issue_scores = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        if (!ptx::mbar_wait(&ctl->k_full[st], ph, abort_flag, p.wait_cycles)) return false;
        if (!ptx::mbar_wait(&ctl->s_empty[st], ph ^ 1u, abort_flag, p.wait_cycles)) return false;
        ptx::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t a = qa + (kk >> 2) * (kBM * 128) + (kk & 3) * 32;
          const uint32_t bb = ka + st * C::kKBytes + (kk >> 2) * (kBN * 128) + (kk & 3) * 32;
          ptx::umma_bf16(tmem_base + (uint32_t)(st * kBN), ptx::umma_desc_k_sw128(a), ptx::umma_desc_k_sw128(bb), idesc_s,
                         kk > 0 ? 1u : 0u);
        }
        ptx::umma_commit(&ctl->s_full[st]);
        ptx::umma_commit(&ctl->k_empty[st]);
        return true;
      };
      if (ok) ok = issue_scores(0);
      for (int j = 0; j < n && ok; ++j) {
        if (j + 1 < n && !issue_scores(j + 1)) { ok = false; break; }
        const int st = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        if (!ptx::mbar_wait(&ctl->v_full[st], ph, abort_flag, p.wait_cycles)) { ok = false; break; }
        if (!ptx::mbar_wait(&ctl->p_full, (uint32_t)j & 1u, abort_flag, p.wait_cycles)) { ok = false; break; }
        ptx::tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < kBN / 16; ++ks) {
          // A = P: K-major, 16 keys = 32 bytes further along the 128-byte row.  B = V: MN-major, 16 keys = 16 rows of
          // 128 bytes further; the second 64 columns of head_dim follow one [64 keys][128 B] block later.
          const uint64_t da = ptx::umma_desc_k_sw128(pa + ks * 32);
          const uint64_t db = ptx::umma_desc_mn_sw128(va + st * C::kVBytes + ks * (16 * 128), kBN * 128, 1024);
          ptx::umma_bf16(tmem_base + C::kOCol, da, db, idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
        }
        ptx::umma_commit(&ctl->o_done);
        ptx::umma_commit(&ctl->v_empty[st]);
      }
      if (!ok) { p.status[0] = (uint32_t)(-RB_ERR_TIMEOUT); p.status[1] = 0xA7C2u; p.status[2] = blockIdx.x; p.status[3] = blockIdx.z; }
    }
  } else if (layout_ok) {
    // ------------------------------------------------------------------ softmax + output (warps 2..5)
    const int quarter = warp & 3;             // the 32 TMEM lanes this warp may touch
    const int row = quarter * 32 + lane;      // query row inside the tile
    const int row_abs = base + q0 + row;      // its absolute position = its causal limit
    const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const bool windowed = p.window < (1 << 30);
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
#ifdef RB_DEBUG_AIDS
    const bool tracing = p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 64;
    unsigned long long tr[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    long long t_prev = clock64();
#endif
    for (int j = 0; j < n; ++j) {
      const int st = j & 1;
      const uint32_t ph = (uint32_t)(j >> 1) & 1u;
      const int key0 = (tile_lo + j) * kBN;
      // the four warps run warp-wide TMEM accesses below: a give-up must be a whole-warp decision
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctl->s_full[st], ph, abort_flag, p.wait_cycles))) { ok = false; break; }
      ptx::tc_fence_after();
      RB_TICK(0);  // waiting for the scores
      float s[kBN];
      {
        uint32_t r0[32], r1[32];
        ptx::tmem_ld_32x32(t_row + (uint32_t)(st * kBN), r0);
        ptx::tmem_ld_32x32(t_row + (uint32_t)(st * kBN + 32), r1);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) { s[i] = __uint_as_float(r0[i]); s[32 + i] = __uint_as_float(r1[i]); }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&ctl->s_empty[st]);  // the score buffer may be overwritten
      RB_TICK(1);  // reading them out of tensor memory
      // mask (only tiles that the causal diagonal or the window actually cuts), then the row max over the raw scores;
      // the scale is positive, so it commutes with the max and rides in the exponent's multiply-add below
      const bool causal_edge = key0 + kBN - 1 > base + q0;
      const bool window_edge = windowed && key0 + kBN > base && base + q0 + kBM - 1 - p.window > key0;
      if (causal_edge || window_edge) {
#pragma unroll
        for (int i = 0; i < kBN; ++i) {
          const int key = key0 + i;
          const bool seen = key <= row_abs && (key < base || key + p.window >= row_abs);
          s[i] = seen ? s[i] : -INFINITY;
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four independent chains
#pragma unroll
      for (int i = 0; i < kBN; i += 4) {
        mx4[0] = fmaxf(mx4[0], s[i]); mx4[1] = fmaxf(mx4[1], s[i + 1]);
        mx4[2] = fmaxf(mx4[2], s[i + 2]); mx4[3] = fmaxf(mx4[3], s[i + 3]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      // The reference point of the exponentials follows the running max lazily: it moves only when the max has grown
      // by more than 2^kSlack since it was last set.  softmax is invariant to the reference point (numerator and
      // denominator carry the same factor), the terms stay below 2^kSlack, well inside float32 and bf16 range, and the
      // rescaling of O below - a read-modify-write of the whole accumulator row - happens a handful of times per
      // walk instead of at nearly every tile.
      constexpr float kSlack = 8.0f;
      const float m_new = (mx > m_run + kSlack || m_run == -INFINITY) ? mx : m_run;
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = ex2_fast(m_run - m_use);
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t packed[kBN / 2];
#pragma unroll
      for (int i = 0; i < kBN; i += 4) {
        const float p0 = ex2_fast(fmaf(s[i], p.scale_log2, -m_use)), p1 = ex2_fast(fmaf(s[i + 1], p.scale_log2, -m_use));
        const float p2 = ex2_fast(fmaf(s[i + 2], p.scale_log2, -m_use)), p3 = ex2_fast(fmaf(s[i + 3], p.scale_log2, -m_use));
        sum4[0] += p0; sum4[1] += p1; sum4[2] += p2; sum4[3] += p3;
        __nv_bfloat162 h0 = __floats2bfloat162_rn(p0, p1), h1 = __floats2bfloat162_rn(p2, p3);
        packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h0);
        packed[(i >> 1) + 1] = *reinterpret_cast<uint32_t*>(&h1);
      }
      const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      l_run = l_run * corr + sum;
      RB_TICK(2);  // scale, max, exp, sum, pack
      bool rescaled = false;
      if (j > 0) {
        // P.V of the previous tile must be done before P is overwritten or O is touched
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctl->o_done, (uint32_t)(j - 1) & 1u, abort_flag, p.wait_cycles))) { ok = false; break; }
        ptx::tc_fence_after();
        RB_TICK(3);  // waiting for the previous P.V
        if (__any_sync(0xffffffffu, m_new != m_run)) {   // warp-uniform: the TMEM accesses below are warp-wide
          rescaled = true;
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t r[32];
            ptx::tmem_ld_32x32(t_row + C::kOCol + (uint32_t)c0, r);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * corr);
            ptx::tmem_st_32x32(t_row + C::kOCol + (uint32_t)c0, r);
          }
        }
      }
      RB_TICK(4);  // rescaling O
      // P row -> shared memory, K-major with the 128-byte swizzle (16-byte chunk c of row r sits at c ^ (r & 7))
      uint8_t* prow = p_s + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) =
            make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
      ptx::fence_proxy_async();   // generic-proxy writes of P become visible to the tensor core's reads
      if (rescaled) ptx::tmem_wait_st();
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&ctl->p_full);
      m_run = m_new;
      RB_TICK(5);  // storing P, fences, hand-over
    }
#ifdef RB_DEBUG_AIDS
    if (tracing) { for (int i = 0; i < 6; ++i) p.trace[i] = tr[i]; p.trace[6] = (unsigned long long)n; }
#endif
    if (ok) ok = __all_sync(0xffffffffu, ptx::mbar_wait(&ctl->o_done, (uint32_t)(n - 1) & 1u, abort_flag, p.wait_cycles));
    if (ok) {
      ptx::tc_fence_after();
      const float inv = 1.0f / l_run;
      const bool store = q0 + row < p.s_new;
      bf16* dst = p.out + (((size_t)b * p.s_new + q0 + row) * p.q_heads + head) * D;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(t_row + C::kOCol + (uint32_t)c0, r);
        ptx::tmem_wait_ld();
        if (store) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            float v[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = __uint_as_float(r[i + k]) * inv;
            *reinterpret_cast<uint4*>(dst + c0 + i) = pack8_bf16(v);
          }
        }
      }
    } else if (lane == 0) {
      p.status[0] = (uint32_t)(-RB_ERR_TIMEOUT); p.status[1] = 0xA7C3u; p.status[2] = blockIdx.x; p.status[3] = blockIdx.z;
    }
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // copies already handed to the copy engine get a bounded chance to land before the shared memory is released
    volatile uint32_t never = 0;
    ptx::mbar_wait(&ctl->q_full, 0u, &never, p.wait_cycles);
    for (uint32_t i = (ctl->k_issued > 2 ? ctl->k_issued - 2 : 0); i < ctl->k_issued; ++i)
      ptx::mbar_wait(&ctl->k_full[i & 1], (i >> 1) & 1u, &never, p.wait_cycles);
    for (uint32_t i = (ctl->v_issued > 2 ? ctl->v_issued - 2 : 0); i < ctl->v_issued; ++i)
      ptx::mbar_wait(&ctl->v_full[i & 1], (i >> 1) & 1u, &never, p.wait_cycles);
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int D>
int launch_tc(rb_ctx* ctx, const void* q, rb_kv_cache* c, int layer, int batch, int s_new, int q_heads, float scale, void* out) {
  using C = TCfg<D>;
  const size_t loff = (size_t)layer * c->layer_stride_elems();
  const bf16* kbase = (const bf16*)c->k + loff;
  const bf16* vbase = (const bf16*)c->v + loff;
  CUtensorMap tq, tk, tv;
  // q rows are (sequence, position), columns (head, lane): 128-row x 64-column boxes
  RB_TRY(tmap_2d_bf16(ctx, q, (int64_t)batch * s_new, (int64_t)q_heads * D, (int64_t)q_heads * D, kBM, &tq));
  // one map per layer and operand: rows are (page, KV head, token), 64-row x 64-column boxes
  const int64_t rows = (int64_t)c->num_pages * c->kv_heads * kBN;
  RB_TRY(tmap_2d_bf16(ctx, kbase, rows, D, D, kBN, &tk));
  RB_TRY(tmap_2d_bf16(ctx, vbase, rows, D, D, kBN, &tv));
  auto kern = attention_prefill_tc_kernel<D>;
  static bool set[64] = {};  // the attribute belongs to the (kernel, device) pair
  const int dv = ctx->device & 63;
  if (!set[dv]) { RB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes)); set[dv] = true; }
  TParams p{};
  p.block_table = c->block_table;
  p.seq_lens = c->seq_lens;
  p.pages_per_seq = c->pages_per_seq;
  p.s_new = s_new;
  p.q_heads = q_heads;
  p.kv_heads = c->kv_heads;
  p.group = q_heads / c->kv_heads;
  p.window = c->window;
  p.scale_log2 = scale * kLog2e;
  p.out = (bf16*)out;
  p.status = ctx->status_dev;
  p.wait_cycles = ctx->local_wait_cycles();
  dim3 grid((unsigned)((s_new + kBM - 1) / kBM), (unsigned)q_heads, (unsigned)batch);
#ifdef RB_DEBUG_AIDS
  static const bool trace = getenv("RAI_B200_ATTN_TRACE") != nullptr;
  static int traced = 0;
  if (trace && traced < 3 && layer == 0) {  // developer build: synchronous, prints where one softmax thread's cycles went
    ++traced;
    unsigned long long* tr = nullptr;
    RB_CUDA(cudaMalloc(&tr, 8 * sizeof(unsigned long long)));
    RB_CUDA(cudaMemset(tr, 0, 8 * sizeof(unsigned long long)));
    p.trace = tr;
    RB_CUDA(launch_kernel(kern, grid, dim3(kThreads), (size_t)C::kSmemBytes, ctx->stream, false, tq, tk, tv, p));
    RB_CUDA(cudaStreamSynchronize(ctx->stream));
    unsigned long long h[8];
    RB_CUDA(cudaMemcpy(h, tr, sizeof(h), cudaMemcpyDeviceToHost));
    cudaFree(tr);
    const double nt = h[6] ? (double)h[6] : 1.0;
    fprintf(stderr, "attention_prefill_tc<%d> s_new=%d tiles=%llu | cycles per tile: wait-scores %.0f  tmem-ld %.0f  softmax-math %.0f  "
            "wait-prev-PV %.0f  rescale-O %.0f  store-P+handover %.0f\n", D, s_new, h[6], h[0] / nt, h[1] / nt, h[2] / nt, h[3] / nt,
            h[4] / nt, h[5] / nt);
    ctx->launches++;
    return RB_OK;
  }
#endif
  RB_CUDA(launch_kernel(kern, grid, dim3(kThreads), (size_t)C::kSmemBytes, ctx->stream, ctx->pdl, tq, tk, tv, p));
  ctx->launches++;
  return RB_OK;
}

}  // namespace

bool attention_prefill_tc_supported(const rb_kv_cache* c, int s_new, int q_heads, const void* q, const void* out) {
  auto al16 = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; };
  return c->dtype == RB_BF16 && (c->head_dim == 64 || c->head_dim == 128) && s_new >= kBM && q_heads % c->kv_heads == 0 &&
         al16(q) && al16(out);
}

int attention_prefill_tc(rb_ctx* ctx, const void* q, rb_kv_cache* c, int layer, int batch, int s_new, int q_heads, float scale,
                         void* out) {
  if (c->head_dim == 64) return launch_tc<64>(ctx, q, c, layer, batch, s_new, q_heads, scale, out);
  if (c->head_dim == 128) return launch_tc<128>(ctx, q, c, layer, batch, s_new, q_heads, scale, out);
  return fail(RB_ERR_UNIMPLEMENTED, "tensor-core prefill attention: head_dim %d unsupported (64, 128)", c->head_dim);
}

}  // namespace rb
