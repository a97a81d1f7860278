// Attention over the paged bf16 KV cache, replacing repeat_kv + QK^T*scale + mask + softmax + PV
// (rai-models/src/llm/qwen2.rs:205-216, phi2.rs:245-261, phi3.rs:199-209, gemma.rs:238-249).
// Scores, masks and repeated KV heads are never materialised: a 64-key tile of K and V is staged
// in shared memory with 16-byte cp.async copies (a cache page IS one tile, so every copy is a
// contiguous 64 x head_dim block), scores live in registers as mma.sync fragments, and the softmax
// is the online (running max / running sum) form in float32.
//
//   prefill  grid (q tiles of 64 rows, q heads, batch): each of the 4 warps owns 16 query rows and
//            walks the causal range of key tiles.
//   decode   grid (KV splits, kv heads, batch): the G = q_heads / kv_heads query heads that share
//            a KV head are packed as the 16 rows of one MMA tile, so K and V are read from HBM once
//            per KV head instead of G times; the 4 warps split each key tile 16 keys apiece and
//            merge their (max, sum, O) at the end.  With more than one split a small kernel merges
//            the per-split partials.
// HBM-bound at decode: algorithmic bytes = 2 * len * kv_heads * head_dim * 2 per sequence and layer.
#include <stdlib.h>

#include <algorithm>
#include <mutex>

#include "ctx.h"
#include "ptx.cuh"

namespace rb {

using bf16 = __nv_bfloat16;

int attention_decode_splits(rb_ctx* ctx, int batch, int kv_heads, int max_len, int head_dim);

// Split-KV scratch of the context, grow-only.  A captured decode step has the buffer's address baked in, and other
// models or direct calls on the same context may need more later: a buffer that has been handed out is therefore
// never freed before rb_destroy - growing allocates a new one and retires the old one.  Models reserve their
// worst case when they are created, so a generation does not allocate.
int attention_reserve_scratch(rb_ctx* ctx, size_t bytes) {
  if (ctx->attn_scratch_bytes >= bytes) return RB_OK;
  float* fresh = nullptr;
  RB_CUDA(cudaMalloc(&fresh, bytes));
  if (ctx->attn_scratch) ctx->retired.push_back(ctx->attn_scratch);
  ctx->attn_scratch = fresh;
  ctx->attn_scratch_bytes = bytes;
  return RB_OK;
}

namespace {

constexpr int kTile = 64;  // keys per tile == tokens per cache page
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// TMA = true: K/V tiles arrive by tiled bulk copies (one elected thread, completion on an mbarrier)
// in the 128-byte-swizzled layout [D/64 column blocks][64 keys][128 bytes]; the copy engine keeps
// far more bytes in flight than 16-byte cp.async requests through the load/store unit can.
// TMA = false: padded rows filled with cp.async (head sizes that are not a multiple of 64).
template <int D, bool DECODE, bool TMA = false>
struct ACfg {
  static constexpr int kDP = D + 8;                      // padded row: conflict-free ldmatrix
  static constexpr int kRowBytes = kDP * 2;              // Q rows always, K/V rows when !TMA
  static constexpr int kStages = (DECODE && D <= 128) ? 3 : 2;
  static constexpr int kQRows = DECODE ? 16 : 64;
  static constexpr int kTileBytes = TMA ? kTile * D * 2 : kTile * kRowBytes;   // one of K or V
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kQBytes = kQRows * kRowBytes;
  static constexpr int kMergeBytes = DECODE ? (4 * 16 * D + 2 * 4 * 16) * 4 : 0;
  static constexpr int kPipeBytes = kStages * kStageBytes + kQBytes + (TMA ? 1024 : 0);
  static constexpr int kSmemBytes = kPipeBytes > kMergeBytes ? kPipeBytes : kMergeBytes;
  static constexpr bool kQInRegs = D <= 128;
  static constexpr int kKeysPerWarp = DECODE ? 16 : 64;
  static constexpr int kNtS = kKeysPerWarp / 8;
};

struct AParams {
  const bf16* q;
  const bf16* k;  // layer base
  const bf16* v;
  const int32_t* block_table;
  const int32_t* seq_lens;
  int pages_per_seq, s_new, q_heads, kv_heads, group;
  int n_splits;
  int window;      // sliding window (qwen2.rs:316-327): among the tokens of one call, key j is hidden from row i when j + window < i
  long long wait_cycles;  // give-up budget of the bounded waits
  float scale_log2;
  bf16* out;
  float* part_o;   // [batch*q_heads][n_splits][D]
  float* part_ml;  // [batch*q_heads][n_splits][2]
  uint32_t* split_count;  // [batch][kv_heads] arrivals; non-null: the last split block of a (sequence, KV head) merges
  uint32_t* status;
  // Fused single-token step (decode, tiled-copy path): the new token's q, k and v are taken straight from
  // the q/k/v projection's output (bf16 rows and/or float32 split-K partials, plus bias), rotated, and the
  // k/v rows appended to the cache by this kernel, which then needs no separate RoPE/append launch and
  // can request its first K/V tiles before the projection has even finished.
  int fuse;
  const bf16* f_qkv;     // [batch, (q_heads + 2 kv_heads) * D] or null
  const float* f_acc;    // [f_n_acc][batch, ...] partial sums or null
  int f_n_acc;
  size_t f_acc_stride;
  const bf16* f_bias;    // [(q_heads + 2 kv_heads) * D] or null
  const float* f_cos;    // [max_pos, rot/2]
  const float* f_sin;
  int f_rot, f_max_seq;
  bf16* f_k;             // the layer's K and V pages, writable
  bf16* f_v;
};

template <int D, bool DECODE, bool TMA>
__global__ void __launch_bounds__(128, (D <= 128) ? 2 : 1)
attention_kernel(const AParams p, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
  using C = ACfg<D, DECODE, TMA>;
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ __align__(8) uint64_t full_bar[C::kStages];
  __shared__ volatile uint32_t abort_flag;
  // K/V stages first (1024-byte aligned for the swizzled layout), Q after them
  uint8_t* kv_s = TMA ? reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~uintptr_t(1023)) : smem;
  uint8_t* q_s = kv_s + C::kStages * C::kStageBytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  pdl_launch_dependents();
  if (TMA && threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) ptx::mbar_init(&full_bar[s], 1);
    abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::tma_prefetch_desc(&tm_k);
    ptx::tma_prefetch_desc(&tm_v);
  }
  if (TMA) __syncthreads();
  // Fused step: everything up to the first use of the projection's output runs BEFORE the wait on the
  // previous kernel.  What it reads there is older than that kernel: the block table never changes, the
  // sequence lengths are set by a kernel that does not release its dependents early (so it completed before
  // anything after it started), and K/V rows of earlier tokens were written by earlier steps.  The one
  // row that is not there yet, the new token's, is patched into the staged tile from registers below.
  const bool fuse = DECODE && p.fuse != 0;
  if (!fuse) pdl_wait();  // q and the newest K/V rows come from the kernel before this one

  int b, head, kvh, q0 = 0, split = 0;
  if (DECODE) {
    split = blockIdx.x; kvh = blockIdx.y; b = blockIdx.z; head = kvh * p.group;
  } else {
    q0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * 64;  // longest causal ranges first
    head = blockIdx.y; b = blockIdx.z; kvh = head / p.group;
  }
  // (fused step: read before the dependency wait, so straight from L2, where the kernel that set it left it)
  const int len = fuse ? __ldcg(p.seq_lens + b) : p.seq_lens[b];
  const int base = len - p.s_new;  // absolute position of query row 0

  // key tiles this CTA walks
  int tile_lo, tile_hi;
  if (DECODE) {
    const int total = (len + kTile - 1) / kTile;
    const int per = (total + p.n_splits - 1) / p.n_splits;
    tile_lo = split * per;
    tile_hi = min(total, tile_lo + per);
  } else {
    // The reference's window term acts among the tokens of ONE call only (qwen2.rs:316-334: the mask block of the
    // cached prefix is all zeros, and a single-token call builds no mask at all, qwen2.rs:340-342), so whole tiles
    // can be skipped only when nothing is cached.
    tile_lo = base == 0 ? max(0, q0 - p.window) / kTile : 0;
    tile_hi = (min(base + q0 + 64, len) + kTile - 1) / kTile;
  }
  if (fuse && (len < 1 || len > p.f_max_seq)) {  // the same guard the separate RoPE/append kernel has
    if (threadIdx.x == 0) { p.status[0] = (uint32_t)(-RB_ERR_INVALID); p.status[1] = 0x20BEu; p.status[2] = (uint32_t)(len - 1); }
    pdl_wait();
    return;
  }

  int armed_it[C::kStages];  // thread 0: iteration whose tile was last requested into each stage
#pragma unroll
  for (int s = 0; s < C::kStages; ++s) armed_it[s] = -1;
  auto load_tile = [&](int tile, int stage) {
    if (TMA) {
      if (threadIdx.x == 0) {
        armed_it[stage] = tile - tile_lo;
        const int page = p.block_table[(size_t)b * p.pages_per_seq + tile];
        const int y = (page * p.kv_heads + kvh) * kTile;  // first row of this (page, KV head) in the layer
        uint8_t* ks = kv_s + stage * C::kStageBytes;
        uint8_t* vs = ks + C::kTileBytes;
        ptx::mbar_expect_tx(&full_bar[stage], C::kStageBytes);
#pragma unroll
        for (int cb = 0; cb < D / 64; ++cb) {
          ptx::tma_load_2d(ks + cb * (kTile * 128), &tm_k, &full_bar[stage], cb * 64, y);
          ptx::tma_load_2d(vs + cb * (kTile * 128), &tm_v, &full_bar[stage], cb * 64, y);
        }
      }
      return;
    }
    const int page = p.block_table[(size_t)b * p.pages_per_seq + tile];
    const size_t off = ((size_t)page * p.kv_heads + kvh) * kTile * D;
    const bf16* ksrc = p.k + off;
    const bf16* vsrc = p.v + off;
    uint8_t* ks = kv_s + stage * C::kStageBytes;
    uint8_t* vs = ks + C::kTileBytes;
    constexpr int chunks_per_row = D / 8;
    for (int i = threadIdx.x; i < kTile * chunks_per_row; i += blockDim.x) {
      const int r = i / chunks_per_row, c = i % chunks_per_row;
      cp_async16(s_u32(ks + r * C::kRowBytes + c * 16), ksrc + (size_t)r * D + c * 8);
      cp_async16(s_u32(vs + r * C::kRowBytes + c * 16), vsrc + (size_t)r * D + c * 8);
    }
  };
  // byte offset of the 16-byte chunk holding (key, dcol..dcol+8) inside a K or V tile
  auto tile_off = [&](int key, int dc) -> int {
    if (TMA) return (dc >> 6) * (kTile * 128) + key * 128 + ((((dc & 63) >> 3) ^ (key & 7)) << 4);
    return key * C::kRowBytes + dc * 2;
  };

  // the new token's tile and slot, and whether this block is the one that walks it (fused step)
  const int new_tile = (len - 1) / kTile, new_slot = (len - 1) % kTile;
  const bool owns_new = fuse && new_tile >= tile_lo && new_tile < tile_hi;
  __shared__ __align__(16) bf16 new_kv[DECODE ? 2 * D : 8];  // the new token's k row, then its v row

  if (fuse) {
    if constexpr (DECODE) {
      // first tiles on their way before the projection's output exists (one commit group each, like the other path)
#pragma unroll
      for (int s = 0; s < C::kStages - 1; ++s) {
        if (tile_lo + s < tile_hi) load_tile(tile_lo + s, s);
        cp_async_commit();
      }
      pdl_wait();
      // q heads of this KV head, its k head and its v head out of the projection's row of this sequence
      const int ncol = (p.q_heads + 2 * p.kv_heads) * D;
      const size_t row = (size_t)b * ncol;
      const int pos = len - 1;
      const int half = p.f_rot >> 1;
      const int pair_items = half >> 3, pass_items = (D - p.f_rot) >> 3;
      const int per_rot_head = pair_items + pass_items;
      const int rot_items = (p.group + 1) * per_rot_head;  // q heads, then the k head
      const int total = rot_items + (D >> 3);
      auto gather = [&](int col, float* v) {  // same order of additions as the separate kernel
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
        float t8[8];
        if (p.f_qkv) { load8(p.f_qkv + row + col, t8);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] += t8[i]; }
        add_slabs<4>(p.f_acc, p.f_n_acc, p.f_acc_stride, row + col, v);
        if (p.f_bias) { load8(p.f_bias + col, t8);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] += t8[i]; }
      };
      const int page = p.block_table[(size_t)b * p.pages_per_seq + new_tile];
      const size_t new_row = (((size_t)page * p.kv_heads + kvh) * kTile + new_slot) * D;
      // r < group: query head r of this group; r == group: the k head; r == group + 1: the v head
      auto emit = [&](int r, int lane0, const float* v) {
        if (r < p.group) { store8(reinterpret_cast<bf16*>(q_s + r * C::kRowBytes) + lane0, v); return; }
        bf16* stash = new_kv + (r - p.group) * D + lane0;
        store8(stash, v);
        if (owns_new) *reinterpret_cast<uint4*>((r == p.group ? p.f_k : p.f_v) + new_row + lane0) = *reinterpret_cast<const uint4*>(stash);
      };
      for (int it = threadIdx.x; it < total; it += blockDim.x) {
        if (it < rot_items) {
          const int r = it / per_rot_head, j = it % per_rot_head;
          const int col0 = (r < p.group ? head + r : p.q_heads + kvh) * D;
          if (j < pair_items) {
            const int i0 = j * 8;
            float lo[8], hi[8], cs[8], sn[8], ylo[8], yhi[8];
            gather(col0 + i0, lo);
            gather(col0 + i0 + half, hi);
            load8(p.f_cos + (size_t)pos * half + i0, cs);
            load8(p.f_sin + (size_t)pos * half + i0, sn);
            rope_rotate8(lo, hi, cs, sn, ylo, yhi);
            emit(r, i0, ylo);
            emit(r, i0 + half, yhi);
          } else {
            const int i0 = p.f_rot + (j - pair_items) * 8;
            float v[8];
            gather(col0 + i0, v);
            emit(r, i0, v);
          }
        } else {
          const int i0 = (it - rot_items) * 8;
          float v[8];
          gather((p.q_heads + p.kv_heads + kvh) * D + i0, v);
          emit(p.group + 1, i0, v);
        }
      }
      // unused query rows of the 16-row tile are zero
      constexpr int chunks_per_row = D / 8;
      for (int i = threadIdx.x; i < (C::kQRows - p.group) * chunks_per_row; i += blockDim.x) {
        const int r = p.group + i / chunks_per_row, c = i % chunks_per_row;
        *reinterpret_cast<uint4*>(q_s + r * C::kRowBytes + c * 16) = make_uint4(0, 0, 0, 0);
      }
    }
  } else {
    // ---- stage Q (rows beyond the valid range are zero)
    constexpr int chunks_per_row = D / 8;
    for (int i = threadIdx.x; i < C::kQRows * chunks_per_row; i += blockDim.x) {
      const int r = i / chunks_per_row, c = i % chunks_per_row;
      const bf16* src = nullptr;
      if (DECODE) {
        if (r < p.group) src = p.q + ((size_t)b * p.q_heads + head + r) * D + c * 8;
      } else {
        if (q0 + r < p.s_new) src = p.q + (((size_t)b * p.s_new + q0 + r) * p.q_heads + head) * D + c * 8;
      }
      const uint32_t dst = s_u32(q_s + r * C::kRowBytes + c * 16);
      if (src) cp_async16(dst, src);
      else *reinterpret_cast<uint4*>(q_s + r * C::kRowBytes + c * 16) = make_uint4(0, 0, 0, 0);
    }
    // prologue: Q + the first kStages-1 tiles, one commit group each
#pragma unroll
    for (int s = 0; s < C::kStages - 1; ++s) {
      if (tile_lo + s < tile_hi) load_tile(tile_lo + s, s);
      cp_async_commit();
    }
  }

  const int qrow0 = DECODE ? 0 : warp * 16;  // first Q row (inside the CTA tile) of this warp
  const int kw0 = DECODE ? warp * 16 : 0;    // first key (inside the tile) of this warp
  uint32_t qf[C::kQInRegs ? D / 16 : 1][4];
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  // causal limit per row half (g, g+8): last visible key index
  int lim[2];
  if (DECODE) { lim[0] = lim[1] = len - 1; }
  else { lim[0] = base + q0 + qrow0 + g; lim[1] = lim[0] + 8; }

  bool q_loaded = false;
  bool aborted = false;
  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    const int it = tile - tile_lo;
    {  // keep kStages-1 tiles in flight
      const int nxt = tile + C::kStages - 1;
      if (nxt < tile_hi) load_tile(nxt, (it + C::kStages - 1) % C::kStages);
      cp_async_commit();
    }
    if (TMA) {
      if (it == 0) cp_async_wait<0>();  // Q
      const bool mine = ptx::mbar_wait(&full_bar[it % C::kStages], (uint32_t)(it / C::kStages) & 1u, &abort_flag, p.wait_cycles);
      if (!__syncthreads_and(mine)) { aborted = true; break; }  // uniform decision: nobody computes on a tile that never came
    } else {
      cp_async_wait<C::kStages - 1>();
      __syncthreads();
    }
    if (owns_new && tile == new_tile) {
      // the copy of this tile may predate the new token's row: put the row in place from the block's own copy
      uint8_t* ks_w = kv_s + (it % C::kStages) * C::kStageBytes;
      for (int i = threadIdx.x; i < 2 * (D / 8); i += blockDim.x) {
        const int is_v = i / (D / 8), c = i % (D / 8);
        *reinterpret_cast<uint4*>(ks_w + is_v * C::kTileBytes + tile_off(new_slot, c * 8)) =
            *reinterpret_cast<const uint4*>(new_kv + is_v * D + c * 8);
      }
      __syncthreads();
    }
    if (C::kQInRegs && !q_loaded) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk)
        ldsm_x4(qf[kk], s_u32(q_s + (qrow0 + (lane & 15)) * C::kRowBytes + (kk * 16 + (lane >> 4) * 8) * 2));
      q_loaded = true;
    }
    const uint8_t* ks = kv_s + (it % C::kStages) * C::kStageBytes;
    const uint8_t* vs = ks + C::kTileBytes;
    const int tile_start = tile * kTile;
    // a warp whose rows all precede this tile has nothing to do (prefill, diagonal tiles only)
    // (warp-uniform by construction: mma.sync and ldmatrix need every lane)
    const bool warp_active = DECODE ? (tile_start + kw0 < len) : (tile_start <= base + q0 + qrow0 + 15);
    if (warp_active) {
      float s[C::kNtS][4];
#pragma unroll
      for (int i = 0; i < C::kNtS; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4];
        if (C::kQInRegs) { a[0] = qf[kk][0]; a[1] = qf[kk][1]; a[2] = qf[kk][2]; a[3] = qf[kk][3]; }
        else ldsm_x4(a, s_u32(q_s + (qrow0 + (lane & 15)) * C::kRowBytes + (kk * 16 + (lane >> 4) * 8) * 2));
#pragma unroll
        for (int np = 0; np < C::kNtS / 2; ++np) {
          uint32_t bb[4];
          const int key = kw0 + np * 16 + (lane & 7) + ((lane >> 4) << 3);
          const int dc = kk * 16 + (((lane >> 3) & 1) << 3);
          ldsm_x4(bb, s_u32(ks + tile_off(key, dc)));
          mma16816(s[2 * np], a, bb[0], bb[1]);
          mma16816(s[2 * np + 1], a, bb[2], bb[3]);
        }
      }
      // scale, mask, online softmax
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < C::kNtS; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key_abs = tile_start + kw0 + nt * 8 + 2 * t + (e & 1);
          const int hf = e >> 1;
          // causal limit (lim is the row's own position) and, among the new tokens only, the sliding window
          const bool seen = key_abs <= lim[hf] && (DECODE || key_abs < base || key_abs + p.window >= lim[hf]);
          const float v = seen ? s[nt][e] * p.scale_log2 : -INFINITY;
          s[nt][e] = v;
          mx[hf] = fmaxf(mx[hf], v);
        }
      float corr[2], m_use[2];
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        mx[hf] = fmaxf(mx[hf], __shfl_xor_sync(0xffffffffu, mx[hf], 1));
        mx[hf] = fmaxf(mx[hf], __shfl_xor_sync(0xffffffffu, mx[hf], 2));
        const float m_new = fmaxf(m_run[hf], mx[hf]);
        m_use[hf] = (m_new == -INFINITY) ? 0.f : m_new;
        corr[hf] = exp2f(m_run[hf] - m_use[hf]);
        m_run[hf] = m_new;
        l_run[hf] *= corr[hf];
      }
      uint32_t pa[C::kKeysPerWarp / 16][4];
#pragma unroll
      for (int nt = 0; nt < C::kNtS; ++nt) {
        const float p0 = exp2f(s[nt][0] - m_use[0]), p1 = exp2f(s[nt][1] - m_use[0]);
        const float p2 = exp2f(s[nt][2] - m_use[1]), p3 = exp2f(s[nt][3] - m_use[1]);
        l_run[0] += p0 + p1;
        l_run[1] += p2 + p3;
        pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p0, p1);
        pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
#pragma unroll
      for (int i = 0; i < D / 8; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
      // O += P V
#pragma unroll
      for (int k2 = 0; k2 < C::kKeysPerWarp / 16; ++k2)
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
          uint32_t bb[4];
          const int key = kw0 + k2 * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
          const int dc = dp * 16 + ((lane >> 4) << 3);
          ldsm_x4_t(bb, s_u32(vs + tile_off(key, dc)));
          mma16816(o[2 * dp], pa[k2], bb[0], bb[1]);
          mma16816(o[2 * dp + 1], pa[k2], bb[2], bb[3]);
        }
    }
    __syncthreads();  // the stage is overwritten by the next iteration's prefetch
  }
  cp_async_wait<0>();
  if (TMA && aborted) {
    // a tile never arrived: report, give copies already handed to the copy engine a bounded chance to land
    // (the stages are about to be reused as merge space or released), and produce no output
    if (threadIdx.x == 0) {
      p.status[0] = (uint32_t)(-RB_ERR_TIMEOUT); p.status[1] = 0xA77Eu; p.status[2] = blockIdx.x; p.status[3] = blockIdx.z;
      volatile uint32_t never = 0;
#pragma unroll
      for (int s = 0; s < C::kStages; ++s)
        if (armed_it[s] >= 0) ptx::mbar_wait(&full_bar[s], (uint32_t)(armed_it[s] / C::kStages) & 1u, &never, p.wait_cycles);
    }
    __syncthreads();
    return;
  }

  // row sums across the quad
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    l_run[hf] += __shfl_xor_sync(0xffffffffu, l_run[hf], 1);
    l_run[hf] += __shfl_xor_sync(0xffffffffu, l_run[hf], 2);
  }

  if (!DECODE) {
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int row = q0 + qrow0 + g + hf * 8;
      if (row >= p.s_new) continue;
      const float inv = 1.0f / l_run[hf];
      bf16* dst = p.out + (((size_t)b * p.s_new + row) * p.q_heads + head) * D;
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
        *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t) = pack_bf16(o[i][hf * 2] * inv, o[i][hf * 2 + 1] * inv);
    }
    return;
  }

  // ---- decode: merge the 4 warps' partial states through shared memory
  __syncthreads();
  float* mo = reinterpret_cast<float*>(smem);          // [4][16][D]
  float* mm = mo + 4 * 16 * D;                         // [4][16]
  float* ml = mm + 4 * 16;                             // [4][16]
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const int row = g + hf * 8;
    if (t == 0) { mm[warp * 16 + row] = m_run[hf]; ml[warp * 16 + row] = l_run[hf]; }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      mo[(warp * 16 + row) * D + i * 8 + 2 * t] = o[i][hf * 2];
      mo[(warp * 16 + row) * D + i * 8 + 2 * t + 1] = o[i][hf * 2 + 1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < p.group * D; idx += blockDim.x) {
    const int row = idx / D, dd = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, mm[w * 16 + row]);
    const float Mu = (M == -INFINITY) ? 0.f : M;
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float sc = exp2f(mm[w * 16 + row] - Mu);
      L += ml[w * 16 + row] * sc;
      O += mo[(w * 16 + row) * D + dd] * sc;
    }
    const size_t bh = (size_t)b * p.q_heads + head + row;
    if (p.n_splits == 1) {
      p.out[bh * D + dd] = __float2bfloat16_rn(O / L);
    } else {
      p.part_o[(bh * p.n_splits + split) * D + dd] = O;
      if (dd == 0) { p.part_ml[(bh * p.n_splits + split) * 2] = M; p.part_ml[(bh * p.n_splits + split) * 2 + 1] = L; }
    }
  }
  if (p.n_splits == 1 || !p.split_count) return;
  // The split block that arrives last for this (sequence, KV head) merges all of them: same sums, in the
  // same split order, as attention_merge_kernel, without the extra launch.
  __shared__ uint32_t is_last;
  __threadfence();   // this block's partials are visible device-wide before it is counted
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* cnt = p.split_count + (size_t)b * p.kv_heads + kvh;
    const uint32_t arrived = atomicAdd(cnt, 1u);
    is_last = (arrived == (uint32_t)p.n_splits - 1u) ? 1u : 0u;
    if (is_last) *cnt = 0u;  // re-armed for the next launch (which starts after this grid has completed)
    __threadfence();
  }
  __syncthreads();
  if (!is_last) return;
  // The per-split maxima and sums of this block's rows first (a few hundred floats, one round trip to L2), turned
  // into one weight per (row, split) in shared memory; then every output element sums its splits with all loads in
  // flight at once.  Same sums, in the same split order, as attention_merge_kernel.
  float* w_s = reinterpret_cast<float*>(smem);          // [16 rows][32 splits] weights exp2(M_split - M) / L
  const int ns = p.n_splits;                             // <= 32
  for (int i = threadIdx.x; i < p.group * ns; i += blockDim.x) {
    const int row = i / ns, sp = i % ns;
    const size_t bh = (size_t)b * p.q_heads + head + row;
    w_s[row * 32 + sp] = __ldcg(p.part_ml + (bh * ns + sp) * 2);            // max, for now
    w_s[512 + row * 32 + sp] = __ldcg(p.part_ml + (bh * ns + sp) * 2 + 1);  // sum
  }
  __syncthreads();
  if (threadIdx.x < p.group) {
    const int row = threadIdx.x;
    float M = -INFINITY;
    for (int sp = 0; sp < ns; ++sp) M = fmaxf(M, w_s[row * 32 + sp]);
    const float Mu = (M == -INFINITY) ? 0.f : M;
    float L = 0.f;
    for (int sp = 0; sp < ns; ++sp) L += w_s[512 + row * 32 + sp] * exp2f(w_s[row * 32 + sp] - Mu);
    for (int sp = 0; sp < ns; ++sp) w_s[row * 32 + sp] = exp2f(w_s[row * 32 + sp] - Mu);
    w_s[1024 + row] = L;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < p.group * D; idx += blockDim.x) {
    const int row = idx / D, dd = idx % D;
    const size_t bh = (size_t)b * p.q_heads + head + row;
    const float* o_p = p.part_o + bh * ns * D + dd;
    float O = 0.f;
    for (int s0 = 0; s0 < ns; s0 += 8) {
      float t[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) t[k] = (s0 + k < ns) ? __ldcg(o_p + (size_t)(s0 + k) * D) : 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (s0 + k < ns) O += t[k] * w_s[row * 32 + s0 + k];
    }
    p.out[bh * D + dd] = __float2bfloat16_rn(O / w_s[1024 + row]);
  }
}

// Merges the per-split (max, sum, O) of the decode kernel: one block per (sequence, head).
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       int n_splits, int d, bf16* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t bh = blockIdx.x;
  float M = -INFINITY;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(bh * n_splits + s) * 2]);
  const float Mu = (M == -INFINITY) ? 0.f : M;
  float L = 0.f;
  for (int s = 0; s < n_splits; ++s) L += part_ml[(bh * n_splits + s) * 2 + 1] * exp2f(part_ml[(bh * n_splits + s) * 2] - Mu);
  for (int dd = threadIdx.x; dd < d; dd += blockDim.x) {
    float O = 0.f;
    for (int s = 0; s < n_splits; ++s)
      O += part_o[(bh * n_splits + s) * d + dd] * exp2f(part_ml[(bh * n_splits + s) * 2] - Mu);
    out[bh * d + dd] = __float2bfloat16_rn(O / L);
  }
}

// Launches attention_kernel<D, DECODE> with tiled-copy loading when the head size allows it.
template <int D, bool DECODE>
int launch_attn_kernel(rb_ctx* ctx, rb_kv_cache* c, const AParams& p, dim3 grid) {
  constexpr bool kTma = (D % 64) == 0;
  using C = ACfg<D, DECODE, kTma>;
  auto kern = attention_kernel<D, DECODE, kTma>;
  static bool set[64] = {};  // the attribute belongs to the (kernel, device) pair
  const int dv = ctx->device & 63;
  if (!set[dv]) { RB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes)); set[dv] = true; }
  CUtensorMap tk{}, tv{};
  if (kTma) {
    // one map per layer and operand: rows are (page, KV head, token), 64-row x 64-column boxes
    const int64_t rows = (int64_t)c->num_pages * c->kv_heads * kTile;
    RB_TRY(tmap_2d_bf16(ctx, p.k, rows, D, D, kTile, &tk));
    RB_TRY(tmap_2d_bf16(ctx, p.v, rows, D, D, kTile, &tv));
  }
  RB_CUDA(launch_kernel(kern, grid, dim3(128), (size_t)C::kSmemBytes, ctx->stream, ctx->pdl, p, tk, tv));
  ctx->launches++;
  return RB_OK;
}

template <int D>
int launch_attention(rb_ctx* ctx, rb_kv_cache* c, AParams& p, int batch, int max_len) {
  if (p.s_new > 1) {
    dim3 grid((unsigned)((p.s_new + 63) / 64), (unsigned)p.q_heads, (unsigned)batch);
    p.n_splits = 1;
    return launch_attn_kernel<D, false>(ctx, c, p, grid);
  }
  // Split the keys of a sequence over several blocks only when (sequence, KV head) pairs alone leave
  // the GPU under-filled: one long block per pair keeps its copy pipeline full and needs no merge.
  const int splits = attention_decode_splits(ctx, batch, p.kv_heads, max_len, D);
  p.n_splits = splits;
  if (splits > 1) {
    RB_TRY(attention_reserve_scratch(ctx, (size_t)batch * p.q_heads * splits * (D + 2) * sizeof(float)));
    p.part_o = ctx->attn_scratch;
    p.part_ml = ctx->attn_scratch + (size_t)batch * p.q_heads * splits * D;
  }
  dim3 grid((unsigned)splits, (unsigned)p.kv_heads, (unsigned)batch);
  static const bool separate_merge = getenv("RAI_B200_ATTN_MERGE_KERNEL") != nullptr;  // debugging aid
  p.split_count = (splits > 1 && !separate_merge) ? c->split_count : nullptr;
  RB_TRY((launch_attn_kernel<D, true>(ctx, c, p, grid)));
  if (splits > 1 && !p.split_count) {
    RB_CUDA(launch_kernel(attention_merge_kernel, dim3((unsigned)(batch * p.q_heads)), dim3(128), 0, ctx->stream, ctx->pdl,
                          (const float*)p.part_o, (const float*)p.part_ml, splits, D, p.out));
    ctx->launches++;
  }
  return RB_OK;
}

}  // namespace

// ------------------------------------------------------------------------------------------
// Decode attention that allocates nothing.  The split-KV partials (per sequence, head and split:
// head_dim running sums plus a max and a sum) normally live in a buffer that the library grows
// with cudaMalloc when a larger shape arrives.  Some callers cannot have that happen under them:
// a host runtime that hands all device memory to its own pool and treats a foreign cudaMalloc as
// an error, or a serving loop that cannot afford the device-wide synchronisation an allocation may
// imply.  For them the same kernels run here with the partials in a fixed array that is part of
// the library image: every GPU that loads the library holds these 2 MiB until the process exits.
// (What the entry point cannot rule out is the CUDA runtime loading a kernel's code on its first
// launch; a caller whose pool takes all remaining memory makes one call per head size first.)
// ------------------------------------------------------------------------------------------
constexpr size_t kStaticScratchFloats = 1u << 19;  // 2 MiB
static __device__ __align__(256) float g_static_attn_scratch[kStaticScratchFloats];
// In host code the array's name is only a handle for the runtime, not a device address: the address
// the kernels need is asked for once per device (with that device current) and kept here.
static float* g_static_attn_scratch_dev[64] = {};
static std::mutex g_static_attn_scratch_lock;

template <int D>
static int launch_attention_decode_static(rb_ctx* ctx, rb_kv_cache* c, AParams& p, int batch, int max_len, float* scratch) {
  const int splits = attention_decode_splits(ctx, batch, p.kv_heads, max_len, D);
  p.n_splits = splits;
  if (splits > 1) {
    const size_t need = (size_t)batch * p.q_heads * splits * (D + 2);
    if (need > kStaticScratchFloats)
      return fail(RB_ERR_INVALID,
                  "rb_attention_decode_static: batch %d x %d heads x %d splits x head_dim %d needs %zu scratch floats, "
                  "the built-in array holds %zu; use rb_attention",
                  batch, p.q_heads, splits, D, need, kStaticScratchFloats);
    p.part_o = scratch;
    p.part_ml = scratch + (size_t)batch * p.q_heads * splits * D;
  }
  dim3 grid((unsigned)splits, (unsigned)p.kv_heads, (unsigned)batch);
  RB_TRY((launch_attn_kernel<D, true>(ctx, c, p, grid)));
  if (splits > 1) {
    RB_CUDA(launch_kernel(attention_merge_kernel, dim3((unsigned)(batch * p.q_heads)), dim3(128), 0, ctx->stream, ctx->pdl,
                          (const float*)p.part_o, (const float*)p.part_ml, splits, D, p.out));
    ctx->launches++;
  }
  return RB_OK;
}

int attention_decode_splits(rb_ctx* ctx, int batch, int kv_heads, int max_len, int head_dim) {
  // One block per (sequence, KV head) keeps its copy pipeline full and needs no merge; splitting the
  // keys only pays when those pairs under-fill the GPU.  Cost model in units of key tiles: a launch
  // runs ceil(blocks / resident blocks) waves, each as long as one block's tiles plus a fixed start-up,
  // and a split launch pays for the merge kernel.
  const int tiles = std::max(1, (max_len + kTile - 1) / kTile);
  const int work = batch * kv_heads;
  const int slots = (head_dim <= 128 ? 2 : 1) * ctx->sm_count;  // blocks resident at once (head size 256: one per SM)
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= std::min(tiles, 32); ++s) {
    const int waves = (work * s + slots - 1) / slots;
    const double cost = (double)waves * ((tiles + s - 1) / s + 2.0) + (s > 1 ? 1.5 : 0.0);
    if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
  }
  static const int forced = getenv("RAI_B200_ATTN_SPLITS") ? atoi(getenv("RAI_B200_ATTN_SPLITS")) : 0;
  if (forced > 0) best = std::max(1, std::min(forced, tiles));
  return best;
}

int attention_mma_bf16(rb_ctx* ctx, const void* q, rb_kv_cache* c, int layer, int batch, int s_new, int q_heads,
                       float scale, void* out) {
  AParams p{};
  const size_t loff = (size_t)layer * c->layer_stride_elems();
  p.q = (const bf16*)q;
  p.k = (const bf16*)c->k + loff;
  p.v = (const bf16*)c->v + loff;
  p.block_table = c->block_table;
  p.seq_lens = c->seq_lens;
  p.pages_per_seq = c->pages_per_seq;
  p.s_new = s_new;
  p.q_heads = q_heads;
  p.kv_heads = c->kv_heads;
  p.group = q_heads / c->kv_heads;
  p.scale_log2 = scale * kLog2e;
  p.out = (bf16*)out;
  p.status = ctx->status_dev;
  p.window = c->window;
  p.wait_cycles = ctx->local_wait_cycles();
  RB_REQUIRE(p.group >= 1 && p.group <= 16 && q_heads % c->kv_heads == 0,
             "attention: %d query heads per KV head unsupported (1..16)", p.group);
  // prefill with at least one 128-row query tile and head size 64 or 128: the tcgen05 kernel
  if (ctx->attn_tc && attention_prefill_tc_supported(c, s_new, q_heads, q, out))
    return attention_prefill_tc(ctx, q, c, layer, batch, s_new, q_heads, scale, out);
  int max_len = 0;
  for (int b = 0; b < batch; ++b) max_len = std::max(max_len, c->host_lens[b]);
  switch (c->head_dim) {
    case 64: return launch_attention<64>(ctx, c, p, batch, max_len);
    case 80: return launch_attention<80>(ctx, c, p, batch, max_len);
    case 96: return launch_attention<96>(ctx, c, p, batch, max_len);
    case 128: return launch_attention<128>(ctx, c, p, batch, max_len);
    case 256: return launch_attention<256>(ctx, c, p, batch, max_len);
  }
  return fail(RB_ERR_UNIMPLEMENTED, "attention: head_dim %d has no tensor-core kernel (64, 80, 96, 128, 256)",
              c->head_dim);
}

bool attention_can_fuse_rope(const rb_kv_cache* c, int q_heads, int rot, const void* qkv, const float* acc, int n_acc,
                             const void* bias, const float* cos_t, const float* sin_t, int batch) {
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const int d = c->head_dim;
  if (c->dtype != RB_BF16 || !(d == 64 || d == 80 || d == 96 || d == 128 || d == 256)) return false;
  if (rot < 0 || rot > d || (rot % 16) != 0 || ((d - rot) % 8) != 0) return false;
  if (q_heads % c->kv_heads != 0 || q_heads / c->kv_heads > 16) return false;
  const size_t acc_stride = (size_t)batch * (q_heads + 2 * c->kv_heads) * d;
  return al16(qkv) && al16(acc) && al16(bias) && al16(cos_t) && al16(sin_t) && ((acc_stride * sizeof(float)) % 16) == 0 &&
         (qkv || (acc && n_acc > 0));
}

int attention_decode_fused_rope(rb_ctx* ctx, const void* qkv, const float* acc, int n_acc, const void* bias,
                                const float* cos_t, const float* sin_t, int rot, rb_kv_cache* c, int layer, int batch,
                                int q_heads, float scale, void* out) {
  AParams p{};
  const size_t loff = (size_t)layer * c->layer_stride_elems();
  p.q = nullptr;
  p.k = (const bf16*)c->k + loff;
  p.v = (const bf16*)c->v + loff;
  p.block_table = c->block_table;
  p.seq_lens = c->seq_lens;
  p.pages_per_seq = c->pages_per_seq;
  p.s_new = 1;
  p.q_heads = q_heads;
  p.kv_heads = c->kv_heads;
  p.group = q_heads / c->kv_heads;
  p.scale_log2 = scale * kLog2e;
  p.out = (bf16*)out;
  p.status = ctx->status_dev;
  p.window = c->window;
  p.wait_cycles = ctx->local_wait_cycles();
  p.fuse = 1;
  p.f_qkv = (const bf16*)qkv;
  p.f_acc = n_acc > 0 ? acc : nullptr;
  p.f_n_acc = acc ? n_acc : 0;
  p.f_acc_stride = (size_t)batch * (q_heads + 2 * c->kv_heads) * c->head_dim;
  p.f_bias = (const bf16*)bias;
  p.f_cos = cos_t;
  p.f_sin = sin_t;
  p.f_rot = rot;
  p.f_max_seq = c->max_seq;
  p.f_k = (bf16*)c->k + loff;
  p.f_v = (bf16*)c->v + loff;
  int max_len = 0;
  for (int b = 0; b < batch; ++b) max_len = std::max(max_len, c->host_lens[b]);
  switch (c->head_dim) {
    case 64: return launch_attention<64>(ctx, c, p, batch, max_len);
    case 80: return launch_attention<80>(ctx, c, p, batch, max_len);
    case 96: return launch_attention<96>(ctx, c, p, batch, max_len);
    case 128: return launch_attention<128>(ctx, c, p, batch, max_len);
    case 256: return launch_attention<256>(ctx, c, p, batch, max_len);
  }
  return fail(RB_ERR_UNIMPLEMENTED, "fused rope + attention: head_dim %d unsupported (64, 80, 96, 128, 256)", c->head_dim);
}

}  // namespace rb

extern "C" int32_t rb_attention_decode_static(rb_ctx* ctx, const void* q, rb_kv_cache* c, int32_t layer, int32_t batch,
                                              int32_t q_heads, float scale, void* out) {
  using namespace rb;
  RB_REQUIRE(ctx && q && c && out, "rb_attention_decode_static: null argument");
  RB_REQUIRE(c->dtype == RB_BF16, "rb_attention_decode_static: bf16 caches only");
  RB_REQUIRE(layer >= 0 && layer < c->layers, "rb_attention_decode_static: layer %d out of range", layer);
  RB_REQUIRE(batch > 0 && batch <= c->max_batch, "rb_attention_decode_static: bad batch");
  RB_REQUIRE(q_heads > 0 && q_heads % c->kv_heads == 0 && q_heads / c->kv_heads <= 16,
             "rb_attention_decode_static: %d query heads over %d KV heads unsupported", q_heads, c->kv_heads);
  RB_REQUIRE(ctx->device >= 0 && ctx->device < 64, "rb_attention_decode_static: device index %d out of range", ctx->device);
  int max_len = 0;
  for (int b = 0; b < batch; ++b) {
    RB_REQUIRE(c->host_lens[b] >= 1, "rb_attention_decode_static: sequence %d is empty", b);
    max_len = std::max(max_len, c->host_lens[b]);
  }
  // One-time set-up per device, done by the first call on it: turn the symbol into a device address.  The lock
  // makes first calls from several host threads safe (the table is read and filled under it).
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> guard(g_static_attn_scratch_lock);
    if (!g_static_attn_scratch_dev[ctx->device]) {
      int current = -1;
      RB_CUDA(cudaGetDevice(&current));
      RB_REQUIRE(current == ctx->device, "rb_attention_decode_static: device %d must be current (it is %d)", ctx->device, current);
      float* ptr = nullptr;
      RB_CUDA(cudaGetSymbolAddress((void**)&ptr, g_static_attn_scratch));
      g_static_attn_scratch_dev[ctx->device] = ptr;
    }
    scratch = g_static_attn_scratch_dev[ctx->device];
  }
  AParams p{};
  const size_t loff = (size_t)layer * c->layer_stride_elems();
  p.q = (const bf16*)q;
  p.k = (const bf16*)c->k + loff;
  p.v = (const bf16*)c->v + loff;
  p.block_table = c->block_table;
  p.seq_lens = c->seq_lens;
  p.pages_per_seq = c->pages_per_seq;
  p.s_new = 1;
  p.q_heads = q_heads;
  p.kv_heads = c->kv_heads;
  p.group = q_heads / c->kv_heads;
  p.scale_log2 = scale * kLog2e;
  p.out = (bf16*)out;
  p.status = ctx->status_dev;
  p.window = c->window;
  p.wait_cycles = ctx->local_wait_cycles();
  switch (c->head_dim) {
    case 64: return launch_attention_decode_static<64>(ctx, c, p, batch, max_len, scratch);
    case 80: return launch_attention_decode_static<80>(ctx, c, p, batch, max_len, scratch);
    case 96: return launch_attention_decode_static<96>(ctx, c, p, batch, max_len, scratch);
    case 128: return launch_attention_decode_static<128>(ctx, c, p, batch, max_len, scratch);
    case 256: return launch_attention_decode_static<256>(ctx, c, p, batch, max_len, scratch);
  }
  return fail(RB_ERR_UNIMPLEMENTED, "rb_attention_decode_static: head_dim %d has no kernel (64, 80, 96, 128, 256)", c->head_dim);
}
