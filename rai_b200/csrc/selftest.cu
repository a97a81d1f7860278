// Self-test of the give-up path of the bounded device-side waits (rb_selftest_wait_gives_up): kernels whose wait can
// never be satisfied run with a short budget, and the host checks that they returned, that the status word
// names them, and that nothing else was written.  Nothing here faults, traps or spins without bound.
#include <vector>

#include "ctx.h"
#include "ptx.cuh"

namespace rb {
namespace {

// One thread waits, with the library's own helper, on an mbarrier that expects an arrival nobody makes.
__global__ void wait_probe_kernel(long long budget, uint32_t* status, uint32_t* returned) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ volatile uint32_t abort_flag;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1);
    abort_flag = 0;
    ptx::fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = ptx::mbar_wait(&bar, 0u, &abort_flag, budget);
    if (!ok) { status[0] = (uint32_t)(-RB_ERR_TIMEOUT); status[1] = 0x5E1Fu; status[2] = blockIdx.x; status[3] = 0u; }
    *returned = ok ? 2u : 1u;
  }
}

struct DevBuf {
  void* p = nullptr;
  ~DevBuf() { if (p) cudaFree(p); }
};

int read_status(rb_ctx* ctx, uint32_t* w) {
  RB_CUDA(cudaStreamSynchronize(ctx->stream));
  RB_CUDA(cudaMemcpy(w, ctx->status_dev, 4 * sizeof(uint32_t), cudaMemcpyDeviceToHost));
  RB_CUDA(cudaMemset(ctx->status_dev, 0, 4 * sizeof(uint32_t)));
  return RB_OK;
}

}  // namespace
}  // namespace rb

using namespace rb;

extern "C" int32_t rb_selftest_wait_gives_up(rb_ctx* ctx, int32_t which, int64_t budget_us) {
  RB_REQUIRE(ctx, "rb_selftest_wait_gives_up: null context");
  RB_REQUIRE(which >= 0 && which <= 3, "rb_selftest_wait_gives_up: unknown test %d", which);
  RB_REQUIRE(budget_us >= 1 && budget_us <= 1000000, "rb_selftest_wait_gives_up: budget %lld us outside [1, 1 000 000]",
             (long long)budget_us);
  RB_TRY(rb_sync(ctx));  // start from a clear status word
  const long long budget = (long long)((double)budget_us * ctx->cycles_per_us);
  uint32_t w[4];
  if (which == 0) {
    DevBuf ret;
    RB_CUDA(cudaMalloc(&ret.p, sizeof(uint32_t)));
    RB_CUDA(cudaMemsetAsync(ret.p, 0, sizeof(uint32_t), ctx->stream));
    wait_probe_kernel<<<1, 32, 0, ctx->stream>>>(budget, ctx->status_dev, (uint32_t*)ret.p);
    RB_CUDA(cudaGetLastError());
    ctx->launches++;
    RB_TRY(read_status(ctx, w));
    uint32_t returned = 0;
    RB_CUDA(cudaMemcpy(&returned, ret.p, sizeof(uint32_t), cudaMemcpyDeviceToHost));
    if (returned != 1u || w[0] != (uint32_t)(-RB_ERR_TIMEOUT) || w[1] != 0x5E1Fu)
      return fail(RB_ERR_CUDA, "wait self-test: expected a recorded give-up at 0x5E1F, got returned=%u status={%u, 0x%x}",
                  returned, w[0], w[1]);
    return RB_OK;
  }
  // ---- the tensor-parallel exchange over a two-member group that lives entirely in this GPU's memory; this launch
  // plays member 0 and nobody plays member 1.  which == 1: the flag-array form; 2: the flag inside the data, direct;
  // 3: the flag inside the data over two hops (row 0 is member 0's to finish, row 1 member 1's).
  const bool in_data = which >= 2;
  const bool two_hop = which == 3;
  const int rows = 2, hidden = 256;
  DevBuf region, part, h, wt, out, sum;
  const size_t slot_elems = (size_t)kTpMaxRows * hidden;
  const size_t region_bytes = kTpFlagBytes + 512 + (2 * 2 + (two_hop ? 2 : 0)) * slot_elems * (in_data ? 4 : 2);   // flags | counters | 2 slots x 2 sources (| 2 slots of finished rows)
  const size_t act_bytes = (size_t)rows * hidden * 2;
  RB_CUDA(cudaMalloc(&region.p, region_bytes));
  RB_CUDA(cudaMalloc(&part.p, act_bytes));
  RB_CUDA(cudaMalloc(&h.p, act_bytes));
  RB_CUDA(cudaMalloc(&wt.p, (size_t)hidden * 2));
  RB_CUDA(cudaMalloc(&out.p, act_bytes));
  RB_CUDA(cudaMalloc(&sum.p, act_bytes));
  RB_CUDA(cudaMemsetAsync(region.p, 0, region_bytes, ctx->stream));
  RB_CUDA(cudaMemsetAsync(h.p, 0, act_bytes, ctx->stream));
  std::vector<uint16_t> ones((size_t)rows * hidden, 0x3F80u);  // bf16 1.0
  RB_CUDA(cudaMemcpyAsync(wt.p, ones.data(), (size_t)hidden * 2, cudaMemcpyHostToDevice, ctx->stream));
  RB_CUDA(cudaMemcpyAsync(part.p, ones.data(), act_bytes, cudaMemcpyHostToDevice, ctx->stream));
  RB_CUDA(cudaMemsetAsync(out.p, 0x5A, act_bytes, ctx->stream));
  RB_CUDA(cudaMemsetAsync(sum.p, 0x5A, act_bytes, ctx->stream));
  TpPeers tp{};
  uint32_t* flags = (uint32_t*)region.p;          // [2 slots][kTpMaxRanks][kTpMaxRows]
  tp.flags[0] = tp.flags[1] = flags;
  tp.seq = (uint32_t*)((char*)region.p + kTpFlagBytes);
  tp.xbuf[0] = tp.xbuf[1] = (const char*)region.p + kTpFlagBytes + 512;
  tp.rank = 0; tp.size = 2; tp.slot_elems = (int64_t)slot_elems; tp.form = two_hop ? kTpInDataTwoHop : in_data ? kTpInDataDirect : kTpFlagArray;
  RB_CUDA(cudaStreamSynchronize(ctx->stream));  // the host buffers above are read by the copies
  const long long keep = ctx->wait_budget_cycles;
  ctx->wait_budget_cycles = budget;
  // exchange number 1 (parity 0): member 1 never raises its flags
  int st = exchange_norm(ctx, tp, 0, RB_NORM_RMS, h.p, nullptr, 0, nullptr, part.p, wt.p, nullptr, 1e-6f, rows, hidden, out.p, sum.p);
  ctx->wait_budget_cycles = keep;
  RB_TRY(st);
  RB_TRY(read_status(ctx, w));
  std::vector<uint16_t> got((size_t)rows * hidden), got_sum((size_t)rows * hidden);
  RB_CUDA(cudaMemcpy(got.data(), out.p, act_bytes, cudaMemcpyDeviceToHost));
  RB_CUDA(cudaMemcpy(got_sum.data(), sum.p, act_bytes, cudaMemcpyDeviceToHost));
  bool untouched = true;
  for (uint16_t v : got) untouched = untouched && v == 0x5A5Au;
  for (uint16_t v : got_sum) untouched = untouched && v == 0x5A5Au;
  if (w[0] != (uint32_t)(-RB_ERR_TIMEOUT) || w[1] != 0x7A11u || !untouched)
    return fail(RB_ERR_CUDA, "exchange-wait self-test: expected a give-up at 0x7A11 with the outputs untouched, got status={%u, 0x%x}, "
                "outputs %s", w[0], w[1], untouched ? "untouched" : "written");
  // exchange number 2 (parity 1, slot 0) with member 1's rows "arrived" (all zero) and its flags raised: completes,
  // nothing recorded, and the sum is member 0's term alone
  if (two_hop) {
    // exchange 2 lands in slot 0.  Row 0 is ours to finish: member 1's share of it (payload 0) arrives in the
    // gathering slot; row 1 is member 1's: its finished row (1 + 0 = bf16 1.0 in every element) arrives behind the
    // gathering slots
    uint64_t* words0 = (uint64_t*)((char*)region.p + kTpFlagBytes + 512);
    std::vector<uint64_t> share((size_t)hidden / 2, (uint64_t)2u << 32);
    std::vector<uint64_t> done((size_t)hidden / 2, ((uint64_t)2u << 32) | 0x3F803F80u);
    RB_CUDA(cudaMemcpy(words0 + ((((size_t)0 * 2 + 1) * slot_elems + (size_t)0 * hidden) >> 1), share.data(),
                       share.size() * sizeof(uint64_t), cudaMemcpyHostToDevice));
    RB_CUDA(cudaMemcpy(words0 + (((size_t)2 * 2 * slot_elems + (size_t)0 * slot_elems + (size_t)1 * hidden) >> 1), done.data(),
                       done.size() * sizeof(uint64_t), cudaMemcpyHostToDevice));
  } else if (in_data) {
    // member 1's two rows of slot 0: every 8-byte word = payload 0, exchange number 2
    std::vector<uint64_t> words((size_t)rows * hidden / 2, (uint64_t)2u << 32);
    uint64_t* dst = (uint64_t*)((char*)region.p + kTpFlagBytes + 512) + (((size_t)0 * 2 + 1) * slot_elems >> 1);
    RB_CUDA(cudaMemcpy(dst, words.data(), words.size() * sizeof(uint64_t), cudaMemcpyHostToDevice));
  } else {
    const uint32_t twos[2] = {2u, 2u};
    RB_CUDA(cudaMemcpy(flags + ((size_t)0 * kTpMaxRanks + 1) * kTpMaxRows, twos, sizeof(twos), cudaMemcpyHostToDevice));
  }
  RB_TRY(exchange_norm(ctx, tp, 1, RB_NORM_RMS, h.p, nullptr, 0, nullptr, part.p, wt.p, nullptr, 1e-6f, rows, hidden, out.p, sum.p));
  RB_TRY(read_status(ctx, w));
  RB_CUDA(cudaMemcpy(got.data(), out.p, act_bytes, cudaMemcpyDeviceToHost));
  RB_CUDA(cudaMemcpy(got_sum.data(), sum.p, act_bytes, cudaMemcpyDeviceToHost));
  bool written = true;
  for (uint16_t v : got) written = written && v == 0x3F80u;      // an all-ones row, RMS-normalised with unit weights
  for (uint16_t v : got_sum) written = written && v == 0x3F80u;  // 0 + (1 + 0)
  if (w[0] != 0u || !written)
    return fail(RB_ERR_CUDA, "exchange-wait self-test: the healthy call after the give-up failed (status %u, outputs %s)", w[0],
                written ? "as expected" : "wrong");
  return RB_OK;
}
