"""Benchmark of the decoder hot path on B200: batch-64 KV-cached decode (the headline) and 8 x 4096
prefill of the Qwen2-7B architecture in bf16, tensor-parallel over --gpus ranks.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" is one decode step of the whole batch (64 new tokens at a 2048-token context that grows by
one per step).  Rank 0 prints ONE JSON line.  Weights are random-init N(0, 0.02) bf16 and token ids
uniform random (no checkpoints or datasets are available offline); the KV cache is filled by really
prefilling random prompts.  `--impl reference` times the CPU restatement of rai's own Cpu path
(oracle/rai_cpu.py; rai itself cannot be built here) on the host cores, on a bounded sample.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NOMINAL_HBM_GBS = 8000.0        # the roofline basis the benchmark definition names
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="qwen2-7b")
    ap.add_argument("--decode-batch", type=int, default=64)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--prefill-batch", type=int, default=8)
    ap.add_argument("--prefill-len", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (debugging only)")
    ap.add_argument("--skip-prefill", action="store_true")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--profile-steps", type=int, default=8)
    ap.add_argument("--skip-timeline", action="store_true")
    ap.add_argument("--timeline", default="", help="write a per-kernel device timeline of a few decode steps (as replayed, "
                    "overlap included) to this JSON file; a tracing pass of its own, never part of the timed region")
    ap.add_argument("--shard-of", type=int, default=0,
                    help="developer aid: time ONE rank's shard of an N-way tensor-parallel model on one GPU, without its "
                         "peers (results are not the model's outputs; the line is labelled)")
    ap.add_argument("--skip-parity", action="store_true", help="skip the oracle comparison that follows the timed region")
    ap.add_argument("--skip-other-configs", action="store_true",
                    help="skip the short decode runs of the other benchmark configurations (single-GPU default run only)")
    ap.add_argument("--skip-fill", action="store_true",
                    help="leave the KV cache zero-filled instead of prefilling it (same traffic; for profiler runs)")
    return ap.parse_args()


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"]))}, "measured"
    except Exception:
        return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while a timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def mark(self):
        return time.perf_counter()

    def stop(self):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()   # our own child, by handle
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass

    def summary(self, t_begin=None, t_end=None):
        """Median SM clock and the throttle reasons seen between the two marks (all samples if none)."""
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = [r for t, r in self.rows if (t_begin is None or t >= t_begin) and (t_end is None or t <= t_end + 0.12)]
        if not rows:
            rows = [r for _, r in self.rows[-3:]]
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
                for n, v in zip(names, r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def decode_step_bytes(cfg, param_bytes_no_embed, batch, ctx):
    """Algorithmic HBM bytes of one decode step: every streamed parameter once, `batch` embedding
    rows, the K and V of `ctx` cached tokens per sequence, and the new token's K and V."""
    from rai_b200 import configs
    L, d = cfg["num_hidden_layers"], configs.head_dim(cfg)
    nkv = cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    kv_token = 2 * L * nkv * d * 2
    return param_bytes_no_embed + batch * cfg["hidden_size"] * 2 + batch * ctx * kv_token + batch * kv_token


def prefill_flops(cfg, batch, seq):
    """2*params*tokens for the linears, last-position lm_head, causal attention (QK^T and PV)."""
    from rai_b200 import configs
    H, I, L, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"], cfg["vocab_size"]
    nq, d = cfg["num_attention_heads"], configs.head_dim(cfg)
    nkv = cfg.get("num_key_value_heads") or nq
    per_layer = H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I
    linear = 2.0 * per_layer * L * batch * seq + 2.0 * H * V * batch
    attn = L * batch * 2.0 * nq * seq * seq * d  # = 4 * nq * d * seq^2 / 2
    return linear, attn


# --------------------------------------------------------------------------------------------------
# CPU arm: the oracle on the host cores, bounded sample
# --------------------------------------------------------------------------------------------------
def cpu_decode_sample(cfg, batch, ctx, steps, warmup, params=None):
    """Times the CPU restatement on a bounded sample of the same workload: the full-width model with
    1 and 2 layers, batch `batch`, a `ctx`-token cache injected as random K/V, `steps` (>= 5) decode steps
    each after `warmup` untimed ones.  Per-layer and outside-the-layers times are separated by the difference of the
    two medians and extrapolated to the full depth; the spread of the step times is reported with the figure."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import torch
    import adapter
    import rai_cpu
    from rai_b200 import configs, synth

    steps = max(5, int(steps))
    warmup = max(1, int(warmup))
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(1234)
    full_layers = cfg["num_hidden_layers"]
    cfg2 = dict(cfg, num_hidden_layers=2, max_position_embeddings=ctx + steps + warmup + 8)
    if params is None:
        params = {}
        for name, shape, kind in synth.param_shapes(cfg2):
            if kind == "norm_w":
                params[name] = torch.ones(shape)
            else:
                params[name] = torch.randn(shape, generator=g) * 0.02
    nkv = cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    d = configs.head_dim(cfg)
    times, all_ts = {}, {}
    t_wall = time.perf_counter()
    for n_layers in (1, 2):
        c = dict(cfg2, num_hidden_layers=n_layers)
        model = rai_cpu.build(adapter.oracle_config(c), adapter.oracle_params(c, params))
        model.kv = [(torch.randn(batch, nkv, ctx, d, generator=g), torch.randn(batch, nkv, ctx, d, generator=g))
                    for _ in range(n_layers)]
        ids = torch.randint(0, cfg["vocab_size"], (batch, 1), generator=g)
        ts = []
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            logits = model.forward(ids, ctx + i)
            ids = logits.reshape(batch, -1).argmax(-1, keepdim=True)
            if i >= warmup:
                ts.append(time.perf_counter() - t0)
        times[n_layers] = statistics.median(ts)
        all_ts[n_layers] = ts
        del model
    wall = time.perf_counter() - t_wall
    per_layer = max(times[2] - times[1], 1e-9)
    outside = max(times[1] - per_layer, 0.0)
    step_s = outside + full_layers * per_layer
    spread = {n: {"min_ms": min(v) * 1e3, "median_ms": statistics.median(v) * 1e3, "max_ms": max(v) * 1e3} for n, v in all_ts.items()}
    n_run = 2 * (steps + warmup)
    return {"value": batch / step_s, "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": (f"torch-CPU float32 restatement of rai's Cpu path, full-width {cfg['arch']} layers: 1- and 2-layer "
                       f"models, batch {batch}, {ctx}-token cache injected, {steps} timed decode steps each (median) after "
                       f"{warmup} warm-up; per-layer {per_layer * 1e3:.0f} ms, outside layers {outside * 1e3:.0f} ms, "
                       f"extrapolated to {full_layers} layers = {step_s:.2f} s/step"),
            "ms_per_step": step_s * 1e3, "extrapolated": True, "sample_steps_run": n_run,
            "sample_ms_per_step": wall / n_run * 1e3, "sample_wall_s": wall, "spread": spread}


def decode_timeline(model, dev, rewind, first, T0, path=None, steps=4):
    """Kernel start/end times of `steps` decode steps as the device ran them (graph replay, dependent launches
    overlapping), from the CUDA activity records torch's profiler collects.  With dependent launches a kernel's own
    duration includes the time it sits waiting for its predecessor, so the figure kept per kernel name is its
    `advance`: how far it moves the end of the step (its end minus the latest end before it).  One more step is
    traced than is kept: the first traced step starts from an idle device (its first kernel's advance would include the
    profiler's own start-up gap) and is dropped.  Returns the summary (None when no activity records are available) and
    writes it, with the raw sequence of one step, to `path`."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    rewind(T0)
    model.decode_loop(first, T0, 2)
    dev.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        model.decode_loop(first, T0 + 2, steps + 1)
        dev.synchronize()
    evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and e.time_range.end > e.time_range.start]
    evs.sort(key=lambda e: e.time_range.start)
    if not evs:
        return None
    t0 = evs[0].time_range.start
    seq, prev_end = [], None
    for e in evs:
        name = e.name.replace("(anonymous namespace)::", "").replace("void ", "").replace("rb::", "").split("(")[0]
        start, end = e.time_range.start - t0, e.time_range.end - t0
        advance = (end - start) if prev_end is None else max(0.0, end - prev_end)
        prev_end = end if prev_end is None else max(prev_end, end)
        seq.append({"name": name, "start_us": round(start, 2), "dur_us": round(end - start, 2), "advance_us": round(advance, 2)})
    n = len(seq) // (steps + 1)
    kept = seq[n:]                      # drop the first traced step
    by_name = {}
    for x in kept:
        a = by_name.setdefault(x["name"], {"launches": 0, "advance_us": 0.0})
        a["launches"] += 1
        a["advance_us"] += x["advance_us"]
    span = (max(x["start_us"] + x["dur_us"] for x in kept) - max(x["start_us"] + x["dur_us"] for x in seq[:n])) if n else 0.0
    per_step = {k: {kk: round(vv / steps, 2) for kk, vv in v.items()} for k, v in by_name.items()}
    out = {"steps": steps, "span_us_per_step": round(span / steps, 1), "per_kernel_per_step": per_step}
    if path:
        json.dump(dict(out, one_step=seq[n:2 * n]), open(path, "w"), indent=1)
    return out


CPU_SAMPLE_STEPS, CPU_SAMPLE_WARMUP = 6, 1   # the same sample in the GPU arm's cpu_baseline and in the reference arm


def run_reference(args):
    """The reference arm: rai's Cpu path (its op-for-op restatement; rai itself cannot be built here) on the host
    cores.  Every "step" it runs is one decode step of a bounded sample (full-width 1- and 2-layer models); the
    line's `steps` and `ms_per_step` describe exactly what ran, so that steps x ms_per_step is this run's own
    time, and `value` is the tokens/s extrapolated to the full depth (`extrapolated: true`)."""
    from rai_b200 import configs
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = configs.get(args.config)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    t0 = time.perf_counter()
    base = cpu_decode_sample(cfg, args.decode_batch, args.context, CPU_SAMPLE_STEPS, CPU_SAMPLE_WARMUP)
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": base["value"], "unit": "tok/s",
        "n_gpus": args.gpus, "steps": base["sample_steps_run"], "warmup": 0, "ms_per_step": base["sample_ms_per_step"],
        "requested_steps": args.steps, "requested_warmup": args.warmup,
        "extrapolated": True, "full_depth_ms_per_step": base["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, cfg, args.gpus),
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample", "spread")},
        "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t0,
        "note": ("rai's Cpu (candle) path cannot be built in this environment (no Rust toolchain); this is its "
                 f"op-for-op restatement timed on {base['cores']} host threads.  `steps` and `ms_per_step` are the sample "
                 "steps actually run (1- and 2-layer full-width models) and their mean duration; `value` extrapolates the "
                 "per-layer time to the full depth"),
    }
    print(json.dumps(line), flush=True)


def workload_config(args, cfg, n):
    return {"workload": (f"{args.config} architecture, bf16, batch-{args.decode_batch} greedy decode with KV cache at a "
                         f"{args.context}-token context (+1 per step); prefill {args.prefill_batch} x {args.prefill_len}"),
            "layers": cfg["num_hidden_layers"], "decode_batch": args.decode_batch, "context": args.context,
            "prefill_batch": args.prefill_batch, "prefill_len": args.prefill_len,
            "parallelism": f"tp{n}", "l2": "inputs larger than L2 (>= 14 GB of weights and KV streamed per step)"}


OTHER_CONFIGS = [  # (name, decode batch, context): configurations 1-4 of the benchmark definition
    ("qwen2-0.5b", 1, 128), ("phi2", 8, 512), ("phi3-mini", 4, 2048), ("gemma-2b", 32, 1024)]


def other_configs():
    """Decode ms/step and whole-step roofline fraction of the other benchmark configurations: a short run of this
    same script per configuration, each in a process of its own."""
    out = {}
    for name, batch, ctx in OTHER_CONFIGS:
        cmd = [sys.executable, os.path.abspath(__file__), "--config", name, "--decode-batch", str(batch), "--context", str(ctx),
               "--steps", "24", "--warmup", "3", "--profile-steps", "1", "--skip-cpu", "--skip-e2e", "--skip-prefill",
               "--skip-timeline", "--skip-parity", "--skip-other-configs"]
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
            d = json.loads(r.stdout.strip().splitlines()[-1])
            out[name] = {"decode_batch": batch, "context": ctx, "ms_per_step": d["ms_per_step"], "tok_s": d["value"],
                         "frac_of_measured_copy": d["roofline"]["whole_step"]["frac_of_measured_copy"],
                         "frac_of_nominal_8tbs": d["roofline"]["whole_step"]["frac_of_nominal_8tbs"],
                         "graph": d["decode_step_is_cuda_graph"]}
        except Exception as e:
            out[name] = {"error": f"{type(e).__name__}: {e}"}
    return out


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    if args.shard_of > 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1:
        # developer aid: needs the developer build of the library (python -m rai_b200.build --debug-aids)
        os.environ["RAI_B200_DEBUG_AIDS"] = "1"
        os.environ["RAI_B200_SHARD_ONLY"] = "1"
    from rai_b200 import _lib, configs, synth
    from rai_b200.device import Cuda
    from rai_b200.models import Model

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    cfg = configs.get(args.config)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    B, T0, K, W = args.decode_batch, args.context, args.steps, args.warmup
    PB, PS = args.prefill_batch, args.prefill_len
    chunk = 256
    max_seq = max(T0 + K + W + 64, 0 if args.skip_prefill else PS)
    cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], max_seq)
    max_tokens = max(B * chunk, 0 if args.skip_prefill else PB * PS)
    dev = Cuda(local)
    model = Model(cfg, _lib.BF16, dev, max(B, PB), max_seq, max_tokens, tp_rank=rank,
                  tp_size=args.shard_of if (args.shard_of > 1 and world == 1) else world)
    if world > 1:
        uid = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            buf = ctypes.create_string_buffer(128)
            _lib.call("rb_tp_unique_id", buf)
            uid = torch.tensor(list(buf.raw), dtype=torch.uint8, device="cuda")
        dist.broadcast(uid, 0)
        model.tp_init(bytes(uid.cpu().tolist()))

    # ---- random-init weights, generated on the device (identical on every rank; the library shards)
    gen = torch.Generator(device="cuda").manual_seed(1234)
    for name, shape, kind in synth.param_shapes(cfg):
        if kind == "norm_w":
            w = torch.ones(shape, device="cuda", dtype=torch.bfloat16)
        else:
            w = (torch.randn(shape, generator=gen, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
        model.update_param(name, w)
        del w
    model.finalize()
    torch.cuda.empty_cache()
    cache = ctypes.c_void_p(_lib.lib().rb_model_kv_cache(model._m))
    tok_gen = torch.Generator(device="cuda").manual_seed(99)

    def rewind(n_tokens):
        _lib.call("rb_kv_cache_set_len", cache, B, n_tokens)

    # ---- fill the cache to the decode context by really prefilling random prompts, chunk by chunk
    model.clear_kv_cache()
    logits_buf = torch.empty((max(B, PB), cfg["vocab_size"]), dtype=torch.bfloat16, device="cuda")
    for pos in range(0, 0 if args.skip_fill else T0, chunk):
        n = min(chunk, T0 - pos)
        ids = torch.randint(0, cfg["vocab_size"], (B, n), generator=tok_gen, device="cuda", dtype=torch.int32)
        _lib.call("rb_model_forward", model._m, ctypes.c_void_p(ids.data_ptr()), B, n, pos,
                  ctypes.c_void_p(logits_buf.data_ptr()))
    dev.synchronize()
    if args.skip_fill:
        rewind(T0)
        logits_buf.zero_()
    first = logits_buf[:B].float().argmax(-1).to(torch.int32).contiguous()

    # ---- decode: W warm-up steps, rewind, then exactly K timed steps on the device
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    if W > 0:
        model.decode_loop(first, T0, W)
        dev.synchronize()
    rewind(T0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    launches0 = dev.launch_count()
    t_begin = sampler.mark()
    torch.cuda.nvtx.range_push("decode_timed")
    e0.record()
    out_tokens = model.decode_loop(first, T0, K)
    e1.record()
    barrier()
    dev.synchronize()
    torch.cuda.nvtx.range_pop()
    t_end = sampler.mark()
    decode_ms = max_over_ranks(e0.elapsed_time(e1))
    launches = dev.launch_count() - launches0
    if rank == 0:
        sampler.stop()
    clocks = sampler.summary(t_begin, t_end) if rank == 0 else None
    decode_tok_s = B * K / (decode_ms / 1e3)
    graph_active = bool(_lib.lib().rb_model_decode_graph_active(model._m))
    if not graph_active and os.environ.get("RAI_B200_GRAPH") != "0":
        # a capture that failed would fall back to plain launches for the model's life: not a number to report quietly
        raise SystemExit("bench: the decode step did not run as a captured graph (RAI_B200_VERBOSE=1 says why)")

    # ---- per-kernel-class timing of the same steps (event pair around every launch; separate pass)
    classes = ["gemm", "attention", "norm", "rope_kv", "embed", "argmax", "other"]
    prof = {}
    PK = max(1, min(args.profile_steps, K))
    rewind(T0)
    _lib.call("rb_profile_start", dev.ctx)
    plain_tokens = model.decode_loop(first, T0, PK)   # launch by launch (profiling switches the captured step off)
    for i, cname in enumerate(classes):
        out4 = (ctypes.c_double * 4)()
        _lib.call("rb_profile_read", dev.ctx, i, out4)
        if out4[0] > 0:
            prof[cname] = {"launches_per_step": out4[0] / PK, "ms_per_step": out4[1] / PK,
                           "gbytes_per_step": out4[2] / PK / 1e9, "avg_launch_us": out4[1] / out4[0] * 1e3,
                           "achieved_gbs": out4[2] / 1e9 / (out4[1] / 1e3) if out4[1] > 0 else None}
    dev.synchronize()
    # the captured, replayed step and the launch-by-launch step must produce the same tokens
    graph_equals_plain = bool(torch.equal(plain_tokens, out_tokens[:PK]))

    # ---- the same steps as the device ran them (graph replay, overlap included): a tracing pass of its own
    # (single GPU only: the decode steps of a tensor-parallel group are collective, so a pass that one rank runs
    # alone would leave it waiting for peers that never come)
    in_graph = None
    if world == 1 and not args.skip_timeline:
        try:
            in_graph = decode_timeline(model, dev, rewind, first, T0, args.timeline or None)
        except Exception as e:  # tracing is an extra: the bench line does not depend on it
            in_graph = {"error": f"{type(e).__name__}: {e}"}

    # ---- end to end through the generation-step call: pinned host tokens in, token ids out, per step
    e2e = None
    if not args.skip_e2e:
        rewind(T0)
        tin = first.cpu().reshape(B, 1).pin_memory()
        tout = torch.empty(B, dtype=torch.int32).pin_memory()
        for i in range(min(W, 3)):
            model.generate_step(tin, T0 + i, tout)
            tin.copy_(tout.reshape(B, 1))
        rewind(T0)
        tin.copy_(first.cpu().reshape(B, 1))
        barrier()
        t0 = time.perf_counter()
        for i in range(K):
            model.generate_step(tin, T0 + i, tout)
            tin.copy_(tout.reshape(B, 1))
        barrier()
        e2e_s = max_over_ranks(time.perf_counter() - t0)
        e2e = {"value": B * K / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": B * 4, "d2h_bytes_per_step": B * 4,
               "ms_per_step": e2e_s / K * 1e3,
               "api": "rb_model_generate_step: pinned host token ids -> H2D -> forward -> on-device argmax -> D2H"}

    # ---- prefill: PB x PS tokens from an empty cache
    prefill = None
    if not args.skip_prefill:
        ids = torch.randint(0, cfg["vocab_size"], (PB, PS), generator=tok_gen, device="cuda", dtype=torch.int32)

        def one_prefill():
            model.clear_kv_cache()
            _lib.call("rb_model_forward", model._m, ctypes.c_void_p(ids.data_ptr()), PB, PS, 0,
                      ctypes.c_void_p(logits_buf.data_ptr()))
        psampler = ClockSampler(local)
        if rank == 0:
            psampler.start()
        one_prefill()
        dev.synchronize()
        reps = 3
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        pt0 = psampler.mark()
        torch.cuda.nvtx.range_push("prefill_timed")
        p0.record()
        for _ in range(reps):
            one_prefill()
        p1.record()
        barrier()
        dev.synchronize()
        torch.cuda.nvtx.range_pop()
        pt1 = psampler.mark()
        if rank == 0:
            psampler.stop()
        pms = max_over_ranks(p0.elapsed_time(p1)) / reps
        lin, att = prefill_flops(cfg, PB, PS)
        prefill = {"tokens_per_s": PB * PS / (pms / 1e3), "ms_per_pass": pms, "tflops": (lin + att) / 1e12 / (pms / 1e3),
                   "flops_linear": lin, "flops_attention_causal": att, "passes": reps,
                   "clocks": psampler.summary(pt0, pt1) if rank == 0 else None}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peaks, peak_kind = measured_peaks()
    # whole-model parameter bytes streamed per step: everything but the embedding table (of which only
    # `batch` rows are read), unless the table doubles as lm_head
    param_no_embed = sum(2 * int(__import__("math").prod(shape)) for name, shape, _ in synth.param_shapes(cfg)
                         if name != "model.embed_tokens.weight" or configs.tied(cfg))
    bytes_first = decode_step_bytes(cfg, param_no_embed, B, T0)
    bytes_last = decode_step_bytes(cfg, param_no_embed, B, T0 + K - 1)
    step_bytes = 0.5 * (bytes_first + bytes_last)
    step_gbs = step_bytes / 1e9 / (decode_ms / K / 1e3)
    gemm = prof.get("gemm", {})
    # The dominant kernel class, per GPU: rank 0's launches over rank 0's shard against ONE GPU's peak.
    profiled_case = world == 1 and args.config == "qwen2-7b" and B == 64
    roofline = {
        "bound": "hbm", "kernel": "gemm_tc_kernel (weight-streaming tcgen05 GEMM; all Linear layers of a decode step)",
        "achieved": gemm.get("achieved_gbs"), "peak": peaks["hbm_gbs"], "unit": "GB/s",
        "frac": (gemm["achieved_gbs"] / peaks["hbm_gbs"]) if gemm.get("achieved_gbs") else None,
        "peak_kind": f"{peak_kind} stream-copy bandwidth of one GPU; achieved is rank 0's own launches over its own shard",
        # DRAM bytes per launch are not measured by this run: ncu measured 478.6 MB of DRAM read+write for the four
        # GEMMs of one layer against 486.2 MB of algorithmic bytes (0.98; the float32 split-K partials mostly stay in
        # L2) on the 2-layer single-GPU case of the summary named below.  Given for that configuration only.
        "traffic": (0.98 * gemm["gbytes_per_step"] * 1e9 / gemm["launches_per_step"]) if (gemm and profiled_case) else None,
        "traffic_source": ("profiles/gemm_tc_decode_2layer_b64.md (ncu dram__bytes_read+write on a 2-layer case, 0.98 of "
                           "algorithmic, scaled by this run's algorithmic bytes per launch)") if profiled_case else None,
        "algorithmic_bytes_per_launch": (gemm["gbytes_per_step"] * 1e9 / gemm["launches_per_step"]) if gemm else None,
        "avg_launch_us": gemm.get("avg_launch_us"), "launches_per_step": gemm.get("launches_per_step"),
        "algorithmic_gbytes_per_step": gemm.get("gbytes_per_step"),
        # the whole model's algorithmic bytes per step over the whole job's time, against N GPUs' bandwidth
        "whole_step": {"algorithmic_gbytes": step_bytes / 1e9, "achieved_gbs": step_gbs, "gpus": world,
                       "frac_of_measured_copy": step_gbs / (peaks["hbm_gbs"] * world),
                       "frac_of_nominal_8tbs": step_gbs / (NOMINAL_HBM_GBS * world)},
        "per_class": prof,
    }
    if in_graph and "per_kernel_per_step" in in_graph and gemm:
        # The per-launch figures above time every launch alone (an event pair around it, no overlap with its
        # neighbours).  In the replayed step consecutive kernels overlap (dependent launches, weights requested
        # ahead of the dependency), so there the GEMMs' share of the step is their `advance`.
        adv = sum(v["advance_us"] for k, v in in_graph["per_kernel_per_step"].items() if k.startswith("gemm_tc_kernel"))
        roofline["in_graph"] = {
            "method": "CUDA activity records of the replayed step; per kernel: its end minus the latest end before it",
            "span_us_per_step": in_graph["span_us_per_step"], "gemm_advance_us_per_step": adv,
            "gemm_achieved_gbs": (gemm["gbytes_per_step"] * 1e6 / adv) if adv > 0 else None,
            "gemm_frac": (gemm["gbytes_per_step"] * 1e6 / adv / peaks["hbm_gbs"]) if adv > 0 else None,
            "per_kernel_per_step": in_graph["per_kernel_per_step"]}
    elif in_graph:
        roofline["in_graph"] = in_graph
    if prefill:
        prefill["frac_of_measured_sustained_bf16"] = prefill["tflops"] / (peaks["bf16_tflops_sustained"] * world)
        prefill["frac_of_nominal_bf16"] = prefill["tflops"] / (NOMINAL_BF16_TFLOPS * world)
    # ---- after the timed region: the CPU arm and the oracle comparison share one set of 2-layer full-width weights
    cpu, parity = None, {"graph_replay_equals_plain_launch_tokens": graph_equals_plain, "steps_compared": PK}
    if world == 1 and (not args.skip_cpu or not args.skip_parity):
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import parity_kit
        cfg2 = dict(cfg, num_hidden_layers=min(2, cfg["num_hidden_layers"]))
        cfg2["max_position_embeddings"] = max(cfg2["max_position_embeddings"], T0 + 64)
        params2 = parity_kit.rounded_params(cfg2, 4321)
        if not args.skip_parity:
            # the timed shape (batch, context) on a 2-layer model of the same widths, from an injected cache, through the
            # same entry points, against the oracle: logits within 2e-2 of the logit range, greedy tokens equal except at
            # reference near-ties
            pm = Model(cfg2, _lib.BF16, dev, B, T0 + 16, B)
            for k, v in params2.items():
                pm.update_param(k, v)
            pm.finalize()
            parity.update(parity_kit.decode_parity(cfg2, params2, pm, B, T0, 2, 4322))
            parity["ok"] = bool(graph_equals_plain and parity["max_logit_err_of_range"] <= parity["tolerance"]
                                and parity["of_which_not_near_ties"] == 0)
            pm.close()
        if not args.skip_cpu:
            base = cpu_decode_sample(cfg, B, T0, CPU_SAMPLE_STEPS, CPU_SAMPLE_WARMUP, params=params2)
            cpu = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample", "spread")}
        del params2
    other = None
    if world == 1 and not args.skip_other_configs and args.config == "qwen2-7b" and not args.layers and not args.shard_of:
        other = other_configs()
    line = {
        "metric": "decode_tokens_per_s", "value": decode_tok_s, "unit": "tok/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": decode_ms / K, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, cfg, world), "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches),
        "roofline": roofline, "cpu_baseline": cpu, "prefill": prefill,
        "decode_step_is_cuda_graph": graph_active,
        "shard_only_of": args.shard_of or None,
        "tokens_checksum": int(out_tokens.to(torch.int64).sum().item()),
        "parity_checked": parity, "other_configs": other,
    }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
