"""Run under torch.distributed.run with N ranks (one GPU each): tensor-parallel forward of tiny
decoders through the C ABI against the CPU oracle.  Exits non-zero on mismatch.  Used by
tests/test_gpu_50_tp.py; NCCL's in-switch reduction is switched off by the caller."""
import ctypes
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (ROOT, os.path.join(ROOT, "oracle"), HERE):
    sys.path.insert(0, p)

import rai_cpu  # noqa: E402
import util  # noqa: E402
from rai_b200 import _lib, configs, synth  # noqa: E402
from rai_b200.device import Cuda  # noqa: E402
from rai_b200.models import Model  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")   # rendezvous and id exchange only; the data path is the library's NCCL
    dev = Cuda(local)
    failures = []
    cases = [("tiny-qwen2", _lib.F32, 1e-4), ("tiny-qwen2", _lib.BF16, 2e-2), ("tiny-qwen2-28h", _lib.BF16, 2e-2),
             ("tiny-qwen2-g7", _lib.BF16, 2e-2), ("tiny-phi2", _lib.BF16, 2e-2), ("tiny-phi3", _lib.BF16, 2e-2),
             ("tiny-gemma", _lib.BF16, 2e-2)]
    # the benchmark's own shard shapes: full-width qwen2-7b (at 8 ranks: 4 query heads per rank with a padded head,
    # a KV head shared by a rank pair, 2368 intermediate units) and phi2, cut to two layers so that the CPU oracle
    # finishes in seconds
    if os.environ.get("TP_CHECK_FULL", "1") == "1":
        cases += [("qwen2-7b", _lib.BF16, 2e-2), ("phi2", _lib.BF16, 2e-2)]
    only = os.environ.get("TP_CHECK_ONLY")          # debugging: comma-separated configuration names
    prompts = [int(x) for x in os.environ.get("TP_CHECK_PROMPTS", "40,150").split(",")]
    for name, dtype, tol in cases:
        if only and name not in only.split(","):
            continue
        cfg = configs.get(name)
        full_width = name in configs.BASELINE
        if full_width:
            cfg["num_hidden_layers"] = 2
        nkv = cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
        if not ((world <= nkv and nkv % world == 0) or (world > nkv and world % nkv == 0)):
            continue
        if cfg["intermediate_size"] % world or cfg["vocab_size"] % world:
            continue
        w = synth.weights(cfg, 31)
        m = Model(cfg, dtype, dev, 2, 256, tp_rank=rank, tp_size=world)
        uid = [None]
        if rank == 0:
            buf = ctypes.create_string_buffer(128)
            _lib.call("rb_tp_unique_id", buf)
            uid = [buf.raw]
        dist.broadcast_object_list(uid, 0)
        m.tp_init(uid[0])
        m.update_params(w)
        # 80 prompt rows go through the peer-memory exchange, 300 rows through NCCL; decode steps
        # (2 rows) always through the exchange
        for plen in (prompts[:1] if full_width else prompts):
            prompt = synth.prompt(cfg, 2, plen, 31)
            want = ref = None
            if rank == 0:
                want, ref = rai_cpu.greedy_generate(util.build_oracle(cfg, w), torch.from_numpy(prompt.astype(np.int64)), 6, True)
            box = [want]
            dist.broadcast_object_list(box, 0)     # every rank is fed the reference's tokens (teacher forcing)
            want_all = box[0]
            m.clear_kv_cache()
            ids, pos, errs, flips = prompt, 0, [], 0
            for t in range(6):
                logits = m.forward(ids, pos).reshape(2, -1).float().cpu()
                pos += ids.shape[1]
                ids = want_all[:, t:t + 1].numpy()
                if rank == 0:
                    errs.append(util.logit_error(logits, ref[t]) if dtype == _lib.BF16 else util.rel_error(logits, ref[t]))
                    for b in range(2):
                        if int(logits[b].argmax()) != int(want[b, t]):
                            margin = float(util.top2_margin(ref[t, b]))
                            rng = float(ref[t, b].max() - ref[t, b].min())
                            flips += 1
                            if dtype == _lib.F32 or margin >= tol * rng:   # a flip is only excused at a genuine near-tie
                                failures.append(f"{name} prompt {plen} step {t} seq {b}: token differs, margin {margin / rng:.1e}")
            if rank == 0:
                print(f"tp{world} {name} dtype {dtype} prompt {plen}: logits error per step " + " ".join(f"{e:.1e}" for e in errs)
                      + f", greedy tokens differing at near-ties: {flips}", flush=True)
                if max(errs) > tol:
                    failures.append(f"{name} prompt {plen}: logits error {max(errs):.2e}")
        m.close()
        dist.barrier()
    dist.destroy_process_group()
    if failures:
        print("FAILURES:", failures, flush=True)
    sys.exit(1 if failures else 0)


if __name__ == "__main__":
    main()
