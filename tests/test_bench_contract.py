"""The benchmark's reference arm (the CPU restatement timed on the host cores) on a tiny configuration: one JSON
line on stdout with the keys the contract names.  The GPU arm shares the line-building code but needs a B200."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--config", "tiny-qwen2",
                        "--decode-batch", "2", "--context", "16", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.strip().splitlines() if l.strip()]
    assert len(lines) == 1, "exactly one line on stdout"
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "decode_tokens_per_s" and d["unit"] == "tok/s"
    for key in ("value", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline", "dtype",
                "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["value"] > 0 and d["higher_is_better"] is True and d["vs_baseline"] is None
    assert set(("kind", "cores", "sample", "value", "unit")) <= set(d["cpu_baseline"])
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"]["value"] == d["value"] and d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in d["config"] and "model" not in d["config"]
    # the line describes what actually ran: the sample steps and their mean duration, flagged as extrapolated
    assert d["extrapolated"] is True and d["steps"] >= 10 and d["full_depth_ms_per_step"] > 0
    assert d["steps"] * d["ms_per_step"] / 1e3 <= d["wall_s"] + 0.5
    assert "spread" in d["cpu_baseline"]


def test_other_ranks_of_the_reference_arm_exit_quietly():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--config",
                        "tiny-qwen2", "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_single_rank_passes_of_the_gpu_arm_are_not_collective():
    """A tensor-parallel decode step is collective (exchange flags, NCCL gathers): any extra pass over decode steps must
    run on every rank or on single-GPU runs only.  The device-timeline pass is the one extra that is rank-local."""
    import re
    src = open(os.path.join(ROOT, "bench.py")).read()
    calls = [m.start() for m in re.finditer(r"in_graph = decode_timeline\(", src)]
    assert len(calls) == 1
    guard = src.rfind("if ", 0, calls[0])
    assert "world == 1" in src[guard:calls[0]], "the timeline pass must be limited to single-GPU runs"


def test_every_committed_profile_names_a_safe_reproducible_command():
    """Each summary under profiles/ gives the command that made it; every ncu command among them leaves the clocks
    alone, runs a committed file, and asks for whole sections only on the reduced (2-layer) case."""
    import glob
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    files = sorted(glob.glob(os.path.join(root, "profiles", "*.md")))
    assert files, "no profile summaries committed"
    for path in files:
        text = open(path).read()
        commands = re.findall(r"```\n(.*?)\n```", text, flags=re.S)
        assert commands, f"{os.path.basename(path)} does not say how it was made"
        for cmd in commands:
            assert "bench.py" in cmd, f"{os.path.basename(path)}: the command runs something other than the bench"
            if cmd.lstrip().startswith("ncu"):
                assert "--clock-control none" in cmd, f"{os.path.basename(path)}: ncu would lock the clocks"
                if "--set full" in cmd or "--section" in cmd:
                    assert "--layers 2" in cmd and re.search(r"-c [1-4]\b", cmd), \
                        f"{os.path.basename(path)}: a multi-pass capture must stay on the small case, a few launches"
