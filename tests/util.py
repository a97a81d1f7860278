"""Helpers shared by the tests: build the CPU oracle and the CUDA model from one seeded weight set."""
import numpy as np
import torch

import rai_cpu  # noqa: F401  (oracle/rai_cpu.py, test infrastructure)
from adapter import build_oracle, oracle_config, oracle_params  # noqa: F401  (oracle/adapter.py)


def logit_error(got: torch.Tensor, want: torch.Tensor) -> float:
    """max |got - want| relative to the range of the reference logits."""
    got, want = got.float().cpu().reshape(-1), want.float().reshape(-1)
    rng = float(want.max() - want.min())
    return float((got - want).abs().max()) / max(rng, 1e-12)


def rel_error(got: torch.Tensor, want: torch.Tensor) -> float:
    """max |got - want| / max |want| — the "relative" error used for float32 comparisons."""
    got, want = got.float().cpu().reshape(-1), want.float().reshape(-1)
    return float((got - want).abs().max()) / max(float(want.abs().max()), 1e-12)


def top2_margin(logits: torch.Tensor) -> torch.Tensor:
    v = logits.float().topk(2, dim=-1).values
    return v[..., 0] - v[..., 1]
