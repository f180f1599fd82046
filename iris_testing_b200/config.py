"""Frozen configuration of one expert-parallel MoE layer.

The reference project configures everything through environment variables
(benchmark.py:17-22, benchmark.py:446-453); :func:`MoEConfig.from_env` accepts
the same names, and the dataclass is what the rest of this package consumes.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, replace
from typing import Optional

import torch


@dataclass(frozen=True)
class MoEConfig:
    hidden_dim: int                 # D (reference: HIDDEN)
    ffn_dim: int                    # F; ignored when ``gated`` is False and ``ffn_dim`` == 0
    num_experts: int                # E over the whole expert-parallel group
    topk: int
    world_size: int = 1
    gated: bool = True              # SiLU-gated MLP (W1, W3, W2); False: a single Linear D -> ffn_dim
    renormalize: bool = False       # renormalise the top-k softmax weights to sum to 1
    dtype: torch.dtype = torch.bfloat16
    capacity_factor: Optional[float] = 1.25   # receive capacity over the balanced load; None: worst case
                                              # (every routed copy of every rank), world_size x the memory
    wait_budget_ms: float = 2000.0  # budget of every bounded device-side wait
    cta_pair: Optional[bool] = None  # two CTAs per MMA (cta_group::2); None: when experts average >= 128 rows

    def __post_init__(self) -> None:
        if self.num_experts % self.world_size != 0:
            # reference intent: utils.py:197-198 (layers/all_to_all.py:80 has the test inverted)
            raise ValueError("num_experts must be divisible by world_size")
        if not (1 <= self.topk <= self.num_experts):
            raise ValueError("topk must be in [1, num_experts]")

    @property
    def e_local(self) -> int:
        return self.num_experts // self.world_size

    @property
    def out_dim(self) -> int:
        return self.hidden_dim if self.gated else (self.ffn_dim or self.hidden_dim)

    def with_world(self, world_size: int) -> "MoEConfig":
        return replace(self, world_size=world_size)

    @staticmethod
    def from_env(world_size: Optional[int] = None) -> "MoEConfig":
        """Build a config from the reference's environment variables.

        ``HIDDEN``, ``TOPK``, ``E_LOCAL``, ``WORLD_SIZE`` keep the meaning they
        have in benchmark.py:446-453; ``FFN`` is new (0 selects the ungated
        single-Linear expert of layers/expert.py).
        """
        w = world_size if world_size is not None else int(os.getenv("WORLD_SIZE", "8"))
        e_local = int(os.getenv("E_LOCAL", "4"))
        ffn = int(os.getenv("FFN", "0"))
        return MoEConfig(
            hidden_dim=int(os.getenv("HIDDEN", "4096")),
            ffn_dim=ffn,
            num_experts=w * e_local,
            topk=int(os.getenv("TOPK", "2")),
            world_size=w,
            gated=ffn > 0,
        )


# Named shapes used by the benchmark drivers.
PRESETS = {
    # Mixtral-8x7B MoE block: the flagship benchmark shape.
    "mixtral-8x7b": dict(hidden_dim=4096, ffn_dim=14336, num_experts=8, topk=2, gated=True),
    # Fine-grained experts (DeepSeek-style block size).
    "fine-grained": dict(hidden_dim=2048, ffn_dim=1408, num_experts=64, topk=8, gated=True),
    # Large experts with skewed routing.
    "large": dict(hidden_dim=6144, ffn_dim=16384, num_experts=8, topk=2, gated=True),
    # Two Mixtral-sized experts: same tiles as the flagship, small enough for a profiler capture.
    "mixtral-2e": dict(hidden_dim=4096, ffn_dim=14336, num_experts=2, topk=2, gated=True),
    # Small shape for smoke tests.
    "tiny": dict(hidden_dim=256, ffn_dim=512, num_experts=8, topk=2, gated=True),
}


def preset(name: str, world_size: int = 1, **overrides) -> MoEConfig:
    kw = dict(PRESETS[name])
    kw.update(overrides)
    return MoEConfig(world_size=world_size, **kw)
