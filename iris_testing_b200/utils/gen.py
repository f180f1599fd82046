"""Deterministic synthetic data: seeds, tokens, router and expert weights.

Behavioural counterparts of the reference generators (utils.py:125-173,
utils.py:248-261): tokens differ per rank (seed + rank), the router is the same
on every rank (seed + 777), expert weights differ per rank (seed + 12345 + rank).
Unlike the reference these work on any device, so the CPU/gloo tests and the
GPU paths draw from the same functions.
"""
from __future__ import annotations

import random
from typing import Optional, Tuple

import numpy as np
import torch

ROUTER_SEED_OFFSET = 777
WEIGHT_SEED_OFFSET = 12345


def set_seed(base_seed: int, rank: int = 0) -> None:
    """Seed python, numpy and torch (CPU and every visible GPU) with base_seed + rank."""
    s = int(base_seed) + int(rank)
    random.seed(s)
    np.random.seed(s % (2 ** 32))
    torch.manual_seed(s)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(s)


def _generator(device: torch.device, seed: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def gen_local_tokens(batch: int, seq: int, hidden_dim: int, dtype: torch.dtype,
                     device, base_seed: int, rank: int, dist: str = "uniform") -> torch.Tensor:
    """This rank's tokens, shape [batch*seq, hidden_dim].

    ``dist="uniform"`` draws from U[0, 1) as the reference does (utils.py:153);
    ``dist="normal"`` draws from N(0, 1), which the benchmark shapes use.
    """
    device = torch.device(device)
    g = _generator(device, int(base_seed) + int(rank))
    shape = (batch * seq, hidden_dim)
    if dist == "uniform":
        x = torch.rand(shape, generator=g, device=device, dtype=torch.float32)
    elif dist == "normal":
        x = torch.randn(shape, generator=g, device=device, dtype=torch.float32)
    else:
        raise ValueError(f"unknown token distribution {dist!r}")
    return x.to(dtype)


def gen_router(hidden_dim: int, num_experts: int, dtype: torch.dtype, device, base_seed: int,
               std: Optional[float] = 0.001) -> torch.Tensor:
    """Router matrix [hidden_dim, num_experts], identical on every rank.

    ``std=0.001`` is the reference's scale (utils.py:171-172); ``std=None``
    selects N(0, 1/hidden_dim), the scale of the benchmark shapes.
    """
    device = torch.device(device)
    g = _generator(device, int(base_seed) + ROUTER_SEED_OFFSET)
    if std is None:
        std = float(hidden_dim) ** -0.5
    w = torch.randn((hidden_dim, num_experts), generator=g, device=device, dtype=torch.float32) * std
    return w.to(dtype)


def gen_local_weights(e_local: int, hidden_dim: int, out_dim: int, dtype: torch.dtype, device,
                      base_seed: int, rank: int, std: float = 0.02) -> torch.Tensor:
    """Per-rank expert weights [e_local, hidden_dim, out_dim] ~ N(0, std)."""
    device = torch.device(device)
    g = _generator(device, int(base_seed) + WEIGHT_SEED_OFFSET + int(rank))
    w = torch.randn((e_local, hidden_dim, out_dim), generator=g, device=device, dtype=torch.float32) * std
    return w.to(dtype)


def gen_gated_expert_weights(e_local: int, hidden_dim: int, ffn_dim: int, dtype: torch.dtype, device,
                             base_seed: int, rank: int, std: float = 0.02
                             ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(W1 [e, D, F], W3 [e, D, F], W2 [e, F, D]) of a SiLU-gated expert MLP."""
    device = torch.device(device)
    g = _generator(device, int(base_seed) + WEIGHT_SEED_OFFSET + int(rank))
    w1 = torch.randn((e_local, hidden_dim, ffn_dim), generator=g, device=device, dtype=torch.float32) * std
    w3 = torch.randn((e_local, hidden_dim, ffn_dim), generator=g, device=device, dtype=torch.float32) * std
    w2 = torch.randn((e_local, ffn_dim, hidden_dim), generator=g, device=device, dtype=torch.float32) * std
    return w1.to(dtype), w3.to(dtype), w2.to(dtype)


def zipf_expert_bias(num_experts: int, s: float = 1.2, scale: float = 1.0, seed: int = 0,
                     device="cpu") -> torch.Tensor:
    """Per-expert logit bias whose ranking follows a Zipf(s) law (skewed load).

    Expert ranks are a seeded permutation; the bias of the expert with rank r is
    ``scale * log(r ** -s)`` shifted to zero mean.
    """
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))
    perm = torch.randperm(num_experts, generator=g)
    ranks = torch.empty(num_experts, dtype=torch.float32)
    ranks[perm] = torch.arange(1, num_experts + 1, dtype=torch.float32)
    bias = scale * (-s) * torch.log(ranks)
    return (bias - bias.mean()).to(device)
