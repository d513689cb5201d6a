"""Seeded synthetic inputs for the named gdn_forward shapes.

Real activations are not available offline, so every benchmark and parity case uses
CPU-generated tensors with the shapes and value distributions of the named
configurations: q,k ~ N(0,1) L2-normalised per head vector (BF16); v ~ N(0,1) BF16;
g a natural-log decay (FP32 or BF16); beta in (0,1) BF16; optional FP32 initial state.
Generation is on the CPU with an explicit ``torch.Generator`` so that the device path
and the CPU checker always see identical bits.
"""
from __future__ import annotations

from dataclasses import dataclass, replace

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class Workload:
    name: str
    batch: int
    length: int
    key_heads: int
    value_heads: int
    gate: str = "logsigmoid"      # "logsigmoid": logsigmoid(N(0,1)+2); "slow": -0.01*U(0,1)
    gate_dtype: str = "fp32"      # "fp32" | "bf16"
    beta_shift: float = 0.0       # beta = sigmoid(N(0,1) + beta_shift)
    initial: float | None = None  # std of the FP32 initial state; 0.0 = zero tensor; None = absent
    seed: int = 1000

    @property
    def shape(self):
        return (self.batch, self.length, self.key_heads, self.value_heads)

    @property
    def tokens(self):
        return self.batch * self.length

    def sliced(self, **changes):
        return replace(self, **changes)


WORKLOADS = {
    # headline metric shape
    "headline": Workload("headline", 1, 8192, 16, 32, seed=999),
    "cfg0": Workload("cfg0", 1, 2048, 16, 32, seed=1000),
    "cfg1": Workload("cfg1", 1, 8192, 16, 48, initial=0.05, seed=1001),
    "cfg2": Workload("cfg2", 8, 4096, 16, 32, gate_dtype="bf16", initial=0.0, seed=1002),
    "cfg3": Workload("cfg3", 4, 3000, 8, 32, gate="slow", beta_shift=1.0, initial=0.1, seed=1003),
    "cfg4": Workload("cfg4", 1, 131072, 16, 32, initial=0.0, seed=1004),
}


def make_inputs(w: Workload, device="cpu", pin=False):
    """Returns (q, k, v, g, beta, initial_state_or_None) generated on CPU, then moved."""
    gen = torch.Generator().manual_seed(w.seed)
    b, t, hk, hv = w.shape

    def normal(*shape):
        return torch.randn(*shape, generator=gen)

    q = F.normalize(normal(b, t, hk, 128), dim=-1).to(torch.bfloat16)
    k = F.normalize(normal(b, t, hk, 128), dim=-1).to(torch.bfloat16)
    v = normal(b, t, hv, 128).to(torch.bfloat16)
    if w.gate == "logsigmoid":
        g = F.logsigmoid(normal(b, t, hv) + 2.0)
    elif w.gate == "slow":
        g = -0.01 * torch.rand(b, t, hv, generator=gen)
    else:
        raise ValueError(f"unknown gate distribution {w.gate!r}")
    g = g.to(torch.bfloat16 if w.gate_dtype == "bf16" else torch.float32)
    beta = torch.sigmoid(normal(b, t, hv) + w.beta_shift).to(torch.bfloat16)
    if w.initial is None:
        initial = None
    elif w.initial == 0.0:
        initial = torch.zeros(b, hv, 128, 128)
    else:
        initial = w.initial * normal(b, hv, 128, 128)
    tensors = [q, k, v, g, beta, initial]
    if pin:
        tensors = [x.pin_memory() if x is not None else None for x in tensors]
    if device != "cpu":
        tensors = [x.to(device, non_blocking=pin) if x is not None else None for x in tensors]
    return tuple(tensors)


def algorithmic_flops(w: Workload):
    """Eight dense contractions of the WY chunk form: 180,224 FLOP per (token, value head)."""
    return 180224 * w.batch * w.length * w.value_heads


def algorithmic_bytes(w: Workload, output_final_state=True):
    """Each tensor once: q,k,v,out, g, beta, optional initial and final state."""
    b, t, hk, hv = w.shape
    gate_bytes = 4 if w.gate_dtype == "fp32" else 2
    total = 2 * b * t * hk * 256 + 2 * b * t * hv * 256 + b * t * hv * (gate_bytes + 2)
    if w.initial is not None:
        total += b * hv * 65536
    if output_final_state:
        total += b * hv * 65536
    return total
