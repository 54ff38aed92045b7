"""Seeded synthetic inputs for one palettized Linear in the native layout
(W [N, K], indices packed 4 per byte along K, one palette per output row and 256 input columns,
index logits / Gumbel noise fp32 [N, K, 4], LoRA A [r, K], B [N, r]).

Everything is drawn on the CPU from one torch.Generator so that a CPU checker and the GPU see identical
bits.  For large shapes the per-weight tensors are drawn in row blocks to bound host memory.
"""
from __future__ import annotations

import torch

GS_K = 256


def make_linear_inputs(M: int, N: int, K: int, seed: int = 0, rank: int = 16, soft: bool = True, lora: bool = True,
                       with_dy: bool = True, lora_scale: float = 1.0):
    """Returns a dict of CPU tensors:
    x bf16 [M, K] ~ N(0,1); idx uint8 [N, K] uniform {0..3}; palette bf16 [N, K/256, 4], each 4-tuple sorted
    N(0, 0.02^2); logits fp32 [N, K, 4] ~ N(0,1); noise fp32 [N, K, 4] = -log(-log U), U ~ Uniform clamped to
    [1e-7, 1); lora_a bf16 [r, K] ~ N(0, 1/K); lora_b bf16 [N, r] ~ N(0, 0.01^2); dy bf16 [M, N] ~ N(0,1)."""
    assert K % GS_K == 0
    g = torch.Generator().manual_seed(seed)
    out = {"M": M, "N": N, "K": K, "gs_n": 1, "gs_k": GS_K, "rank": rank, "lora_scale": lora_scale}
    out["x"] = torch.randn(M, K, generator=g).to(torch.bfloat16)
    out["idx"] = torch.randint(0, 4, (N, K), generator=g, dtype=torch.uint8)
    out["palette"] = (torch.randn(N, K // GS_K, 4, generator=g) * 0.02).sort(dim=-1).values.to(torch.bfloat16)
    if soft:
        out["logits"] = torch.randn(N, K, 4, generator=g)
        u = torch.rand(N, K, 4, generator=g).clamp_(min=1e-7)
        out["noise"] = -torch.log(-torch.log(u))
        del u
    if lora:
        out["lora_a"] = (torch.randn(rank, K, generator=g) * (K ** -0.5)).to(torch.bfloat16)
        out["lora_b"] = (torch.randn(N, rank, generator=g) * 0.01).to(torch.bfloat16)
    if with_dy:
        out["dy"] = torch.randn(M, N, generator=g).to(torch.bfloat16)
    return out


def make_linear_inputs_cuda(M: int, N: int, K: int, seed: int = 0, rank: int = 16, device="cuda"):
    """Same distributions drawn directly on the device (different bits than the CPU generator): for timing
    runs at sizes where host generation would dominate the run time."""
    g = torch.Generator(device=device).manual_seed(seed)
    out = {"M": M, "N": N, "K": K, "gs_n": 1, "gs_k": GS_K, "rank": rank, "lora_scale": 1.0}
    out["x"] = torch.randn(M, K, generator=g, device=device).to(torch.bfloat16)
    out["idx"] = torch.randint(0, 4, (N, K), generator=g, device=device, dtype=torch.uint8)
    out["palette"] = (torch.randn(N, K // GS_K, 4, generator=g, device=device) * 0.02).sort(dim=-1).values.to(torch.bfloat16)
    out["logits"] = torch.randn(N, K, 4, generator=g, device=device)
    u = torch.rand(N, K, 4, generator=g, device=device).clamp_(min=1e-7)
    out["noise"] = -torch.log(-torch.log(u))
    del u
    out["lora_a"] = (torch.randn(rank, K, generator=g, device=device) * (K ** -0.5)).to(torch.bfloat16)
    out["lora_b"] = (torch.randn(N, rank, generator=g, device=device) * 0.01).to(torch.bfloat16)
    out["dy"] = torch.randn(M, N, generator=g, device=device).to(torch.bfloat16)
    return out
