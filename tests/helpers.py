"""Shared helpers of the test-suite."""
import numpy as np
import torch

# Parity contract for tensor-core products and gradients (bf16 inputs, fp32 accumulation):
# max |a - b| / max |b| <= 1e-2 and cosine >= 0.9999 per tensor.
REL_TOL = 1e-2
COS_TOL = 0.9999


def bf16_from_bits(a) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


def assert_close(got: torch.Tensor, want: torch.Tensor, what: str, rel=REL_TOL, cos=COS_TOL):
    import plz_oracle as O
    g, w = got.detach().float().cpu(), want.detach().float().cpu()
    assert g.shape == w.shape, f"{what}: shape {tuple(g.shape)} vs {tuple(w.shape)}"
    assert torch.isfinite(g).all(), f"{what}: non-finite values"
    r, c = O.max_rel_err(g, w), O.cosine(g, w)
    assert r <= rel and c >= cos, f"{what}: max rel err {r:.3e} (<= {rel}), cosine {c:.6f} (>= {cos})"


def check_status():
    import plz_native as P
    st = P.device_status()
    assert st[0] == 0, f"device status {st}"


def assert_close_rows(got: torch.Tensor, want: torch.Tensor, what: str, rel=REL_TOL, floor=0.02):
    """The per-tensor metric again, but per ROW (a palette group, a LoRA rank row...): max |a - b| over the row divided by
    that row's own max |b| (not below `floor` x the tensor's max, so that a row that is all noise cannot fail alone).
    One large element elsewhere in the tensor cannot hide a wrong small row."""
    g, w = got.detach().double().cpu(), want.detach().double().cpu()
    assert g.shape == w.shape, f"{what}: shape {tuple(g.shape)} vs {tuple(w.shape)}"
    g, w = g.reshape(g.shape[0], -1), w.reshape(w.shape[0], -1)
    den = w.abs().amax(1).clamp(min=floor * w.abs().max().item())
    err = (g - w).abs().amax(1) / den
    worst = int(err.argmax())
    assert err[worst].item() <= rel, f"{what}: row {worst} has max rel err {err[worst].item():.3e} (<= {rel})"
