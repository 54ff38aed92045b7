"""A stand-in for the CALLER side of the drop-in boundary, for machines without the reference checkout.

It restates how the reference's module reaches its kernels -- by module NAME, at construction time, Triton first, then
`fused_lut_linear_cuda` (scripts/qwen_model.py:104-130) -- and how it dispatches in forward (:147-196): soft kernel when
training with index logits, hard kernel otherwise, tensors in the reference's runtime layout (indices (K, N) int8,
palette (N/gs, 4) bf16, logits (4, K, N) fp16 initialised one-hot at +-10, :135-143).  The LoRA wrapper follows
scripts/qwen_model.py:291-304 (bf16 rounding after each of the three ops, scaling = alpha / rank).
"""
import torch
from torch import nn


class RefLikePalettizedLinear(nn.Module):
    def __init__(self, indices_kn, palette, group_size, bias=None, use_soft_indices=True):
        super().__init__()
        self.register_buffer("indices", indices_kn.long())
        self.register_buffer("indices_int8", indices_kn.to(torch.int8).contiguous())
        self.palette = nn.Parameter(palette.clone().to(torch.bfloat16))
        self.group_size, self.tau, self.use_soft_indices = group_size, 1.0, use_soft_indices
        self.register_buffer("bias", bias)
        self._use_triton = self._use_cuda = False
        self._hard_kernel = self._soft_kernel = None
        try:
            from triton_soft_forward import triton_soft_linear  # noqa: F401
            from triton_hard_forward import triton_hard_linear  # noqa: F401
            self._use_triton = True
        except Exception:
            pass
        if not self._use_triton:
            import fused_lut_linear_cuda
            self._hard_kernel = fused_lut_linear_cuda.fused_lut_linear
            self._soft_kernel = fused_lut_linear_cuda.fused_lut_linear_soft
            self._use_cuda = True
        if use_soft_indices:
            K, N = indices_kn.shape
            lg = torch.full((4, K, N), -10.0, dtype=torch.float16, device=indices_kn.device)
            for p in range(4):
                lg[p][indices_kn == p] = 10.0
            self.index_logits = nn.Parameter(lg)
        else:
            self.index_logits = None

    def forward(self, x):
        lead = x.shape[:-1]
        xf = x.reshape(-1, x.shape[-1])
        if self.training and self.use_soft_indices and self.index_logits is not None:
            y = self._soft_kernel(xf, self.palette, self.index_logits, self.bias, self.group_size, self.tau)
        else:
            y = self._hard_kernel(xf, self.palette, self.indices_int8, self.bias, self.group_size)
        return y.reshape(*lead, -1)


class RefLikeLoRA(nn.Module):
    def __init__(self, base, in_dim, out_dim, rank=16, alpha=32.0):
        super().__init__()
        self.base, self.scaling = base, alpha / rank
        g = torch.Generator().manual_seed(3)
        self.lora_A = nn.Parameter((torch.randn(in_dim, rank, generator=g) * 0.01).to(torch.bfloat16))
        self.lora_B = nn.Parameter((torch.randn(out_dim, rank, generator=g) * 0.01).to(torch.bfloat16))

    def forward(self, x):
        return self.base(x) + ((x @ self.lora_A) @ self.lora_B.T) * self.scaling
