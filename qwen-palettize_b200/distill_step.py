"""One distillation training step of a super-block of palettized decoder layers against a dense bf16 teacher: teacher
forward (second stream), student forward in soft mode (Gumbel-Softmax over the index logits, straight-through), loss,
backward, data-parallel gradient exchange and the optimizer step of palettes, LoRA factors, index logits and norm weights.

This is the inner loop of the reference's trainer (scripts/train_qwen.py:1217-1290: teacher targets on a side stream, student
forward under autocast, compute_loss, backward, FP32MasterAdamW steps, clamp of the logits) with every op on this library's
kernels and an explicit backward. Per Linear of the student:

    forward   plz_soft_select (logits + counter-based Gumbel noise -> packed argmax indices), LUT GEMM with the LoRA block
    backward  dX LUT GEMM; weight-gradient GEMM whose epilogue recomputes the softmax and produces dLogits, dPalette, dA, dB
    exchange  world > 1: dLogits leave the weight-gradient epilogue straight into the owner ranks' staging slots
              (dp.LogitGradScatter, reduce-scatter fused into the kernel); the owner reduces its rows, steps them (AdamW state
              for 1 / world of the rows) and the updated logit rows are gathered by the copy engines; dPalette / dA / dB go
              through the small NCCL all-reduce that doubles as the barrier of the exchange
    optimizer fused fp32-master AdamW (plz_adamw_step; logits clamped), run as soon as a Linear's gradients exist, so a
              full-size dLogits tensor lives for one Linear at a time

Norm-weight gradients are summed over ranks in one bucket at the end of the step (dp.GradExchange)."""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

_HERE = os.path.dirname(os.path.abspath(__file__))
if _HERE not in sys.path:
    sys.path.insert(0, _HERE)

import dp  # noqa: E402
import plz_ops as ops  # noqa: E402
from decoder_layer import LINEARS, LayerConfig, layer_backward, layer_forward  # noqa: E402
from distill import TeacherOverlap  # noqa: E402


@dataclass
class Hyper:
    lr_logits: float = 1e-2
    lr_palette: float = 1e-4
    lr_lora: float = 1e-4
    lr_norm: float = 1e-5
    betas: tuple = (0.9, 0.95)
    eps: float = 1e-8
    clamp: tuple = (-10.0, 10.0)     # the logits are clamped after every step
    tau: float = 1.0
    w_cos: float = 0.5
    w_mse: float = 0.5


class AdamParam:
    """fp32 master + Adam moments of one tensor; `param` is the model copy (bf16) the kernels read, or None when the master
    itself is what they read (the fp32 index logits)."""

    def __init__(self, value: torch.Tensor, keep_param: bool = True):
        self.master = value.detach().float().contiguous().clone() if keep_param else value
        self.param = value if keep_param else None
        self.m = torch.zeros(self.master.numel(), dtype=torch.float32, device=value.device)
        self.v = torch.zeros_like(self.m)

    def step(self, grad: torch.Tensor, t: int, lr: float, hp: Hyper, grad_scale: float = 1.0, clamp=None):
        ops.adamw_step(self.master.view(-1), self.m, self.v, grad.contiguous().view(-1), t, lr, betas=hp.betas, eps=hp.eps,
                       grad_scale=grad_scale, clamp=clamp, clamp_master=clamp is not None,
                       param=self.param.view(-1) if self.param is not None else None)


class SoftLinear:
    """One palettized Linear in training mode: index logits fp32 [N, K, 4], palette bf16 [N * K / 256, 4], LoRA A [r, K],
    B [N, r], the packed-index scratch the soft forward writes, optimizer state, and (world > 1) its fused exchange."""

    def __init__(self, N: int, K: int, logits: torch.Tensor, palette: torch.Tensor, lora_a: torch.Tensor, lora_b: torch.Tensor,
                 lora_scale: float, seed: int, fused_exchange: bool = True):
        dev = logits.device
        self.N, self.K, self.seed, self.scale = N, K, seed, lora_scale
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.w = ops.PackedWeight(ops.empty_packed(N, K, dev), palette, N, K, 1, 256)
        self.lora_a, self.lora_b = lora_a, lora_b
        self.scatter = None
        if self.world > 1 and fused_exchange:
            self.scatter = dp.LogitGradScatter(N, K, dev, mode="slots", shard_optimizer=True)
            self.scatter.param.copy_(logits)
            self.logits = self.scatter.param              # peer-visible: updated rows are pushed straight into it
            r0, r1 = self.scatter.shard_rows()
            self.opt_logits = AdamParam(self.logits[r0:r1], keep_param=False)    # state for this rank's rows only
        else:
            self.logits = logits
            self.opt_logits = AdamParam(self.logits, keep_param=False)
        self.opt_pal = AdamParam(self.w.palette)
        self.opt_a, self.opt_b = AdamParam(lora_a), AdamParam(lora_b)
        self.handle = None

    @property
    def lora(self):
        return (self.lora_a, self.lora_b, self.scale)

    def close(self):
        if self.scatter is not None:
            self.scatter.close()


class SoftLinears:
    """The seven Linears of a student layer for decoder_layer.layer_forward / layer_backward. The optimizer step of a Linear
    runs inside bwd(), right after its gradients exist."""

    def __init__(self, lin: dict, hp: Hyper, step_no: int, exch: dp.GradExchange | None = None, keep_debug: bool = False):
        self.lin, self.hp, self.t, self.exch = lin, hp, step_no, exch
        self.grads, self.debug = {}, ({} if keep_debug else None)
        self.world = dist.get_world_size() if dist.is_initialized() else 1

    def fwd(self, name, x):
        L = self.lin[name]
        ops.soft_select(L.w, L.logits, "nk4", noise="hash", tau=self.hp.tau, seed=L.seed + self.t, want_packed=True)
        return ops.hard_forward(L.w, x, L.lora)

    def bwd(self, name, x_in, t_in, d_out):
        L, hp, t = self.lin[name], self.hp, self.t
        dxi, dti = ops.backward_dx(L.w, d_out, L.lora)          # reads the packed indices and the palette: before their update
        gs = 1.0 / self.world                                   # the loss is a mean over the global batch
        if L.scatter is not None:
            dpal, da, db = L.scatter.dw(L.w, x_in, d_out, L.logits, "hash", hp.tau, seed=L.seed + t, lora_ws=(t_in, dti))
            if L.handle is not None:
                raise RuntimeError("the previous exchange of this Linear was not finished")
            L.handle = L.scatter.start([dpal, da, db], step_fn=lambda p_, g_: L.opt_logits.step(g_, t, hp.lr_logits, hp, gs, hp.clamp))
        else:
            dlog, dpal, da, db = ops.backward_dw_soft(L.w, x_in, d_out, L.logits, "nk4", noise="hash", tau=hp.tau, seed=L.seed + t,
                                                      lora_ws=(t_in, dti))
            if self.world > 1:                                  # unfused exchange: plain all-reduce of everything
                for g in (dlog, dpal, da, db):
                    dist.all_reduce(g)
            if self.debug is not None:
                self.debug[name] = (x_in, d_out, dlog.clone(), dpal.clone(), L.w.palette.clone())
            L.opt_logits.step(dlog, t, hp.lr_logits, hp, gs, hp.clamp)
        L.opt_pal.step(dpal, t, hp.lr_palette, hp, gs)
        L.opt_a.step(da, t, hp.lr_lora, hp, gs)
        L.opt_b.step(db, t, hp.lr_lora, hp, gs)
        return dxi

    def finish(self):
        """Wait for the exchanges this layer started (the gathered logit rows are in place afterwards)."""
        for L in self.lin.values():
            if L.handle is not None:
                L.scatter.finish(L.handle)
                L.handle = None


class DenseLinears:
    """Teacher Linears: dense bf16 weights [N, K] through the dense-B GEMM, forward only."""

    def __init__(self, weights: dict):
        self.weights = weights

    def fwd(self, name, x):
        return ops.dense_forward(self.weights[name], x)[0], None


@dataclass
class Norms:
    input_ln: torch.Tensor
    post_ln: torch.Tensor
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    opt: dict = field(default_factory=dict)

    def names(self):
        return ("input_ln", "post_ln", "q_norm", "k_norm")


class Superblock:
    """Student (soft, trainable) and teacher (dense, frozen) copies of a few decoder layers, and the training step."""

    def __init__(self, cfg: LayerConfig, n_layers: int, device, seed: int = 0, hp: Hyper | None = None, fused_exchange: bool = True,
                 max_positions: int = 4096):
        self.cfg, self.hp, self.device = cfg, hp or Hyper(), device
        g = torch.Generator(device=device).manual_seed(seed)          # same seed on every rank: replicated parameters
        self.student, self.norms, self.teacher, self.teacher_norms = [], [], [], []
        for li in range(n_layers):
            lin, dense = {}, {}
            for name, (N, K) in cfg.shapes().items():
                logits = torch.randn(N, K, 4, generator=g, device=device)
                pal = (torch.randn(N * (K // 256), 4, generator=g, device=device) * 0.02).sort(-1).values.to(torch.bfloat16)
                a = (torch.randn(cfg.lora_rank, K, generator=g, device=device) * K ** -0.5).to(torch.bfloat16)
                b = (torch.randn(N, cfg.lora_rank, generator=g, device=device) * 0.01).to(torch.bfloat16)
                lin[name] = SoftLinear(N, K, logits, pal, a, b, cfg.lora_scale, seed=1000 * li + 17 * len(lin), fused_exchange=fused_exchange)
                dense[name] = (torch.randn(N, K, generator=g, device=device) * 0.02).to(torch.bfloat16)
                del logits
            self.student.append(lin)
            self.teacher.append(dense)
            nw = lambda n: (1.0 + 0.1 * torch.randn(n, generator=g, device=device)).to(torch.bfloat16)
            nm = Norms(nw(cfg.hidden), nw(cfg.hidden), nw(cfg.head_dim), nw(cfg.head_dim))
            nm.opt = {k: AdamParam(getattr(nm, k)) for k in nm.names()}
            self.norms.append(nm)
            self.teacher_norms.append(Norms(nm.input_ln.clone(), nm.post_ln.clone(), nm.q_norm.clone(), nm.k_norm.clone()))
        self.cos, self.sin = ops.rope_tables(max_positions, cfg.head_dim, cfg.rope_theta, device)
        self.overlap = TeacherOverlap(device)
        self.exch = dp.GradExchange()
        self.t = 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1

    def teacher_forward(self, x, B, S):
        h = x
        for dense, nm in zip(self.teacher, self.teacher_norms):
            h, _ = layer_forward(self.cfg, nm, h, B, S, self.cos[:S], self.sin[:S], keep=False, lin=DenseLinears(dense))
        return h

    def step(self, x: torch.Tensor, B: int, S: int, keep_debug: bool = False):
        """x bf16 [B * S, hidden]: this rank's tokens. Returns the loss statistics (fp32 [4] on the device: loss, 1 - cos, MSE
        term, mean t^2) of this rank's tokens."""
        cfg, hp = self.cfg, self.hp
        self.t += 1
        cos, sin = self.cos[:S], self.sin[:S]
        self.overlap.produce(lambda: self.teacher_forward(x, B, S))      # side stream, beside the student forward
        lins = [SoftLinears(lin, hp, self.t, keep_debug=keep_debug) for lin in self.student]
        ctxs, h = [], x
        for nm, sl in zip(self.norms, lins):
            h, ctx = layer_forward(cfg, nm, h, B, S, cos, sin, keep=True, lin=sl)
            ctxs.append(ctx)
        target = self.overlap.target()
        stats, d = ops.distill_loss(h, target, hp.w_cos, hp.w_mse)
        self.overlap.release()
        norm_grads = []
        for nm, sl, ctx in zip(reversed(self.norms), reversed(lins), reversed(ctxs)):
            d, g = layer_backward(cfg, nm, ctx, d, B, S, cos, sin, lin=sl)
            norm_grads.append((nm, g))
            ctx.t.clear()
        flat = [g[k] for nm, g in norm_grads for k in nm.names()]
        hnd = self.exch.start(flat) if self.world > 1 else None
        for sl in lins:
            sl.finish()
        if hnd is not None:
            self.exch.finish(hnd)
        for nm, g in norm_grads:
            for k in nm.names():
                nm.opt[k].step(g[k], self.t, hp.lr_norm, hp, 1.0 / self.world)
        self.last_debug = [sl.debug for sl in lins] if keep_debug else None
        return stats

    def close(self):
        for lin in self.student:
            for L in lin.values():
                L.close()
