"""The assembled distillation step (teacher forward on a side stream, soft student forward, loss, backward, optimizer):
gradients of one Linear inside the step against the oracle, and the loss going down when the student can fix what
separates it from the teacher."""
import pytest
import torch

import plz_oracle as O
from helpers import assert_close, check_status

pytestmark = pytest.mark.gpu


def _make(hp):
    import decoder_layer as DL
    import distill_step as DS
    import plz_ops as ops
    cfg = DL.LayerConfig(hidden=256, n_heads=2, n_kv_heads=1, head_dim=128, intermediate=512, lora_rank=16, lora_scale=2.0)
    dev = torch.device("cuda", 0)
    sb = DS.Superblock(cfg, 2, dev, seed=11, hp=hp, max_positions=256)
    # teacher = the student's own starting weights (argmax of the logits, LoRA merged) with every palette 5 % larger
    for lin, dense in zip(sb.student, sb.teacher):
        for name, L in lin.items():
            ops.soft_select(L.w, L.logits, "nk4", noise=None, tau=1.0, want_packed=True)
            w = ops.dequantize(L.w).float() * 1.05 + L.scale * (L.lora_b.float() @ L.lora_a.float())
            dense[name] = w.to(torch.bfloat16)
    return cfg, dev, sb


def test_step_gradients_match_the_oracle_and_loss_goes_down():
    import distill_step as DS
    hp = DS.Hyper(lr_logits=0.0, lr_lora=0.0, lr_norm=0.0, lr_palette=2e-4, tau=1.0)
    cfg, dev, sb = _make(hp)
    B, S = 2, 128
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(B * S, cfg.hidden, generator=g, device=dev).to(torch.bfloat16)
    stats = sb.step(x, B, S, keep_debug=True)
    check_status()
    first = stats.cpu()
    assert torch.isfinite(first).all() and first[0] > 0
    # the weight-gradient launch of one Linear inside the step against the oracle on the tensors it saw
    L = sb.student[1]["down"]
    x_in, d_out, dlog, dpal, pal_before = sb.last_debug[1]["down"]
    noise = O.gumbel_hash(L.seed + 1, L.N, L.K)
    logits = L.logits.cpu()                       # unchanged by the step: lr_logits = 0 and |logits| < clamp
    p, _, hard, w_hard = O.soft_weights(logits, noise, pal_before.cpu(), hp.tau, 1, 256)
    _, want_dlog, want_dpal, _ = O.soft_backward(x_in.cpu(), d_out.cpu(), w_hard, p, pal_before.cpu(), 1, 256)
    assert_close(dlog, want_dlog, "dLogits inside the step", rel=1e-2, cos=0.9999)
    assert_close(dpal, want_dpal, "dPalette inside the step", rel=1e-2, cos=0.9999)
    losses = [first[0].item()]
    for _ in range(14):
        losses.append(sb.step(x, B, S)[0].item())
    check_status()
    assert losses[-1] < 0.5 * losses[0], losses
    sb.close()


def test_step_moves_every_kind_of_parameter():
    import distill_step as DS
    hp = DS.Hyper(lr_logits=1e-2, lr_lora=1e-3, lr_norm=1e-3, lr_palette=1e-4)
    cfg, dev, sb = _make(hp)
    B, S = 1, 256
    g = torch.Generator(device=dev).manual_seed(2)
    x = torch.randn(B * S, cfg.hidden, generator=g, device=dev).to(torch.bfloat16)
    L = sb.student[0]["gate"]
    before = [L.logits.clone(), L.w.palette.clone(), L.lora_a.clone(), L.lora_b.clone(), sb.norms[0].post_ln.clone()]
    for _ in range(2):
        stats = sb.step(x, B, S)
    check_status()
    assert torch.isfinite(stats).all()
    after = [L.logits, L.w.palette, L.lora_a, L.lora_b, sb.norms[0].post_ln]
    for name, a, b in zip(("logits", "palette", "lora_a", "lora_b", "post_ln"), before, after):
        assert torch.isfinite(b.float()).all() and not torch.equal(a, b), name
    assert L.logits.abs().max() <= 10.0
    sb.close()
