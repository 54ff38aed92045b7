"""Fused fp32-master AdamW (+ clip scale + clamp) and the distillation loss on the GPU against the CPU oracle and
against the golden vectors produced by the reference's compute_loss / FP32MasterAdamW."""
import pytest
import torch

import plz_oracle as O
from helpers import assert_close, bf16_from_bits, check_status

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("gdtype,pdtype,clamp,clamp_master,wd", [
    (torch.float32, torch.float32, None, False, 0.0),
    (torch.float16, torch.float16, (-2.0, 2.0), False, 0.0),
    (torch.float32, torch.bfloat16, (-1.0, 1.0), True, 0.01),
])
def test_adamw_matches_torch(gdtype, pdtype, clamp, clamp_master, wd):
    import plz_ops as ops
    g = torch.Generator().manual_seed(1)
    n = 100_003
    p0 = (torch.randn(n, generator=g) * 2).to(pdtype)
    grads = [(torch.randn(n, generator=g) * 0.1).to(gdtype) for _ in range(4)]
    master = p0.float().cuda()
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    param = p0.clone().cuda()
    for step, gr in enumerate(grads, 1):
        ops.adamw_step(master, m, v, gr.cuda(), step, 0.05, betas=(0.9, 0.95), eps=1e-8, weight_decay=wd, grad_scale=0.5,
                       clamp=clamp, clamp_master=clamp_master, param=param)
    check_status()
    ma, mo, m_ref, v_ref = O.adamw_reference(p0, grads, 0.05, weight_decay=wd, clamp=clamp, clamp_master=clamp_master, grad_scale=0.5)
    assert_close(master, ma, "master", rel=1e-5, cos=0.999999)
    assert_close(m, m_ref, "m", rel=1e-5, cos=0.999999)
    assert_close(v, v_ref, "v", rel=1e-5, cos=0.999999)
    assert_close(param, mo.float(), "model copy", rel=4e-3 if pdtype != torch.float32 else 1e-5)
    if clamp is not None:
        assert param.float().max() <= clamp[1] and param.float().min() >= clamp[0]


def test_adamw_against_reference_vectors(golden):
    import plz_ops as ops
    p0 = torch.from_numpy(golden["adam_p0"])
    grads = torch.from_numpy(golden["adam_grads"])
    master = p0.float().cuda()
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    param = p0.clone().cuda()
    for step in range(grads.shape[0]):
        ops.adamw_step(master, m, v, grads[step].cuda(), step + 1, 0.05, clamp=(-2.0, 2.0), param=param)
    check_status()
    want = torch.from_numpy(golden["adam_model"]).float()
    # fp16 model copy after three steps: at most one fp16 ulp away from FP32MasterAdamW + clamp
    assert (param.float().cpu() - want).abs().max() <= 2e-3


@pytest.mark.parametrize("M,H", [(48, 64), (1000, 2560)])
def test_distill_loss_matches_oracle(M, H):
    import plz_ops as ops
    g = torch.Generator().manual_seed(M)
    s = torch.randn(M, H, generator=g).to(torch.bfloat16)
    t = (s.float() + 0.5 * torch.randn(M, H, generator=g)).to(torch.bfloat16)
    s[0] = 0
    out4, ds = ops.distill_loss(s.cuda(), t.cuda(), 0.5, 0.5, grad_dtype=torch.float32)
    check_status()
    (loss, l_cos, l_mse, t_var), ds_ref = O.distill_loss(s, t, 0.5, 0.5)
    got = out4.cpu()
    for a, b in zip(got.tolist(), (loss, l_cos, l_mse, t_var)):
        assert abs(a - b) <= 1e-4 * max(1.0, abs(b)), (got.tolist(), (loss, l_cos, l_mse, t_var))
    assert_close(ds, ds_ref, "dLoss/ds", rel=1e-3, cos=0.99999)
    _, ds16 = ops.distill_loss(s.cuda(), t.cuda(), 0.5, 0.5, grad_dtype=torch.bfloat16)
    assert_close(ds16, ds_ref, "dLoss/ds (bf16)")


def test_distill_loss_against_reference_vectors(golden):
    import plz_ops as ops
    s, t = bf16_from_bits(golden["loss_s"]), bf16_from_bits(golden["loss_t"])
    out4, ds = ops.distill_loss(s.cuda(), t.cuda(), 0.5, 0.5, grad_dtype=torch.float32)
    check_status()
    assert abs(out4[0].item() - float(golden["loss_vals"][0])) <= 1e-5
    assert abs(out4[1].item() - float(golden["loss_vals"][1])) <= 1e-5
    assert_close(ds.reshape(-1), torch.from_numpy(golden["loss_ds"]).reshape(-1), "dLoss/ds vs compute_loss autograd", rel=1e-3, cos=0.99999)
