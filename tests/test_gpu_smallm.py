"""Small-M (token decode) hard forward on the GPU against the CPU oracle and against the large-M kernel."""
import pytest
import torch

import plz_oracle as O
from helpers import assert_close, check_status

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K,gs_n,gs_k", [(1, 256, 256, 1, 256), (1, 9728, 2560, 1, 256), (2, 1000, 2560, 1, 256), (3, 2560, 9728, 1, 256), (8, 1024, 2560, 1, 256), (16, 9728, 2560, 1, 256),
                                             (12, 4096, 4096, 1, 256), (7, 72, 768, 1, 256), (16, 2560, 9728, 1, 256), (9, 151936 // 16, 2560, 1, 256),
                                             (33, 1000, 512, 1, 64), (64, 2560, 9728, 1, 256), (4, 1024, 1024, 256, 1024)])
def test_small_m_forward(M, N, K, gs_n, gs_k):
    import plz_ops as ops
    g = torch.Generator().manual_seed(M * 31 + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    idx = torch.randint(0, 4, (N, K), generator=g, dtype=torch.uint8)
    pal = (torch.randn((N // gs_n) * (K // gs_k), 4, generator=g) * 0.02).sort(-1).values.to(torch.bfloat16)
    w = ops.PackedWeight(torch.from_numpy(O.pack_rows(idx.numpy())).cuda(), pal.cuda(), N, K, gs_n, gs_k)
    y = ops.hard_forward_smallm(w, x.cuda())
    check_status()
    assert_close(y, O.hard_forward(x, O.dequantize(idx.long(), pal, gs_n, gs_k)), "y")
    if N % 8 == 0:
        y_big, _ = ops.hard_forward(w, x.cuda())
        assert_close(y, y_big, "small-M kernel vs tiled kernel", rel=4e-3)


@pytest.mark.parametrize("M,Ns,K", [(1, (9728, 9728), 2560), (8, (4096, 1024, 1024), 2560), (16, (264, 72, 1000, 8), 512), (5, (2560,), 9728)])
def test_small_m_multi(M, Ns, K):
    """Several matrices that share x in one launch against the oracle and the single-matrix calls (same arithmetic; the
    order in which the partial sums of the ten 256-column groups meet in shared memory is not fixed, so not bit for bit)."""
    import plz_ops as ops
    g = torch.Generator().manual_seed(M + sum(Ns))
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    ws, refs = [], []
    for N in Ns:
        idx = torch.randint(0, 4, (N, K), generator=g, dtype=torch.uint8)
        pal = (torch.randn(N * (K // 256), 4, generator=g) * 0.02).sort(-1).values.to(torch.bfloat16)
        ws.append(ops.PackedWeight(torch.from_numpy(O.pack_rows(idx.numpy())).cuda(), pal.cuda(), N, K, 1, 256))
        refs.append(O.hard_forward(x.cpu(), O.dequantize(idx.long(), pal, 1, 256)))
    ys = ops.hard_forward_smallm_multi(ws, x)
    check_status()
    for y, w, ref in zip(ys, ws, refs):
        assert_close(y, ref, "y of one matrix of the group")
        assert_close(y, ops.hard_forward_smallm(w, x), "multi vs single launch", rel=4e-3)


def test_small_m_overlapped_launches():
    """Programmatic dependent launch on: a chain y1 = x W1^T, y2 = y1[:, :K] W2^T ... whose every launch may start under the
    tail of the previous one must give what the serialized chain gives (the kernel waits for its predecessor before it
    reads x or writes y)."""
    import plz_native as P
    import plz_ops as ops
    N = K = 2560
    g = torch.Generator().manual_seed(7)
    ws = []
    for _ in range(6):
        idx = torch.randint(0, 4, (N, K), generator=g, dtype=torch.uint8)
        pal = (torch.randn(N * (K // 256), 4, generator=g) * 0.02).sort(-1).values.to(torch.bfloat16)
        ws.append(ops.PackedWeight(torch.from_numpy(O.pack_rows(idx.numpy())).cuda(), pal.cuda(), N, K, 1, 256))
    x0 = torch.randn(8, K, generator=g).to(torch.bfloat16).cuda()

    def chain():
        h = x0
        for w in ws:
            h = ops.hard_forward_smallm(w, h)
            h = (h * 16.0).to(torch.bfloat16)  # keep the magnitude; a torch kernel between the launches
        return h

    want = chain()
    P.check(P.lib().plz_set_smallm_overlap(1), "plz_set_smallm_overlap")
    try:
        outs = [chain() for _ in range(5)]
        h = x0
        for w in ws:  # and back to back, without anything in between
            h = ops.hard_forward_smallm(w, h)
        torch.cuda.synchronize()
    finally:
        P.check(P.lib().plz_set_smallm_overlap(0), "plz_set_smallm_overlap")
    check_status()
    for o in outs:
        assert_close(o, want, "overlapped chain", rel=8e-3)
    h2 = x0
    for w in ws:
        h2 = ops.hard_forward_smallm(w, h2)
    assert_close(h, h2, "back-to-back overlapped chain", rel=8e-3)
