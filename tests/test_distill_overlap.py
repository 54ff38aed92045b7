"""Teacher / student overlap: the ordering rules on fake streams (CPU), and on the GPU that the overlapped pipeline gives
exactly the losses and gradients of the serial order."""
import pytest
import torch


class _Log:
    def __init__(self):
        self.ops = []


class _FakeEvent:
    n = 0

    def __init__(self, log):
        _FakeEvent.n += 1
        self.id, self.log = _FakeEvent.n, log

    def record(self, stream):
        self.log.ops.append(("record", self.id, stream.name))


class _FakeStream:
    def __init__(self, name, log):
        self.name, self.log = name, log

    def wait_event(self, ev):
        self.log.ops.append(("wait", ev.id, self.name))

    def wait_stream(self, other):
        self.log.ops.append(("wait_stream", other.name, self.name))


class _Ctx:
    def __init__(self, s):
        pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def test_ordering_rules_on_fake_streams():
    import distill
    log = _Log()
    compute, teacher = _FakeStream("compute", log), _FakeStream("teacher", log)
    ov = distill.TeacherOverlap(None, stream_factory=lambda: teacher, event_factory=lambda: _FakeEvent(log),
                                current_stream=lambda: compute)
    filled, released = [e.id for e in ov._filled], [e.id for e in ov._released]
    for step in range(5):
        ov.produce(lambda: torch.full((2, 3), float(step)), stream_ctx=_Ctx)
        with pytest.raises(RuntimeError):
            ov.produce(lambda: torch.zeros(2, 3), stream_ctx=_Ctx)          # one target in flight at a time
        t = ov.target()
        assert t[0, 0].item() == step                                        # the buffer of THIS step
        ov.release()
    with pytest.raises(RuntimeError):
        ov.target()
    ops = log.ops
    for step in range(5):
        b = step & 1
        i_fill = [i for i, o in enumerate(ops) if o == ("record", filled[b], "teacher")][step // 2]
        i_wait = [i for i, o in enumerate(ops) if o == ("wait", filled[b], "compute")][step // 2]
        i_rel = [i for i, o in enumerate(ops) if o == ("record", released[b], "compute")][step // 2]
        assert i_fill < i_wait < i_rel                                        # rule 2, then rule 3
        if step >= 2:
            # rule 1: before the teacher refills buffer b it waits for the release recorded two steps earlier
            waits = [i for i, o in enumerate(ops) if o == ("wait", released[b], "teacher")]
            prev_rel = [i for i, o in enumerate(ops) if o == ("record", released[b], "compute")][step // 2 - 1]
            assert prev_rel < waits[step // 2 - 1] < i_fill
    # buffers are reused, not reallocated
    assert ov._buf[0] is not None and ov._buf[1] is not None and ov._buf[0].data_ptr() != ov._buf[1].data_ptr()


@pytest.mark.gpu
def test_overlapped_equals_serial_on_the_gpu():
    import distill
    import palettized_linear as PL
    import plz_ops as ops
    import synth
    from helpers import check_status
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    M, K, N = 1024, 512, 512
    d = synth.make_linear_inputs(M, N, K, seed=2, rank=16)
    wt = [(torch.randn(K, K, device=dev) * K ** -0.5).to(torch.bfloat16) for _ in range(6)]    # dense teacher: 6 Linears

    def teacher(x):
        h = x
        for w in wt:
            h = ops.dense_forward(w, h)[0]
        return h

    def make_student():
        m = PL.PalettizedLinear(K, N, rank=16, lora_scale=1.0)
        with torch.no_grad():
            m.palette.copy_(d["palette"].cuda()); m.index_logits.copy_(d["logits"].cuda())
            m.lora_A.copy_(d["lora_a"].cuda()); m.lora_B.copy_(d["lora_b"].cuda())
        m.noise = d["noise"].cuda()
        return m.train()
    batches = [(d["x"].cuda() * (1 + 0.1 * i)).to(torch.bfloat16) for i in range(5)]

    def run(overlapped):
        m = make_student()
        ov = distill.TeacherOverlap(dev)
        losses, grads = [], []
        for x in batches:
            if overlapped:
                ready = torch.cuda.Event()
                ready.record()                      # the batch exists: the teacher need not wait for the previous backward
                ov.produce(lambda: teacher(x), inputs_ready=ready)
                s = m(x)
                stats, ds = ov.loss(s)
            else:
                t = teacher(x)
                torch.cuda.synchronize()
                s = m(x)
                stats, ds = ops.distill_loss(s, t)
            m.zero_grad(set_to_none=True)
            s.backward(ds)
            losses.append(stats.clone())
            grads.append(m.index_logits.grad.clone())
        torch.cuda.synchronize()
        return losses, grads
    la, ga = run(True)
    lb, gb = run(False)
    check_status()
    for i in range(len(batches)):
        assert torch.equal(la[i], lb[i]), f"step {i}: loss statistics differ between the overlapped and the serial order"
        assert torch.equal(ga[i], gb[i]), f"step {i}: logit gradients differ"
    assert len({float(l[0]) for l in la}) == len(batches)         # the five steps saw five different targets
