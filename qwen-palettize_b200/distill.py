"""The distillation step around the palettized layers: teacher forward overlapped with the student on a second stream,
ping-pong target buffers, and the fused loss kernel.

Follows the reference's training loop (scripts/train_qwen.py:1112-1124 set-up, :1217-1249 teacher side, :1251-1287 student
side and loss), with its three ordering rules:
  1. the teacher never overwrites a target buffer the student still reads: before writing buffer b the teacher stream
     waits for the `released` event of b, recorded two steps earlier;
  2. the student never reads a buffer the teacher is still writing: the compute stream waits for the `filled` event of b
     before the loss;
  3. `released` is recorded IMMEDIATELY after the loss kernel has been enqueued, before the backward: the student needs the
     target only for the loss, so the next-but-one teacher forward can start under the current backward.
The loss itself is plz_distill_loss (one fused kernel: per-token 1 - cos plus normalised MSE, and dLoss/ds), the
reference's compute_loss (scripts/train_qwen.py:229-249).
"""
from __future__ import annotations

import os
import sys

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
if _HERE not in sys.path:
    sys.path.insert(0, _HERE)


class TeacherOverlap:
    """Double-buffered teacher targets produced on a side stream.

        ov = TeacherOverlap(device)
        for step, batch in enumerate(data):
            ov.produce(lambda: teacher(batch))        # enqueued on the teacher stream, returns at once
            s = student(batch)                        # compute stream, runs beside the teacher
            stats, ds = ov.loss(s)                    # waits for the target, fused loss + gradient, releases the buffer
            s.backward(ds)                            # the teacher of the next steps may already overwrite the other buffer

    `stream_factory` / `event_factory` / `current_stream` exist so that the ordering logic can be exercised without a GPU."""

    def __init__(self, device=None, stream_factory=None, event_factory=None, current_stream=None):
        self.device = device
        self._stream = (stream_factory or (lambda: torch.cuda.Stream(device=device)))()
        ev = event_factory or (lambda: torch.cuda.Event())
        self._filled = [ev(), ev()]
        self._released = [ev(), ev()]
        self._current = current_stream or (lambda: torch.cuda.current_stream(device))
        self._buf = [None, None]
        self._idx = 0          # buffer of the step in flight
        self._produced = 0     # number of produce() calls
        self._pending = False  # a target has been produced and not yet consumed

    @property
    def stream(self):
        return self._stream

    def produce(self, teacher_fn, inputs_ready=None, stream_ctx=None):
        """Run teacher_fn() (no grad) on the teacher stream and keep its result as the target of this step.
        inputs_ready: an event after which the teacher's inputs (the batch) are valid. With it the teacher waits for nothing
        else, so it can run under the PREVIOUS step's backward and optimizer work still queued on the compute stream (the
        reference's behaviour: its side stream never waits for the default stream). Without it the teacher stream waits for
        everything enqueued on the compute stream so far, which is always safe and still overlaps the teacher with this
        step's student forward and backward."""
        if self._pending:
            raise RuntimeError("TeacherOverlap.produce(): the previous target has not been consumed by loss() / release()")
        b = self._idx
        if self._produced >= 2:
            self._stream.wait_event(self._released[b])                    # rule 1
        if inputs_ready is not None:
            self._stream.wait_event(inputs_ready)
        else:
            self._stream.wait_stream(self._current())
        ctx = stream_ctx or torch.cuda.stream
        with ctx(self._stream):
            with torch.no_grad():
                t = teacher_fn()
                if self._buf[b] is not None and self._buf[b].shape == t.shape and self._buf[b].dtype == t.dtype:
                    self._buf[b].copy_(t)                                 # keep one allocation per buffer
                else:
                    self._buf[b] = t.detach()
        self._filled[b].record(self._stream)
        self._produced += 1
        self._pending = True

    def target(self):
        """The compute stream waits for this step's target (rule 2) and gets the buffer."""
        if not self._pending:
            raise RuntimeError("TeacherOverlap.target(): produce() has not been called for this step")
        self._current().wait_event(self._filled[self._idx])
        return self._buf[self._idx]

    def release(self):
        """Record that the compute stream is done with this step's target (rule 3) and switch buffers."""
        self._released[self._idx].record(self._current())
        self._idx ^= 1
        self._pending = False

    def loss(self, student_out, w_cos: float = 0.5, w_mse: float = 0.5, want_grad: bool = True, grad_dtype=torch.bfloat16,
             upstream: float = 1.0):
        """Fused distillation loss of the student output against this step's target; releases the buffer right after the
        kernel has been enqueued.  Returns (stats fp32 [4] on the device: loss, 1 - cos, normalised MSE, mean(t^2); dLoss/ds)."""
        import plz_ops as ops
        t = self.target()
        out = ops.distill_loss(student_out, t, w_cos=w_cos, w_mse=w_mse, want_grad=want_grad, grad_dtype=grad_dtype, upstream=upstream)
        self.release()
        return out
