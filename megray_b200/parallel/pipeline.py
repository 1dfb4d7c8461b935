"""Pipeline parallelism: the one-forward-one-backward (1F1B) schedule over the communicator's
send / recv.

Stage ``s`` of ``P`` (= rank ``s`` of the communicator) runs ``min(P - s - 1, M)`` warm-up
forwards, then alternates one forward with one backward, then drains the remaining backwards, so
at most ``P - s`` micro-batches are alive on a stage at any time.  Where a stage has something to
send in one direction and to receive from the other in the same slot (the steady state), both
transfers go into one ``group_start`` / ``group_end`` bracket, so neighbouring stages that send to
each other at the same moment cannot block each other.

The reference library offers the primitives this is built from (``send`` / ``recv`` and the group
calls, include/megray/communicator.h:51-57,107-109) and no schedule.  Works with CUDA tensors on
the NVL / NCCL backends and with CPU tensors on the host backend.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch


def one_f_one_b(num_stages: int, num_microbatches: int, stage: int) -> List[Tuple[str, int]]:
    """The order of work on ``stage``: a list of ("F", micro-batch) / ("B", micro-batch)."""
    if not 0 <= stage < num_stages or num_microbatches < 1:
        raise ValueError("bad stage or micro-batch count")
    warmup = min(num_stages - stage - 1, num_microbatches)
    steady = num_microbatches - warmup
    order = [("F", i) for i in range(warmup)]
    for i in range(steady):
        order += [("F", warmup + i), ("B", i)]
    order += [("B", steady + i) for i in range(warmup)]
    return order


class PipelineStage:
    """One stage of a pipeline whose stages exchange activations of one fixed shape.

    ``forward(mb, x) -> y`` and ``backward(mb, dy) -> dx`` are the stage's own computation (they
    keep whatever they need between the two calls).  The first stage reads its inputs from
    ``inputs[mb]``; the last stage turns its output into the gradient of the loss with
    ``loss_grad(mb, y) -> dy``.
    """

    def __init__(self, comm, forward: Callable, backward: Callable, activation_shape, dtype=torch.float32,
                 device="cpu"):
        self.comm, self.forward, self.backward = comm, forward, backward
        self.stage, self.stages = comm.rank, comm.nranks
        self.shape, self.dtype, self.device = tuple(activation_shape), dtype, device
        self.first, self.last = self.stage == 0, self.stage == comm.nranks - 1

    def _buf(self) -> torch.Tensor:
        return torch.empty(self.shape, dtype=self.dtype, device=self.device)

    # -- single transfers -------------------------------------------------------------------
    def _recv_forward(self, mb, inputs):
        if self.first:
            return inputs[mb]
        x = self._buf()
        self.comm.recv(x, self.stage - 1)
        return x

    def _send_forward(self, y):
        if not self.last:
            self.comm.send(y.contiguous(), self.stage + 1)

    def _recv_backward(self, mb, y, loss_grad):
        if self.last:
            return loss_grad(mb, y)
        dy = self._buf()
        self.comm.recv(dy, self.stage + 1)
        return dy

    def _send_backward(self, dx):
        if not self.first:
            self.comm.send(dx.contiguous(), self.stage - 1)

    # -- combined transfers of the steady state ---------------------------------------------
    def _send_forward_recv_backward(self, mb_b, y, y_b, loss_grad):
        if self.last:
            return loss_grad(mb_b, y_b)
        dy = self._buf()
        self.comm.group_start()
        self.comm.send(y.contiguous(), self.stage + 1)
        self.comm.recv(dy, self.stage + 1)
        self.comm.group_end()
        return dy

    def _send_backward_recv_forward(self, mb_f, dx, inputs):
        if self.first:
            return inputs[mb_f]
        x = self._buf()
        self.comm.group_start()
        self.comm.send(dx.contiguous(), self.stage - 1)
        self.comm.recv(x, self.stage - 1)
        self.comm.group_end()
        return x

    # -- the schedule -----------------------------------------------------------------------
    def run(self, num_microbatches: int, inputs: Optional[List[torch.Tensor]] = None,
            loss_grad: Optional[Callable] = None) -> List[torch.Tensor]:
        """Runs all micro-batches through this stage under 1F1B.  Returns the stage's outputs per
        micro-batch (the model's outputs on the last stage)."""
        if self.first and inputs is None:
            raise ValueError("the first stage needs the micro-batch inputs")
        if self.last and loss_grad is None:
            raise ValueError("the last stage needs loss_grad")
        M = num_microbatches
        warmup = min(self.stages - self.stage - 1, M)
        steady = M - warmup
        outputs: List[Optional[torch.Tensor]] = [None] * M
        for i in range(warmup):
            x = self._recv_forward(i, inputs)
            outputs[i] = self.forward(i, x)
            self._send_forward(outputs[i])
        x = self._recv_forward(warmup, inputs) if steady > 0 else None
        for i in range(steady):
            mb_f, mb_b = warmup + i, i
            outputs[mb_f] = self.forward(mb_f, x)
            dy = self._send_forward_recv_backward(mb_b, outputs[mb_f], outputs[mb_b], loss_grad)
            dx = self.backward(mb_b, dy)
            if i + 1 < steady:
                x = self._send_backward_recv_forward(mb_f + 1, dx, inputs)
            else:
                self._send_backward(dx)
        for i in range(warmup):
            mb_b = steady + i
            dy = self._recv_backward(mb_b, outputs[mb_b], loss_grad)
            self._send_backward(self.backward(mb_b, dy))
        return outputs
