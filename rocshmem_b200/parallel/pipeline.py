"""Point-to-point activations between pipeline stages: put with signal on the host API.

A channel is a symmetric buffer plus two counters. ``send`` waits until the receiver has consumed the previous
message (its acknowledgement counter), puts the payload into the receiver's buffer, orders the put before the
signal with ``quiet`` and then bumps the receiver's arrival counter with a remote atomic; ``recv`` waits for that
counter (bounded wait: a sender that never comes is reported, not waited for for ever), copies the payload out and
acknowledges. This is the put_signal / wait_until pairing of the device API (reference:
src/ipc/context_ipc_device.cpp:221-324) used from the host.
"""
from __future__ import annotations

import torch

from .. import runtime as rt


class P2PChannel:
    """One direction between a fixed pair of PEs; both create it collectively with the same arguments."""

    def __init__(self, shape, dtype: torch.dtype, src_pe: int, dst_pe: int):
        self.src_pe, self.dst_pe = src_pe, dst_pe
        self.buf = rt.zeros(shape, dtype)
        self.arrived = rt.zeros(1, torch.int64)     # on the receiver: messages delivered
        self.consumed = rt.zeros(1, torch.int64)    # on the sender: messages the receiver has taken
        self.count = 0

    def destroy(self) -> None:
        """Collective: free the buffer and the two counters."""
        rt.free_all([self.buf, self.arrived, self.consumed])
        self.buf = self.arrived = self.consumed = None

    def send(self, t: torch.Tensor) -> None:
        """Put the tensor into the receiver's buffer once the previous message has been taken, then signal."""
        if rt.my_pe() != self.src_pe:
            raise RuntimeError("send on a PE that is not the channel's source")
        if self.count and rt.wait_until(self.consumed, rt.CMP_GE, self.count) != rt.SUCCESS:
            raise TimeoutError(f"PE {self.dst_pe} did not take message {self.count}")
        rt.putmem(self.buf, t.contiguous(), self.dst_pe)
        rt.quiet()
        rt.atomic_fetch_add(self.arrived, 1, self.dst_pe)
        self.count += 1

    def recv(self) -> torch.Tensor:
        """Wait for the next message, return a copy and tell the sender the buffer is free."""
        if rt.my_pe() != self.dst_pe:
            raise RuntimeError("recv on a PE that is not the channel's destination")
        self.count += 1
        if rt.wait_until(self.arrived, rt.CMP_GE, self.count) != rt.SUCCESS:
            raise TimeoutError(f"message {self.count} from PE {self.src_pe} did not arrive")
        out = self.buf.clone()
        rt.atomic_fetch_add(self.consumed, 1, self.src_pe)
        return out


class PipelineStage:
    """One stage of a pipeline-parallel model with the all-forward, all-backward (GPipe) schedule.

    Stage ``s`` runs on PE ``first_pe + s`` of the world; activations travel to the next stage and gradients with
    respect to them travel back through :class:`P2PChannel` pairs. All PEs of the pipeline create the object
    collectively with the same ``num_stages``, shapes and dtype; every micro-batch has the activation shape
    ``act_shape`` at every stage boundary.

        stage = PipelineStage(module, num_stages=4, act_shape=(mb, d), dtype=torch.float32)
        losses = stage.run(micro_batches, loss_fn, targets)   # inputs on stage 0, targets on the last stage
        # module's parameters now hold the gradients of the summed loss

    The schedule keeps one saved activation per micro-batch alive between its forward and backward, as GPipe does.
    """

    def __init__(self, module: torch.nn.Module, num_stages: int, act_shape, dtype: torch.dtype = torch.float32,
                 first_pe: int = 0):
        self.module = module
        self.num_stages = num_stages
        self.stage = rt.my_pe() - first_pe
        self.act_shape, self.dtype = tuple(act_shape), dtype
        # Channels are symmetric objects: every PE creates all of them, in the same order.
        self.fwd = [P2PChannel(act_shape, dtype, first_pe + s, first_pe + s + 1) for s in range(num_stages - 1)]
        self.bwd = [P2PChannel(act_shape, dtype, first_pe + s + 1, first_pe + s) for s in range(num_stages - 1)]

    @property
    def active(self) -> bool:
        """False on PEs outside ``[first_pe, first_pe + num_stages)``: they only take part in creation and destruction."""
        return 0 <= self.stage < self.num_stages

    def destroy(self) -> None:
        """Collective: free all channels."""
        for ch in reversed(self.fwd + self.bwd):
            ch.destroy()
        self.fwd, self.bwd = [], []

    def run(self, micro_batches=None, loss_fn=None, targets=None, num_micro: int = 0):
        """Forward all micro-batches, then backward in reverse order. ``micro_batches`` is needed on the first
        stage, ``loss_fn`` and ``targets`` on the last; the other stages pass ``num_micro``. Returns the list of
        losses on the last stage (detached), ``None`` elsewhere."""
        if not self.active:
            return None
        s, last = self.stage, self.num_stages - 1
        m = len(micro_batches) if micro_batches is not None else (len(targets) if targets is not None else num_micro)
        dev = rt.device()
        saved_in, saved_out, losses = [], [], []
        for i in range(m):
            if s == 0:
                x = micro_batches[i].to(dev)
            else:
                x = self.fwd[s - 1].recv().requires_grad_(True)
            y = self.module(x)
            saved_in.append(x)
            if s == last:
                loss = loss_fn(y, targets[i].to(dev))
                losses.append(loss.detach())
                saved_out.append(loss)
            else:
                saved_out.append(y)
                self.fwd[s].send(y.detach().to(self.dtype))
        for i in reversed(range(m)):
            if s == last:
                saved_out[i].backward()
            else:
                saved_out[i].backward(self.bwd[s].recv().to(saved_out[i].dtype))
            if s > 0:
                self.bwd[s - 1].send(saved_in[i].grad.to(self.dtype))
            saved_in[i] = saved_out[i] = None
        return losses if s == last else None
