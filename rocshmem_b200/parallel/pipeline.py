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
