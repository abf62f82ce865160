"""Point-to-point transport between pipeline stages.

The reference pickles a 1 KB header per message and synchronises the CUDA stream around every send / recv
(fairscale/nn/pipe/messages.py:109-151).  Here a message is a fixed int64 header (ndim, dtype code, dims) plus
the payload, both sent with ``torch.distributed`` p2p (NCCL over NVLink on GPUs, gloo on CPU) without host
synchronisation: NCCL orders the transfers on its own stream and the consumer kernel waits on it.
"""

from __future__ import annotations

from typing import Any, List, Optional

import torch
import torch.distributed as dist
from torch import Tensor

_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.int64, torch.int32, torch.uint8, torch.bool, torch.float64]
_HEADER = 10  # ndim, dtype, requires_grad, up to 7 dims


class SendRecvTransport:
    """Blocking-receive / async-send tensor transport for one pipeline group."""

    def __init__(self, group: Any, device: torch.device):
        self.group = group
        self.device = device
        self._pending: List[Any] = []

    def _global(self, group_rank: int) -> int:
        return dist.get_global_rank(self.group, group_rank) if self.group is not None and self.group is not dist.group.WORLD else group_rank

    def send(self, t: Tensor, dst: int) -> None:
        t = t.contiguous()
        assert t.dim() <= 7
        head = torch.zeros(_HEADER, dtype=torch.int64)
        head[0], head[1], head[2] = t.dim(), _DTYPES.index(t.dtype), int(t.requires_grad)
        for i, s in enumerate(t.shape):
            head[3 + i] = s
        head = head.to(self.device)
        self._pending.append(dist.isend(head, self._global(dst), group=self.group))
        self._pending.append(dist.isend(t.detach(), self._global(dst), group=self.group))
        self._pending.append((head, t))  # keep the buffers alive until the sends completed

    def recv(self, src: int) -> Tensor:
        head = torch.zeros(_HEADER, dtype=torch.int64, device=self.device)
        dist.recv(head, self._global(src), group=self.group)
        h = head.tolist()
        shape = tuple(h[3 : 3 + h[0]])
        out = torch.empty(shape, dtype=_DTYPES[h[1]], device=self.device)
        dist.recv(out, self._global(src), group=self.group)
        if h[2] and out.is_floating_point():
            out.requires_grad_()
        return out

    def flush(self) -> None:
        for w in self._pending:
            if hasattr(w, "wait"):
                w.wait()
        self._pending.clear()
