"""Point-to-point transport between pipeline stages.

The reference pickles a 1 KB header per message and synchronises the CUDA stream around every send / recv
(fairscale/nn/pipe/messages.py:109-151).  Here a message is a fixed int64 header (ndim, dtype code, dims) plus the
payload, both sent with ``torch.distributed`` p2p (NCCL over NVLink on GPUs, gloo on CPU).  Reading the header costs
the receiver one host synchronisation.  With ``static_shapes=True`` and a ``slot`` per message (the micro-batch index)
the header travels only the first time a (peer, slot) pair is used: from then on both sides rely on the recorded
shape / dtype contract, the receive is posted straight into a correctly sized buffer and nothing is read on the host.
A sender whose tensor no longer matches its contract raises instead of sending.
"""

from __future__ import annotations

import os
import queue
import threading
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.int64, torch.int32, torch.uint8, torch.bool, torch.float64]
_HEADER = 10  # ndim, dtype, requires_grad, up to 7 dims


def to_input_device(tensors: Any, input_device: Optional[torch.device]) -> Any:
    """Move a tuple of tensors to ``input_device`` (no-op when it is None)."""
    if input_device is None:
        return tensors
    return tuple(t.to(input_device) for t in tensors)


class Transport:
    """Interface of a stage-to-stage tensor transport: ``send(tensor, dst_rank)``, ``recv(src_rank) -> tensor`` (blocking,
    messages of one pair arrive in the order they were sent) and ``flush()`` (wait for outstanding sends)."""

    device: torch.device

    def send(self, t: Tensor, dst: int, slot: Optional[int] = None) -> None:
        raise NotImplementedError

    def recv(self, src: int, slot: Optional[int] = None) -> Tensor:
        raise NotImplementedError

    def flush(self) -> None:
        raise NotImplementedError

    def prefetch(self, src: int, slot: Optional[int]) -> bool:
        """Optionally start receiving the next message from ``src`` ahead of the ``recv`` that will ask for it; the default
        does nothing."""
        return False


Signature = Tuple[Tuple[int, ...], torch.dtype, bool]  # shape, dtype, requires_grad


class SendRecvTransport(Transport):
    """Blocking-receive / async-send tensor transport for one pipeline group."""

    def __init__(self, group: Any, device: torch.device, static_shapes: bool = False):
        self.group = group
        self.device = device
        self.static_shapes = static_shapes
        self._pending: List[Any] = []
        self._sent: Dict[Tuple[int, int], Signature] = {}      # (destination, slot) -> contract
        self._expected: Dict[Tuple[int, int], Signature] = {}  # (source, slot) -> contract
        self.headers_sent = 0      # instrumentation: how many messages carried a header ...
        self.headers_received = 0  # ... and how many receives had to read one on the host
        self._prefetched: Dict[Tuple[int, Optional[int]], Tuple[Tensor, Any]] = {}  # (source, slot) -> (buffer, pending receive)
        self.prefetches = 0        # receives that were posted ahead of their use

    def _global(self, group_rank: int) -> int:
        return dist.get_global_rank(self.group, group_rank) if self.group is not None and self.group is not dist.group.WORLD else group_rank

    def send(self, t: Tensor, dst: int, slot: Optional[int] = None) -> None:
        t = t.contiguous()
        assert t.dim() <= 7
        signature: Signature = (tuple(t.shape), t.dtype, bool(t.requires_grad))
        contract = self._sent.get((dst, slot)) if (self.static_shapes and slot is not None) else None
        if contract is not None and contract != signature:
            raise RuntimeError(f"message for stage {dst}, slot {slot} is {signature} but the static contract says {contract}; "
                               "create the transport with static_shapes=False for varying shapes")
        keep: List[Any] = [t]
        if contract is None:
            head = torch.zeros(_HEADER, dtype=torch.int64)
            head[0], head[1], head[2] = t.dim(), _DTYPES.index(t.dtype), int(t.requires_grad)
            for i, s in enumerate(t.shape):
                head[3 + i] = s
            head = head.to(self.device)
            self._pending.append(dist.isend(head, self._global(dst), group=self.group))
            self.headers_sent += 1
            keep.append(head)
            if self.static_shapes and slot is not None:
                self._sent[(dst, slot)] = signature
        self._pending.append(dist.isend(t.detach(), self._global(dst), group=self.group))
        self._pending.append(keep)  # the buffers stay alive until the sends have completed

    def prefetch(self, src: int, slot: Optional[int]) -> bool:
        """Post the receive of the next message from ``src`` now, so that the transfer runs while the caller computes.
        Possible when the message's shape is known (static-shape contract already established for ``(src, slot)``); the
        caller must ask for this message next among those from ``src``.  Returns whether a receive was posted."""
        contract = self._expected.get((src, slot)) if (self.static_shapes and slot is not None) else None
        if contract is None or (src, slot) in self._prefetched:
            return False
        shape, dtype, _ = contract
        buf = torch.empty(shape, dtype=dtype, device=self.device)
        self._prefetched[(src, slot)] = (buf, dist.irecv(buf, self._global(src), group=self.group))
        self.prefetches += 1
        return True

    def recv(self, src: int, slot: Optional[int] = None) -> Tensor:
        pending = self._prefetched.pop((src, slot), None)
        if pending is not None:
            out, work = pending
            work.wait()
            if self._expected[(src, slot)][2] and out.is_floating_point():
                out.requires_grad_()
            return out
        contract = self._expected.get((src, slot)) if (self.static_shapes and slot is not None) else None
        if contract is None:
            head = torch.zeros(_HEADER, dtype=torch.int64, device=self.device)
            dist.recv(head, self._global(src), group=self.group)
            h = head.tolist()  # the one host synchronisation of a message with a header
            self.headers_received += 1
            contract = (tuple(h[3 : 3 + h[0]]), _DTYPES[h[1]], bool(h[2]))
            if self.static_shapes and slot is not None:
                self._expected[(src, slot)] = contract
        shape, dtype, requires_grad = contract
        out = torch.empty(shape, dtype=dtype, device=self.device)
        dist.recv(out, self._global(src), group=self.group)
        if requires_grad and out.is_floating_point():
            out.requires_grad_()
        return out

    def flush(self) -> None:
        for w in self._pending:
            if hasattr(w, "wait"):
                w.wait()
        self._pending.clear()


# ---------------------------------------------------------------------------------------------------------------------
# RPC transport: the same send / recv / flush interface carried by torch.distributed.rpc (TensorPipe).  Tensors travel
# as CPU copies into per-(transport, source) queues of the destination process, as in the reference's RpcTransport
# (fairscale/nn/pipe/messages.py:55-107).  It needs no process-group p2p support and is meant for control-plane sized
# traffic and for clusters without NCCL p2p; activations of real models belong on SendRecvTransport.
# ---------------------------------------------------------------------------------------------------------------------
_rpc_queues: Dict[Tuple[int, int], "queue.Queue[Any]"] = {}
_rpc_queues_lock = threading.Lock()


def _rpc_queue(channel: int, src: int) -> "queue.Queue[Any]":
    with _rpc_queues_lock:
        q = _rpc_queues.get((channel, src))
        if q is None:
            q = _rpc_queues[(channel, src)] = queue.Queue()
        return q


def rpc_push_queue(channel: int, src: int, seq: int, payload: Tensor, requires_grad: bool) -> None:
    """Runs on the destination worker: file message number ``seq`` from group rank ``src`` under ``channel``."""
    _rpc_queue(channel, src).put((seq, payload, requires_grad))


class RpcTransport(Transport):
    """``send`` / ``recv`` / ``flush`` over ``torch.distributed.rpc``.

    Args:
        rank: this process's rank in the pipeline group.
        worker_name: maps a group rank to its RPC worker name (default ``"Test<rank>"``, the reference's test naming).
        device: where received tensors are placed.
        channel: distinguishes independent transports between the same workers.
        timeout: seconds a ``recv`` waits before raising ``TimeoutError``.
    """

    def __init__(self, rank: int, device: torch.device, worker_name: Optional[Callable[[int], str]] = None, channel: int = 0,
                 timeout: float = 120.0) -> None:
        from torch.distributed import rpc

        self.rpc = rpc
        self.rank = rank
        self.device = device
        self.worker_name = worker_name or (lambda r: f"Test{r}")
        self.channel = channel
        self.timeout = timeout
        self._pending: List[Any] = []
        # RPC calls to one worker may run out of order there: messages are numbered per destination and put back in
        # order by the receiver
        self._next_send: Dict[int, int] = {}
        self._next_recv: Dict[int, int] = {}
        self._early: Dict[Tuple[int, int], Any] = {}

    def send(self, t: Tensor, dst: int, slot: Optional[int] = None) -> None:
        seq = self._next_send.get(dst, 0)
        self._next_send[dst] = seq + 1
        args = (self.channel, self.rank, seq, t.detach().cpu(), bool(t.requires_grad))
        self._pending.append(self.rpc.rpc_async(self.worker_name(dst), rpc_push_queue, args=args))

    def recv(self, src: int, slot: Optional[int] = None) -> Tensor:
        want = self._next_recv.get(src, 0)
        self._next_recv[src] = want + 1
        q = _rpc_queue(self.channel, src)
        while (src, want) not in self._early:
            try:
                seq, payload, requires_grad = q.get(timeout=self.timeout)
            except queue.Empty:
                raise TimeoutError(f"no message from pipeline rank {src} within {self.timeout} s") from None
            self._early[(src, seq)] = (payload, requires_grad)
        payload, requires_grad = self._early.pop((src, want))
        out = payload.to(self.device)
        if requires_grad and out.is_floating_point():
            out.requires_grad_()
        return out

    def flush(self) -> None:
        for f in self._pending:
            f.wait()
        self._pending.clear()


def get_transport(group: Any, device: torch.device, **rpc_kwargs: Any) -> Any:
    """p2p transport unless ``FORCE_RPC`` is set (the reference picks RPC unless it runs under MPI,
    fairscale/nn/pipe/async_pipeline.py:39-43; here p2p over NCCL / gloo is the default because it always exists)."""
    if os.environ.get("FORCE_RPC", "").lower() in ("1", "true", "yes"):
        return RpcTransport(dist.get_rank(group), device, **rpc_kwargs)
    # FSB200_PIPE_STATIC_SHAPES=1: every (peer, micro-batch) message keeps its shape from step to step, headers are sent once
    return SendRecvTransport(group, device, static_shapes=os.environ.get("FSB200_PIPE_STATIC_SHAPES", "0") == "1")


def MakeTransport(use_rpc: bool, worker_map: Optional[Dict[int, str]], input_device: Optional[torch.device], group: Any = None) -> Transport:
    """Explicit choice of transport (parity: fairscale/nn/pipe/messages.py:50-58): RPC needs the rank -> worker name map."""
    device = input_device if input_device is not None else torch.device("cpu")
    if use_rpc:
        if worker_map is None:
            raise ValueError("'RpcTransport' requires 'worker_map' to be set")
        names = dict(worker_map)
        return RpcTransport(dist.get_rank(group), device, worker_name=lambda r: names[r])
    return SendRecvTransport(group if group is not None else dist.group.WORLD, device)
