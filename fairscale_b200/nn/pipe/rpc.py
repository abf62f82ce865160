"""Drive a multi-process pipeline from rank 0 over ``torch.distributed.rpc`` (parity: fairscale/nn/pipe/rpc.py:85-285).

Control plane only: rank 0 tells every worker to construct its :class:`AsyncPipe` stage, to run forward for a
batch and to run its share of backward; tensors travel between stages over p2p as in :class:`AsyncPipe`.
"""

from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional

import torch
import torch.distributed as dist
from torch import Tensor, nn

from .async_pipe import AsyncPipe

def set_device_based_on_group(group: Any = None) -> None:
    """One GPU per rank of the node: global rank modulo the number of visible devices."""
    torch.cuda.set_device(dist.get_rank() % torch.cuda.device_count())


def get_shapes(tensor: Any) -> Any:
    return tensor.shape if isinstance(tensor, Tensor) else [t.shape for t in tensor]


def get_dtype(tensor: Any) -> Any:
    return tensor.dtype if isinstance(tensor, Tensor) else [t.dtype for t in tensor]


def get_global_ranks_from_group(group: Any) -> List[int]:
    return [dist.get_global_rank(group, r) for r in range(dist.get_world_size(group))]


def callback_with_model(callback: Callable[[Any, AsyncPipe], None], ctx: Any, pipe_id: int = 0) -> None:
    """Run ``callback(ctx, model)`` on this worker's stage with the device of its group selected."""
    if torch.cuda.is_available():
        set_device_based_on_group()
    callback(ctx, _PIPES[pipe_id])


_PIPES: Dict[int, AsyncPipe] = {}
_OUTPUTS: Dict[int, Any] = {}  # what the last forward returned on this worker
_NEXT_ID = 0


def _build(pipe_id: int, module_factory: Callable[[], nn.Sequential], args: tuple, kwargs: dict) -> None:
    _PIPES[pipe_id] = AsyncPipe(module_factory(), *args, **kwargs)


def _forward(pipe_id: int, training: bool, grad_enabled: bool = True) -> None:
    pipe = _PIPES[pipe_id]
    pipe.train(training)
    with torch.set_grad_enabled(grad_enabled):  # grad mode is per thread: mirror the caller's on this worker
        out = pipe(None)
    _OUTPUTS[pipe_id] = out
    if pipe.rank == pipe.final_stage and pipe.rank != 0 and isinstance(out, Tensor):
        pipe.transport.send(out, 0)  # rank 0 computes the loss on the pipeline's output


def _backward(pipe_id: int) -> None:
    pipe = _PIPES[pipe_id]
    out = _OUTPUTS.pop(pipe_id, None)
    if pipe.rank == pipe.final_stage and pipe.rank != 0 and isinstance(out, Tensor) and out.requires_grad:
        torch.autograd.backward(out, pipe.transport.recv(0))  # d(loss)/d(output) as computed on rank 0
        pipe.back_helper()
    else:
        pipe.back_helper(out if isinstance(out, list) else None)


def _call(pipe_id: int, fn: Callable[[AsyncPipe], Any]) -> Any:
    return fn(_PIPES[pipe_id])


class PipeBackRedirect(torch.autograd.Function):
    """Identity on the final stage's output as seen by rank 0.  When the loss computed on rank 0 back-propagates, its
    backward tells every worker to run its share of the pipeline's backward, so the caller needs no explicit
    ``wrapper.backward()`` (parity: fairscale/nn/pipe/rpc.py:53-71)."""

    @staticmethod
    def forward(ctx: Any, inputs: Tensor, wrapper: "PipeRPCWrapper") -> Tensor:  # type: ignore[override]
        ctx.wrapper = wrapper
        return inputs.view_as(inputs)

    @staticmethod
    def backward(ctx: Any, *grad: Tensor) -> Any:  # type: ignore[override]
        ctx.wrapper.backward(grad[0])
        return None, None


class PipeRPCWrapper(nn.Module):
    """Rank 0 owns the object; workers are addressed by the names in ``worker_map`` (group rank -> rpc name)."""

    def __init__(self, module_factory: Callable[[], nn.Sequential], *args: Any, worker_map: Optional[Dict[int, str]] = None, **kwargs: Any):
        super().__init__()
        from torch.distributed import rpc

        global _NEXT_ID
        self.pipe_id = _NEXT_ID
        _NEXT_ID += 1
        self.worker_map = worker_map or {r: f"Test{r}" for r in range(dist.get_world_size())}
        self.rpc = rpc
        futs = [rpc.rpc_async(name, _build, args=(self.pipe_id, module_factory, args, kwargs)) for r, name in self.worker_map.items() if r != 0]
        _build(self.pipe_id, module_factory, args, kwargs)
        for f in futs:
            f.wait()
        self.model = _PIPES[self.pipe_id]

    @property
    def final_stage(self) -> int:
        """Group rank of the stage that produces the pipeline's output."""
        return self.model.final_stage

    def foreach_worker(self, callback: Callable[[AsyncPipe], Any], include_self: bool = False) -> List[Any]:
        futs = [self.rpc.rpc_async(name, _call, args=(self.pipe_id, callback)) for r, name in self.worker_map.items() if r != 0]
        out = [callback(self.model)] if include_self else []
        return out + [f.wait() for f in futs]

    def forward(self, tensor: Tensor) -> Any:  # type: ignore[override]
        """Feed ``tensor`` to stage 0 (this process) and return the pipeline's output here on rank 0.  When the last
        stage lives on another worker its output is shipped back, and back-propagating through the returned tensor
        runs every worker's share of backward (:class:`PipeBackRedirect`)."""
        futs = [self.rpc.rpc_async(name, _forward, args=(self.pipe_id, self.training, torch.is_grad_enabled())) for r, name in self.worker_map.items() if r != 0]
        out = self.model(tensor)
        self._pending = futs
        self._stage0_outputs = out if isinstance(out, list) else None
        if self.model.final_stage == 0 or self.model.partition is None:
            return out
        remote = self.model.transport.recv(self.model.final_stage)
        if remote.requires_grad and torch.is_grad_enabled():
            return PipeBackRedirect.apply(remote, self)
        return remote.detach()

    def backward(self, output_grad: Optional[Tensor] = None) -> None:
        """Run backward on every stage.  Called by :class:`PipeBackRedirect` with the gradient of the output; call it
        directly (no argument) after ``loss.backward()`` when the last stage is this process."""
        for f in getattr(self, "_pending", []):
            f.wait()
        if output_grad is not None:
            self.model.transport.send(output_grad, self.model.final_stage)
        futs = [self.rpc.rpc_async(name, _backward, args=(self.pipe_id,)) for r, name in self.worker_map.items() if r != 0]
        self.model.back_helper(self._stage0_outputs)
        for f in futs:
            f.wait()
