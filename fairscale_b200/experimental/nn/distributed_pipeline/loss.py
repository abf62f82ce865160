"""A loss evaluated on the worker that holds the pipeline's output.

``DistributedLoss(nn.MSELoss, reduction="sum")`` builds the loss module once, in the driver; calling the result with the
output RRef of a :class:`DistributedPipeline` and an RRef of the target sends both references (not the tensors) to the
output's owner, which fetches the target, evaluates the loss next to the output and keeps the result: the caller gets an
RRef to a scalar and passes it to ``backward(context_id)``.  Same call convention as
fairscale/experimental/nn/distributed_pipeline/loss.py:10-22.
"""

from typing import Any

from torch.distributed import rpc


class _LossOnOwner:
    """The callable handed back to the user: a loss module plus the remote evaluation."""

    def __init__(self, module: Any) -> None:
        self.module = module

    @staticmethod
    def evaluate(module: Any, output: rpc.RRef, target: rpc.RRef) -> Any:
        # runs on the output's owner: the output is local there, the target is pulled over
        return module(output.to_here(), target.to_here())

    def __call__(self, output: rpc.RRef, target: rpc.RRef) -> rpc.RRef:
        return rpc.remote(output.owner(), _LossOnOwner.evaluate, args=(self.module, output, target))


def DistributedLoss(loss: Any, *args: Any, **kwargs: Any) -> _LossOnOwner:
    """``loss`` is a loss class (or factory); ``args`` / ``kwargs`` are its constructor arguments."""
    return _LossOnOwner(loss(*args, **kwargs))
