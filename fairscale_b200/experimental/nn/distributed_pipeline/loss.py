"""Loss evaluated where the model output lives (parity: .../distributed_pipeline/loss.py:10-22)."""

from typing import Any, Callable

from torch.distributed import rpc


def _rloss(loss_func: Callable, input_rref: rpc.RRef, target_rref: rpc.RRef) -> Any:
    return loss_func(input_rref.to_here(), target_rref.to_here())


def DistributedLoss(loss: Any, *args: Any, **kwargs: Any) -> Callable:
    """``DistributedLoss(nn.MSELoss)(output_rref, target_rref)`` returns an RRef to the loss on the output's owner."""
    loss_func = loss(*args, **kwargs)

    def dloss(input_rref: rpc.RRef, target_rref: rpc.RRef) -> rpc.RRef:
        return rpc.remote(input_rref.owner(), _rloss, args=(loss_func, input_rref, target_rref))

    return dloss
