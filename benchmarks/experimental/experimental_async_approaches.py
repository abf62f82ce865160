"""Asynchronous (stale-weight) pipeline training with weight-prediction optimizers: plain AMPnet, SpecTrain and XPipe
(reference driver: benchmarks/experimental/experimental_async_approaches.py:129-873).

The optimizers expose ``update_weight_using_future_predictions(rank, n_stages, index, chunks, forward)``, the hook
``AMPnetPipe.interleave(..., weight_prediction=True)`` calls before every forward / backward: it moves the weights to where
they are predicted to be when the gradient of this micro-batch is finally applied (s steps of the smoothed update ahead,
s = staleness of the stage), and ``step()`` restores the real weights before applying the gradient.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/experimental/experimental_async_approaches.py [--optimizer spectrain|xpipe|sgd]
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist
from torch import nn
from torch.optim import Optimizer
from torch.utils.data import DataLoader

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from benchmarks.experimental.benchmark_dataset import BenchmarkLMDataset, collate_sentences_lm  # noqa: E402
from fairscale_b200.experimental.nn.ampnet_pipe import AMPnetPipe  # noqa: E402
from fairscale_b200.models.transformer_lm import TransformerLM  # noqa: E402


class _PredictingOptimizer(Optimizer):
    """Base: keeps the real weights aside while predicted ones are installed."""

    def __init__(self, params, defaults):
        super().__init__(params, defaults)
        self._real = None

    def _velocity(self, p, group):  # smoothed update direction per unit step, provided by subclasses
        raise NotImplementedError

    @staticmethod
    def staleness(rank: int, n_stages: int, forward: bool) -> int:
        """Optimizer steps between this pass and the moment its gradient lands (version difference of the stage)."""
        return (n_stages - 1 - rank) if forward else 0

    @torch.no_grad()
    def update_weight_using_future_predictions(self, rank, n_stages, index, chunks, forward):
        self._restore()
        s = self.staleness(rank, n_stages, forward)
        if s == 0:
            return
        self._real = []
        for group in self.param_groups:
            for p in group["params"]:
                v = self._velocity(p, group)
                if v is None:
                    continue
                self._real.append((p, p.detach().clone()))
                p.add_(v, alpha=-group["lr"] * s)

    @torch.no_grad()
    def _restore(self):
        if self._real:
            for p, saved in self._real:
                p.copy_(saved)
        self._real = None


class SpectrainSGDMomentum(_PredictingOptimizer):
    """SGD with momentum; prediction along the momentum buffer (SpecTrain, arXiv:1809.02839)."""

    def __init__(self, params, lr, momentum=0.9, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay))

    def _velocity(self, p, group):
        return self.state[p].get("momentum_buffer")

    @torch.no_grad()
    def step(self, closure=None):
        self._restore()
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad.add(p, alpha=group["weight_decay"]) if group["weight_decay"] else p.grad
                buf = self.state[p].get("momentum_buffer")
                buf = self.state[p]["momentum_buffer"] = g.clone() if buf is None else buf.mul_(group["momentum"]).add_(g)
                p.add_(buf, alpha=-group["lr"])


class XpipeAdam(_PredictingOptimizer):
    """Adam; prediction along m / (sqrt(v) + eps) (XPipe, arXiv:1911.04610)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps))

    def _velocity(self, p, group):
        st = self.state[p]
        if "exp_avg" not in st:
            return None
        return st["exp_avg"] / (st["exp_avg_sq"].sqrt() + group["eps"])

    @torch.no_grad()
    def step(self, closure=None):
        self._restore()
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "exp_avg" not in st:
                    st["step"], st["exp_avg"], st["exp_avg_sq"] = 0, torch.zeros_like(p), torch.zeros_like(p)
                st["step"] += 1
                st["exp_avg"].mul_(b1).add_(p.grad, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(p.grad, p.grad, value=1 - b2)
                step_size = group["lr"] * (1 - b2 ** st["step"]) ** 0.5 / (1 - b1 ** st["step"])
                p.addcdiv_(st["exp_avg"], st["exp_avg_sq"].sqrt() + group["eps"], value=-step_size)


class _Delegate:
    def __init__(self):
        self.losses = []

    def transform_input(self, b):
        return b["input"]

    def transform_target(self, b):
        return b["target"].reshape(-1)

    def transform_output_before_loss(self, out):
        return out.reshape(-1, out.shape[-1]).float()

    def log_loss(self, batch, loss, count):
        self.losses.append(float(loss.detach()))

    def check_and_save_weights(self, n):
        pass


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--optimizer", default="spectrain", choices=["sgd", "spectrain", "xpipe"])
    ap.add_argument("--samples", type=int, default=64)
    ap.add_argument("--seq", type=int, default=32)
    args = ap.parse_args()
    cuda = torch.cuda.is_available()
    rank = int(os.environ.get("LOCAL_RANK", "0"))
    if cuda:
        torch.cuda.set_device(rank)
    dist.init_process_group("nccl" if cuda else "gloo")
    world = dist.get_world_size()
    torch.manual_seed(0)
    model = TransformerLM(1000, 64, 4, 128, 0.0, 0.1, 2)
    base, rem = divmod(len(model), world)
    pipe = AMPnetPipe(model, balance=[base + (1 if i < rem else 0) for i in range(world)], chunks=1, checkpoint="never")
    params = list(pipe.partition.parameters())
    opt = {"sgd": lambda: torch.optim.SGD(params, lr=0.05), "spectrain": lambda: SpectrainSGDMomentum(params, lr=0.05),
           "xpipe": lambda: XpipeAdam(params, lr=1e-3)}[args.optimizer]()
    data = DataLoader(BenchmarkLMDataset(1000, args.seq, args.samples), batch_size=4, collate_fn=collate_sentences_lm)
    delegate = _Delegate()
    pipe.interleave(data, nn.CrossEntropyLoss(), opt, delegate, weight_prediction=args.optimizer != "sgd")
    if dist.get_rank() == world - 1:
        n = len(delegate.losses)
        print(json.dumps({"benchmark": "async_pipe", "optimizer": args.optimizer, "stages": world, "first_losses": sum(delegate.losses[: n // 4]) / (n // 4),
                          "last_losses": sum(delegate.losses[-(n // 4):]) / (n // 4)}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
