"""Fused multi-tensor Adam.

API parity with fairscale/optim/adam.py:19-300 (``Adam`` + ``Precision``); the kernel is
``csrc/adam.cu``.  Differences that matter on B200:

* bf16 parameters / gradients / low-precision copies are supported (the reference asserts fp16);
* all tensors of a param group on one device are updated by ONE launch driven by a table in device
  memory, filled through a pinned host buffer (no per-launch 4 KB argument packing);
* an optional device-side ``inv_scale`` (AMP unscale or clip coefficient) and ``noop_flag`` fold
  gradient unscaling / skipped steps into the same pass without a host sync;
* only ``Precision.PURE_FP16`` (scaled fp16 moments) needs to read ``found_inf`` back.

On CPU tensors the same class runs a pure PyTorch restatement of the kernel math, which is also the
oracle of the GPU numerics tests.
"""

from __future__ import annotations

from enum import Enum, auto
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
from torch.optim import Optimizer

from ..ops import _bind


class Precision(Enum):
    FULL_PRECISION = auto()
    MIXED_PRECISION = auto()
    MEMORY_EFFICIENT_MIXED_PRECISION = auto()
    PURE_FP16 = auto()


_LOW = (torch.float16, torch.bfloat16)


def adam_reference_step(
    p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, *, step_size: float, lr: float, beta1: float,
    beta2: float, eps: float, eps_mode: int, weight_decay: float, grad_scale: float = 1.0, optim_scale: float = 1.0,
    adamw: bool = False, p_copy: Optional[torch.Tensor] = None,
) -> bool:
    """fp32 restatement of the kernel's update for one tensor (in place).  Returns True if a scaled
    fp16 moment overflowed."""
    pf = p.detach().float()
    gf = g.detach().float() / grad_scale
    scaled = m.dtype != torch.float32
    mf = m.float() / optim_scale if scaled else m.float()
    vf = v.float() / optim_scale if scaled else v.float()
    mf = beta1 * mf + (1 - beta1) * gf
    vf = beta2 * vf + (1 - beta2) * gf * gf
    denom = torch.sqrt(vf + eps) if eps_mode == 0 else torch.sqrt(vf) + eps
    if adamw:
        pf = pf * (1 - lr * weight_decay) - step_size * (mf / denom)
    else:
        pf = pf - step_size * (mf / denom + weight_decay * pf)
    overflow = False
    if scaled:
        ms, vs = (mf * optim_scale).to(m.dtype), (vf * optim_scale).to(v.dtype)
        overflow = not (bool(torch.isfinite(ms).all()) and bool(torch.isfinite(vs).all()))
        m.copy_(ms)
        v.copy_(vs)
    else:
        m.copy_(mf)
        v.copy_(vf)
    p.detach().copy_(pf)
    if p_copy is not None:
        p_copy.copy_(pf)
    return overflow


class _DeviceTable:
    """Pinned host staging (a small ring, guarded by events) + device copy of one launch's pointer table."""

    RING = 4

    def __init__(self, device: torch.device, capacity: int):
        self.capacity = capacity
        self.hosts = [torch.zeros((capacity, 8), dtype=torch.int64).pin_memory() for _ in range(self.RING)]
        self.events: List[Optional[torch.cuda.Event]] = [None] * self.RING
        self.devs = [torch.zeros((capacity, 8), dtype=torch.int64, device=device) for _ in range(self.RING)]
        self.cursor = 0

    def upload(self, rows: List[Tuple[int, ...]]) -> torch.Tensor:
        i = self.cursor
        self.cursor = (i + 1) % self.RING
        ev = self.events[i]
        if ev is not None:
            ev.synchronize()  # the kernel that read this slot (RING steps ago) has finished
        n = len(rows)
        self.hosts[i][:n] = torch.tensor(rows, dtype=torch.int64)
        self.devs[i][:n].copy_(self.hosts[i][:n], non_blocking=True)
        return self.devs[i]

    def mark_used(self) -> None:
        """Record, after the consuming kernel was launched, when the most recent slot may be reused."""
        i = (self.cursor - 1) % self.RING
        ev = self.events[i] or torch.cuda.Event()
        ev.record()
        self.events[i] = ev


class Adam(Optimizer):
    """Adam / AdamW with one fused kernel launch per (param group, device).

    Args follow the reference: ``lr, bias_correction, betas, eps, eps_inside_sqrt, weight_decay,
    max_grad_norm (unused, kept for signature parity), amsgrad (must be False), precision``.
    ``weight_decay`` is classic L2 (added to the update) unless ``decoupled_weight_decay=True``.

    Precision modes: FULL (params and state in the param dtype's fp32), MIXED (fp16/bf16 params, fp32
    master copy held by the optimizer, low-precision copy written by the kernel),
    MEMORY_EFFICIENT_MIXED (fp16/bf16 params updated directly, fp32 moments), PURE_FP16 (fp16 moments
    stored times ``optim_scale``, halved on overflow and doubled every 2000 clean steps).
    """

    def __init__(
        self,
        params: Any,
        lr: float = 1e-3,
        bias_correction: bool = True,
        betas: Tuple[float, float] = (0.9, 0.999),
        eps: float = 1e-8,
        eps_inside_sqrt: bool = False,
        weight_decay: float = 0.0,
        max_grad_norm: float = 0.0,
        amsgrad: bool = False,
        precision: Optional[Precision] = None,
        decoupled_weight_decay: bool = False,
    ):
        parameters: List[Any] = list(params)
        first = parameters[0]["params"][0] if isinstance(parameters[0], dict) else parameters[0]
        self.precision = precision
        if self.precision is None:
            self.precision = Precision.FULL_PRECISION if first.dtype == torch.float32 else Precision.MIXED_PRECISION
        if self.precision is not Precision.FULL_PRECISION:
            assert first.dtype in _LOW, "mixed / pure low-precision modes expect fp16 or bf16 parameters"
        self.optim_type = torch.float16 if precision is Precision.PURE_FP16 else torch.float32
        self._optim_scale = float(2**16) if precision is Precision.PURE_FP16 else 1.0
        self._steps_since_optim_scale_change = 0
        self._optim_scale_update_freq = 2000
        if amsgrad:
            raise RuntimeError("FusedAdam does not support the AMSGrad variant.")
        if lr < 0.0 or eps < 0.0 or weight_decay < 0.0:
            raise ValueError(f"lr, eps and weight_decay must not be negative (got lr={lr}, eps={eps}, weight_decay={weight_decay})")
        if not (0.0 <= betas[0] < 1.0 and 0.0 <= betas[1] < 1.0):
            raise ValueError(f"betas must lie in [0, 1), got {betas}")
        defaults = dict(lr=lr, bias_correction=bias_correction, betas=betas, eps=eps, weight_decay=weight_decay,
                        max_grad_norm=max_grad_norm)
        super().__init__(parameters, defaults)
        self.eps_mode = 0 if eps_inside_sqrt else 1
        self.adamw = decoupled_weight_decay
        self.fp32_param_groups: List[Any] = []
        if self.mixed_precision:
            self._build_fp32_params()
        self._tables: Dict[Tuple[int, torch.device], _DeviceTable] = {}
        self._found_inf: Dict[torch.device, torch.Tensor] = {}
        # optional extras set by wrappers: device scalar multiplied into every gradient, and a skip flag
        self.inv_scale: Optional[torch.Tensor] = None
        self.noop_flag: Optional[torch.Tensor] = None
        # param -> low-precision tensor that should receive the updated value (e.g. FSDP compute shard)
        self.param_copies: Dict[torch.Tensor, torch.Tensor] = {}

    def _build_fp32_params(self) -> None:
        self.fp32_param_groups = []
        for group in self.param_groups:
            masters = []
            for p in group["params"]:
                p32 = torch.nn.Parameter(p.data.float())
                masters.append(p32)
            self.fp32_param_groups.append({"params": masters})

    @property
    def supports_memory_efficient_fp16(self) -> bool:
        return True

    @property
    def _step_supports_amp_scaling(self) -> bool:
        return False

    @property
    def mixed_precision(self) -> bool:
        return self.precision is Precision.MIXED_PRECISION

    def state_dict(self) -> Dict[str, Any]:
        d = super().state_dict()
        d["optim_scale"] = self._optim_scale
        return d

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        state_dict = dict(state_dict)
        scale = state_dict.pop("optim_scale", self._optim_scale)
        super().load_state_dict(state_dict)
        self._optim_scale = scale
        # torch casts loaded state to the dtype of its parameter, which would round fp32 moments of fp16 / bf16 parameters
        # (the reference accepts that loss, fairscale/optim/adam.py:169-181): take the moments from the saved tensors instead
        saved_state = state_dict.get("state", {})
        for group, saved_group in zip(self.param_groups, state_dict["param_groups"]):
            for p, saved_id in zip(group["params"], saved_group["params"]):
                st, saved = self.state.get(p), saved_state.get(saved_id)
                if not st or "exp_avg" not in st:
                    continue
                for key in ("exp_avg", "exp_avg_sq"):
                    src = saved[key] if saved is not None and torch.is_tensor(saved.get(key)) else st[key]
                    st[key] = src.detach().to(device=p.device, dtype=self.optim_type, copy=True)

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure: Optional[Callable[[], float]] = None) -> Optional[float]:
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()

        any_overflow = False
        for gi, group in enumerate(self.param_groups):
            beta1, beta2 = group["betas"]
            per_device: Dict[torch.device, List[Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, Optional[torch.Tensor]]]] = {}
            step_no = None
            for pj, p in enumerate(group["params"]):
                if p.grad is None:
                    continue
                grad = p.grad.data
                if grad.is_sparse:
                    raise RuntimeError("FusedAdam does not support sparse gradients, please consider SparseAdam instead")
                state = self.state[p]
                if len(state) == 0:
                    state["step"] = 0
                    state["exp_avg"] = torch.zeros_like(p, dtype=self.optim_type)
                    state["exp_avg_sq"] = torch.zeros_like(p, dtype=self.optim_type)
                state["step"] += 1
                step_no = state["step"]
                if self.mixed_precision:
                    master = self.fp32_param_groups[gi]["params"][pj].data
                    copy: Optional[torch.Tensor] = p.data
                else:
                    master = p.data
                    copy = self.param_copies.get(p)
                per_device.setdefault(p.device, []).append((master, grad, state["exp_avg"], state["exp_avg_sq"], copy))
            if step_no is None:
                continue
            if group["bias_correction"]:
                step_size = group["lr"] * (1 - beta2**step_no) ** 0.5 / (1 - beta1**step_no)
            else:
                step_size = group["lr"]
            for device, items in per_device.items():
                if device.type == "cuda":
                    self._launch(gi, device, items, group, step_size)
                else:
                    for master, grad, m, v, copy in items:
                        g = grad if self.inv_scale is None else grad.float() * self.inv_scale.to(grad.device)
                        if self.noop_flag is not None and bool(self.noop_flag.item()):
                            continue
                        any_overflow |= adam_reference_step(
                            master, g, m, v, step_size=step_size, lr=group["lr"], beta1=beta1, beta2=beta2, eps=group["eps"],
                            eps_mode=self.eps_mode, weight_decay=group["weight_decay"], optim_scale=self._optim_scale,
                            adamw=self.adamw, p_copy=copy,
                        )

        if self.precision is Precision.PURE_FP16:
            for t in self._found_inf.values():
                any_overflow |= bool(t.item())
                t.zero_()
            self._update_optim_scale(any_overflow)
        return loss

    # ------------------------------------------------------------------ step fused into the gradient reduction
    def group_of(self, p: torch.Tensor) -> Optional[Dict[str, Any]]:
        for group in self.param_groups:
            if any(q is p for q in group["params"]):
                return group
        return None

    def can_fuse_reduce_scatter(self, p: torch.Tensor) -> bool:
        """Whether :meth:`reduce_scatter_step` may update ``p``: plain fp32 Adam state, nothing that has to look at all
        gradients first (a loss scaler's skip flag, a clip coefficient) and the parameter known to this optimizer."""
        return (self.precision is Precision.FULL_PRECISION and p.dtype == torch.float32 and self.inv_scale is None
                and self.noop_flag is None and self.group_of(p) is not None)

    @torch.no_grad()
    def reduce_scatter_step(self, p: torch.Tensor, workspace: Any, flat_grad: torch.Tensor, scale: float,
                            gnorm_sq: Optional[torch.Tensor] = None) -> None:
        """This optimizer's step for the single (sharded, fp32) parameter ``p``, executed inside the reduce-scatter of its
        unreduced flat gradient ``flat_grad``: one NVLink kernel sums the peers' slices, applies Adam to ``p`` and its
        moments and writes the compute-dtype copy registered in ``param_copies``.  The caller leaves ``p.grad`` unset, so
        the regular :meth:`step` of the same iteration skips ``p``."""
        group = self.group_of(p)
        assert group is not None
        state = self.state[p]
        if len(state) == 0:
            state["step"] = 0
            state["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
            state["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
        state["step"] += 1
        t = state["step"]
        beta1, beta2 = group["betas"]
        step_size = group["lr"] * (1 - beta2**t) ** 0.5 / (1 - beta1**t) if group["bias_correction"] else group["lr"]
        found = self._found_inf.get(p.device)
        if found is None:
            found = self._found_inf[p.device] = torch.zeros(1, dtype=torch.int32, device=p.device)
        workspace.reduce_scatter_adam(flat_grad, p.data.view(-1), state["exp_avg"].view(-1), state["exp_avg_sq"].view(-1),
                                      self.param_copies.get(p), scale, step_size, group["lr"], beta1, beta2, group["eps"],
                                      group["weight_decay"], self.eps_mode == 0, self.adamw, gnorm_sq=gnorm_sq, found_inf=found)

    def _launch(self, gi: int, device: torch.device, items: List[Any], group: Dict[str, Any], step_size: float) -> None:
        chunk = _bind.fn("fsb_adam_chunk_size")()
        # one launch per distinct dtype signature (normally exactly one)
        buckets: Dict[Tuple[torch.dtype, torch.dtype, torch.dtype, Optional[torch.dtype]], List[Any]] = {}
        for it in items:
            master, grad, m, v, copy = it
            key = (master.dtype, grad.dtype, m.dtype, None if copy is None else copy.dtype)
            buckets.setdefault(key, []).append(it)
        found = self._found_inf.get(device)
        if found is None:
            found = self._found_inf[device] = torch.zeros(1, dtype=torch.int32, device=device)
        beta1, beta2 = group["betas"]
        with torch.cuda.device(device):
            for bi, (key, its) in enumerate(buckets.items()):
                rows, chunks = [], 0
                for master, grad, m, v, copy in its:
                    assert master.is_contiguous() and grad.is_contiguous() and m.is_contiguous() and v.is_contiguous()
                    n = master.numel()
                    rows.append((master.data_ptr(), grad.data_ptr(), m.data_ptr(), v.data_ptr(),
                                 0 if copy is None else copy.data_ptr(), n, chunks, 0))
                    chunks += (n + chunk - 1) // chunk
                tkey = (gi * 16 + bi, device)
                table = self._tables.get(tkey)
                if table is None or table.capacity < len(rows):
                    table = self._tables[tkey] = _DeviceTable(device, max(16, 2 * len(rows)))
                dev_table = table.upload(rows)
                pd, gd, sd, cd = key
                _bind.call(
                    "fsb_multi_tensor_adam", dev_table.data_ptr(), len(rows), chunks, _bind.dtype_code(pd), _bind.dtype_code(gd),
                    _bind.dtype_code(sd), _bind.dtype_code(cd) if cd is not None else 0, step_size, group["lr"], beta1, beta2,
                    group["eps"], 1.0, self._optim_scale, group["weight_decay"], self.eps_mode, int(self.adamw),
                    _bind.ptr(self.noop_flag), found.data_ptr(), _bind.ptr(self.inv_scale), _bind.stream_ptr(device),
                )
                table.mark_used()

    def _update_optim_scale(self, overflow: bool) -> None:
        if overflow:
            self._steps_since_optim_scale_change = 0
            self._optim_scale /= 2
            if self._optim_scale < 1.0:
                raise RuntimeError("Optimizer state scale < 1. This may mean that gradients are exploding")
            for group in self.param_groups:
                for p in group["params"]:
                    if p in self.state and "exp_avg" in self.state[p]:
                        self.state[p]["exp_avg"] = torch.zeros_like(p, dtype=self.optim_type)
                        self.state[p]["exp_avg_sq"] = torch.zeros_like(p, dtype=self.optim_type)
        else:
            self._steps_since_optim_scale_change += 1
        if self._steps_since_optim_scale_change == self._optim_scale_update_freq:
            self._steps_since_optim_scale_change = 0
            if self._optim_scale < 2**16:
                self._optim_scale *= 2


FusedAdam = Adam
