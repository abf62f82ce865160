"""Coalesce many small gradient reduce-scatters into few large ones.

Parity: fairscale/internal/reduce_scatter_bucketer.py:24-204.  A staging buffer of
shape ``[world, slots]`` per (dtype, device, group) collects the ``world`` chunks of
each small gradient column-wise; one reduce-scatter of the filled prefix yields the
local result of every queued gradient at once.  Inputs larger than a staging row go
out directly.  Staging memory only exists between the first queued gradient and
``teardown()`` (i.e. during backward).

On NVSwitch the collective cost is dominated by launch latency rather than link
count, so the default capacity (25 MB) is kept for API parity while the collective
itself is routed through :mod:`fairscale_b200.parallel.comm`.
"""

from __future__ import annotations

from typing import TYPE_CHECKING, Any, Callable, Dict, List, Optional, Tuple

import torch
from torch import Tensor

from ..parallel import comm

if TYPE_CHECKING:
    from torch.distributed import ProcessGroup


def _release(t: Tensor) -> None:
    t.untyped_storage().resize_(0)


def _materialize(t: Tensor) -> None:
    st = t.untyped_storage()
    want = t.numel() * t.element_size()
    if st.size() != want:
        st.resize_(want)


class Bucket:
    """One ``[world, slots]`` staging buffer plus the shard the reduction lands in."""

    def __init__(self, data: Tensor, group: "ProcessGroup"):
        self.data = data
        self.group = group
        self.offset = 0
        self.callbacks: List[Callable[[], None]] = []
        self.output_shard = torch.zeros_like(data[0])

    def flush(self) -> None:
        if self.offset == 0:
            assert not self.callbacks
            return
        used = self.offset
        comm.reduce_scatter_into(self.output_shard[:used], self.data[:, :used].contiguous(), group=self.group)
        for cb in self.callbacks:
            cb()
        # the staging rows are reused; callbacks keep views of the landed shard, so it is replaced
        self.data[:, :used].zero_()
        self.offset = 0
        self.callbacks.clear()
        self.output_shard = torch.zeros_like(self.data[0])

    def setup(self) -> None:
        for t in (self.data, self.output_shard):
            if t.untyped_storage().size() == 0:
                _materialize(t)
                t.zero_()

    def teardown(self) -> None:
        assert self.offset == 0 and not self.callbacks, "Incorrect call of teardown"
        for t in (self.data, self.output_shard):
            _release(t)


class ReduceScatterBucketer:
    """Queue reduce-scatters; small ones share a bucket, big ones run immediately.

    Callbacks receive the reduced local shard and are only guaranteed to have run
    after :meth:`flush`.  ``bucket_cap_mb <= 0`` disables bucketing.
    """

    def __init__(self, bucket_cap_mb: int = 25):
        self.bucket_cap_mb = bucket_cap_mb
        self.buckets: Dict[Tuple[torch.dtype, torch.device, Any], Bucket] = {}
        self._shard_size_cache: Dict[Tuple[int, int], int] = {}

    @torch.no_grad()
    def reduce_scatter_async(
        self, input_list: List[Tensor], group: "ProcessGroup", callback_fn: Optional[Callable] = None
    ) -> None:
        world = group.size()
        assert len(input_list) == world, (
            f"reduce_scatter received {len(input_list)} inputs, expected group.size() ({world})"
        )
        first = input_list[0]
        n = first.numel()
        slots = self._get_shard_size(first.element_size(), world)

        if n > slots:
            out = torch.zeros_like(first)
            flat = _as_flat(input_list)
            comm.reduce_scatter_into(out, flat, group=group)
            if callback_fn is not None:
                callback_fn(out)
            return

        bucket = self._get_bucket(first, group)
        if n > bucket.data.size(1) - bucket.offset:
            bucket.flush()
        lo = bucket.offset
        for r, piece in enumerate(input_list):
            bucket.data[r, lo : lo + n].copy_(piece.reshape(-1))
        bucket.offset = lo + n
        if callback_fn is not None:
            landed = bucket.output_shard[lo : lo + n].view_as(first)
            bucket.callbacks.append(lambda cb=callback_fn, v=landed: cb(v))

    @torch.no_grad()
    def flush(self) -> None:
        for b in self.buckets.values():
            b.flush()

    @torch.no_grad()
    def teardown(self) -> None:
        for b in self.buckets.values():
            b.teardown()

    def _get_shard_size(self, element_size: int, num_shards: int) -> int:
        key = (element_size, num_shards)
        if key not in self._shard_size_cache:
            if self.bucket_cap_mb <= 0:
                size = 0
            else:
                size = int((self.bucket_cap_mb * 1024 * 1024 / element_size) // num_shards)
            self._shard_size_cache[key] = size
        return self._shard_size_cache[key]

    def _get_bucket(self, tensor: Tensor, group: "ProcessGroup") -> Bucket:
        key = (tensor.dtype, tensor.device, group)
        if key not in self.buckets:
            world = group.size()
            slots = self._get_shard_size(tensor.element_size(), world)
            self.buckets[key] = Bucket(tensor.new_zeros((world, slots)), group)
        self.buckets[key].setup()
        return self.buckets[key]


def _as_flat(chunks: List[Tensor]) -> Tensor:
    """Return the chunks as one contiguous 1-D tensor, without a copy when they already are
    consecutive views of one storage (the common case: ``chunk_and_pad`` of an unpadded grad)."""
    first = chunks[0]
    n = first.numel()
    base_ptr = first.data_ptr()
    step = n * first.element_size()
    if all(c.is_contiguous() and c.numel() == n and c.data_ptr() == base_ptr + i * step for i, c in enumerate(chunks)):
        try:
            return torch.as_strided(first.reshape(-1), (n * len(chunks),), (1,))
        except RuntimeError:
            pass
    return torch.cat([c.reshape(-1) for c in chunks])
