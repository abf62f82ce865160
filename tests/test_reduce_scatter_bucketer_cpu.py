"""ReduceScatterBucketer on gloo ranks: small inputs share a bucket and are reduced at flush, large ones at once; the
callbacks receive the reduced shard of exactly their tensor."""
import torch
import torch.distributed as dist

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.internal.reduce_scatter_bucketer import ReduceScatterBucketer
from fairscale_b200.parallel import comm


def _worker(rank, world):
    group = dist.group.WORLD
    bucketer = ReduceScatterBucketer(bucket_cap_mb=1)  # 1 MiB / 4 bytes / 2 ranks = 131072 fp32 slots per rank
    results = {}
    sizes = [(3, 2), (5,), (200000,), (7, 3)]  # the third one does not fit a bucket row
    comm.reset_counters()
    for idx, shape in enumerate(sizes):
        n = 1
        for s in shape:
            n *= s
        # rank r contributes (r + 1) * (idx + 1) to every chunk; chunk c additionally carries c
        inputs = [torch.full(shape, float((rank + 1) * (idx + 1) + c)) for c in range(world)]
        bucketer.reduce_scatter_async(inputs, group, callback_fn=lambda t, i=idx: results.__setitem__(i, t.clone()))
        if n > 131072:
            assert idx in results and comm.counters()["reduce_scatter"] == 1  # ran immediately, on its own
        else:
            assert idx not in results  # waits in the bucket
    bucketer.flush()
    assert comm.counters()["reduce_scatter"] == 2  # one for the large tensor, one for the whole bucket
    total = sum(r + 1 for r in range(world))
    for idx, shape in enumerate(sizes):
        expect = torch.full(shape, float(total * (idx + 1) + world * rank))
        torch.testing.assert_close(results[idx], expect)
        assert results[idx].shape == torch.Size(shape)
    # a second round reuses the bucket; teardown releases it
    bucketer.reduce_scatter_async([torch.ones(4) for _ in range(world)], group, callback_fn=lambda t: results.__setitem__("again", t.clone()))
    bucketer.flush()
    torch.testing.assert_close(results["again"], torch.full((4,), float(world)))
    bucketer.teardown()
    # bucketing switched off: every call reduces at once
    direct = ReduceScatterBucketer(bucket_cap_mb=0)
    got = []
    direct.reduce_scatter_async([torch.ones(2) * (rank + 1) for _ in range(world)], group, callback_fn=got.append)
    assert len(got) == 1 and torch.equal(got[0], torch.full((2,), float(total)))


def test_reduce_scatter_bucketer():
    spawn_ranks(_worker, 2, (), backend="gloo")
