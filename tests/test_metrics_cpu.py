"""StepMetrics counts the collectives of an FSDP step and emits one JSON line per step."""
import io
import json

import torch
from torch import nn

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn import FullyShardedDataParallel as FSDP
from fairscale_b200.utils.metrics import StepMetrics


def _worker(rank, world):
    torch.manual_seed(0)
    model = FSDP(nn.Sequential(nn.Linear(16, 16), nn.ReLU(), nn.Linear(16, 4)), compute_device=torch.device("cpu"), bucket_cap_mb=0)
    n_params = sum(p.numel() for p in model.parameters()) * world  # shards -> padded full size
    sink = io.StringIO()
    with StepMetrics(sink, tokens_per_step=8, roofline_ms=0.001, device_timing=False) as m:
        for _ in range(2):
            m.begin_step()
            model(torch.randn(8, 16)).sum().backward()
            rec = m.end_step(loss=1.5)
    lines = [json.loads(l) for l in sink.getvalue().splitlines()]
    assert [l["step"] for l in lines] == [0, 1] and lines[1] == rec == m.last
    assert rec["comm_calls"]["all_gather"] >= 1 and rec["comm_calls"]["reduce_scatter"] == 1
    assert rec["comm_bytes"]["reduce_scatter"] == n_params * 4  # the full fp32 gradient goes into the reduce-scatter
    assert rec["comm_bytes"]["all_gather"] % (n_params * 4) == 0
    assert rec["tokens_per_s"] > 0 and 0 < rec["roofline_fraction"] < 1 and rec["loss"] == 1.5
    # after the context the listener is gone
    before = dict(m._calls)
    model(torch.randn(8, 16)).sum().backward()
    assert m._calls == before


def test_step_metrics_counts_fsdp_traffic():
    spawn_ranks(_worker, 2, (), backend="gloo")


def _timer(rank, world):
    import time

    from fairscale_b200.utils.profiling import device_timer

    with device_timer(steps=2) as t:
        time.sleep(0.05 * (rank + 1))  # rank 1 is the slow one
    assert t.ms >= 95 and abs(t.ms_per_step - t.ms / 2) < 1e-9
    both = [None, None]
    import torch.distributed as dist

    dist.all_gather_object(both, t.ms)
    assert both[0] == both[1]  # every rank reports the maximum


def test_device_timer_reports_the_slowest_rank():
    spawn_ranks(_timer, 2, (), backend="gloo")
