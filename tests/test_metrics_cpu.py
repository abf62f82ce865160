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


def test_ncu_summary_reads_a_raw_page_csv():
    """The profile summariser on a hand-made raw-page CSV: units row, per-launch rows, kernel filter, achieved rates."""
    from fairscale_b200.utils import ncu_summary

    header = ["ID", "Kernel Name", "gpu__time_duration.sum", "launch__grid_size", "dram__bytes_read.sum",
              "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active",
              "smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio",
              "smsp__average_warps_issue_stalled_selected_per_issue_active.ratio"]
    units = ["", "", "us", "", "Mbyte", "%", "inst", "inst"]
    rows = [["0", "gemm_kernel(Params)", "200.0", "148", "100.5", "79.25", "11.5", "1.0"],
            ["1", "copy_kernel(void *)", "50,000", "296", "2,048.0", "0", "30.25", "1.0"]]
    text = "==PROF== noise before the table\n" + "\n".join(",".join(f'"{c}"' for c in r) for r in [header, units] + rows) + "\n"
    h, u, launches = ncu_summary.parse_csv(text)
    assert h == header and u == units and len(launches) == 2
    report = ncu_summary.summarise(h, u, launches, kernel="gemm", flops=2 * 8192 * 8192 * 2048, peaks={"bf16_tflops": 1600.0})
    assert "gemm_kernel" in report and "copy_kernel" not in report
    assert "200.0 us" in report and "79.2 %" in report and "100.5 MB" in report
    assert "long_scoreboard 11.50" in report and "selected" not in report
    assert "1374.4 TFLOP/s = 0.86 of measured" in report
    everything = ncu_summary.summarise(h, u, launches, nbytes=2048e6 * 2)
    assert "50000.0 us" in everything and "81.9 GB/s" in everything
