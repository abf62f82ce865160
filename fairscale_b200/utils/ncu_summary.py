"""Turn an Nsight Compute report into the short text summary kept under ``profiles/``.

    python -m fairscale_b200.utils.ncu_summary report.ncu-rep [--kernel REGEX] [--flops F] [--bytes B]

The report is read with ``ncu -i <report> --page raw --csv`` (works on a machine without a GPU); alternatively a CSV that
was produced that way can be passed directly.  For every captured launch the summary lists duration, launch shape, the
tensor-pipe and DRAM figures a roofline needs, occupancy and the largest warp-stall reasons.  ``--flops`` / ``--bytes``
(algorithmic work of one launch) add the achieved rate and, with ``MEASURED_PEAKS.json`` in the working directory, the
fraction of the measured peak - under a profiler durations are serialised and cold-cache, so those fractions are a lower
bound and timings for a report belong to CUDA events outside the profiler.
"""

from __future__ import annotations

import argparse
import csv
import io
import json
import os
import re
import subprocess
import sys
from typing import Dict, Iterable, List, Optional, Tuple

# metric -> label; the order is the order of the report
FIGURES: List[Tuple[str, str]] = [
    ("gpu__time_duration.sum", "duration"),
    ("launch__grid_size", "grid"),
    ("launch__block_size", "block"),
    ("launch__registers_per_thread", "registers / thread"),
    ("launch__shared_mem_per_block_dynamic", "dynamic shared memory / block"),
    ("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active", "tensor pipe busy (of active cycles)"),
    ("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed", "tensor pipe busy (of elapsed cycles)"),
    ("sm__throughput.avg.pct_of_peak_sustained_elapsed", "SM throughput"),
    ("dram__bytes_read.sum", "DRAM read"),
    ("dram__bytes_write.sum", "DRAM written"),
    ("gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "DRAM throughput"),
    ("lts__throughput.avg.pct_of_peak_sustained_elapsed", "L2 throughput"),
    ("sm__warps_active.avg.pct_of_peak_sustained_active", "warps active (of maximum)"),
    ("smsp__issue_active.avg.pct_of_peak_sustained_active", "issue slots busy"),
]
STALL = re.compile(r"smsp__average_warps_issue_stalled_(\w+)_per_issue_active\.ratio")


def read_rows(path: str) -> Tuple[List[str], List[str], List[List[str]]]:
    """``(header, units, launches)`` of a report (``.ncu-rep``) or of a raw-page CSV made from one."""
    if path.endswith(".csv"):
        text = open(path).read()
    else:
        text = subprocess.run(["ncu", "-i", path, "--page", "raw", "--csv"], check=True, capture_output=True, text=True).stdout
    return parse_csv(text)


def parse_csv(text: str) -> Tuple[List[str], List[str], List[List[str]]]:
    rows = [r for r in csv.reader(io.StringIO(text)) if r]
    # ncu prints ==PROF== lines before the table on some versions: the table starts at the row that names the ID column;
    # the row after it holds the units (its first cell is empty), the launches follow
    start = next(i for i, r in enumerate(rows) if r[0] == "ID")
    return rows[start], rows[start + 1], [r for r in rows[start + 2:] if len(r) == len(rows[start])]


def _number(cell: str) -> Optional[float]:
    try:
        return float(cell.replace(",", ""))
    except ValueError:
        return None


def _scaled(value: float, unit: str) -> str:
    unit = unit.strip()
    if unit in ("ns", "nsecond"):
        return f"{value / 1e3:.1f} us"
    if unit in ("us", "usecond"):
        return f"{value:.1f} us"
    if unit in ("ms", "msecond"):
        return f"{value * 1e3:.1f} us"
    if unit == "%":
        return f"{value:.1f} %"
    if unit in ("byte", "Kbyte", "Mbyte", "Gbyte"):
        mb = value * {"byte": 1e-6, "Kbyte": 1e-3, "Mbyte": 1.0, "Gbyte": 1e3}[unit]
        return f"{mb:.1f} MB"
    if unit in ("Kbyte/block",):
        return f"{value:.1f} KB"
    if unit in ("byte/block",):
        return f"{value / 1024:.1f} KB"
    return f"{value:g}" + (f" {unit}" if unit else "")


def _microseconds(value: float, unit: str) -> float:
    return value * {"ns": 1e-3, "nsecond": 1e-3, "us": 1.0, "usecond": 1.0, "ms": 1e3, "msecond": 1e3, "s": 1e6, "second": 1e6}.get(unit.strip(), 1.0)


def summarise(header: List[str], units: List[str], launches: Iterable[List[str]], kernel: Optional[str] = None,
              flops: Optional[float] = None, nbytes: Optional[float] = None, peaks: Optional[Dict[str, float]] = None) -> str:
    col = {name: i for i, name in enumerate(header)}
    name_col = col.get("Kernel Name")
    want = re.compile(kernel) if kernel else None
    out: List[str] = []
    for row in launches:
        name = row[name_col] if name_col is not None else "?"
        if want is not None and not want.search(name):
            continue
        out.append(name if len(name) <= 110 else name[:107] + "...")
        duration_us = None
        for metric, label in FIGURES:
            i = col.get(metric)
            value = _number(row[i]) if i is not None and i < len(row) else None
            if value is None:
                continue
            if metric == "gpu__time_duration.sum":
                duration_us = _microseconds(value, units[i])
            out.append(f"    {label:<40s} {_scaled(value, units[i])}")
        stalls = []
        for i, metric in enumerate(header):
            m = STALL.fullmatch(metric)
            value = _number(row[i]) if m and i < len(row) else None
            if m and value is not None and m.group(1) != "selected":
                stalls.append((value, m.group(1)))
        if stalls:
            top = ", ".join(f"{n} {v:.2f}" for v, n in sorted(stalls, reverse=True)[:5])
            out.append(f"    {'warp stall per issue (largest)':<40s} {top}")
        if duration_us:
            if flops:
                rate = flops / duration_us / 1e6  # TFLOP/s
                line = f"    {'achieved':<40s} {rate:.1f} TFLOP/s"
                if peaks and peaks.get("bf16_tflops"):
                    line += f" = {rate / peaks['bf16_tflops']:.2f} of measured ({peaks['bf16_tflops']:.1f})"
                out.append(line)
            if nbytes:
                rate = nbytes / duration_us / 1e3  # GB/s
                line = f"    {'achieved':<40s} {rate:.1f} GB/s"
                if peaks and peaks.get("hbm_gbs"):
                    line += f" = {rate / peaks['hbm_gbs']:.2f} of measured ({peaks['hbm_gbs']:.1f})"
                out.append(line)
        out.append("")
    return "\n".join(out)


def _peaks() -> Optional[Dict[str, float]]:
    path = os.path.join(os.getcwd(), "MEASURED_PEAKS.json")
    try:
        data = json.load(open(path))
        return {k: float(v) for k, v in data.items() if isinstance(v, (int, float))}
    except Exception:
        return None


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("report", help=".ncu-rep file, or a CSV made with `ncu -i <rep> --page raw --csv`")
    ap.add_argument("--kernel", help="only launches whose kernel name matches this regular expression")
    ap.add_argument("--flops", type=float, help="algorithmic floating-point operations of one launch")
    ap.add_argument("--bytes", type=float, dest="nbytes", help="algorithmic bytes moved by one launch")
    args = ap.parse_args(argv)
    header, units, launches = read_rows(args.report)
    sys.stdout.write(summarise(header, units, launches, args.kernel, args.flops, args.nbytes, _peaks()))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
