"""Helpers for single-node multi-process tests.

Capability parity with fairscale/fair_dev/testing/testing.py:61-774: ranks are spawned
as child processes of the test and rendezvous over loopback TCP on 127.0.0.1 (or a
temporary ``file://`` store), NCCL when every rank can have its own GPU, gloo otherwise.
Nothing here faults or hangs a device: delays are bounded sleep kernels and failures are
raised on the host.
"""

from __future__ import annotations

import contextlib
import functools
import gc
import logging
import os
import random
import socket
import tempfile
import traceback
from typing import Any, Callable, Dict, Generator, List, Optional, Tuple, Union

import numpy
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import Tensor, nn

skip_if_cuda = pytest.mark.skipif(torch.cuda.is_available(), reason="Testing only on CPUs to save time")
skip_if_no_cuda = pytest.mark.skipif(
    not torch.cuda.is_available() or torch.cuda.device_count() < 1, reason="CUDA required"
)
skip_if_single_gpu = pytest.mark.skipif(
    not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="multiple GPUs required"
)
skip_if_less_than_four_gpu = pytest.mark.skipif(
    not torch.cuda.is_available() or torch.cuda.device_count() < 4, reason="4 GPUs or more required"
)
skip_due_to_flakyness = pytest.mark.skip(reason="Flaky test to be fixed or removed")
available_devices = ["cpu"] + (["cuda"] if torch.cuda.is_available() else [])


class IdentityLayer(nn.Module):
    """A module whose output is its own (random) weight; used by tensor-parallel tests."""

    def __init__(self, size: Union[int, Tuple[int, ...]], scale: float = 1.0) -> None:
        super().__init__()
        self.weight = nn.Parameter(scale * torch.randn(size))

    def forward(self, *_: Any, **__: Any) -> Tensor:
        return self.weight


def set_random_seed(seed: int, model_parallel: bool = True) -> None:
    random.seed(seed)
    numpy.random.seed(seed)
    torch.manual_seed(seed)
    if model_parallel:
        from ...nn.model_parallel.random import model_parallel_cuda_manual_seed

        model_parallel_cuda_manual_seed(seed)


def make_cudnn_deterministic() -> None:
    torch.backends.cudnn.deterministic = True
    torch.backends.cudnn.benchmark = False
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False


def find_free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def dist_init(rank: int, world_size: int, filename: str, filename_rpc: str = "", backend: Optional[str] = None) -> bool:
    """Initialise the default group of a spawned rank.

    ``filename`` is either a path (→ ``file://`` store) or ``tcp://127.0.0.1:port``.
    Returns False when NCCL was requested but there are fewer GPUs than ranks.
    """
    os.environ["WORLD_SIZE"] = str(world_size)
    os.environ["RANK"] = str(rank)
    url = filename if "://" in filename else "file://" + filename
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() and torch.cuda.device_count() >= world_size else "gloo"
    if backend == "nccl":
        if torch.cuda.device_count() < world_size:
            logging.warning("Requested world size cannot be reached on this machine, not enough GPUs")
            return False
        torch.cuda.set_device(rank % torch.cuda.device_count())
    dist.init_process_group(backend=backend, rank=rank, world_size=world_size, init_method=url)
    if filename_rpc:
        from torch.distributed import rpc

        rpc.init_rpc(
            f"Test{rank}",
            rank=rank,
            world_size=world_size,
            backend=rpc.BackendType.TENSORPIPE,
            rpc_backend_options=rpc.TensorPipeRpcBackendOptions(init_method="file://" + filename_rpc),
        )
    return True


def get_worker_map() -> Dict[Any, Any]:
    return {rank: f"Test{rank}" for rank in range(dist.get_world_size())}


def get_world_sizes() -> List[int]:
    limit = torch.cuda.device_count() if torch.cuda.is_available() else 4
    return [x for x in [1, 2, 4, 8] if x <= limit]


def teardown() -> None:
    from ...internal.parallel import reset_process_group_cache

    with contextlib.suppress(ImportError):
        from ...nn.model_parallel.initialize import destroy_model_parallel

        destroy_model_parallel()
    reset_process_group_cache()
    if dist.is_initialized():
        dist.destroy_process_group()
    try:
        from torch.distributed import rpc

        if rpc.api._is_current_rpc_agent_set():
            rpc.shutdown(graceful=False)
    except Exception:
        pass


def _rank_entry(rank: int, fn: Callable, world_size: int, url: str, backend: Optional[str], args: Tuple, err_q: Any,
                env: Optional[Dict[str, str]] = None) -> None:
    if env:
        os.environ.update(env)  # a forkserver child starts from the server's environment, not from the caller's
    if not torch.cuda.is_available():
        # CPU ranks: several processes with a full-size OpenMP pool each oversubscribe the cores, and the tiny tensors of the
        # tests then spend their time in thread hand-offs (a 3-step conv net: 2 s with 8 threads per rank, 0.04 s with one)
        torch.set_num_threads(int(os.environ.get("FSB_TEST_THREADS", "1")))
    try:
        ok = dist_init(rank, world_size, url, backend=backend)
        if not ok:
            return
        fn(rank, world_size, *args)
    except BaseException:
        err_q.put((rank, traceback.format_exc()))
        raise
    finally:
        with contextlib.suppress(Exception):
            teardown()


def _start_context() -> Any:
    """How rank processes are started.  With a GPU: ``spawn`` (a fresh interpreter per rank).  On CPU-only machines:
    ``forkserver`` with torch and this package preloaded in the server, so a rank starts in a fraction of a second instead
    of re-importing torch; the server is forked before any thread pool exists, which a plain ``fork`` of the test process
    would not guarantee.  ``FSB_TEST_START_METHOD`` overrides the choice."""
    method = os.environ.get("FSB_TEST_START_METHOD", "spawn" if torch.cuda.is_available() else "forkserver")
    ctx = mp.get_context(method)
    if method == "forkserver":
        # torch._dynamo is pulled in by the first non-reentrant torch.utils.checkpoint call and torch.distributed.optim by
        # DistributedOptimizer: seconds each, paid once in the server instead of in every rank of every test
        ctx.set_forkserver_preload(["torch", "torch.distributed", "torch.distributed.rpc", "torch.distributed.autograd", "torch.distributed.optim",
                                    "torch.utils.checkpoint", "torch._dynamo", "numpy", "fairscale_b200", "fairscale_b200.nn", "fairscale_b200.optim",
                                    "fairscale_b200.experimental.nn"])
    return ctx


def spawn_ranks(fn: Callable, world_size: int, args: Tuple = (), backend: Optional[str] = None, timeout: float = 300.0) -> None:
    """Run ``fn(rank, world_size, *args)`` in ``world_size`` child processes with an initialised default group.

    Raises ``RuntimeError`` with the child's traceback if a rank fails or the run exceeds
    ``timeout`` seconds (children are then terminated by pid).
    """
    ctx = _start_context()
    err_q = ctx.SimpleQueue()
    url = f"tcp://127.0.0.1:{find_free_port()}"
    procs = [
        ctx.Process(target=_rank_entry, args=(r, fn, world_size, url, backend, args, err_q, dict(os.environ)), daemon=False)
        for r in range(world_size)
    ]
    for p in procs:
        p.start()
    import time

    deadline = time.time() + timeout
    failed: Optional[str] = None
    while True:
        alive = [p for p in procs if p.is_alive()]
        bad = [p for p in procs if not p.is_alive() and p.exitcode not in (0, None)]
        if bad:
            failed = f"rank process exited with code {bad[0].exitcode}"
            break
        if not alive:
            break
        if time.time() > deadline:
            failed = f"timeout after {timeout}s"
            break
        time.sleep(0.05)
    if failed is not None:
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(10)
        details = []
        while not err_q.empty():
            r, tb = err_q.get()
            details.append(f"--- rank {r} ---\n{tb}")
        raise RuntimeError(failed + "\n" + "\n".join(details))
    for p in procs:
        p.join()


def spawn_for_all_world_sizes(test_func: Callable, world_sizes: Optional[List[int]] = None, args: Any = ()) -> None:
    """Call ``test_func(rank, world_size, *args)`` under each world size (default 1,2,4,8 capped by devices)."""
    for ws in world_sizes if world_sizes is not None else get_world_sizes():
        spawn_ranks(test_func, ws, tuple(args))


def torch_spawn(world_sizes: Optional[List[int]] = None) -> Callable:
    """Decorator: turn ``fn(rank, world_size, *args)``-style function into a pytest test per world size."""
    sizes = world_sizes if world_sizes is not None else get_world_sizes()

    def wrap(func: Callable) -> Callable:
        @functools.wraps(func)
        def runner(*args: Any) -> None:
            for ws in sizes:
                spawn_ranks(_call_without_rank, ws, (func,) + tuple(args))

        return runner

    return wrap


def _call_without_rank(rank: int, world_size: int, func: Callable, *args: Any) -> None:
    func(*args)


class _Block(nn.Module):
    def __init__(self, embed_dim: int, num_heads: int) -> None:
        super().__init__()
        self.ln_1 = nn.LayerNorm(embed_dim)
        self.ln_2 = nn.LayerNorm(embed_dim)
        self.attn = nn.MultiheadAttention(embed_dim, num_heads)
        self.mlp = nn.Sequential(nn.Linear(embed_dim, embed_dim * 4), nn.GELU(), nn.Linear(embed_dim * 4, embed_dim))

    def forward(self, x: Tensor) -> Tensor:
        n = x.size(0)
        mask = torch.full((n, n), -float("Inf"), device=x.device, dtype=x.dtype).triu(diagonal=1)
        h = self.ln_1(x)
        a, _ = self.attn(h, h, h, attn_mask=mask, need_weights=False)
        x = x + a
        return x + self.mlp(self.ln_2(x))


class GPT2(nn.Module):
    """Small GPT-2 style model for tests (token + position embeddings, pre-LN blocks, LM or classifier head)."""

    def __init__(
        self, embed_dim: int, num_heads: int, num_layers: int, num_positions: int, num_vocab: int, num_classes: int
    ) -> None:
        super().__init__()
        self.embed_dim = embed_dim
        self.sos = nn.Parameter(torch.zeros(embed_dim))
        nn.init.normal_(self.sos)
        self.token_embeddings = nn.Embedding(num_vocab, embed_dim)
        self.position_embeddings = nn.Embedding(num_positions, embed_dim)
        self.layers = nn.ModuleList([_Block(embed_dim, num_heads) for _ in range(num_layers)])
        self.ln_f = nn.LayerNorm(embed_dim)
        self.head = nn.Linear(embed_dim, num_vocab, bias=False)
        self.clf_head = nn.Linear(embed_dim, num_classes)

    def forward(self, x: Tensor, classify: bool = False) -> Any:  # x: [batch, seq] token ids
        length, batch = x.shape[1], x.shape[0]
        h = self.token_embeddings(x.t().contiguous())  # [seq, batch, dim]
        sos = self.sos.expand(1, batch, self.embed_dim)
        h = torch.cat([sos, h[:-1]], dim=0)
        pos = torch.arange(length, device=x.device).unsqueeze(-1)
        h = h + self.position_embeddings(pos).expand_as(h)
        for layer in self.layers:
            h = layer(h)
        h = self.ln_f(h)
        logits = self.head(h)
        if not classify:
            return logits
        return self.clf_head(h.mean(dim=0)), logits


def objects_are_equal(a: Any, b: Any, raise_exception: bool = False, dict_key: Optional[str] = None,
                      rtol: Optional[float] = None, atol: Optional[float] = None) -> bool:
    """Deep comparison of nested containers of tensors (``torch.testing.assert_close`` on leaves)."""
    if type(a) is not type(b):
        if raise_exception:
            raise ValueError(f"type mismatch {type(a)} vs. {type(b)}")
        return False
    if isinstance(a, dict):
        if set(a.keys()) != set(b.keys()):
            if raise_exception:
                raise ValueError(f"keys mismatch {a.keys()} vs. {b.keys()}")
            return False
        return all(objects_are_equal(a[k], b[k], raise_exception, k, rtol, atol) for k in a.keys())
    if isinstance(a, (list, tuple, set)):
        if len(a) != len(b):
            if raise_exception:
                raise ValueError(f"length mismatch {len(a)} vs. {len(b)}")
            return False
        return all(objects_are_equal(x, y, raise_exception, dict_key, rtol, atol) for x, y in zip(a, b))
    if torch.is_tensor(a):
        try:
            a_cmp, b_cmp = a, b.to(a.device)
            torch.testing.assert_close(a_cmp, b_cmp, rtol=rtol, atol=atol)
            return True
        except (AssertionError, RuntimeError) as e:
            if raise_exception:
                if dict_key:
                    raise ValueError(f"for dict key '{dict_key}': {e}")
                raise
            return False
    return bool(a == b)


def check_same_model_params(model_a: nn.Module, model_b: nn.Module, message: str = "") -> None:
    for pa, pb in zip(model_a.parameters(), model_b.parameters()):
        assert torch.allclose(pa, pb, atol=1e-3), f"Model parameters differ\n{pa} {pb}\n" + message
    for ba, bb in zip(model_a.buffers(), model_b.buffers()):
        assert torch.allclose(ba, bb), f"Model buffers differ {ba} - {bb}\n" + message


def check_same_models_across_ranks(model: nn.Module, process_group: Any, params_should_be_equal: bool,
                                   check_broadcast_buffers: bool) -> None:
    world = dist.get_world_size(process_group)
    rank = dist.get_rank(process_group)
    for p in model.parameters():
        gathered = [torch.empty_like(p) for _ in range(world)] if rank == 0 else []
        dist.gather(p, gathered, group=process_group)
        if rank == 0:
            for other in gathered[1:]:
                assert not params_should_be_equal or torch.allclose(gathered[0], other), (
                    f"Models differ in between ranks {gathered[0]} - {other}"
                )
    if check_broadcast_buffers:
        for b in model.buffers():
            gathered = [torch.empty_like(b) for _ in range(world)] if rank == 0 else []
            dist.gather(b, gathered, group=process_group)
            if rank == 0:
                for other in gathered[1:]:
                    assert torch.allclose(gathered[0], other), f"Buffers differ in between ranks {gathered[0]} - {other}"


class DeviceAndTypeCheckModule(nn.Module):
    """Asserts device/dtype of its input, parameter and buffer, then returns a scalar loss."""

    def __init__(self, expected_input_dtype: Optional[torch.dtype] = None, expected_input_device: Optional[torch.device] = None,
                 expected_param_dtype: Optional[torch.dtype] = None, expected_param_device: Optional[torch.device] = None,
                 expected_loss_dtype: Optional[torch.dtype] = None, expected_loss_device: Optional[torch.device] = None,
                 expected_buffer_dtype: Optional[torch.dtype] = None):
        super().__init__()
        self.expected_input_dtype = expected_input_dtype
        self.expected_input_device = expected_input_device
        self.expected_param_dtype = expected_param_dtype
        self.expected_param_device = expected_param_device
        self.expected_loss_dtype = expected_loss_dtype
        self.expected_loss_device = expected_loss_device
        self.expected_buffer_dtype = expected_buffer_dtype
        self.linear = nn.Linear(5, 5)
        self.register_buffer("buffer", torch.rand((5,)))

    @staticmethod
    def _check(key: str, x: Union[torch.device, torch.dtype], expected: Any) -> None:
        assert expected in {None, x}, f"{key} ({x}) != expected ({expected})"

    def forward(self, *inputs: Tensor, **kwargs: Any) -> Tensor:
        x = inputs[0]
        self._check("input.dtype", x.dtype, self.expected_input_dtype)
        self._check("input.device", x.device, self.expected_input_device)
        p = self.linear.weight
        self._check("param.dtype", p.dtype, self.expected_param_dtype)
        self._check("param.device", p.device, self.expected_param_device)
        self._check("buffer.dtype", self.buffer.dtype, self.expected_buffer_dtype)
        loss = (self.linear(x) + self.buffer).sum()
        self._check("loss.dtype", loss.dtype, self.expected_loss_dtype)
        self._check("loss.device", loss.device, self.expected_loss_device)
        return loss


@functools.lru_cache()
def get_cycles_per_ms() -> float:
    """GPU cycles per millisecond for ``torch.cuda._sleep`` (median of several bounded probes)."""

    def measure() -> float:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        torch.cuda._sleep(1000000)
        end.record()
        end.synchronize()
        return 1000000 / start.elapsed_time(end)

    vals = sorted(measure() for _ in range(10))
    core = vals[2:-2]
    return sum(core) / len(core)


def in_circle_ci() -> bool:
    """True on the reference project's CI machines (kept so ported test code keeps working)."""
    return os.path.exists("/home/circleci")


def skip_a_test_if_in_CI() -> None:
    if in_circle_ci():
        import pytest

        pytest.skip("Sometimes a CI test failure is not reproducible locally, we skip them")


def torch_cuda_version(compiled: bool = False) -> Tuple[int, ...]:
    """CUDA version torch was built with (``compiled=True``) or the one the driver reports (needs a GPU)."""
    if compiled or not torch.cuda.is_available():
        numbering = (torch.version.cuda or "0.0").split(".")[:2]
    else:
        import subprocess

        out = subprocess.check_output(["nvidia-smi"]).decode("utf-8")
        found = [line.split("CUDA Version:")[1].split()[0] for line in out.splitlines() if "CUDA Version:" in line]
        numbering = (found[0] if found else "0.0").split(".")[:2]
    return tuple(int(n) for n in numbering)


def test_runner(rank: int, test_func: Callable, deterministic: bool = False, *args: Any, **kwargs: Any) -> None:
    """Entry of a spawned test process: optionally fix the seeds, then call ``test_func(rank, ...)``."""
    if deterministic:
        torch.backends.cudnn.deterministic = True
        torch.backends.cudnn.benchmark = False
        torch.manual_seed(1357)
    test_func(rank, *args, **kwargs)


test_runner.__test__ = False  # type: ignore[attr-defined]  # a helper, not a pytest test


def worker_process(rank: int, world_size: int, filename: str, filename_rpc: str, func: Callable, args: Any, error_queue: Any) -> None:
    """Main of a process started by a spawn helper: bring up torch.distributed (and RPC), one model-parallel group of
    size 1 with ``world_size`` pipeline stages, run ``func(*args)``, tear down; exceptions travel through ``error_queue``."""
    if not dist_init(rank, world_size, filename, filename_rpc):
        teardown()
        return
    from ...nn.model_parallel import initialize_model_parallel

    initialize_model_parallel(1, world_size)
    try:
        func(*args)
        teardown()
    except BaseException as e:  # noqa: B902
        teardown()
        import pytest

        if isinstance(e, pytest.skip.Exception):
            error_queue.put(str(e))
        else:
            raise


def gpu_delay(ms: float, stream: Optional[Any] = None) -> None:
    """Keep ``stream`` (default: the current one) busy for ``ms`` milliseconds with the library's delay kernel.

    The kernel polls the global nanosecond timer and is capped at one second, so unlike a cycle-count sleep it needs
    no clock calibration and cannot outlive a test.
    """
    from ...ops import _bind

    s = torch.cuda.current_stream() if stream is None else stream
    _bind.call("fsb_delay", int(ms * 1e6), s.cuda_stream)


def gpu_occupy_sms(ms: float, sms: int, stream: Optional[Any] = None) -> None:
    """Take ``sms`` whole SMs of the current device for ``ms`` milliseconds on ``stream`` (each CTA of the kernel claims
    200 KB of shared memory): a stand-in for a foreign kernel that leaves a persistent kernel of another stream fewer SMs
    than its grid has CTAs.  Capped at one second like :func:`gpu_delay`."""
    from ctypes import c_int, c_ulonglong, c_void_p

    from ...ops import _bind

    _bind._SIGNATURES.setdefault("fsb_delay_wide", [c_ulonglong, c_int, c_void_p])
    s = torch.cuda.current_stream() if stream is None else stream
    _bind.call("fsb_delay_wide", int(ms * 1e6), int(sms), s.cuda_stream)


class DummyProcessGroup:
    """Stands in for a process group in single-process unit tests (no collectives are issued)."""

    def __init__(self, rank: int, size: int):
        self._rank = rank
        self._size = size

    def rank(self) -> int:
        return self._rank

    def size(self) -> int:
        return self._size


class SGDWithPausingCompute(torch.optim.SGD):
    """SGD whose step first stalls the GPU for a bounded time and then perturbs the weights,
    to expose missing stream synchronisation after the optimizer step."""

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        self.rank = kwargs.pop("rank")
        super().__init__(*args, **kwargs)

    def step(self, closure: Optional[Any] = None) -> Any:
        loss = super().step(closure=closure)
        with torch.cuda.stream(torch.cuda.Stream()):
            gpu_delay(0.1)
            for group in self.param_groups:
                for p in group["params"]:
                    with torch.no_grad():
                        p *= 1.0 + self.rank / 10.0
        return loss


def state_dict_norm(state: Dict[str, torch.Tensor]) -> torch.Tensor:
    norm = torch.zeros(1)
    for v in state.values():
        if v.is_floating_point():
            norm += v.norm().cpu()
    return norm


def rmf(filename: str) -> None:
    with contextlib.suppress(FileNotFoundError):
        os.remove(filename)


@contextlib.contextmanager
def in_temporary_directory() -> Generator:
    old = os.getcwd()
    with tempfile.TemporaryDirectory() as d:
        os.chdir(d)
        try:
            yield d
        finally:
            os.chdir(old)


@contextlib.contextmanager
def temp_files_ctx(num: int) -> Generator:
    files = [tempfile.mkstemp()[1] for _ in range(num)]
    try:
        yield tuple(files)
    finally:
        for f in files:
            rmf(f)


def dump_all_tensors(rank: int) -> None:
    """Debug aid: print every live tensor on rank ``rank``."""
    if dist.is_initialized() and dist.get_rank() != rank:
        return
    for obj in gc.get_objects():
        with contextlib.suppress(Exception):
            if torch.is_tensor(obj):
                print(type(obj), obj.dtype, obj.device, tuple(obj.shape))
    if torch.cuda.is_available():
        print(torch.cuda.memory_summary())


def get_smi_memory() -> float:
    """MiB used by this process on the current GPU according to NVML (0 when unknown)."""
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
        for proc in pynvml.nvmlDeviceGetComputeRunningProcesses(h):
            if proc.pid == os.getpid():
                return proc.usedGpuMemory / 2**20
    except Exception:
        pass
    return 0.0
