"""A tiny end-to-end check of an installation: one FSDP forward + backward + optimizer step of a two-layer GPT on
``cuda:0`` through the native kernels.

    python -m fairscale_b200._native         # build the native library (nvcc, sm_100a) inside the package
    python -m fairscale_b200.utils.smoke     # run the check
"""

from __future__ import annotations


def smoke() -> None:
    """Raises if the native library is missing, a kernel reports an error or the losses are not finite."""
    import socket

    import torch
    import torch.distributed as dist

    from fairscale_b200 import _native
    from fairscale_b200.models.gpt import GPTConfig, build_fsdp_gpt
    from fairscale_b200.ops import _bind
    from fairscale_b200.optim import FusedAdam

    if not _native.available():
        _native.build()
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    created = False
    if not dist.is_initialized():
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        dist.init_process_group("nccl", rank=0, world_size=1, init_method=f"tcp://127.0.0.1:{port}")
        created = True
    cfg = GPTConfig.tiny(vocab=1024, d_model=256, n_heads=2, n_layers=2, ffn=1024, max_seq=256)
    torch.manual_seed(0)
    model = build_fsdp_gpt(cfg, device)
    opt = FusedAdam(model.parameters(), lr=1e-3)
    model.attach_optimizer(opt)
    tokens = torch.randint(0, cfg.vocab_size, (2, 257), device=device)
    before = _bind.launch_count()
    losses = []
    for _ in range(2):
        loss = model(tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous())
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        losses.append(float(loss.item()))
    torch.cuda.synchronize()
    status = _native.read_status(device)
    assert status == 0, f"a kernel reported status {status}"
    assert all(l == l and l < 20 for l in losses), losses
    assert _bind.launch_count() > before, "native kernels were not launched"
    print(f"smoke ok: losses {losses}, native launches {_bind.launch_count() - before}")
    if created:
        dist.destroy_process_group()



if __name__ == "__main__":
    smoke()
