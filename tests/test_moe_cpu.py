"""Top-2 gating numerics and MOELayer (index path == dense einsum path) on CPU / gloo."""
import pytest
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn.moe import MOELayer, Top2Gate, top2gating
from fairscale_b200.nn.moe.top2gate import dense_from_route, top2_route


def test_top2gating_reference_values():
    # same construction as the reference's unit test: 12 tokens, 4 experts, uniform logits except a bump
    torch.manual_seed(3)
    logits = torch.rand(12, 4)
    l_aux, combine, mask = top2gating(logits)
    assert combine.shape == (12, 4, 6) and mask.shape == (12, 4, 6)
    assert mask.dtype == torch.bool
    # every kept (token, expert) pair owns exactly one slot and no slot is used twice
    assert (mask.sum(dim=(1, 2)) <= 2).all()
    assert (mask.sum(dim=0) <= 1).all()
    # weights of a token sum to 1 when both choices were kept
    sums = combine.sum(dim=(1, 2))
    both = mask.sum(dim=(1, 2)) == 2
    torch.testing.assert_close(sums[both], torch.ones_like(sums[both]))
    assert 0.0 < l_aux.item() < 1.0


def test_capacity_overflow_drops_tokens():
    logits = torch.zeros(8, 4)
    logits[:, 0] = 10.0  # everyone wants expert 0 first; capacity is 4
    route = top2_route(logits, noise=torch.zeros_like(logits))
    assert route.capacity == 4
    assert route.keep[:, 0].sum().item() == 4
    assert (route.slot[route.keep[:, 0], 0] == torch.arange(4)).all()  # token order decides the slots
    combine, mask = dense_from_route(route, torch.float32)
    assert mask[:, 0].sum().item() == 4


class _Expert(nn.Module):
    def __init__(self, d, scale):
        super().__init__()
        self.fc = nn.Linear(d, d, bias=False)
        with torch.no_grad():
            self.fc.weight.copy_(torch.eye(d) * scale)

    def forward(self, x):
        return self.fc(x)


class _DenseGate(nn.Module):
    """Wraps a Top2Gate but only exposes the dense contract (forces the einsum path)."""

    def __init__(self, inner):
        super().__init__()
        self.inner = inner
        self.noise = None

    def forward(self, x):
        route = top2_route(self.inner.wg(x), noise=self.noise)
        c, m = dense_from_route(route, x.dtype)
        return route.l_aux, c, m


class _IndexGate(Top2Gate):
    noise = None

    def route(self, x):
        return top2_route(self.wg(x), noise=self.noise)


def _moe(rank, world):
    torch.manual_seed(0)
    d, n_local = 8, 2
    E = world * n_local
    gate = _IndexGate(d, E)
    dist.broadcast(gate.wg.weight.data, 0)
    experts = nn.ModuleList([_Expert(d, 1.0 + rank * n_local + i) for i in range(n_local)])
    fast = MOELayer(gate, experts)
    dense_gate = _DenseGate(gate)
    slow = MOELayer(dense_gate, experts)
    for p in experts.parameters():
        assert p.expert is True
    torch.manual_seed(10 + rank)
    x = torch.randn(4, 4, d, requires_grad=True)  # 16 tokens, divisible by E
    noise = torch.randn(16, E)
    gate.noise = noise
    dense_gate.noise = noise
    y_fast = fast(x)
    g = torch.randn_like(y_fast)
    gx_fast, gw_fast = torch.autograd.grad(y_fast, [x, gate.wg.weight], g, retain_graph=True)
    ge_fast = torch.autograd.grad(y_fast, list(experts.parameters()), g)
    y_slow = slow(x)
    gx_slow, gw_slow = torch.autograd.grad(y_slow, [x, gate.wg.weight], g, retain_graph=True)
    ge_slow = torch.autograd.grad(y_slow, list(experts.parameters()), g)
    torch.testing.assert_close(y_fast, y_slow, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(gx_fast, gx_slow, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(gw_fast, gw_slow, atol=1e-5, rtol=1e-5)
    for a, b in zip(ge_fast, ge_slow):
        torch.testing.assert_close(a, b, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(fast.l_aux, slow.l_aux)


def test_moe_index_path_matches_dense_path():
    spawn_ranks(_moe, 2, (), backend="gloo")


def test_grouped_experts_match_module_list():
    spawn_ranks(_grouped_vs_list, 1, (), backend="gloo")


def _grouped_vs_list(rank, world):
    """Stacked experts (one grouped call) give the same layer output and gradients as a ModuleList of FFNs."""
    import torch
    from torch import nn

    from fairscale_b200.nn.moe import GroupedExperts, MOELayer, Top2Gate

    torch.manual_seed(0)
    d, f, n_exp = 8, 16, 4
    grouped = GroupedExperts(n_exp, d, f)

    class FFN(nn.Module):
        def __init__(self, e):
            super().__init__()
            self.l1, self.l2 = nn.Linear(d, f), nn.Linear(f, d)
            with torch.no_grad():
                self.l1.weight.copy_(grouped.w1[e]); self.l1.bias.copy_(grouped.b1[e])
                self.l2.weight.copy_(grouped.w2[e]); self.l2.bias.copy_(grouped.b2[e])

        def forward(self, x):
            return self.l2(torch.nn.functional.gelu(self.l1(x)))

    gate = Top2Gate(d, n_exp)
    a = MOELayer(gate, grouped)
    b = MOELayer(gate, nn.ModuleList([FFN(e) for e in range(n_exp)]))
    x = torch.randn(4, 8, d)
    from fairscale_b200.nn.moe import top2gate as tg

    noise = tg.gumbel_rsample((32, n_exp), x.device)
    orig = tg.gumbel_rsample
    tg.gumbel_rsample = lambda shape, device: noise  # same routing for both layers
    try:
        ya, yb = a(x), b(x)
        torch.testing.assert_close(ya, yb, rtol=1e-4, atol=1e-5)
        ya.pow(2).sum().backward()
        g_grouped = grouped.w1.grad.clone()
        gate.zero_grad()
        yb.pow(2).sum().backward()
    finally:
        tg.gumbel_rsample = orig
    torch.testing.assert_close(g_grouped[1], b.experts[1].l1.weight.grad, rtol=1e-3, atol=1e-5)


class _RoundRobinGate(nn.Module):
    """Deterministic dense gate (any gate returning ``(l_aux, combine_weights, dispatch_mask)`` is accepted): token i goes
    to expert ``i % E``, slot ``i // E``."""

    def __init__(self, num_experts):
        super().__init__()
        self.num_experts = num_experts

    def forward(self, x):
        s = x.shape[0]
        capacity = 2 * s // self.num_experts
        out = torch.zeros(s, self.num_experts, capacity, dtype=x.dtype)
        for i in range(s):
            out[i, i % self.num_experts, i // self.num_experts] = 1.0
        return 0.0, out, out.bool()


def _round_robin(rank, world, n_local):
    d = 8
    E = world * n_local
    x = torch.randn(4 * n_local, 16, d)
    experts = []
    for i in range(n_local):
        lin = nn.Linear(d, d, bias=False)
        lin.weight = nn.Parameter(torch.eye(d) * (rank * n_local + i + 1))  # a scale that names the expert
        experts.append(lin)
    moe = MOELayer(_RoundRobinGate(E), experts[0] if n_local == 1 else nn.ModuleList(experts))
    y = moe(x)
    assert y.shape == x.shape
    flat_in, flat_out = x.reshape(-1, d), y.reshape(-1, d)
    for i in range(flat_in.shape[0]):  # every token came back scaled by the expert it was routed to
        torch.testing.assert_close(flat_out[i], flat_in[i] * (i % E + 1))
    # gradients reach the local experts only, and they are tagged for the data-parallel reducers
    y.sum().backward()
    assert all(p.grad is not None and p.expert for e in experts for p in e.parameters())


@pytest.mark.parametrize("n_local", [1, 2])
def test_moe_round_robin_gate_routes_to_the_right_expert(n_local):
    spawn_ranks(_round_robin, 2, (n_local,), backend="gloo")


def _identity_experts(rank, world):
    torch.manual_seed(1)
    d, n_local = 8, 2
    x = torch.randn(4 * n_local, 16, d)
    experts = nn.ModuleList()
    for _ in range(n_local):
        lin = nn.Linear(d, d, bias=False)
        lin.weight = nn.Parameter(torch.eye(d))
        experts.append(lin)
    gate = Top2Gate(d, world * n_local)
    dist.broadcast(gate.wg.weight.data, 0)
    y = MOELayer(gate, experts)(x)
    assert y.shape == x.shape
    kept = y.abs().sum(-1) > 0
    assert kept.float().mean() > 0.9  # nearly every token found room in one of its two experts
    # identity experts and gates that sum to one: a routed token comes back unchanged
    torch.testing.assert_close(y[kept], x[kept], atol=1e-5, rtol=1e-5)


def test_moe_identity_experts_reassemble_the_input():
    spawn_ranks(_identity_experts, 2, (), backend="gloo")


def test_gate_takes_low_precision_activations_and_routes_in_fp32():
    """A bf16 activation against the fp32 gate weight: logits (and so the softmax over experts) come out in fp32."""
    from fairscale_b200.nn.moe.top2gate import Top2Gate, gate_logits

    torch.manual_seed(0)
    gate = Top2Gate(16, 4)
    x = torch.randn(12, 16).bfloat16().requires_grad_()
    logits = gate_logits(x, gate.wg)
    assert logits.dtype == torch.float32
    torch.testing.assert_close(logits, torch.nn.functional.linear(x.float(), gate.wg.weight))
    l_aux, combine, mask = gate(x)
    assert combine.dtype == torch.float32 and mask.dtype == torch.bool
    (l_aux + combine.sum()).backward()
    assert x.grad is not None and gate.wg.weight.grad is not None


def _identity_backward(rank, world):
    """fairscale tests/nn/moe/test_moe_layer.py `backward`: one identity expert per rank and as many experts as ranks; every
    token finds room (capacity is 2 * tokens / experts), so the layer returns its input and an MSE loss against the input
    leaves no gradient on the expert."""
    torch.manual_seed(2)
    d = 8
    x = torch.randn(4, 16, d)
    expert = nn.Linear(d, d, bias=False)
    expert.weight = nn.Parameter(torch.eye(d))
    gate = Top2Gate(d, world)
    dist.broadcast(gate.wg.weight.data, 0)
    moe = MOELayer(gate, expert)
    y = moe(x)
    assert y.shape == x.shape
    torch.testing.assert_close(y, x, atol=1e-5, rtol=1e-5)
    nn.functional.mse_loss(y, x).backward()
    torch.testing.assert_close(expert.weight.grad, torch.zeros_like(expert.weight), atol=1e-6, rtol=0)
    assert moe.l_aux is not None and moe.l_aux.requires_grad


def test_moe_identity_expert_gets_no_gradient_from_a_loss_against_the_input():
    spawn_ranks(_identity_backward, 2, (), backend="gloo")
