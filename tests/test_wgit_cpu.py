import os

import pytest
import torch

from fairscale_b200.experimental.wgit import Algo, EnergyConcentrationProfile, Repo, RepoStatus, SHA1_Store, SignalSparsity, random_sparse_mask
from fairscale_b200.experimental.wgit.cli import main


def test_sha1_store_dedup_and_refcount(tmp_path):
    store = SHA1_Store(tmp_path / "s", init=True)
    a, b = torch.arange(1000.0), torch.ones(10)
    h1 = store.add(a, name="a")
    assert store.add(a.clone(), name="a2") == h1
    sd = store.add({"x": a, "y": {"z": b}})
    assert sd["x"] == h1 and isinstance(sd["y"]["z"], str)
    orig, dedup, comp = store.size_info()
    assert orig > dedup > 0 and comp > 0
    torch.testing.assert_close(store.get(h1), a)
    assert store.names(h1) == {"a": 1, "a2": 1, "x": 1}
    for _ in range(3):
        store.delete(h1)
    with pytest.raises(ValueError):
        store.get(h1)
    with pytest.raises(ValueError):
        store.add(b, compress=False)


@pytest.mark.parametrize("algo", [Algo.FFT, Algo.DCT])
def test_signal_sparsity(algo):
    torch.manual_seed(0)
    x = torch.randn(6, 32)
    full = SignalSparsity(algo=algo, sst_top_k_percent=100, dst_top_k_percent=100)
    assert full.lossy_compress(x)[0] is x
    s = SignalSparsity(algo=algo, sst_top_k_element=32, dst_top_k_element=1)
    torch.testing.assert_close(s.sst_dst_to_dense(s.dense_to_sst(x)), x, rtol=1e-4, atol=1e-4)  # transform round trip
    s = SignalSparsity(algo=algo, sst_top_k_element=8, dst_top_k_element=4)
    rec, sst, dst = s.lossy_compress(x)
    assert (sst != 0).sum(-1).max() <= 8 and (dst != 0).sum(-1).max() <= 4
    err_sst = (x - s.sst_dst_to_dense(sst)).norm()
    assert (x - rec).norm() < err_sst < x.norm()
    flat = SignalSparsity(algo=algo, sst_top_k_dim=None, dst_top_k_dim=None, sst_top_k_percent=10, dst_top_k_percent=10)
    rec2, sst2, _ = flat.lossy_compress(x)
    assert int((sst2 != 0).sum()) == 19 and rec2.shape == x.shape
    with pytest.raises(ValueError):
        SignalSparsity(sst_top_k_element=1, sst_top_k_percent=5.0)
    m = random_sparse_mask(x, 25, -1)
    assert torch.all(m.sum(-1) == 8)
    prof = EnergyConcentrationProfile(dim=-1, top_k_percents=[10, 100])
    lo, hi = prof.measure(x)
    assert 0 < float(lo) < float(hi) and abs(float(hi) - 1) < 1e-6
    assert len(prof.measure_fft(x)) == 2


def test_repo_add_commit_status_and_get(tmp_path, capsys):
    cwd = os.getcwd()
    os.chdir(tmp_path)
    try:
        main(["init"])
        sd = {"w": torch.randn(16, 16), "b": torch.zeros(16), "step": 3}
        torch.save(sd, "ckpt.pt")
        repo = Repo(tmp_path)
        repo.add("ckpt.pt")
        assert repo.status() == {"ckpt.pt": RepoStatus.CHANGES_ADDED_NOT_COMMITED}
        repo.commit("first")
        assert repo.status() == {"ckpt.pt": RepoStatus.CLEAN}
        got = repo.get("ckpt.pt")
        torch.testing.assert_close(got["w"], sd["w"])
        assert got["step"] == 3
        sd["b"] = torch.ones(16)
        torch.save(sd, "ckpt.pt")
        assert repo.status() == {"ckpt.pt": RepoStatus.CHANGES_NOT_ADDED}
        before = repo.size_info().deduped
        repo.add("ckpt.pt")
        repo.commit("second")
        grown = repo.size_info().deduped - before
        assert 0 < grown < 3000  # only the changed bias was stored again
        main(["log"])
        assert "second" in capsys.readouterr().out
        torch.save({"w": torch.randn(8, 64)}, "sp.pt")
        repo.add("sp.pt", sparsify=True, sparsify_policy=SignalSparsity(sst_top_k_percent=50, dst_top_k_percent=50))
        assert repo.get("sp.pt")["w"].shape == (8, 64)
        main(["version"])
    finally:
        os.chdir(cwd)


def _golden_cases():
    """Fixed inputs with the SST / DST / reconstruction recorded by the reference's
    tests/experimental/wgit/test_signal_sparsity.py:118-200 (FFT, top-k over the flattened tensor and over dim 0)."""
    t0 = torch.arange(12).sin().reshape(4, 3).float()
    sst0 = torch.zeros(4, 3, dtype=torch.complex64)
    sst0[0, 2] = complex(-1.3618, -5.7650)
    sst0[3, 1] = complex(-1.3618, 5.7650)
    dst0 = torch.zeros(4, 3)
    dst0[0, 0], dst0[3, 0] = 0.22696666419506072998, 0.18515183031558990479
    rt0 = torch.tensor([[0.0, 0.71862268447875976562, 0.94558942317962646484],
                        [0.22696666419506072998, -0.71862268447875976562, -0.94558942317962646484],
                        [-0.22696666419506072998, 0.71862268447875976562, 0.94558942317962646484],
                        [0.41211849451065063477, -0.71862268447875976562, -0.94558942317962646484]])
    t1 = torch.arange(50, 62).sin().reshape(4, 3) / 100
    sst1 = torch.zeros(4, 3, dtype=torch.complex64)
    sst1[2] = torch.tensor([-1.81658901274204254150e-02, 1.96999348700046539307e-02, 3.94537299871444702148e-02], dtype=torch.complex64)
    dst1 = torch.zeros(4, 3)
    dst1[0, 0], dst1[3, 1], dst1[3, 2] = 0.00191772403195500374, 0.00187687762081623077, 0.00020225439220666885
    rt1 = torch.tensor([[-0.00262374849990010262, 0.00492498371750116348, 0.00986343249678611755],
                        [0.00454147253185510635, -0.00492498371750116348, -0.00986343249678611755],
                        [-0.00454147253185510635, 0.00492498371750116348, 0.00986343249678611755],
                        [0.00454147253185510635, -0.00304810609668493271, -0.00966117810457944870]])
    return [(t0, sst0, dst0, rt0, None, 2), (t1, sst1, dst1, rt1, 0, 1)]


@pytest.mark.parametrize("tensor,sst,dst,rt,dim,k", _golden_cases())
def test_signal_sparsity_reference_golden_values(tensor, sst, dst, rt, dim, k):
    s = SignalSparsity(sst_top_k_element=k, sst_top_k_dim=dim, dst_top_k_percent=100)
    torch.testing.assert_close(s.dense_to_sst(tensor), sst, rtol=1e-4, atol=1e-5)
    s = SignalSparsity(sst_top_k_element=k, sst_top_k_dim=dim, dst_top_k_element=k, dst_top_k_dim=dim)
    lossy, got_sst, got_dst = s.lossy_compress(tensor)
    torch.testing.assert_close(got_sst, sst, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(got_dst, dst, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(lossy, rt, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(s.sst_dst_to_dense(sst, dst), rt, rtol=1e-4, atol=1e-5)
