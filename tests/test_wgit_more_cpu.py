"""Weight-tracking tool, case by case: configuration checks and the transform identities of SignalSparsity (perfect
reconstruction, top-k by element / percent / dimension, disabled halves, nothing-to-drop shortcut, random masks), the energy
profile, the content-addressed store with and without compression (files, state dicts, tensors, reference counts, sizes,
names, deletion), the git wrapper, the Repo API through its status transitions, and the command line.  Cases of the
reference's tests/experimental/wgit/test_{signal_sparsity,signal_sparsity_profiling,sha1_store,pygit,api,cli}.py."""
import json
import os
import shutil
from pathlib import Path

import pytest
import torch

from fairscale_b200.experimental.wgit import Algo, EnergyConcentrationProfile, Repo, RepoStatus, SHA1_Store, SignalSparsity, random_sparse_mask
from fairscale_b200.experimental.wgit.cli import main
from fairscale_b200.experimental.wgit.pygit import PyGit
from fairscale_b200.fair_dev.testing.testing import objects_are_equal


# ------------------------------------------------------------------------------------------------ SignalSparsity
@pytest.mark.parametrize("kwargs", [
    dict(sst_top_k_element=1, dst_top_k_element=1),
    dict(sst_top_k_percent=1.0, dst_top_k_element=5),
    dict(sst_top_k_element=3, dst_top_k_percent=100.0),
    dict(sst_top_k_percent=0.5, dst_top_k_percent=0.5, sst_top_k_dim=0, dst_top_k_dim=None),
    dict(),  # both halves off is a legal (if useless) configuration
])
def test_valid_configurations_are_accepted(kwargs):
    SignalSparsity(**kwargs)


@pytest.mark.parametrize("kwargs", [
    dict(sst_top_k_element=1, sst_top_k_percent=1.0),
    dict(dst_top_k_element=1, dst_top_k_percent=1.0),
    dict(sst_top_k_percent=0.0), dict(sst_top_k_percent=100.5), dict(dst_top_k_percent=-1.0),
    dict(sst_top_k_element=0), dict(dst_top_k_element=-3),
])
def test_invalid_configurations_are_refused(kwargs):
    with pytest.raises(ValueError):
        SignalSparsity(**kwargs)


@pytest.mark.parametrize("algo", [Algo.FFT, Algo.DCT])
@pytest.mark.parametrize("shape,dim", [((5,), 0), ((4, 6), 0), ((4, 6), 1), ((4, 6), -1), ((3, 4, 5), 1), ((4, 6), None)])
def test_keeping_every_coefficient_reconstructs_the_tensor(algo, shape, dim):
    torch.manual_seed(3)
    x = torch.randn(*shape)
    n = x.numel() if dim is None else x.shape[dim]
    s = SignalSparsity(algo=algo, sst_top_k_element=n, sst_top_k_dim=dim, dst_top_k_element=1, dst_top_k_dim=dim)
    sst = s.dense_to_sst(x)
    assert sst.shape == x.shape
    torch.testing.assert_close(s.sst_dst_to_dense(sst), x, atol=2e-5, rtol=1e-4)
    # whatever the SST keeps, an SST plus a full DST is exact
    s = SignalSparsity(algo=algo, sst_top_k_element=1, sst_top_k_dim=dim, dst_top_k_element=n, dst_top_k_dim=dim)
    rec, sst, dst = s.lossy_compress(x)
    torch.testing.assert_close(rec, x, atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("dim,k", [(0, 1), (0, 3), (1, 2), (1, 6), (None, 5)])
def test_top_k_counts_by_element_and_by_percent_agree(dim, k):
    torch.manual_seed(4)
    x = torch.randn(4, 6)
    total = x.numel() if dim is None else x.shape[dim]
    by_element = SignalSparsity(sst_top_k_element=k, sst_top_k_dim=dim, dst_top_k_element=k, dst_top_k_dim=dim)
    by_percent = SignalSparsity(sst_top_k_percent=100.0 * k / total, sst_top_k_dim=dim, dst_top_k_percent=100.0 * k / total, dst_top_k_dim=dim)
    a, b = by_element.dense_to_sst(x), by_percent.dense_to_sst(x)
    torch.testing.assert_close(a, b)
    kept = (a != 0).sum() if dim is None else (a != 0).sum(dim=dim).max()
    assert int(kept) <= k
    if dim is not None:
        other = (a != 0).sum(dim=dim)
        assert int(other.min()) >= 1  # each slice along the dimension keeps its own top k
    torch.testing.assert_close(by_element.dense_sst_to_dst(x, a), by_percent.dense_sst_to_dst(x, b))


def test_one_half_disabled():
    x = torch.arange(20.0).reshape(4, 5).cos()
    only_dst = SignalSparsity(dst_top_k_element=2)
    assert only_dst.dense_to_sst(x) is None
    dst = only_dst.dense_sst_to_dst(x, None)
    assert int((dst != 0).sum(-1).max()) == 2
    # the two largest magnitudes of every row, at their places
    top = x.abs().topk(2, dim=-1)
    torch.testing.assert_close(dst.gather(-1, top.indices).abs(), top.values)
    rec, sst, dst2 = only_dst.lossy_compress(x)
    assert sst is None and torch.equal(rec, dst2) and torch.equal(dst, dst2)

    only_sst = SignalSparsity(sst_top_k_element=2)
    sst = only_sst.dense_to_sst(x)
    assert only_sst.dense_sst_to_dst(x, sst) is None
    rec, sst2, none = only_sst.lossy_compress(x)
    assert none is None and torch.equal(sst, sst2)
    torch.testing.assert_close(rec, only_sst.sst_dst_to_dense(sst))
    with pytest.raises(AssertionError):
        only_sst.sst_dst_to_dense(None, None)
    with pytest.raises(ValueError):
        SignalSparsity(sst_top_k_element=2, dst_top_k_element=2).dense_sst_to_dst(x, torch.zeros(2, 2, dtype=torch.complex64))


@pytest.mark.parametrize("dim", [0, 1, None])
def test_nothing_to_drop_returns_the_input_itself(dim):
    x = torch.randn(3, 7)
    s = SignalSparsity(sst_top_k_percent=100, sst_top_k_dim=dim, dst_top_k_percent=100, dst_top_k_dim=dim)
    rec, sst, dst = s.lossy_compress(x)
    assert rec is x and sst is None and dst is x


def test_random_mask_has_the_requested_density_along_the_dimension():
    torch.manual_seed(0)
    x = torch.randn(10, 40)
    for percent, dim, expect in ((10, 1, 4), (50, 0, 5), (100, 1, 40), (1, 1, 1)):
        m = random_sparse_mask(x, percent, dim)
        assert m.shape == x.shape and set(m.unique().tolist()) <= {0.0, 1.0}
        assert torch.all(m.sum(dim) == expect)
    a, b = random_sparse_mask(x, 10, 1), random_sparse_mask(x, 10, 1)
    assert not torch.equal(a, b)  # drawn afresh every call
    with pytest.raises(AssertionError):
        random_sparse_mask(x, 0, 1)


def test_energy_profile_on_known_signals():
    # all of the energy in one entry per row
    x = torch.zeros(4, 100)
    x[:, 7] = 3.0
    prof = EnergyConcentrationProfile(dim=1, top_k_percents=[1, 10, 100])
    assert [round(float(v), 6) for v in prof.measure(x)] == [1.0, 1.0, 1.0]
    # flat signal: the share equals the percentage
    flat = torch.ones(4, 100)
    assert [round(float(v), 6) for v in prof.measure(flat)] == [0.01, 0.1, 1.0]
    # a pure tone concentrates in the frequency domain, not in the time domain
    t = torch.arange(256.0)
    tone = torch.cos(2 * torch.pi * 8 * t / 256).unsqueeze(0)
    p = EnergyConcentrationProfile(dim=1, top_k_percents=[1])
    assert float(p.measure_fft(tone)[0]) > 0.99 > 0.05 > float(p.measure(tone)[0])
    with pytest.raises(AssertionError):
        EnergyConcentrationProfile(dim=0, top_k_percents=[0.0])
    with pytest.raises(AssertionError):
        prof.measure(torch.ones(2, 2, dtype=torch.int64))


# ------------------------------------------------------------------------------------------------ SHA1_Store
def _checkpoints(tmp_path):
    """Five files: four networks of different widths, and a byte-for-byte copy of the last one (a second ``torch.save`` would
    not do: the archive records the file's own name)."""
    paths = []
    for i, width in enumerate([10, 20, 30, 40]):
        torch.manual_seed(i)
        path = tmp_path / f"ckpt_{i}.pt"
        torch.save(torch.nn.Linear(width, width).state_dict(), path)
        paths.append(path)
    paths.append(tmp_path / "ckpt_4.pt")
    shutil.copy(paths[3], paths[4])
    return paths


@pytest.mark.parametrize("compress", [True, False])
def test_store_files_state_dicts_and_tensors(tmp_path, compress):
    store = SHA1_Store(tmp_path / "store", init=True)
    paths = _checkpoints(tmp_path)
    keys = [store.add(p, compress) for p in paths]
    assert keys[3] == keys[4] and len(set(keys)) == 4
    meta = json.loads((tmp_path / "store" / "sha1_store.json").read_text())
    entries = {k: v for k, v in meta.items() if isinstance(v, dict)}
    assert sorted(e["ref_count"] for e in entries.values()) == [1, 1, 1, 2]

    # a state dict is stored tensor by tensor: adding the same one twice doubles every count
    sd = torch.nn.Sequential(torch.nn.Linear(8, 8), torch.nn.Linear(8, 4)).state_dict()
    first = store.add(sd, compress)
    assert store.add(sd, compress) == first and set(first.keys()) == set(sd.keys())
    meta = json.loads((tmp_path / "store" / "sha1_store.json").read_text())
    counts = sorted(v["ref_count"] for v in meta.values() if isinstance(v, dict))
    assert counts == [1, 1, 1, 2, 2, 2, 2, 2]

    t = torch.arange(77.0)
    key = store.add(t, compress)
    assert torch.equal(store.get(key), t)
    # what comes back equals what went in
    assert objects_are_equal(store.get(keys[0]), torch.load(paths[0]))
    assert objects_are_equal({k: store.get(v) for k, v in first.items()}, dict(sd))
    with pytest.raises(ValueError):
        store.get("0" * 40)


@pytest.mark.parametrize("compress", [True, False])
def test_store_delete_counts_down_and_then_forgets(tmp_path, compress):
    store = SHA1_Store(tmp_path / "store", init=True)
    with pytest.raises(ValueError):
        store.delete("0" * 40)
    path = _checkpoints(tmp_path)[0]
    key = store.add(path, compress)
    assert store.add(path, compress) == key
    store.delete(key)
    assert objects_are_equal(store.get(key), torch.load(path))  # one reference is left
    store.delete(key)
    with pytest.raises(ValueError):
        store.get(key)
    with pytest.raises(ValueError):
        store.delete(key)
    assert store.size_info() == (0, 0, 0)


@pytest.mark.parametrize("compress", [True, False])
def test_store_sizes_and_names(tmp_path, compress):
    store = SHA1_Store(tmp_path / "store", init=True)
    t = torch.zeros(4000)  # compresses well
    key = store.add(t, compress, name="first")
    orig, dedup, comp = store.size_info(key)
    assert orig == dedup and (comp < orig if compress else comp == orig)
    assert store.size_info() == (orig, dedup, comp)
    assert store.names(key) == {"first": 1}
    assert store.add(t.clone(), compress, name="second") == key
    orig2, dedup2, comp2 = store.size_info(key)
    assert orig2 == 2 * orig and dedup2 == dedup and comp2 == comp
    assert store.names(key) == {"first": 1, "second": 1}
    store.add(t, compress, name="second")
    assert store.names(key) == {"first": 1, "second": 2}


def test_store_open_create_and_reopen(tmp_path):
    with pytest.raises(RuntimeError):
        SHA1_Store(tmp_path / "nothing_here" / "x")  # opening a store that was never created
    store = SHA1_Store(tmp_path / "s", init=True, tmp_dir=str(tmp_path / "staging"))
    assert (tmp_path / "staging").is_dir()
    key = store.add(torch.ones(3))
    again = SHA1_Store(tmp_path / "s")
    assert torch.equal(again.get(key), torch.ones(3))
    with pytest.raises(SystemExit):
        SHA1_Store(tmp_path / "s", init=True)  # refuses to initialise over an existing directory


# ------------------------------------------------------------------------------------------------ git wrapper
def test_git_wrapper_add_commit_status_log(tmp_path):
    root = tmp_path / ".wgit"
    root.mkdir()
    git = PyGit(root, gitignore=["sha1_store"])
    assert Path(git.path) == root / ".git" and (root / ".gitignore").read_text() == "sha1_store\n"
    (root / "a.pt").write_text("1")
    (root / "b.pt").write_text("2")
    assert set(git.status()) == {".gitignore", "a.pt", "b.pt"} and all(v == "??" for v in git.status().values())
    git.add()
    assert all(v.strip() == "A" for v in git.status().values())
    git.commit("first files")
    assert git.status() == {} and "first files" in git.log()
    (root / "a.pt").write_text("changed")
    assert git.status() == {"a.pt": " M"}
    git.add()
    git.commit("second")
    assert len(git.log("a.pt").splitlines()) == 2 and len(git.log("b.pt").splitlines()) == 1
    # opening an existing repository keeps its history and its ignore file
    again = PyGit(root)
    assert "second" in again.log() and (root / ".gitignore").read_text() == "sha1_store\n"
    with pytest.raises(RuntimeError):
        again.checkout("not-a-revision")


# ------------------------------------------------------------------------------------------------ Repo API and CLI
@pytest.fixture
def in_tmp(tmp_path):
    cwd = os.getcwd()
    os.chdir(tmp_path)
    yield tmp_path
    os.chdir(cwd)


@pytest.mark.parametrize("per_tensor", [True, False])
@pytest.mark.parametrize("gzip", [True, False])
def test_repo_api_status_transitions(in_tmp, per_tensor, gzip):
    repo = Repo(in_tmp, init=True)
    assert (in_tmp / ".wgit" / "sha1_store").is_dir() and (in_tmp / ".wgit" / ".git").exists() and (in_tmp / ".wgit" / ".gitignore").is_file()
    assert repo.status() == {}

    (in_tmp / "sub").mkdir()
    first, second = "sub/ckpt_a.pt", "ckpt_b.pt"
    torch.save(torch.nn.Linear(6, 6).state_dict(), first)
    ret = repo.add(first, per_tensor=per_tensor, gzip=gzip)
    assert (ret is not None and set(ret) == {"weight", "bias"}) if per_tensor else ret is None
    assert repo.status() == {first: RepoStatus.CHANGES_ADDED_NOT_COMMITED}
    meta = json.loads((in_tmp / ".wgit" / first).read_text())
    assert meta["file_path"] == first and meta["last_modified_time_stamp"] == (in_tmp / first).stat().st_mtime
    repo.commit("epoch 1")
    assert repo.status() == {first: RepoStatus.CLEAN}

    torch.save(torch.nn.Linear(6, 6).state_dict(), first)
    os.utime(first, (1_000_000_000, 1_000_000_000))  # a new modification time whatever the clock resolution
    assert repo.status() == {first: RepoStatus.CHANGES_NOT_ADDED}
    repo.add(first, per_tensor=per_tensor, gzip=gzip)
    assert json.loads((in_tmp / ".wgit" / first).read_text())["SHA1"] != meta["SHA1"]
    assert repo.status() == {first: RepoStatus.CHANGES_ADDED_NOT_COMMITED}

    torch.save(torch.ones(5), second)
    repo.add(second, per_tensor=per_tensor, gzip=gzip)
    assert repo.status() == {first: RepoStatus.CHANGES_ADDED_NOT_COMMITED, second: RepoStatus.CHANGES_ADDED_NOT_COMMITED}
    repo.commit("epoch 2")
    assert repo.status() == {first: RepoStatus.CLEAN, second: RepoStatus.CLEAN}
    if per_tensor:
        assert torch.equal(repo.get(second), torch.ones(5))
        assert objects_are_equal(repo.get(first), dict(torch.load(first)))
    info = repo.size_info()
    assert info.original >= info.deduped > 0 and (info.gzipped <= info.deduped)
    one = repo.size_info(first) if per_tensor else None
    assert one is None or 0 < one.deduped < info.deduped


def test_repo_refuses_missing_things(in_tmp, capsys):
    with pytest.raises(SystemExit):
        Repo(in_tmp)  # not a repository
    assert "not a wgit repository" in capsys.readouterr().err
    repo = Repo(in_tmp, init=True)
    with pytest.raises(SystemExit):
        repo.add("no_such_file.pt")
    torch.save(torch.ones(2), "x.pt")
    with pytest.raises(ValueError):
        repo.add("x.pt", per_tensor=False, sparsify=True)
    with pytest.raises(NotImplementedError):
        repo.checkout_by_steps()
    with pytest.raises(RuntimeError):
        repo.checkout("0123456789abcdef0123456789abcdef01234567")  # no such revision


def test_repo_checkout_moves_the_metadata_back(in_tmp):
    repo = Repo(in_tmp, init=True)
    torch.save({"w": torch.zeros(4)}, "m.pt")
    repo.add("m.pt")
    repo.commit("zeros")
    first_rev = repo._pygit.log().split()[0]
    torch.save({"w": torch.ones(4)}, "m.pt")
    os.utime("m.pt", (1_000_000_000, 1_000_000_000))
    repo.add("m.pt")
    repo.commit("ones")
    assert torch.equal(repo.get("m.pt")["w"], torch.ones(4))
    repo.checkout(first_rev)
    assert torch.equal(repo.get("m.pt")["w"], torch.zeros(4))


def test_repo_sparsified_checkpoint_with_a_policy_per_tensor(in_tmp):
    torch.manual_seed(0)
    repo = Repo(in_tmp, init=True)
    sd = {"big": torch.randn(16, 64), "small": torch.randn(4, 4), "steps": torch.tensor(7), "note": "hello"}
    torch.save(sd, "s.pt")
    seen = []

    def policy(name):
        seen.append(name)
        keep = 100 if name == "small" else 25
        return SignalSparsity(sst_top_k_percent=keep, dst_top_k_percent=keep)

    repo.add("s.pt", sparsify=True, sparsify_policy=policy)
    assert sorted(seen) == ["big", "small"]  # only floating tensors with a dimension are sparsified
    got = repo.get("s.pt")
    torch.testing.assert_close(got["small"], sd["small"])   # nothing dropped
    assert int(got["steps"]) == 7 and got["note"] == "hello"
    err = (got["big"] - sd["big"]).norm() / sd["big"].norm()
    assert 0.0 < float(err) < 0.9 and got["big"].shape == sd["big"].shape


def test_command_line_round(in_tmp, capsys):
    main(["init"])
    assert Path(".wgit/sha1_store").is_dir() and Path(".wgit/.gitignore").is_file() and Path(".wgit/.git").exists()
    torch.save(torch.nn.Linear(3, 3).state_dict(), "checkpoint_0.pt")
    main(["add", "checkpoint_0.pt"])
    first = json.loads(Path(".wgit/checkpoint_0.pt").read_text())["SHA1"]
    torch.save(torch.nn.Linear(3, 3).state_dict(), "checkpoint_0.pt")
    main(["add", "--no_per_tensor", "checkpoint_0.pt"])
    second = json.loads(Path(".wgit/checkpoint_0.pt").read_text())["SHA1"]
    assert isinstance(first, dict) and isinstance(second, str)
    main(["commit", "-m", "epoch_1"])
    capsys.readouterr()
    main(["status"])
    assert capsys.readouterr().out == "{'checkpoint_0.pt': <RepoStatus.CLEAN: 1>}\n"
    main(["log"])
    out = capsys.readouterr()
    assert out.out.startswith("wgit log\n") and "epoch_1" in out.out and out.err == ""
    main(["log", "--file", "checkpoint_0.pt"])
    assert capsys.readouterr().out.startswith("wgit log of the file: checkpoint_0.pt\n")
    main(["version"])
    assert capsys.readouterr().out.strip().count(".") == 2
    main([])
    assert "usage" in capsys.readouterr().out.lower()
    with pytest.raises(SystemExit):
        main(["commit"])  # a message is required
