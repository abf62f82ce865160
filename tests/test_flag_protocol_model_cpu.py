"""Exhaustive host-side model of the flag protocol of the NVLink collectives (``csrc/comm_dev.cuh``).

A collective call number ``k`` uses epoch ``e0 + k`` on two channels.  Every rank: (1) has its input in its symmetric
buffer, (2) stores the epoch into its slot of every peer's *entry* pad, (3) waits until all slots of its own entry pad
reached the epoch, (4) reads every peer's buffer, (5) stores the epoch into every peer's *exit* pad, (6) waits for its
own exit pad, and only then returns (the next call may overwrite the buffer).  Waits compare epochs as signed 32-bit
distances, so the counter may wrap.

The model explores EVERY interleaving of the ranks' steps (each flag store and each buffer read is a separate step)
for 2 and 3 ranks over several consecutive calls and checks: a buffer is never read before its owner wrote this call's
input, never overwritten while a peer may still read the previous call's data, and every schedule terminates.  Removing
the exit barrier must be caught by the same checker.
"""
from collections import deque

import pytest

MASK = 0xFFFFFFFF


def _reached(flag: int, epoch: int) -> bool:
    d = (flag - epoch) & MASK
    return d < 0x80000000  # signed distance >= 0


def _program(world: int, rank: int, calls: int, with_exit: bool):
    """The step list of one rank: tuples (op, call, peer)."""
    steps = []
    peers = [p for p in range(world)]
    for k in range(calls):
        steps.append(("write", k, rank))
        steps += [("sig_entry", k, p) for p in peers]
        steps.append(("wait_entry", k, rank))
        steps += [("read", k, p) for p in peers if p != rank]
        if with_exit:
            steps += [("sig_exit", k, p) for p in peers]
            steps.append(("wait_exit", k, rank))
    return steps


def explore(world: int, calls: int, e0: int, with_exit: bool = True):
    """Breadth-first search over all schedules.  Returns (violations, deadlocks, number of states)."""
    progs = [_program(world, r, calls, with_exit) for r in range(world)]
    init_flag = (e0 - 1) & MASK  # pads hold the epoch of the previous call
    # state: pcs, entry pads [dst][src], exit pads [dst][src], buffer versions, readers in flight are implicit in pcs
    start = (tuple([0] * world), tuple([init_flag] * (world * world)), tuple([init_flag] * (world * world)), tuple([-1] * world))
    seen = {start}
    queue = deque([start])
    violations, deadlocks = [], 0
    while queue:
        pcs, entry, exit_, bufs = queue.popleft()
        moved = False
        finished = all(pcs[r] == len(progs[r]) for r in range(world))
        for r in range(world):
            if pcs[r] == len(progs[r]):
                continue
            op, k, peer = progs[r][pcs[r]]
            epoch = (e0 + k) & MASK
            n_entry, n_exit, n_bufs = entry, exit_, bufs
            if op == "write":
                # overwriting the buffer is only safe if no peer can still read the previous call's data from it:
                # a peer that has not yet executed its read of rank r for call k-1 would see the new data
                if k > 0:
                    for q in range(world):
                        if q == r:
                            continue
                        pending = [s for s in progs[q][pcs[q]:] if s[0] == "read" and s[1] == k - 1 and s[2] == r]
                        if pending:
                            violations.append(("overwrite before read", r, q, k))
                n_bufs = bufs[:r] + (k,) + bufs[r + 1:]
            elif op == "sig_entry":
                i = peer * world + r
                n_entry = entry[:i] + (epoch,) + entry[i + 1:]
            elif op == "sig_exit":
                i = peer * world + r
                n_exit = exit_[:i] + (epoch,) + exit_[i + 1:]
            elif op == "wait_entry":
                if not all(_reached(entry[r * world + s], epoch) for s in range(world)):
                    continue  # blocked
            elif op == "wait_exit":
                if not all(_reached(exit_[r * world + s], epoch) for s in range(world)):
                    continue
            elif op == "read":
                if bufs[peer] != k:
                    violations.append(("stale or early read", r, peer, k, bufs[peer]))
            moved = True
            nxt = (pcs[:r] + (pcs[r] + 1,) + pcs[r + 1:], n_entry, n_exit, n_bufs)
            if nxt not in seen:
                seen.add(nxt)
                queue.append(nxt)
        if not moved and not finished:
            deadlocks += 1
    return violations, deadlocks, len(seen)


@pytest.mark.parametrize("world,calls", [(2, 3), (3, 2)])
def test_protocol_is_safe_and_live_under_every_schedule(world, calls):
    violations, deadlocks, states = explore(world, calls, e0=5)
    assert states > 100  # the search really branched
    assert violations == [] and deadlocks == 0


def test_protocol_survives_epoch_wraparound():
    violations, deadlocks, _ = explore(2, 3, e0=0xFFFFFFFE)  # epochs 0xFFFFFFFE, 0xFFFFFFFF, 0
    assert violations == [] and deadlocks == 0
    assert _reached(0, 0xFFFFFFFF) and not _reached(0xFFFFFFFF, 0) and _reached(7, 7)


def test_checker_catches_a_protocol_without_exit_barrier():
    violations, _, _ = explore(2, 2, e0=1, with_exit=False)
    kinds = {v[0] for v in violations}
    assert "overwrite before read" in kinds or "stale or early read" in kinds


# ---------------------------------------------------------------------------------------------------------------------
# GEMM -> reduce-scatter (``gemm_rs`` in csrc/gemm_comm_tcgen05.cu): rank r computes the chunks r+1, r+2, ..., r, writes
# each partial chunk c != r to slot c of its own staging buffer and then raises its flag in owner c's pad; owner c waits
# for every peer's flag and pulls that peer's slot c; an exit barrier ends the call.  Checked: a slot is only read once
# its producer has written this call's partial, and never overwritten by the next call while its owner may still read.
# ---------------------------------------------------------------------------------------------------------------------
def _rs_program(world: int, rank: int, calls: int, with_exit: bool):
    steps = []
    for k in range(calls):
        for i in range(1, world):
            c = (rank + i) % world
            steps.append(("write", k, c))           # my staging slot for chunk c
            steps.append(("flag", k, c))            # tell owner c
        for p in range(world):
            if p != rank:
                steps.append(("wait_flag", k, p))   # peer p finished my chunk
                steps.append(("pull", k, p))        # read slot `rank` of peer p's staging buffer
        if with_exit:
            steps += [("sig_exit", k, p) for p in range(world)]
            steps.append(("wait_exit", k, rank))
    return steps


def explore_rs(world: int, calls: int, e0: int, with_exit: bool = True):
    progs = [_rs_program(world, r, calls, with_exit) for r in range(world)]
    init = (e0 - 1) & MASK
    # flags[owner][src], exit pads [dst][src], staging versions [rank][chunk]
    start = (tuple([0] * world), tuple([init] * (world * world)), tuple([init] * (world * world)), tuple([-1] * (world * world)))
    seen, queue = {start}, deque([start])
    violations, deadlocks = [], 0
    while queue:
        pcs, flags, exit_, stage = queue.popleft()
        moved = False
        for r in range(world):
            if pcs[r] == len(progs[r]):
                continue
            op, k, x = progs[r][pcs[r]]
            epoch = (e0 + k) & MASK
            n_flags, n_exit, n_stage = flags, exit_, stage
            if op == "write":
                if k > 0:  # owner x must be done pulling slot x of rank r for call k-1
                    pending = [s for s in progs[x][pcs[x]:] if s == ("pull", k - 1, r)]
                    if pending:
                        violations.append(("overwrite before pull", r, x, k))
                i = r * world + x
                n_stage = stage[:i] + (k,) + stage[i + 1:]
            elif op == "flag":
                i = x * world + r
                n_flags = flags[:i] + (epoch,) + flags[i + 1:]
            elif op == "wait_flag":
                if not _reached(flags[r * world + x], epoch):
                    continue
            elif op == "pull":
                if stage[x * world + r] != k:
                    violations.append(("pull of a stale or missing partial", r, x, k, stage[x * world + r]))
            elif op == "sig_exit":
                i = x * world + r
                n_exit = exit_[:i] + (epoch,) + exit_[i + 1:]
            elif op == "wait_exit":
                if not all(_reached(exit_[r * world + s], epoch) for s in range(world)):
                    continue
            moved = True
            nxt = (pcs[:r] + (pcs[r] + 1,) + pcs[r + 1:], n_flags, n_exit, n_stage)
            if nxt not in seen:
                seen.add(nxt)
                queue.append(nxt)
        if not moved and not all(pcs[r] == len(progs[r]) for r in range(world)):
            deadlocks += 1
    return violations, deadlocks, len(seen)


@pytest.mark.parametrize("world,calls,e0", [(2, 3, 9), (3, 2, 0xFFFFFFFF)])
def test_gemm_rs_flag_protocol(world, calls, e0):
    violations, deadlocks, states = explore_rs(world, calls, e0)
    assert states > 50 and violations == [] and deadlocks == 0


def test_gemm_rs_checker_needs_the_exit_barrier():
    violations, _, _ = explore_rs(2, 2, e0=1, with_exit=False)
    assert any(v[0] == "overwrite before pull" or v[0].startswith("pull of a stale") for v in violations)
