"""Exhaustive host-side model of the barrier schedule of the ping-pong attention forward
(``csrc/attention_fwd_pingpong.cu``): one TMA producer, one MMA issuer, the in-order tensor pipe, and the softmax
groups of the two query tiles A and B, synchronised by phase-parity mbarriers exactly as in the kernel.

Every interleaving of the actors is explored (TMA loads land and tensor-pipe operations retire at arbitrary later
times).  Checked in every reachable state: no deadlock; a K / V stage is never overwritten by a load while an issued
product has yet to read it; S_t(j) is read by the softmax of step j only (not a stale or a later one); the
probabilities P_t(j), which overwrite the score columns, are consumed by P V of step j before S_t(j+1) lands on them; a
parity wait never passes on an older phase than the one the waiter means.
"""
from collections import deque

import pytest


def _program_producer(n_kv):
    steps = []
    for j in range(n_kv):
        st, par = j & 1, ((j >> 1) & 1) ^ 1
        steps += [("wait", f"k_empty{st}", par, j), ("load", "K", st, j), ("wait", f"v_empty{st}", par, j), ("load", "V", st, j)]
    return steps


def _program_mma(n_kv):
    n_a = n_kv - 1
    steps = []

    def issue_s(t, j):
        return [("wait", f"k_full{j & 1}", (j >> 1) & 1, j), ("mma", "S", t, j), ("commit", f"s_full{t}")]

    def issue_pv(t, j):
        return [("wait", f"p_full{t}", j & 1, j), ("mma", "PV", t, j), ("commit", f"o_done{t}")]

    steps += issue_s(0, 0) + issue_s(1, 0) + [("commit", "k_empty0")]
    for j in range(n_kv):
        steps.append(("wait", f"v_full{j & 1}", (j >> 1) & 1, j))
        if j < n_a:
            steps += issue_pv(0, j)
            if j + 1 < n_a:
                steps += issue_s(0, j + 1)
        steps += issue_pv(1, j) + [("commit", f"v_empty{j & 1}")]
        if j + 1 < n_kv:
            steps += issue_s(1, j + 1) + [("commit", f"k_empty{(j + 1) & 1}")]
    return steps


def _program_softmax(t, n_kv, rescale):
    n_it = n_kv - 1 if t == 0 else n_kv
    steps = []
    for j in range(n_it):
        steps += [("wait", f"s_full{t}", j & 1, j), ("read_s", t, j)]
        if rescale and j > 0:
            steps += [("wait", f"o_done{t}", (j - 1) & 1, j - 1), ("touch_o", t, j - 1)]
        steps += [("write_p", t, j), ("arrive", f"p_full{t}")]
    steps += [("wait", f"o_done{t}", (n_it - 1) & 1, n_it - 1), ("touch_o", t, n_it - 1)]
    return steps


BARS = ["k_full0", "k_full1", "k_empty0", "k_empty1", "v_full0", "v_full1", "v_empty0", "v_empty1",
        "s_full0", "s_full1", "p_full0", "p_full1", "o_done0", "o_done1"]


def explore(n_kv, rescale, break_order=False):
    progs = [_program_producer(n_kv), _program_mma(n_kv), _program_softmax(0, n_kv, rescale), _program_softmax(1, n_kv, rescale)]
    if break_order:  # a wrong schedule: S_A(j+1) issued before P V_A(j) (the checker must notice)
        mma = progs[1]
        for i, s in enumerate(mma):
            if s[:3] == ("mma", "PV", 0) and s[3] == 0:
                k = next(x for x in range(i, len(mma)) if mma[x][:3] == ("mma", "S", 0) and mma[x][3] == 1)
                mma[i - 1 : k + 2] = mma[k - 1 : k + 2] + mma[i - 1 : k - 1]  # move wait+S+commit ahead of wait+PV+commit
                break
    bar_idx = {b: i for i, b in enumerate(BARS)}
    # state: pcs(4), completed phases per barrier, in-flight loads (frozenset), tensor queue (tuple), stage versions
    # (K0,K1,V0,V1), score regions (kind, j) per tile, last P V retired per tile
    start = ((0, 0, 0, 0), tuple([0] * len(BARS)), frozenset(), (), (-1, -1, -1, -1), (("free", -1), ("free", -1)), (-1, -1))
    seen, queue = {start}, deque([start])
    problems, deadlocks = [], 0

    def passes(phases, name, parity, use):
        c = phases[bar_idx[name]]
        ok = parity != (c & 1)
        return ok, c

    while queue:
        state = queue.popleft()
        pcs, phases, loads, tq, stages, regions, pv_done = state
        successors = []
        # --- program steps of the four threads
        for a in range(4):
            if pcs[a] == len(progs[a]):
                continue
            op = progs[a][pcs[a]]
            n_ph, n_loads, n_tq, n_stages, n_regions = phases, loads, tq, stages, regions
            if op[0] == "wait":
                ok, c = passes(phases, op[1], op[2], op[3])
                if not ok:
                    continue
                # the waiter means use number `use_idx` of this barrier: stage barriers count every second step
                name, use = op[1], op[3]
                meant = use // 2 if name[0] in "kv" else use
                if name.endswith("empty0") or name.endswith("empty1"):
                    meant = use // 2 - 1  # the release of the previous occupant; -1 = never occupied
                if meant >= 0 and c < meant + 1:
                    problems.append(("wait passed on an older phase", a, op, c))
            elif op[0] == "load":
                n_loads = loads | {(op[1], op[2], op[3])}
            elif op[0] == "mma":
                n_tq = tq + (op,)
            elif op[0] == "commit":
                n_tq = tq + (op,)
            elif op[0] == "arrive":
                i = bar_idx[op[1]]
                n_ph = phases[:i] + (phases[i] + 1,) + phases[i + 1:]
            elif op[0] == "read_s":
                if regions[op[1]] != ("S", op[2]):
                    problems.append(("softmax read a wrong score tile", op, regions[op[1]]))
            elif op[0] == "write_p":
                n_regions = tuple(("P", op[2]) if t == op[1] else r for t, r in enumerate(regions))
            elif op[0] == "touch_o":
                if pv_done[op[1]] < op[2]:
                    problems.append(("output touched before its P V retired", op, pv_done))
            n_pcs = pcs[:a] + (pcs[a] + 1,) + pcs[a + 1:]
            successors.append((n_pcs, n_ph, n_loads, n_tq, n_stages, n_regions, pv_done))
        # --- a TMA load lands
        for ld in loads:
            kind, st, j = ld
            idx = st if kind == "K" else 2 + st
            pending = [o for o in tq if o[0] == "mma" and ((kind == "K" and o[1] == "S") or (kind == "V" and o[1] == "PV")) and (o[3] & 1) == st and o[3] < j]
            if pending:
                problems.append(("stage overwritten before an issued product read it", ld, pending))
            n_stages = stages[:idx] + (j,) + stages[idx + 1:]
            i = bar_idx[("k_full" if kind == "K" else "v_full") + str(st)]
            n_ph = phases[:i] + (phases[i] + 1,) + phases[i + 1:]
            successors.append((pcs, n_ph, loads - {ld}, tq, n_stages, regions, pv_done))
        # --- the tensor pipe retires its oldest entry
        if tq:
            op = tq[0]
            n_ph, n_regions, n_pv = phases, regions, pv_done
            if op[0] == "commit":
                i = bar_idx[op[1]]
                n_ph = phases[:i] + (phases[i] + 1,) + phases[i + 1:]
            elif op[1] == "S":
                _, _, t, j = op
                if stages[j & 1] != j:
                    problems.append(("S product read a K stage of another step", op, stages))
                if regions[t][0] == "P":
                    problems.append(("scores landed on unconsumed probabilities", op, regions[t]))
                n_regions = tuple(("S", j) if x == t else r for x, r in enumerate(regions))
            else:
                _, _, t, j = op
                if regions[t] != ("P", j):
                    problems.append(("P V read wrong probabilities", op, regions[t]))
                if stages[2 + (j & 1)] != j:
                    problems.append(("P V read a V stage of another step", op, stages))
                n_regions = tuple(("free", j) if x == t else r for x, r in enumerate(regions))
                n_pv = tuple(j if x == t else d for x, d in enumerate(pv_done))
            successors.append((pcs, n_ph, loads, tq[1:], stages, n_regions, n_pv))
        done = all(pcs[a] == len(progs[a]) for a in range(4)) and not tq and not loads
        if not successors and not done:
            deadlocks += 1
        for s in successors:
            if s not in seen:
                seen.add(s)
                queue.append(s)
        if len(problems) > 50:
            break
    return problems, deadlocks, len(seen)


@pytest.mark.parametrize("n_kv", [2, 4])
@pytest.mark.parametrize("rescale", [False, True])
def test_pingpong_schedule_is_safe_and_live(n_kv, rescale):
    problems, deadlocks, states = explore(n_kv, rescale)
    assert states > 200
    assert problems == [] and deadlocks == 0, (problems[:3], deadlocks)


def test_checker_notices_scores_issued_ahead_of_the_product_that_reads_the_probabilities():
    problems, deadlocks, _ = explore(4, False, break_order=True)
    assert problems or deadlocks
