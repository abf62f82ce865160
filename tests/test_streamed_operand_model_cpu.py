"""Index arithmetic of the GEMMs whose operand arrives while they run, restated in Python and checked exhaustively on small
cases and on the shapes of the benchmarks at 2, 4 and 8 ranks.

Host side (``csrc/comm.cu``): ``fsb_comm_gather_flagged_copies`` sends the pieces of the weight cyclically from
``first_piece`` on and raises ``flags[i]`` after the i-th piece sent; ``fsb_comm_gather_blocks_flagged`` sends the row blocks
of an activation own block first, then rank + 1, ... and raises one flag per piece of a block.  Device side
(``csrc/gemm_tcgen05.cu``): ``pair_tile_coords`` orders the tiles, ``wait_b_pieces`` / ``wait_a_rows`` decide which flags a
tile waits for, remembering the highest flag index seen (flags are raised in index order, so a raised flag vouches for
all lower ones).  Checked here: every byte a tile reads is covered by a flag the tile waited for (directly or through
that rule); tiles follow the arrival order, so that consuming tiles in order never needs the piece sent last before the
others; and, for the weight gather, the ranks do not all pull from the same source at once.
"""
import itertools

import pytest

TILE_ROWS, HALF_ROWS = 256, 128  # rows of B (or A) per CTA-pair tile and per CTA


# ------------------------------------------------------------------------------------------------ streamed B (weight)
def _b_tile_rows_in_order(N, K, piece_bytes, first_piece):
    """Yields ``(n0, n1)`` row ranges of B, per CTA of the pair, in the order the kernel visits its N tiles."""
    tiles_n = -(-N // TILE_ROWS)
    tile_bytes = TILE_ROWS * K * 2
    rot = -(-first_piece * piece_bytes // tile_bytes)
    for lin in range(tiles_n):
        tn = (lin + rot) % tiles_n
        for half in range(2):
            n0 = tn * TILE_ROWS + half * HALF_ROWS
            if n0 < N:
                yield n0, min(n0 + HALF_ROWS, N)


def _b_flags_waited(n0, n1, K, piece_bytes, first_piece, num_pieces, upto):
    """``wait_b_pieces``: the flag indices this call polls, and the new ``upto``."""
    lo, hi = n0 * K * 2, n1 * K * 2
    polled = []
    for q in range(lo // piece_bytes, (hi - 1) // piece_bytes + 1):
        i = (q - first_piece + num_pieces) % num_pieces
        if i > upto:
            polled.append(i)
            upto = i
    return polled, upto


def _b_send_order(total_bytes, piece_bytes, first_piece):
    """Host: the byte range sent as the i-th piece, for i = 0, 1, ..."""
    num = -(-total_bytes // piece_bytes)
    for i in range(num):
        q = (first_piece + i) % num
        yield i, q * piece_bytes, min((q + 1) * piece_bytes, total_bytes)


@pytest.mark.parametrize("N,K,piece_bytes", [(6144, 2048, 4 << 20), (512, 256, 64 << 10), (768, 1024, 64 << 10), (1536, 512, 2 << 20),
                                             (264, 72, 8 << 10), (1000, 136, 100_000)])
def test_streamed_b_every_byte_is_vouched_for_and_tiles_follow_arrival(N, K, piece_bytes):
    total = N * K * 2
    num = -(-total // piece_bytes)
    for first in range(num):
        sent_as = {}  # byte -> sending index, by piece
        for i, a, b in _b_send_order(total, piece_bytes, first):
            sent_as[(a, b)] = i
        assert sorted(sent_as.values()) == list(range(num))
        upto, order_of_first_need = -1, []
        for n0, n1 in _b_tile_rows_in_order(N, K, piece_bytes, first):
            polled, upto = _b_flags_waited(n0, n1, K, piece_bytes, first, num, upto)
            # every piece under the tile's rows was sent with an index <= upto: its flag is up once flag `upto` is
            for (a, b), i in sent_as.items():
                if a < n1 * K * 2 and b > n0 * K * 2:
                    assert i <= upto, (first, n0, n1, i, upto)
            order_of_first_need.extend(polled)
        # flags are polled in increasing order only (no wait can be lapped), and every flag is eventually looked at or vouched for
        assert order_of_first_need == sorted(order_of_first_need)
        assert upto == num - 1
        # the first tile visited does not need the piece that is sent last, unless one tile spans every piece
        first_rows = next(_b_tile_rows_in_order(N, K, piece_bytes, first))
        polled, _ = _b_flags_waited(*first_rows, K, piece_bytes, first, num, -1)
        if num > 2 and TILE_ROWS * K * 2 <= piece_bytes:
            assert max(polled) < num - 1, (first, polled)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_weight_gather_ranks_start_at_different_pieces_and_spread_over_the_sources(world):
    """The QKV weight of a GPT block (25 MB at the front of a 96 MB flat parameter) lies in the shards of the first ranks.
    With every rank starting at piece ``rank * pieces // world`` no source serves more than about two thirds of the ranks at
    any step, where the same order on every rank makes all of them read one source."""
    d, ffn = 2048, 8192
    flat = 4 * d * d + 2 * d * ffn + 9 * d + ffn
    shard_bytes = -(-flat // (world * 8)) * 8 * 2
    piece, w_bytes = 4 << 20, 3 * d * d * 2
    num = -(-w_bytes // piece)

    def worst_fan_in(first_of):
        worst = 0
        for step in range(num):
            readers = {}
            for r in range(world):
                q = (first_of(r) + step) % num
                owners = {b // shard_bytes for b in (q * piece, min((q + 1) * piece, w_bytes) - 1)}
                for o in owners - {r}:
                    readers[o] = readers.get(o, 0) + 1
            worst = max(worst, max(readers.values(), default=0))
        return worst

    same_order = worst_fan_in(lambda r: 0)
    rotated = worst_fan_in(lambda r: (r * num) // world)
    assert same_order == world - 1  # everybody but the owner reads the first shard at once
    # the weight only lies in two or three shards, so the ranks cannot be spread over more sources than that
    assert rotated <= -(-2 * world // 3), (world, rotated)
    assert rotated <= same_order and (rotated < same_order or world < 8)  # with 2-4 ranks the weight sits in one or two shards


# ------------------------------------------------------------------------------------------------ streamed A (activation)
def _a_tile_rows_in_order(M, shard_rows, first_shard):
    tiles_m = -(-M // TILE_ROWS)
    rot = -(-first_shard * shard_rows // TILE_ROWS)
    for lin in range(tiles_m):
        tm = (lin + rot) % tiles_m
        for half in range(2):
            m0 = tm * TILE_ROWS + half * HALF_ROWS
            if m0 < M:
                yield m0, min(m0 + HALF_ROWS, M)


def _a_flags_waited(r0, r1, shard_rows, piece_rows, first_shard, num_shards, upto):
    """``wait_a_rows``."""
    pps = -(-shard_rows // piece_rows)
    polled, r = [], r0
    while r < r1:
        shard, in_shard = divmod(r, shard_rows)
        k = (shard - first_shard + num_shards) % num_shards
        j = in_shard // piece_rows
        idx = k * pps + j
        if idx > upto:
            polled.append(idx)
            upto = idx
        r = min(shard * shard_rows + (j + 1) * piece_rows, (shard + 1) * shard_rows)
    return polled, upto


def _a_send_order(world, rank, shard_rows, piece_rows):
    """Host: ``(flag index, first row, last row + 1)`` in sending order (own block, then rank + 1, ...)."""
    pps = -(-shard_rows // piece_rows)
    for k in range(world):
        p = (rank + k) % world
        for j in range(pps):
            yield k * pps + j, p * shard_rows + j * piece_rows, p * shard_rows + min((j + 1) * piece_rows, shard_rows)


@pytest.mark.parametrize("world,shard_rows,piece_rows", [(2, 8192, 512), (4, 4096, 512), (8, 2048, 512), (2, 128, 128), (4, 384, 128),
                                                         (3, 640, 256), (8, 4096, 4096)])
def test_streamed_a_rows_are_vouched_for_and_own_block_comes_first(world, shard_rows, piece_rows):
    M = world * shard_rows
    for rank in range(world):
        sent = list(_a_send_order(world, rank, shard_rows, piece_rows))
        assert [i for i, _, _ in sent] == list(range(len(sent)))
        upto, polled_all = -1, []
        for r0, r1 in _a_tile_rows_in_order(M, shard_rows, rank):
            polled, upto = _a_flags_waited(r0, r1, shard_rows, piece_rows, rank, world, upto)
            for i, a, b in sent:
                if a < r1 and b > r0:
                    assert i <= upto, (rank, r0, r1, i, upto)
            polled_all.extend(polled)
        assert upto == len(sent) - 1
        # flags are only ever polled in increasing order
        assert polled_all == sorted(polled_all)
        # the first tile lies in the rank's own block, which is in place before the kernel starts (when the block is large
        # enough to contain a whole aligned tile)
        start = -(-rank * shard_rows // TILE_ROWS) * TILE_ROWS
        if start + TILE_ROWS <= (rank + 1) * shard_rows:
            for r0, r1 in itertools.islice(_a_tile_rows_in_order(M, shard_rows, rank), 2):  # both CTAs of the first pair
                first_polled, _ = _a_flags_waited(r0, r1, shard_rows, piece_rows, rank, world, -1)
                assert max(first_polled) < -(-shard_rows // piece_rows), (rank, r0, r1, first_polled)


def test_every_tile_is_visited_exactly_once_under_any_rotation():
    for tiles, rot in itertools.product(range(1, 9), range(0, 12)):
        assert sorted((lin + rot) % tiles for lin in range(tiles)) == list(range(tiles))
