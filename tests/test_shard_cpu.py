"""Row-window sharding (host logic) on CPU, including a world_size-2 gloo run.

The property that makes the single-SpMM path collective-free: every window is built and
multiplied independently, so a rank's format arrays are the matching segments of the unsharded
arrays and concatenating the per-rank results reproduces the unsharded result bit for bit.
The CPU oracle stands in for the GPU operators here (no GPU in this test)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as O
from trspmm import graphs, shard


def test_cuts_are_window_aligned_and_balanced():
    rp, col, val = graphs.rmat_graph(12, 16, seed=3)
    n = rp.numel() - 1
    for parts in (1, 2, 3, 8):
        cuts = shard.balanced_window_cuts(rp, parts)
        assert cuts[0] == 0 and cuts[-1] == n and len(cuts) == parts + 1
        assert all(c % 16 == 0 for c in cuts[:-1]) and cuts == sorted(cuts)
        loads = [int(rp[b] - rp[a]) for a, b in zip(cuts[:-1], cuts[1:])]
        heaviest_window = int((rp[16::16] - rp[:-16:16]).max())
        assert max(loads) <= col.numel() / parts + heaviest_window
    # ragged row count and more parts than windows
    rp2, _, _ = graphs.uniform_graph(100, 3, seed=1)
    cuts = shard.balanced_window_cuts(rp2, 16)
    assert cuts[0] == 0 and cuts[-1] == 100 and cuts == sorted(cuts)


def test_shard_formats_are_segments_of_the_full_format():
    rp, col, val = graphs.clustered_graph(1024, 64, 12, 2, seed=2)
    full, _ = O.build_format(rp, col, val)
    named = dict(zip(O.FORMAT_NAMES, full))
    cuts = shard.balanced_window_cuts(rp, 3)
    g0 = t0 = 0
    for a, b in zip(cuts[:-1], cuts[1:]):
        rp_l, col_l, val_l = shard.slice_csr(rp, col, val, a, b)
        part, _ = O.build_format(rp_l, col_l, val_l)
        p = dict(zip(O.FORMAT_NAMES, part))
        G, T = p["s_column"].shape[0], p["s_tile_column"].shape[0]
        assert torch.equal(p["s_column"], named["s_column"][g0:g0 + G])
        assert torch.equal(p["s_value"], named["s_value"][g0:g0 + G])
        assert torch.equal(p["s_packed_a"], named["s_packed_a"][t0:t0 + T])
        assert torch.equal(p["s_packed_meta"], named["s_packed_meta"][t0:t0 + T])
        assert torch.equal(p["s_tile_column"], named["s_tile_column"][t0:t0 + T])
        w0 = a // 16
        assert torch.equal(p["s_offset"], named["s_offset"][w0:w0 + p["s_offset"].numel()] - g0)
        g0 += G
        t0 += T
    assert g0 == named["s_column"].shape[0] and t0 == named["s_tile_column"].shape[0]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rp, col, val = graphs.rmat_graph(10, 8, seed=7)  # same seed on every rank
        n = rp.numel() - 1
        B = torch.randn(n, 16, generator=torch.Generator().manual_seed(0)).half()
        (r0, r1), (rp_l, col_l, val_l) = shard.shard_for_rank(rp, col, val, rank, world)
        fmt, _ = O.build_format(rp_l, col_l, val_l)
        mine = O.spmm_from_format(fmt, B, r1 - r0)
        # gather the row blocks: every rank contributes a different number of rows
        cuts = shard.balanced_window_cuts(rp, world)
        full = torch.zeros(n, 16)
        full[r0:r1] = mine
        ops = []
        for peer in range(world):  # unequal-count all-gather as one batch of sends / receives
            if peer == rank:
                continue
            ops.append(dist.P2POp(dist.irecv, full[cuts[peer]:cuts[peer + 1]], peer))
            ops.append(dist.P2POp(dist.isend, full[r0:r1], peer))
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        if rank == 0:
            whole, _ = O.build_format(rp, col, val)
            q.put(bool(torch.equal(full, O.spmm_from_format(whole, B, n))))
    finally:
        dist.destroy_process_group()


def test_two_ranks_reassemble_the_unsharded_result():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
        assert p.exitcode == 0
    assert q.get(timeout=10) is True


def _failing_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    try:
        if rank == 1:
            raise RuntimeError("injected host-side failure before the collective")
        try:
            t = torch.zeros(4)
            dist.broadcast(t, src=1)  # the peer never joins
            q.put("no error")
        except Exception as exc:  # the survivor sees an error instead of hanging
            q.put("error: " + type(exc).__name__)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_rank_failure_is_seen_on_the_host():
    """Failure detection without touching a GPU: a rank raises before the collective, the other
    rank's collective ends with an error within the process-group timeout."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    assert procs[1].exitcode != 0
    assert q.get(timeout=10).startswith("error")


def test_even_row_split_covers_all_rows():
    from trspmm.shard import even_row_split
    for n, w in ((10, 1), (10, 3), (2097152, 8), (7, 8), (16, 4)):
        per, padded = even_row_split(n, w)
        assert per * w == padded and padded >= n and padded - n < w + per
        covered = sum(max(0, min((r + 1) * per, n) - r * per) for r in range(w))
        assert covered == n


def test_rescale_costs_moves_windows_away_from_the_slow_rank():
    from trspmm.shard import cuts_from_window_costs, rescale_costs
    W, n = 400, 400 * 16
    cost = torch.ones(W)
    cuts = cuts_from_window_costs(cost, 4, n)
    assert cuts == [0, 1600, 3200, 4800, 6400]
    # rank 1 measured 50 % slower than the others: its range must shrink, the total stays covered
    new_cost = rescale_costs(cost, cuts, [1.0, 1.5, 1.0, 1.0])
    new_cuts = cuts_from_window_costs(new_cost, 4, n)
    assert new_cuts[0] == 0 and new_cuts[-1] == n and all(b >= a for a, b in zip(new_cuts, new_cuts[1:]))
    assert new_cuts[2] - new_cuts[1] < cuts[2] - cuts[1]
    assert all(c % 16 == 0 for c in new_cuts)
    # equal times change nothing
    assert cuts_from_window_costs(rescale_costs(cost, cuts, [2.0] * 4), 4, n) == cuts


def test_output_transfers_cover_every_even_share_exactly_once():
    """Re-deal of the computed rows: for any cut, the pieces the ranks send to a peer tile that
    peer's even share of the rows without gap or overlap."""
    import random
    rng = random.Random(5)
    for world in (2, 3, 8):
        for n in (1, 17, 1000, 4099):
            for _ in range(20):
                inner = sorted(rng.randint(0, n) for _ in range(world - 1))
                cuts = [0] + inner + [n]
                got = {p: [] for p in range(world)}
                for r in range(world):
                    for peer, src, dst, cnt in shard.output_transfers(cuts, r):
                        assert cnt > 0 and 0 <= src and src + cnt <= cuts[r + 1] - cuts[r]
                        o0, o1 = shard.even_output_rows(n, world, peer)
                        assert cuts[r] + src == o0 + dst         # the same global row on both sides
                        got[peer].append((dst, cnt))
                for p in range(world):
                    o0, o1 = shard.even_output_rows(n, world, p)
                    pos = 0
                    for dst, cnt in sorted(got[p]):
                        assert dst == pos
                        pos += cnt
                    assert pos == o1 - o0
