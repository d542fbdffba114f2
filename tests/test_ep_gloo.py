"""The expert-parallel exchange plan among CPU ranks (gloo, world size 2 and 4).

On the GPUs the ranks gather their histograms into every rank's count table with peer stores and each derives, from the
table alone, where its rows land in every owner's receive buffer (blok_moe_ep_forward, csrc/ep.cu).  That arithmetic is
shared with blok_ep_plan_host (csrc/ep_plan.h), so the same code runs here: every rank routes its own ragged batch,
gloo carries the histograms, each rank plans with the C entry point, the rows are "sent" as (owner, row) records, and
the owners must find their buffers filled exactly once, grouped by expert, source ranks in order, with the tiles
covering exactly the received rows.  The reference is a single-GPU program; nothing here has a counterpart in it."""
import ctypes as C
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

E, TOPK = 32, 4


def plan_host(lib, table, world, rank, cap, max_tiles=4096):
    per = E // world
    i32 = lambda n: np.zeros(n, np.int32)
    send_base, counts, offsets = i32(E), i32(per), i32(per + 1)
    te, ts, tc, nt = i32(max_tiles), i32(max_tiles), i32(max_tiles), i32(1)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    tab = np.ascontiguousarray(table, np.int32)
    rc = lib.blok_ep_plan_host(p(tab), world, E, rank, C.c_long(cap), max_tiles, p(send_base), p(counts), p(offsets), p(te), p(ts),
                               p(tc), p(nt))
    n = int(nt[0])
    return rc, send_base, counts, offsets, te[:n], ts[:n], tc[:n]


def _worker(rank, world, port, fault, q):
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    # a short process-group timeout: a peer that is gone must end the survivors' next collective with an error
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        if fault == "peer_exits":
            dist.barrier()       # the group is up
            if rank == 1:
                os._exit(0)      # this rank leaves between steps, with nothing of its own in flight
        import blok_b200
        lib = blok_b200.load()
        per = E // world
        rng = np.random.default_rng(100 + rank)
        T = 5 + 3 * rank if fault != "empty_rank" or rank != 0 else 0          # ragged: every rank has a different token count
        ids = np.stack([rng.choice(E, TOPK, replace=False) for _ in range(T)]) if T else np.zeros((0, TOPK), np.int64)
        hist = torch.from_numpy(np.bincount(ids.reshape(-1), minlength=E).astype(np.int32))
        table = [torch.zeros(E, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(table, hist)                                            # every rank's row of the count table
        table = torch.stack(table).numpy()
        cap = 3 if fault == "overflow" else world * 16 * TOPK
        rc, send_base, counts, offsets, te, ts, tc = plan_host(lib, table, world, rank, cap)
        if fault == "overflow":
            q.put((rank, "rc", rc))
            return
        assert rc == 0
        # dispatch: assignment a goes to row send_base[g] + (its position among this rank's assignments to g)
        cursor = np.zeros(E, np.int64)
        rec = []
        for a, g in enumerate(ids.reshape(-1)):
            rec.append((int(g) // per, int(send_base[g] + cursor[g]), int(g), rank, a))
            cursor[g] += 1
        everyone = [None] * world
        dist.all_gather_object(everyone, rec)
        mine = sorted(r for part in everyone for r in part if r[0] == rank)     # what lands in this owner's buffer, by row
        rows = [r[1] for r in mine]
        ok = rows == list(range(len(rows))) and len(rows) == int(offsets[per])                  # filled exactly once, no gaps
        for e in range(per):
            seg = mine[offsets[e]:offsets[e] + counts[e]]
            ok = ok and all(r[2] == rank * per + e for r in seg)                                   # grouped by expert
            ok = ok and [r[3] for r in seg] == sorted(r[3] for r in seg)                           # source ranks in order
        covered = sorted(x for s, c in zip(ts, tc) for x in range(s, s + c))
        ok = ok and covered == list(range(len(rows))) and all(c <= 64 for c in tc)                # tiles cover the rows
        ok = ok and all(offsets[e] <= s < offsets[e] + max(counts[e], 1) for e, s in zip(te, ts))
        q.put((rank, "ok" if ok else "mismatch", dict(received=len(rows), assignments=len(rec),
                                                      remote=sum(1 for r in rec if r[0] != rank))))
    except Exception as e:  # a peer that failed makes the collective fail on the others
        q.put((rank, "error", type(e).__name__))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(world, fault=None):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fault, q)) for r in range(world)]
    for p in procs:
        p.start()
    import queue as _queue
    import time as _time
    res, deadline = {}, _time.time() + 120
    while len(res) < world and _time.time() < deadline:
        try:
            r, status, info = q.get(timeout=2)
            res[r] = (status, info)
        except _queue.Empty:
            if not any(p.is_alive() for p in procs) and q.empty():
                break  # a rank that left without reporting (fault injection) is not waited for
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.terminate()
    return res


@pytest.mark.parametrize("world", [2, 4])
def test_every_assignment_lands_once_grouped_by_expert(world):
    res = _run(world)
    assert len(res) == world and all(v[0] == "ok" for v in res.values()), res
    assert sum(v[1]["received"] for v in res.values()) == sum(v[1]["assignments"] for v in res.values())
    assert any(v[1]["remote"] > 0 for v in res.values())


def test_a_rank_without_tokens_still_takes_part():
    res = _run(2, fault="empty_rank")
    assert len(res) == 2 and all(v[0] == "ok" for v in res.values()), res
    assert res[0][1]["assignments"] == 0 and res[0][1]["received"] > 0


def test_more_rows_than_the_receive_buffer_holds_is_an_error_code():
    res = _run(2, fault="overflow")
    assert all(v == ("rc", -7) for v in res.values()), res       # BLOK_ERR_ROUTE on every rank, nothing written past the buffer


def test_plan_clamps_counts_a_timed_out_peer_may_have_left():
    """A rank whose wait for a peer's counts gave up may read anything in that peer's row: negative or huge counts must
    not turn into positions outside the buffers."""
    import blok_b200
    lib = blok_b200.load()
    table = np.zeros((2, E), np.int32)
    table[0, :4] = 3
    table[1, 0] = -5
    table[1, 1] = 2 ** 31 - 1
    rc, send_base, counts, offsets, te, ts, tc = plan_host(lib, table, 2, 0, cap=64)
    assert rc == -7                                                  # the huge count overflows the buffer: reported
    assert all(0 <= b <= 64 for b in send_base) and int(offsets[-1]) <= 64
    assert all(s + c <= 64 for s, c in zip(ts, tc))


def test_a_peer_that_left_ends_the_collective_with_an_error_not_a_hang():
    """Host-side failure detection: rank 1 exits between steps; rank 0's next exchange fails within the group timeout."""
    import time
    t0 = time.time()
    res = _run(2, fault="peer_exits")
    assert 0 in res and res[0][0] == "error", res
    assert time.time() - t0 < 90
