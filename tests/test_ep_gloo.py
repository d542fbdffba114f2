"""Expert-parallel dispatch/combine logic among CPU ranks (gloo, world size 2 and 4) with stand-in experts:
the sharded result must equal the single-process result, and routing faults must surface as errors."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

E, TOPK, H = 16, 4, 8


def _weights():
    g = torch.Generator().manual_seed(0)
    return torch.randn(E, H, H, generator=g) * 0.3, torch.randn(E, H, generator=g)


def _router(x, wr):
    s = torch.sigmoid(x @ wr.t())
    wts, ids = torch.topk(s, TOPK, dim=-1)
    return ids, (wts / wts.sum(-1, keepdim=True)).float()


def _expert(rows, e_global, W):
    return torch.einsum("nh,nkh->nk", rows, W[e_global])


def _combine(y, wts, shared):
    out = (y.reshape(wts.shape[0], TOPK, -1) * wts[..., None]).sum(1)
    return out + shared if shared is not None else out


def _single(x, W, wr):
    ids, wts = _router(x, wr)
    y = _expert(x.repeat_interleave(TOPK, 0), ids.reshape(-1), W)
    return _combine(y, wts, x * 0.5)


def _worker(rank, world, port, fault, q):
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    # a short process-group timeout: a peer that is gone must end the survivors' next collective with an error
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    if fault == "peer_exits" and rank == 1:
        dist.barrier()       # the group is up; then this rank leaves between steps, with nothing of its own in flight
        os._exit(0)
    if fault == "peer_exits":
        dist.barrier()
    from blok_b200 import ep
    W, wr = _weights()
    per = E // world
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(5 + 3 * rank, H, generator=g)          # ragged: every rank has a different token count

    def experts_fn(rows, local_e):
        if fault == "short" and rank == 0:
            return rows[:-1] if rows.shape[0] else rows
        return _expert(rows, local_e.long() + rank * per, W)

    def router_fn(xx):
        ids, wts = _router(xx, wr)
        if fault == "bad_id" and rank == 1:
            ids = ids.clone()
            ids[0, 0] = E + 3
        return ids, wts

    layer = ep.ExpertParallelMoe(router_fn, experts_fn, _combine, lambda xx: xx * 0.5, E, TOPK)
    try:
        out = layer.forward(x)
        ok = torch.allclose(out, _single(x, W, wr), atol=1e-5)
        q.put((rank, "ok" if ok else "mismatch", layer.last_stats))
    except ep.RoutingError as e:
        q.put((rank, "routing_error", str(e)))
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
def test_sharded_equals_single_process(world):
    res = _run(world)
    assert len(res) == world and all(v[0] == "ok" for v in res.values()), res
    # every assignment is received exactly once across the ranks
    assert sum(v[1]["received"] for v in res.values()) == sum(v[1]["assignments"] for v in res.values())
    assert any(v[1]["remote"] > 0 for v in res.values())


def test_bad_expert_id_is_reported_on_the_routing_rank():
    res = _run(2, fault="bad_id")
    assert res[1][0] == "routing_error" and "expert id outside" in res[1][1]


def test_short_return_from_experts_is_detected():
    res = _run(2, fault="short")
    assert res[0][0] == "routing_error" and "returned" in res[0][1]


def test_plan_dispatch_properties():
    from blok_b200 import ep
    ids = torch.tensor([[0, 15, 7, 8], [3, 4, 12, 1]])
    order, counts, local = ep.plan_dispatch(ids, 16, 4)
    assert counts.tolist() == [3, 2, 1, 2]
    dest = (ids.reshape(-1) // 4)[order]
    assert torch.equal(dest, torch.sort(dest).values)
    assert torch.equal(local.long(), ids.reshape(-1)[order] % 4)
    with pytest.raises(ep.RoutingError):
        ep.plan_dispatch(ids, 16, 3)
    o2, c2, _ = ep.plan_dispatch(torch.zeros((0, 4), dtype=torch.int64), 16, 4)
    assert o2.numel() == 0 and c2.tolist() == [0, 0, 0, 0]


def test_a_peer_that_left_ends_the_collective_with_an_error_not_a_hang():
    """Host-side failure detection: rank 1 exits between steps; rank 0's next exchange fails within the group timeout."""
    import time
    t0 = time.time()
    res = _run(2, fault="peer_exits")
    assert 0 in res and res[0][0] == "error", res
    assert time.time() - t0 < 90
