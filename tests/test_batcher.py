"""The continuous-batching scheduler (blok_batcher_*) driven by a stand-in for the model: runs without a GPU.

Per sequence the rule is the reference's (src/kimi_exec.cu:885-890): the prompt, then one token per iteration until
EOS (not emitted) or max_new tokens.  The scheduler adds admission in arrival order, a budget of pages that is never
exceeded, and slots that are reused."""
import numpy as np
import pytest

from blok_b200 import lib

EOS = 7


def _serve(b, requests, next_token, page_rows, n_pages):
    """Runs the scheduler to completion with next_token(request, step) as the model.  Returns the emitted tokens per
    request and the trace of (admitted, decoded) per iteration; checks the invariants on the way."""
    rids = [b.submit(len(p), mx) for p, mx in requests]
    assert rids == list(range(len(requests)))
    out = {r: [] for r in rids}
    slot_req, steps, trace, admitted_order = {}, {r: 0 for r in rids}, [], []

    def take(slot):
        r = slot_req[slot]
        tok = next_token(r, steps[r])
        steps[r] += 1
        if tok != EOS:
            out[r].append(tok)
        if b.token(slot, tok == EOS):
            del slot_req[slot]

    for _ in range(10000):
        if b.unfinished == 0:
            break
        admit, decode = b.plan()
        assert admit or decode, "an iteration must make progress"
        assert sorted(decode) == sorted(slot_req), "exactly the running sequences step"
        for slot, r in admit:
            assert slot not in slot_req and 0 <= slot < b.slots
            slot_req[slot] = r
            admitted_order.append(r)
        need = sum(-(-(len(requests[r][0]) + requests[r][1]) // page_rows) for r in slot_req.values())
        assert need == b.committed_pages <= n_pages
        trace.append((list(admit), list(decode)))
        for slot in decode:
            take(slot)
        for slot, _ in admit:
            take(slot)
    assert b.unfinished == 0 and b.waiting == 0 and b.committed_pages == 0 and not slot_req
    assert admitted_order == sorted(admitted_order), "first come, first served"
    return out, trace


def test_every_request_gets_its_own_tokens():
    rng = np.random.default_rng(1)
    requests = [([1] * int(rng.integers(1, 40)), int(rng.integers(1, 12))) for _ in range(23)]
    stop_at = {r: int(rng.integers(0, 14)) for r in range(len(requests))}   # some hit EOS before their budget
    tok = lambda r, i: EOS if i == stop_at[r] else 100 + 16 * r + i
    b = lib.Batcher(slots=4, n_pages=9, page_rows=16, max_ctx=64)
    out, trace = _serve(b, requests, tok, 16, 9)
    for r, (p, mx) in enumerate(requests):
        want = [100 + 16 * r + i for i in range(min(mx, stop_at[r]))]
        assert out[r] == want and b.emitted(r) == len(want)
    assert max(len(d) + len(a) for a, d in trace) > 1, "sequences ran side by side"
    b.close()


def test_admission_waits_for_pages_and_for_slots():
    # four pages of 16 rows, each request needs 2 pages (20 + 4 rows): two run and the third waits, for a slot and pages
    # when there are two slots, for pages alone when there are three
    for slots in (2, 3):
        b = lib.Batcher(slots=slots, n_pages=4, page_rows=16, max_ctx=64)
        for _ in range(3):
            b.submit(20, 4)
        admit, decode = b.plan()
        assert [r for _, r in admit] == [0, 1] and decode == [] and b.waiting == 1 and b.committed_pages == 4
        for slot, _ in admit:
            assert not b.token(slot)
        for it in range(3):                      # tokens 2..4 of both; the last one ends them
            admit, decode = b.plan()
            assert admit == [] and len(decode) == 2
            done = [b.token(s) for s in decode]
            assert done == [it == 2] * 2
        admit, decode = b.plan()
        assert [r for _, r in admit] == [2] and decode == [] and b.committed_pages == 2
        b.close()


def test_a_large_request_blocks_the_queue_behind_it_until_it_fits():
    b = lib.Batcher(slots=4, n_pages=4, page_rows=16, max_ctx=64)
    b.submit(10, 2)      # 1 page
    b.submit(40, 20)     # 4 pages: only fits an empty pool
    b.submit(5, 2)       # 1 page, but may not overtake
    admit, _ = b.plan()
    assert [r for _, r in admit] == [0] and b.waiting == 2
    s0 = admit[0][0]
    assert not b.token(s0)
    admit, decode = b.plan()
    assert admit == [] and decode == [s0]
    assert b.token(s0)                           # second token: request 0 is done
    admit, decode = b.plan()
    assert [r for _, r in admit] == [1] and decode == [] and b.waiting == 1   # request 2 still behind it
    b.close()


def test_requests_that_can_never_run_are_refused_at_submit():
    b = lib.Batcher(slots=2, n_pages=2, page_rows=16, max_ctx=64)
    with pytest.raises(lib.BlokError) as e:
        b.submit(60, 5)                          # longer than the context (:784)
    assert e.value.code == -2
    with pytest.raises(lib.BlokError) as e:
        b.submit(30, 10)                         # 3 pages, the pool has 2
    assert e.value.code == -6
    for bad in ((0, 1), (1, 0)):
        with pytest.raises(lib.BlokError):
            b.submit(*bad)
    assert b.unfinished == 0
    with pytest.raises(lib.BlokError):
        b.token(0)                               # no sequence there
    assert b.plan() == ([], [])
    b.close()


def test_eos_as_first_token_emits_nothing_and_frees_the_slot():
    b = lib.Batcher(slots=1, n_pages=8, page_rows=16, max_ctx=64)
    out, trace = _serve(b, [([1, 2, 3], 5), ([4], 3)], lambda r, i: EOS if r == 0 else 50 + i, 16, 8)
    assert out == {0: [], 1: [50, 51, 52]}
    b.close()
