"""The paged latent cache and the prefill chunk of the MLA block, checked against the dense, token-by-token path
(which the other MLA tests pin to the oracle).  The reference has neither: its KvCache is one contiguous region
(src/kimi_exec.cu:192-238) and its prompt is replayed token by token (:885-886), so the dense decode call IS the
reference behaviour these must reproduce.  Collected after the other GPU tests."""
import numpy as np
import pytest
import torch

import util

pytestmark = pytest.mark.gpu

PAGE = 64


def _paged_copy(cache, table_stride, n_pages, seed, device):
    """Scatters a dense cache [B, ctx, 576] (ctx = table_stride * PAGE) into a pool in a random page order.
    Returns pool [n_pages, PAGE, 576] and the int32 table [B, table_stride]."""
    B, ctx, w = cache.shape
    assert ctx == table_stride * PAGE and n_pages >= B * table_stride
    perm = np.random.default_rng(seed).permutation(n_pages)[:B * table_stride].reshape(B, table_stride)
    table = torch.from_numpy(perm.astype(np.int32)).to(device)
    pool = torch.zeros((n_pages, PAGE, w), dtype=torch.bfloat16, device=device)
    pool[table.long().view(-1)] = cache.view(B * table_stride, PAGE, w)
    return pool, table


@pytest.fixture(scope="module")
def layer16(cuda):
    from blok_b200 import lib, synth
    w = synth.mla_weights(cuda, seed=3, std=0.02)
    return w, lib.MlaLayer(w, yarn_factor=32.0, max_batch=16, max_ctx=8192)


def test_attend_paged_equals_dense(cuda, layer16):
    from blok_b200 import synth
    _, layer = layer16
    seqs, stride = [33, 700, 4097, 64], 65
    cache = synth.latent_cache(len(seqs), stride * PAGE, cuda, seed=21)
    pool, table = _paged_copy(cache, stride, 300, 1, cuda)
    g = torch.Generator(device=cuda).manual_seed(8)
    q = (torch.randn((len(seqs), 64, 576), generator=g, device=cuda) * 0.3).bfloat16()
    seq = torch.tensor(seqs, dtype=torch.int32, device=cuda)
    dense = layer.attend(q, cache, seq)
    paged = layer.attend_paged(q, pool, table, seq)
    assert torch.equal(dense, paged)
    # batch entries in another order than the slots
    order = torch.tensor([2, 0, 3, 1], dtype=torch.int32, device=cuda)
    o2 = layer.attend_paged(q[order.long()].contiguous(), pool, table, seq[order.long()].contiguous(), slot_of=order)
    assert torch.equal(o2, dense[order.long()])


def test_decode_paged_equals_dense(cuda, layer16):
    from blok_b200 import synth
    _, layer = layer16
    ctxs, stride = [40, 130, 63, 64], 4
    B = len(ctxs)
    cache = synth.latent_cache(B, stride * PAGE, cuda, seed=22)
    pool, table = _paged_copy(cache, stride, 40, 2, cuda)
    pool_before = pool.clone()
    n = synth.activations(B, 7168, cuda, 5)
    ctx_len = torch.tensor(ctxs, dtype=torch.int32, device=cuda)
    want = layer.decode(n, cache, ctx_len)
    got = layer.decode_paged(n, pool, table, ctx_len)
    assert torch.equal(got, want)
    changed = torch.zeros(pool.shape[:2], dtype=torch.bool, device=cuda)
    for b, pos in enumerate(ctxs):
        page = int(table[b, pos // PAGE])
        assert torch.equal(pool[page, pos % PAGE], cache[b, pos]), "appended row of sequence %d" % b
        changed[page, pos % PAGE] = True
    assert torch.equal(pool[~changed], pool_before[~changed]), "rows other than the appended ones are untouched"


@pytest.mark.parametrize("T", [11, 16])   # 16 entries and more take the GEMM form of the projections
def test_prefill_chunk_equals_token_by_token(cuda, layer16, T):
    from blok_b200 import synth
    _, layer = layer16
    first, cap = 5, 128
    cache = synth.latent_cache(1, cap, cuda, seed=23)
    seq_cache, chunk_cache = cache.clone(), cache[0].clone()
    n = synth.activations(T, 7168, cuda, 6)
    want = []
    for i in range(T):   # the reference's order: one token, one attention pass (:886)
        pos = torch.tensor([first + i], dtype=torch.int32, device=cuda)
        want.append(layer.decode(n[i:i + 1].contiguous(), seq_cache, pos))
    want = torch.cat(want)
    got = layer.prefill(n, chunk_cache, torch.tensor([first], dtype=torch.int32, device=cuda))
    torch.cuda.synchronize()
    for i in range(T):
        util.assert_close(util.t2np_f32(got[i]), util.t2np_f32(want[i]).astype(np.float64), "prefill token %d" % i)
    util.assert_close(util.t2np_f32(chunk_cache[first:first + T]).ravel(), util.t2np_f32(seq_cache[0, first:first + T]).ravel().astype(np.float64),
                      "appended rows")
    keep = torch.ones(cap, dtype=torch.bool, device=cuda)
    keep[first:first + T] = False
    assert torch.equal(chunk_cache[keep], cache[0][keep])
    # a later token must not see an earlier chunk position's successor: token 0 of the chunk equals a lone decode
    lone = layer.decode(n[:1].contiguous(), cache.clone(), torch.tensor([first], dtype=torch.int32, device=cuda))
    util.assert_close(util.t2np_f32(got[0]), util.t2np_f32(lone[0]).astype(np.float64), "causality of the chunk's first token")


def test_more_than_eight_sequences(cuda, layer16):
    from blok_b200 import synth
    _, layer = layer16
    B, cap = 13, 128
    ctxs = [(7 * b + 3) % 100 for b in range(B)]
    cache = synth.latent_cache(B, cap, cuda, seed=24)
    n = synth.activations(B, 7168, cuda, 7)
    one_call = cache.clone()
    got = layer.decode(n, one_call, torch.tensor(ctxs, dtype=torch.int32, device=cuda))
    for lo, hi in ((0, 8), (8, 13)):
        part = cache[lo:hi].clone()
        want = layer.decode(n[lo:hi].contiguous(), part, torch.tensor(ctxs[lo:hi], dtype=torch.int32, device=cuda))
        for b in range(lo, hi):
            util.assert_close(util.t2np_f32(got[b]), util.t2np_f32(want[b - lo]).astype(np.float64), "sequence %d of 13" % b)
        # 13 entries take one pass of the weight-streaming kernel per projection, 8 and 5 the mat-vec kernel: the appended
        # rows agree within the summation order, every other row is untouched
        for b in range(lo, hi):
            util.assert_close(util.t2np_f32(one_call[b, ctxs[b]]), util.t2np_f32(part[b - lo, ctxs[b]]).astype(np.float64), "appended row %d" % b)
            keep = torch.ones(cap, dtype=torch.bool, device=cuda)
            keep[ctxs[b]] = False
            assert torch.equal(one_call[b][keep], cache[b][keep])


def test_paged_prefill_through_one_slot(cuda, layer16):
    """A prefill chunk on the paged pool: the T batch entries name the same slot with consecutive positions."""
    from blok_b200 import synth
    _, layer = layer16
    first, T, stride = 60, 9, 2   # the chunk crosses from the first page into the second
    cache = synth.latent_cache(1, stride * PAGE, cuda, seed=25)
    pool, table = _paged_copy(torch.cat([cache, cache]), stride, 8, 3, cuda)   # slot 1 holds a copy of the same sequence
    n = synth.activations(T, 7168, cuda, 8)
    dense = cache[0].clone()
    want = layer.prefill(n, dense, torch.tensor([first], dtype=torch.int32, device=cuda))
    slot_of = torch.ones(T, dtype=torch.int32, device=cuda)
    ctx_len = torch.arange(first, first + T, dtype=torch.int32, device=cuda)
    got = layer.decode_paged(n, pool, table, ctx_len, slot_of=slot_of)
    assert torch.equal(got, want)
    for i in range(T):
        pos = first + i
        assert torch.equal(pool[int(table[1, pos // PAGE]), pos % PAGE], dense[pos])


def test_paged_arguments_are_checked(cuda, layer16):
    from blok_b200 import lib
    _, layer = layer16
    n = torch.zeros((1, 7168), dtype=torch.bfloat16, device=cuda)
    table = torch.zeros((1, 2), dtype=torch.int32, device=cuda)
    ctx = torch.zeros(1, dtype=torch.int32, device=cuda)
    with pytest.raises(lib.BlokError):   # page rows must be a multiple of the kernel's 32-row tile
        layer.decode_paged(n, torch.zeros((4, 48, 576), dtype=torch.bfloat16, device=cuda), table, ctx)
    with pytest.raises(lib.BlokError):   # a chunk longer than the handle's max_batch
        layer.prefill(torch.zeros((17, 7168), dtype=torch.bfloat16, device=cuda),
                      torch.zeros((64, 576), dtype=torch.bfloat16, device=cuda), ctx)
    with pytest.raises(lib.BlokError):   # a chunk longer than the cache
        layer.prefill(torch.zeros((9, 7168), dtype=torch.bfloat16, device=cuda),
                      torch.zeros((8, 576), dtype=torch.bfloat16, device=cuda), ctx)


# ---- the whole model: prompt chunks and steps of more than 8 sequences against the oracle's token-by-token run ----

CFGP = dict(layers=3, first_dense=1, hidden=1024, vocab=2048, dense_inter=512, inter=512, experts=128, topk=8,
            shared_inter=512, q_rank=256, max_batch=1, max_ctx=64, yarn_factor=64.0)
MARGIN = 0.02   # a bf16 logit step at this magnitude; closer calls may legitimately flip


@pytest.mark.parametrize("chunk", [8, 24])
def test_model_prefill_matches_token_by_token(cuda, oracle, chunk):
    from blok_b200 import lib
    from test_gpu_model import OracleModel, _sharpen
    model = lib.Model(seed=6, **dict(CFGP, prefill_chunk=chunk))
    _sharpen(model)
    orc = OracleModel(oracle, model)
    prompt = [int(t) for t in np.random.default_rng(chunk).integers(0, CFGP["vocab"], size=29)]   # chunks of 8: 8+8+8+5; of 24: 24+5
    for t in prompt:
        want, margin, _ = orc.step(t)
    got = model.prefill(torch.tensor(prompt, dtype=torch.int32, device=cuda))
    checks = [(int(got[0]), want, margin, "after the prompt")]
    # decode on top of the rows the chunks appended
    ids = torch.tensor([want], dtype=torch.int32, device=cuda)
    for step in range(3):
        nxt = model.step(ids)
        want, margin, _ = orc.step(int(ids[0]))
        checks.append((int(nxt[0]), want, margin, "decode step %d after prefill" % step))
        ids = torch.tensor([want], dtype=torch.int32, device=cuda)
    clear = 0
    for g, w, m, what in checks:
        if m > MARGIN:
            clear += 1
            assert g == w, "%s: got %d want %d (margin %.3f)" % (what, g, w, m)
    assert clear >= 2, "too few decisive samples to judge: %s" % (checks,)
    # generate() takes the same path when the model has a prefill chunk, and the chunked prompt agrees with the replay
    a = model.generate(prompt, 4)
    replay = lib.Model(seed=6, **CFGP)
    _sharpen(replay)
    b = replay.generate(prompt, 4)
    if checks[0][2] > MARGIN:
        assert a[:1] == b[:1] == [checks[0][1]]
    with pytest.raises(lib.BlokError):
        replay.prefill(torch.tensor(prompt, dtype=torch.int32, device=cuda))   # prefill_chunk = 0
    replay.close()
    model.close()


def test_model_steps_twelve_sequences(cuda, oracle):
    from blok_b200 import lib
    from test_gpu_model import OracleModel, _sharpen
    B = 12
    model = lib.Model(seed=7, **dict(CFGP, max_batch=B))
    _sharpen(model)
    orc = OracleModel(oracle, model)
    tok, clear = 11, 0
    for step in range(4):
        nxt = model.step(torch.full((B,), tok, dtype=torch.int32, device=cuda))
        want, margin, _ = orc.step(tok)
        if margin > MARGIN:
            clear += 1
            assert nxt.tolist() == [want] * B, "step %d: got %s want %d (margin %.3f)" % (step, nxt.tolist(), want, margin)
        tok = want
    assert clear >= 2
    with pytest.raises(lib.BlokError):
        model.step(torch.zeros(B + 1, dtype=torch.int32, device=cuda))
    model.close()


# ---- the model over a page pool: the same kernels with another address rule, so the tokens must be identical ----

CFGS = dict(layers=3, first_dense=1, hidden=1024, vocab=2048, dense_inter=512, inter=256, experts=16, topk=8,
            shared_inter=256, q_rank=256, max_batch=3, max_ctx=64, yarn_factor=64.0)


def _ids(values, device):
    return torch.tensor(values, dtype=torch.int32, device=device)


def test_paged_model_equals_dense_model(cuda):
    from blok_b200 import lib
    from test_gpu_model import _sharpen
    dense = lib.Model(seed=8, **CFGS)
    paged = lib.Model(seed=8, **dict(CFGS, kv_page_rows=32, kv_pages=6))
    _sharpen(dense)
    _sharpen(paged)
    assert paged.free_pages == 6 and dense.free_pages == -1
    ids = _ids([5, 900, 77], cuda)
    for _ in range(5):
        a, b = dense.step(ids), paged.step(ids)
        assert torch.equal(a, b)
        ids = a
    assert paged.free_pages == 3 and [paged.slot_length(s) for s in range(3)] == [5, 5, 5]
    # a subset of the resident sequences, in another order
    a = dense.step(ids)
    b = paged.step_slots([2, 0], ids[[2, 0]].contiguous())
    assert torch.equal(b, a[[2, 0]])
    assert [paged.slot_length(s) for s in range(3)] == [6, 5, 6]
    # the sequence in slot 1 ends, another one starts there: it must behave like a fresh sequence
    paged.release_slot(1)
    assert paged.free_pages == 4 and paged.slot_length(1) == 0
    fresh = lib.Model(seed=8, **dict(CFGS, max_batch=1))
    _sharpen(fresh)
    tok = _ids([1234], cuda)
    for _ in range(3):
        want, got = fresh.step(tok), paged.step_slots([1], tok)
        assert torch.equal(want, got)
        tok = want
    with pytest.raises(lib.BlokError):
        paged.step_slots([0, 0], _ids([1, 2], cuda))        # a slot twice
    with pytest.raises(lib.BlokError):
        dense.step_slots([1, 0], _ids([1, 2], cuda))        # a dense cache has no slot indirection
    for m in (dense, paged, fresh):
        m.close()


def test_paged_model_pool_exhaustion_is_an_error_not_a_fault(cuda):
    from blok_b200 import lib
    model = lib.Model(seed=9, **dict(CFGS, kv_page_rows=32, kv_pages=4))
    ids = _ids([1, 2, 3], cuda)
    for _ in range(32):                     # every sequence fills its first page
        ids = model.step(ids)
    assert model.free_pages == 1
    with pytest.raises(lib.BlokError) as e:  # three sequences need a second page, one is left
        model.step(ids)
    assert e.value.code == -6
    assert [model.slot_length(s) for s in range(3)] == [32, 32, 32]   # nothing was launched, nothing advanced
    model.release_slot(2)
    nxt = model.step_slots([0, 1], ids[:2].contiguous())
    assert nxt.shape == (2,) and [model.slot_length(s) for s in range(3)] == [33, 33, 0]
    with pytest.raises(lib.BlokError) as e:  # max_ctx bounds a sequence as the reference's capacity check does (:205)
        for _ in range(40):
            nxt = model.step_slots([0], nxt[:1].contiguous())
    assert e.value.code == -2 and model.slot_length(0) == 64
    model.reset()
    assert model.free_pages == 4 and model.slot_length(0) == 0
    model.close()


def test_paged_model_prefill_equals_dense_prefill(cuda):
    from blok_b200 import lib
    from test_gpu_model import _sharpen
    dense = lib.Model(seed=10, **dict(CFGS, max_batch=1, prefill_chunk=8))
    paged = lib.Model(seed=10, **dict(CFGS, prefill_chunk=8, kv_page_rows=32, kv_pages=5))
    _sharpen(dense)
    _sharpen(paged)
    prompt = _ids([int(t) for t in np.random.default_rng(3).integers(0, CFGS["vocab"], size=37)], cuda)  # crosses into a second page
    a, b = dense.prefill(prompt), paged.prefill_slot(2, prompt)
    assert torch.equal(a, b) and paged.slot_length(2) == 37 and paged.free_pages == 3
    for _ in range(3):
        a, b = dense.step(a), paged.step_slots([2], b)
        assert torch.equal(a, b)
    with pytest.raises(lib.BlokError):
        paged.prefill_slot(0, _ids(list(range(65)), cuda))   # longer than max_ctx
    with pytest.raises(lib.BlokError):
        dense.prefill_slot(1, prompt)
    dense.close()
    paged.close()


def test_generate_many_serves_every_request_like_generate_alone(cuda):
    from blok_b200 import lib
    from test_gpu_model import _sharpen
    alone = lib.Model(seed=11, **dict(CFGS, max_batch=1, prefill_chunk=8))
    many = lib.Model(seed=11, **dict(CFGS, prefill_chunk=8, kv_page_rows=32, kv_pages=4))   # 3 slots, pages for 2-4 requests
    _sharpen(alone)
    _sharpen(many)
    rng = np.random.default_rng(5)
    prompts = [[int(t) for t in rng.integers(0, CFGS["vocab"], size=n)] for n in (3, 17, 9, 30, 1, 12, 5)]
    want = [alone.generate(p, 5) for p in prompts]
    got = many.generate_many(prompts, 5)
    assert len(got) == len(prompts) and many.free_pages == 4
    # the prompt goes through the same kernels in both models, so the first token is the same id; later tokens come
    # from steps of 1 sequence there and of up to 3 here (another summation order in the mat-vecs): a near tie may flip
    assert [g[:1] for g in got] == [w[:1] for w in want]
    assert all(1 <= len(g) <= 5 and all(0 <= t < CFGS["vocab"] for t in g) for g in got)
    assert sum(g == w for g, w in zip(got, want)) >= len(prompts) - 2
    assert many.generate_many(prompts, 5) == got, "deterministic"
    with pytest.raises(lib.BlokError):
        alone.generate_many(prompts, 5)        # needs the page pool
    with pytest.raises(lib.BlokError):
        many.generate_many([[1] * 60], 5)      # longer than max_ctx
    alone.close()
    many.close()


def test_cli_prefill_chunk_flag_runs_the_prompt_in_chunks():
    import json
    from test_cli import run, EXE
    from blok_b200 import build
    build.build()
    exe = EXE
    args = ["--index", "unused", "--prompt-tokens", "5,6,7,8,9,10,11", "--tokens", "3", "--synthetic-seed", "1", "--layers", "2",
            "--experts", "16", "--vocab", "4096"]
    replay, chunks = run(exe, *args), run(exe, *args, "--prefill-chunk", "4")
    assert replay.returncode == 0 and chunks.returncode == 0, (replay.stderr, chunks.stderr)
    a, b = json.loads(replay.stdout)["token_ids"], json.loads(chunks.stdout)["token_ids"]
    assert 1 <= len(b) <= 3 and all(0 <= t < 4096 for t in b) and len(a) == len(b)
    p = run(exe, *args, "--prefill-chunk", "65")
    assert p.returncode == 1 and "unsupported configuration" in p.stderr
