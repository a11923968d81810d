"""Continuous batching: requests of different lengths join and leave the decode batch at different
times; every token the engine emits must be the (near-)arg-max of the reference engine's logits when
that engine is fed the same prefix (teacher forcing keeps near-ties from cascading)."""
import torch

from cosmos_b200 import ops
from cosmos_b200.config import tiny_config
from cosmos_b200.models import rope
from cosmos_b200.models.mot import MoTModel
from cosmos_b200.models.reasoner import ReasonerEngine
from cosmos_b200.serve.engine import BatchEngine, EngineWorker


def _model():
    torch.manual_seed(0)
    cfg = tiny_config(n_layers=2, vocab_size=300)
    m = MoTModel(cfg, dtype=torch.float32, device="cpu")
    m.init_weights(seed=11)
    return m


def _check_against_reference(model, req):
    ref = ReasonerEngine(model)
    ids = torch.tensor([req.ids], dtype=torch.long)
    logits, kvs = ref.prefill(ref.embed(ids), rope.text_positions(len(req.ids), 0, "cpu"))
    pos = len(req.ids)
    for tok in req.out:
        lg = logits[0]
        assert lg[tok] >= lg.max() - 1e-3, (req.rid, tok, float(lg[tok]), float(lg.max()))
        logits, kvs = ref.decode_one(torch.tensor([tok]), pos, kvs)
        pos += 1


def test_requests_join_and_leave_the_running_batch():
    model = _model()
    eng = BatchEngine(model, max_batch=3, max_len=64, page_size=4, use_graph=False)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 300, (n,), generator=g).tolist() for n in (5, 9, 3, 12, 7)]
    budgets = [6, 4, 8, 4, 5]
    reqs = [eng.submit(prompts[0], budgets[0]), eng.submit(prompts[1], budgets[1])]
    eng.step()
    assert eng.n_active() == 2 and not eng.waiting
    reqs += [eng.submit(prompts[2], budgets[2]), eng.submit(prompts[3], budgets[3])]   # only one slot is free
    eng.step()
    assert eng.n_active() == 3 and len(eng.waiting) == 1
    reqs.append(eng.submit(prompts[4], budgets[4]))
    eng.run_until_done(max_steps=100)
    assert not eng.has_work() and eng.n_active() == 0
    for r, b in zip(reqs, budgets):
        assert r.finish_reason == "length" and len(r.out) == b
        _check_against_reference(model, r)
    # all pages went back to the pool (the scratch page stays reserved)
    alloc = eng.dec.cache.alloc
    assert alloc.num_free() == eng.max_batch * eng.max_pages + 1 - 1
    # fewer engine steps than running the requests one after the other would need
    assert eng.steps < sum(budgets) - len(budgets)


def test_end_token_retires_a_request_and_page_shortage_defers_admission():
    model = _model()
    eng = BatchEngine(model, max_batch=2, max_len=32, page_size=4, use_graph=False)
    probe = eng.submit([1, 2, 3, 4], 6)
    eng.run_until_done()
    eos = probe.out[2]                      # the third token of this prompt becomes the end token
    r = eng.submit([1, 2, 3, 4], 6, eos_ids=(eos,))
    eng.run_until_done()
    assert r.finish_reason == "stop" and r.out == probe.out[:r.out.index(eos) + 1]
    # a request that needs more pages than are free right now waits, it is not dropped
    small = BatchEngine(model, max_batch=2, max_len=32, page_size=4, use_graph=False)
    while small.dec.cache.alloc.num_free() > 9:      # leave 9 pages = 36 tokens
        assert small.dec.cache.reserve(-100 - small.dec.cache.alloc.num_free(), 4)
    a = small.submit(list(range(10)), 14)            # 24 tokens = 6 pages
    b = small.submit(list(range(8)), 12)             # 20 tokens = 5 pages: does not fit next to a
    small.step()
    assert small.n_active() == 1 and len(small.waiting) == 1
    small.run_until_done()
    assert len(a.out) == 14 and len(b.out) == 12


def test_worker_thread_serves_concurrent_callers():
    model = _model()
    worker = EngineWorker(BatchEngine(model, max_batch=4, max_len=48, page_size=4, use_graph=False))
    try:
        futs = [worker.submit([i + 1, i + 2, i + 3], 5) for i in range(6)]
        outs = [f.result(timeout=120) for f in futs]
        assert all(len(r.out) == 5 for r in outs)
        for r in outs:
            _check_against_reference(model, r)
    finally:
        worker.close()


def test_device_side_sampling_follows_the_truncated_softmax():
    """Top-k / top-p sampling inside the decode step: over many draws the frequencies match the softmax of
    the kept candidates, tokens outside top-k or beyond the top-p mass never appear, and top_k = 1 is greedy."""
    from cosmos_b200.serve.decoder import TPDecoder

    cfg = tiny_config(n_layers=1, vocab_size=300)
    dec = TPDecoder(cfg, 1, 0, None, "cpu", page_size=4, max_batch=4, max_len=16, dtype=torch.float32)
    dec.enable_sampling(4)
    sp = dec.sampling
    logits = torch.full((4, 300), -20.0)
    base = torch.tensor([2.0, 1.5, 1.0, 0.5, 0.0, -0.5])
    logits[:, 10:16] = base
    sp["temperature"][:] = torch.tensor([1.0, 1.0, 0.0, 0.7])
    sp["top_k"][:] = torch.tensor([3, 64, 5, 1])
    sp["top_p"][:] = torch.tensor([1.0, 0.6, 1.0, 1.0])
    g = torch.Generator().manual_seed(0)
    n = 4000
    counts = torch.zeros(4, 300)
    dec.tokens = torch.zeros(4, dtype=torch.long)             # no penalties set: the seen flags change nothing
    dec.next_tokens = torch.zeros(4, dtype=torch.long)
    for _ in range(n):
        dec.refill_noise(g)
        tok = dec._sample(logits)
        counts[torch.arange(4), tok] += 1
    f = counts / n
    want0 = torch.softmax(base[:3], -1)                       # slot 0: top_k = 3
    assert torch.allclose(f[0, 10:13], want0, atol=0.03) and f[0, 13:].sum() == 0
    p = torch.softmax(base, -1)                               # slot 1: top_p = 0.6 keeps tokens while the mass before them < 0.6
    kept = (torch.cumsum(p, 0) - p) < 0.6
    want1 = torch.where(kept, p, torch.zeros_like(p))
    want1 = want1 / want1.sum()
    assert torch.allclose(f[1, 10:16], want1, atol=0.03)
    assert f[2, 10] == 1.0 and f[3, 10] == 1.0                # temperature 0 and top_k = 1 are greedy
    # presence / repetition penalties act on seen tokens only
    dec.tokens = torch.tensor([10, 11, 12, 13])
    sp["presence"][:] = torch.tensor([1.5, 0.0, 0.0, 0.0])
    sp["repetition"][:] = torch.tensor([1.0, 2.0, 1.0, 1.0])
    sp["seen_any"].zero_()
    sp["seen_out"].zero_()
    cand = ops.sample_topk(logits.clone(), sp["seen_any"], sp["seen_out"], dec.tokens, sp["presence"], sp["repetition"], 0)
    vals, ids = cand[..., 0], cand[..., 1].contiguous().view(torch.int32)

    def val(b, tok):
        return vals[b][ids[b] == tok]

    assert torch.isclose(val(0, 10), torch.tensor(0.5)) and torch.isclose(val(1, 11), torch.tensor(0.75))
    assert torch.isclose(val(2, 12), torch.tensor(1.0)) and torch.isclose(val(1, 10), torch.tensor(2.0))
    assert sp["seen_out"][0, 10] and sp["seen_any"][3, 13] and sp["seen_out"].sum() == 4
    assert torch.equal(ids[2, :6].long(), torch.arange(10, 16))   # best first


def test_sampled_requests_run_through_the_engine():
    model = _model()
    eng = BatchEngine(model, max_batch=3, max_len=48, page_size=4, use_graph=False)
    a = eng.submit([5, 6, 7], 8, temperature=0.8, top_k=20, top_p=0.9, presence_penalty=1.5)
    b = eng.submit([5, 6, 7], 8)                              # greedy neighbour in the same batch
    eng.run_until_done()
    assert len(a.out) == 8 and len(b.out) == 8
    _check_against_reference(model, b)                        # the sampled neighbour does not disturb it


def test_request_with_vision_embeddings_joins_the_batch():
    """A prompt with a vision grid (3-D rotary ids, DeepStack features) is prefilled on its own and then
    decodes in the same batch as text requests; its tokens follow the single-request engine's logits."""
    from cosmos_b200.models.vit import VisionEncoder

    torch.manual_seed(0)
    cfg = tiny_config(n_layers=2, vocab_size=300, vit_deepstack=(0,))
    model = MoTModel(cfg, dtype=torch.float32, device="cpu")
    model.init_weights(seed=11)
    vit = VisionEncoder(cfg).float().eval()
    with torch.no_grad():
        emb, grid, deep = vit(torch.rand(2, 3, 64, 64) * 2 - 1, return_deepstack=True)
    n_vis = grid[0] * grid[1] * grid[2]
    pad = 299
    ids = [5, 6] + [pad] * n_vis + [7, 8, 9]
    ref = ReasonerEngine(model, vit)
    ids_t = torch.tensor([ids])
    vmask = ids_t == pad
    x = ref.embed(ids_t, emb, vmask)
    pos = ref.positions(ids_t, vmask, [grid])
    assert rope.next_start(pos) < len(ids)               # the grid advances the ids slower than one per token

    eng = BatchEngine(model, max_batch=3, max_len=64, page_size=4, use_graph=False)
    text = eng.submit([1, 2, 3, 4], 6)
    vis = eng.submit(ids, 6, embeds=x[0], positions=pos, vision_mask=vmask[0], deepstack=deep)
    eng.run_until_done()
    assert len(vis.out) == 6 and len(text.out) == 6
    _check_against_reference(model, text)
    logits, kvs = ref.prefill(x, pos, deep, vmask)
    p = rope.next_start(pos)
    for tok in vis.out:
        lg = logits[0]
        assert lg[tok] >= lg.max() - 1e-3, (tok, float(lg[tok]), float(lg.max()))
        logits, kvs = ref.decode_one(torch.tensor([tok]), p, kvs)
        p += 1


def _tp_engine_ranks(rank, world):
    """Both ranks build the same model; rank 0 submits, rank 1 follows; returns what each rank decoded."""
    import torch.distributed as dist

    model = _model()
    eng = BatchEngine(model, max_batch=3, max_len=48, page_size=4, use_graph=False, group=dist.group.WORLD)
    if rank == 0:
        a = eng.submit([5, 9, 2, 7, 1], 6)
        b = eng.submit([3, 3, 8], 5)
        eng.step()
        c = eng.submit([4, 4, 4, 4, 9, 1, 2], 4, temperature=0.9, top_k=10, top_p=0.9, presence_penalty=1.0)
        d = eng.submit([8, 6], 5)                       # waits for a free slot
        eng.run_until_done()
        eng.shutdown()
        reqs = [a, b, c, d]
    else:
        eng.follow()
        reqs = [eng.finished[i] for i in sorted(eng.finished)]
    return {"outs": [r.out for r in reqs], "ids": [r.ids for r in reqs], "free": eng.dec.cache.alloc.num_free()}


def test_tensor_parallel_engine_runs_in_lock_step_over_gloo():
    from tests.dist_utils import run_ranks

    out = run_ranks(_tp_engine_ranks, 2, timeout=180)
    assert out[0]["outs"] == out[1]["outs"] and out[0]["ids"] == out[1]["ids"]      # followers mirror rank 0
    assert [len(o) for o in out[0]["outs"]] == [6, 5, 4, 5]
    assert out[0]["free"] == out[1]["free"]
    model = _model()
    for ids, toks, greedy in zip(out[0]["ids"], out[0]["outs"], [True, True, False, True]):
        if greedy:                                       # greedy requests follow the single-process reference
            from types import SimpleNamespace
            _check_against_reference(model, SimpleNamespace(ids=ids, out=toks, rid=0))


def _tp_engine_media_ranks(rank, world):
    """Rank 0 encodes an image and submits the request with its embeddings; the follower receives them with the
    request and mirrors prefill and decode."""
    import torch.distributed as dist
    from cosmos_b200.models.vit import VisionEncoder

    torch.manual_seed(0)
    cfg = tiny_config(n_layers=2, vocab_size=300, vit_deepstack=(0,))
    model = MoTModel(cfg, dtype=torch.float32, device="cpu")
    model.init_weights(seed=11)
    eng = BatchEngine(model, max_batch=2, max_len=64, page_size=4, use_graph=False, group=dist.group.WORLD)
    if rank == 0:
        vit = VisionEncoder(cfg).float().eval()
        with torch.no_grad():
            emb, grid, deep = vit(torch.rand(1, 3, 64, 64) * 2 - 1, return_deepstack=True)
        n_vis = grid[0] * grid[1] * grid[2]
        ids = [5, 6] + [299] * n_vis + [7, 8]
        ref = ReasonerEngine(model, vit)
        ids_t = torch.tensor([ids])
        vmask = ids_t == 299
        x = ref.embed(ids_t, emb, vmask)
        pos = ref.positions(ids_t, vmask, [grid])
        text = eng.submit([1, 2, 3], 4)
        vis = eng.submit(ids, 5, embeds=x[0], positions=pos, vision_mask=vmask[0], deepstack=deep)
        eng.run_until_done()
        eng.shutdown()
        logits, kvs = ref.prefill(x, pos, deep, vmask)      # the single-request engine as the oracle
        p = rope.next_start(pos)
        for tok in vis.out:
            assert logits[0][tok] >= logits[0].max() - 1e-3
            logits, kvs = ref.decode_one(torch.tensor([tok]), p, kvs)
            p += 1
        reqs = [text, vis]
    else:
        eng.follow()
        reqs = [eng.finished[i] for i in sorted(eng.finished)]
    return {"outs": [r.out for r in reqs], "had_media": [r.embeds is not None for r in reqs]}


def test_tensor_parallel_engine_serves_a_request_with_media():
    from tests.dist_utils import run_ranks

    out = run_ranks(_tp_engine_media_ranks, 2, timeout=180)
    assert out[0]["outs"] == out[1]["outs"] and [len(o) for o in out[0]["outs"]] == [4, 5]
    assert out[0]["had_media"] == out[1]["had_media"] == [False, True]


def test_a_callback_that_returns_false_retires_the_request():
    """Stop strings are detected by the caller's token callback; returning False ends the request at that token and
    frees its slot and pages, while its neighbours in the batch carry on."""
    model = _model()
    eng = BatchEngine(model, max_batch=2, max_len=48, page_size=4, use_graph=False)
    free0 = eng.dec.cache.alloc.num_free()
    got = []
    a = eng.submit([5, 9, 2, 7, 1], 10, on_token=lambda t: (got.append(t), len(got) < 3)[1])
    b = eng.submit([3, 3, 8], 6)
    eng.run_until_done()
    assert len(a.out) == 3 and a.finish_reason == "stop" and got == a.out
    assert len(b.out) == 6 and b.finish_reason == "length"
    assert eng.dec.cache.alloc.num_free() == free0
    _check_against_reference(model, b)


def test_sampling_over_vocabulary_shards_equals_sampling_over_the_whole_vocabulary():
    """`ops.sample_topk` per shard + `ops.sample_pick` over the gathered candidates (what tensor-parallel ranks do)
    draws the same tokens as one shard holding the whole vocabulary: same candidates after the merge, same noise."""
    g = torch.Generator().manual_seed(5)
    b, v, shards = 6, 1000, 4
    logits = torch.randn(b, v, generator=g) * 3
    seen_any = torch.rand(b, v, generator=g) < 0.2
    seen_out = seen_any & (torch.rand(b, v, generator=g) < 0.5)
    tokens = torch.randint(0, v, (b,), generator=g)
    pres, rep = torch.rand(b, generator=g), 1 + torch.rand(b, generator=g)
    temp = torch.tensor([0.0, 0.5, 1.0, 0.8, 1.3, 0.0])
    top_k = torch.tensor([5, 64, 10, 3, 40, 1])
    top_p = torch.tensor([1.0, 0.9, 0.5, 1.0, 0.7, 1.0])
    noise = torch.rand(b, 64, generator=g).clamp_min(1e-7)
    whole = ops.sample_topk(logits, seen_any.clone(), seen_out.clone(), tokens, pres, rep, 0)
    want = ops.sample_pick(whole, 1, temp, top_k, top_p, noise, v, torch.empty(b, dtype=torch.long))
    vl = v // shards
    parts = []
    for r in range(shards):
        sl = slice(r * vl, (r + 1) * vl)
        parts.append(ops.sample_topk(logits[:, sl].contiguous(), seen_any[:, sl].contiguous(), seen_out[:, sl].contiguous(),
                                     tokens, pres, rep, r * vl))
    got = ops.sample_pick(torch.cat(parts, 0), shards, temp, top_k, top_p, noise, v, torch.empty(b, dtype=torch.long))
    assert torch.equal(got, want)
    assert got[0] == whole[0, 0, 1].view(torch.int32) and got[5] == whole[5, 0, 1].view(torch.int32)   # greedy rows


def test_sample_topk_definition_pads_small_shards_and_takes_no_flags():
    logits = torch.tensor([[0.5, 3.0, -1.0, 2.0]])
    cand = ops.sample_topk(logits, None, None, None, None, None, 100)
    vals, ids = cand[0, :, 0], cand[0, :, 1].contiguous().view(torch.int32)
    assert cand.shape == (1, 64, 2)
    assert vals[:4].tolist() == [3.0, 2.0, 0.5, -1.0] and ids[:4].tolist() == [101, 103, 100, 102]
    assert torch.isinf(vals[4:]).all() and (vals[4:] < 0).all()
    out = ops.sample_pick(cand, 1, torch.tensor([1.0]), torch.tensor([64]), torch.tensor([1.0]),
                          torch.full((1, 64), 0.5), 1000, torch.empty(1, dtype=torch.long))
    assert out.item() == 101      # equal noise: the most likely candidate wins; padded entries never do
