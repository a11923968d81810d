"""Training on CPU ranks over gloo: the FSDP (and FSDP x CP) step must reproduce the single-process
AdamW step on the same global batch; checkpoint/resume must continue bit-identically."""
import torch

from tests.dist_utils import run_ranks


def _cfg():
    from cosmos_b200.config import tiny_config
    return tiny_config(n_layers=2, d_model=128, n_heads=4, n_kv_heads=2, head_dim=32, ffn_dim=256, vocab_size=512,
                       mrope_section=(6, 5, 5), max_text_len=16)


def _data(n_clips):
    g = torch.Generator().manual_seed(11)
    lat = torch.randn(n_clips, 16, 3, 8, 8, generator=g)
    ids = torch.randint(0, 512, (n_clips, 16), generator=g)
    t = torch.rand(n_clips, generator=g)
    eps = torch.randn(lat.shape, generator=g)
    return lat, ids, t, eps


def _worker(rank, world, pc_kw, steps, save_dir=None, resume=False, extra_steps=0):
    from cosmos_b200.config import ParallelConfig
    from cosmos_b200.models.mot import MoTModel
    from cosmos_b200.parallel.mesh import Mesh
    from cosmos_b200.train import TrainConfig, Trainer

    pc = ParallelConfig(**pc_kw)
    shard_ws = pc.dp_shard * pc.cp
    model = MoTModel(_cfg(), pad_to=128 * shard_ws)
    model.init_weights(seed=3)
    mesh = Mesh(pc, world, rank)
    tr = Trainer(model, mesh, TrainConfig(lr=1e-3, max_grad_norm=0.5, fused=False))
    n_dp = pc.dp_shard * pc.dp_replicate
    lat, ids, t, eps = _data(2)
    # one clip per data-parallel rank (replica-major, as train.py shards the data)
    d = (mesh.index("dp_replicate") * pc.dp_shard + mesh.index("dp_shard")) if n_dp > 1 else slice(None)
    lat, ids, t, eps = _data(max(2, n_dp))
    sel = slice(d, d + 1) if isinstance(d, int) else d
    start = 0
    if resume:
        start = tr.load(save_dir)
    logs = []
    for s in range(start, steps + extra_steps):
        out = tr.train_step(lat[sel], ids[sel], t=t[sel], eps=eps[sel])
        logs.append(out)
        if save_dir and not resume and s + 1 == steps:
            tr.save(save_dir, steps)
            break
    full = tr.fsdp.full_state()
    return {k: v.clone() for k, v in full.items()}, logs


def test_fsdp_step_matches_single_process():
    want, logs1 = _worker(0, 1, {}, 2)
    outs = run_ranks(_worker, 2, dict(dp_shard=2), 2)
    for got, logs in outs:
        for k in want:
            assert torch.allclose(got[k], want[k], atol=2e-5), (k, (got[k] - want[k]).abs().max())
        assert abs(logs[0]["loss"] - logs1[0]["loss"]) < 1e-5
        assert abs(logs[0]["grad_norm"] - logs1[0]["grad_norm"]) < 1e-4


def test_fsdp_x_cp_matches_single_process():
    want, _ = _worker(0, 1, {}, 1)
    outs = run_ranks(_worker, 4, dict(dp_shard=2, cp=2), 1)
    for got, _ in outs:
        for k in want:
            assert torch.allclose(got[k], want[k], atol=3e-5), (k, (got[k] - want[k]).abs().max())


def test_replicas_average_their_gradients_and_stay_identical():
    """dp_replicate 2 x dp_shard 2: four ranks, four clips. Each replica pair holds the same shards; their gradients
    are averaged over the replicate axis at the optimizer step, so after two steps the replicas are bit-equal and
    equal the single-process step on the four-clip batch."""
    outs = run_ranks(_worker, 4, dict(dp_replicate=2, dp_shard=2), 2)
    (a0, l0), (a1, _), (b0, _), (b1, _) = outs        # ranks 0, 1 = replica 0; ranks 2, 3 = replica 1
    for k in a0:
        assert torch.equal(a0[k], b0[k]) and torch.equal(a1[k], b1[k]), k
    from cosmos_b200.config import ParallelConfig
    from cosmos_b200.models.mot import MoTModel
    from cosmos_b200.parallel.mesh import Mesh
    from cosmos_b200.train import TrainConfig, Trainer
    model = MoTModel(_cfg(), pad_to=128)
    model.init_weights(seed=3)
    tr = Trainer(model, Mesh(ParallelConfig(), 1, 0), TrainConfig(lr=1e-3, max_grad_norm=0.5, fused=False))
    lat, ids, t, eps = _data(4)
    for _ in range(2):
        log = tr.train_step(lat, ids, t=t, eps=eps)
    want = tr.fsdp.full_state()
    for k in want:
        assert torch.allclose(a0[k], want[k], atol=3e-5), (k, (a0[k] - want[k]).abs().max())
    assert abs(l0[-1]["grad_norm"] - log["grad_norm"]) < 1e-4


def test_checkpoint_resume_continues_identically(tmp_path):
    straight, _ = _worker(0, 1, {}, 3)
    _worker(0, 1, {}, 2, str(tmp_path))
    resumed, _ = _worker(0, 1, {}, 2, str(tmp_path), True, 1)
    for k in straight:
        assert torch.equal(resumed[k], straight[k]), k


def test_gradient_accumulation_equals_the_larger_batch_and_the_schedule_sets_the_rate():
    """Two micro-batches of one clip with grad_accum = 2 give the optimizer step of one batch of two clips; the
    learning rate of each optimizer step follows warm-up + cosine."""
    import math

    from cosmos_b200.config import ParallelConfig
    from cosmos_b200.models.mot import MoTModel
    from cosmos_b200.parallel.mesh import Mesh
    from cosmos_b200.train import TrainConfig, Trainer

    lat, ids, t, eps = _data(2)

    def run(accum):
        model = MoTModel(_cfg(), pad_to=128)
        model.init_weights(seed=3)
        tc = TrainConfig(lr=1e-3, max_grad_norm=0.5, fused=False, grad_accum=accum, warmup_steps=2, total_steps=6, min_lr_ratio=0.1)
        tr = Trainer(model, Mesh(ParallelConfig(), 1, 0), tc)
        logs = []
        for _ in range(3):                                   # three optimizer steps
            if accum == 1:
                logs.append(tr.train_step(lat, ids, t=t, eps=eps))
            else:
                first = tr.train_step(lat[:1], ids[:1], t=t[:1], eps=eps[:1])
                assert "grad_norm" not in first and "lr" not in first        # no step yet
                logs.append(tr.train_step(lat[1:], ids[1:], t=t[1:], eps=eps[1:]))
        return {k: v.clone() for k, v in tr.fsdp.full_state().items()}, logs

    (a, la), (b, lb) = run(1), run(2)
    assert [round(x["lr"], 9) for x in la] == [round(x["lr"], 9) for x in lb] == [0.0005, 0.001, round(1e-3 * (0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi / 4))), 9)]
    assert all(abs(x["grad_norm"] - y["grad_norm"]) < 1e-4 * max(1.0, x["grad_norm"]) for x, y in zip(la, lb))
    for k in a:
        assert torch.allclose(a[k], b[k], atol=2e-6, rtol=1e-5), k
    tc = TrainConfig(lr=2.0, warmup_steps=4, total_steps=12, min_lr_ratio=0.25)
    assert tc.lr_at(1) == 0.5 and tc.lr_at(4) == 2.0 and abs(tc.lr_at(8) - 2.0 * (0.25 + 0.75 * 0.5)) < 1e-12
    assert abs(tc.lr_at(12) - 0.5) < 1e-12 and abs(tc.lr_at(40) - 0.5) < 1e-12
    assert TrainConfig(lr=3.0).lr_at(7) == 3.0
