"""Parallel strategies on CPU ranks over gloo (world_size 2 and 4) against the single-process result."""
import pytest
import torch

from tests.dist_utils import run_ranks


def _gen_worker(rank, world, pc_kw, steps):
    from cosmos_b200.config import ParallelConfig, SamplingConfig, tiny_config
    from cosmos_b200.models.mot import MoTModel
    from cosmos_b200.parallel.mesh import Mesh
    from cosmos_b200.parallel.runtime import build_engine_for_mesh
    from cosmos_b200.pipeline import Cosmos3OmniPipeline

    torch.manual_seed(0)
    cfg = tiny_config(n_layers=2, max_text_len=16)
    model = MoTModel(cfg)
    model.init_weights(seed=5)
    mesh = Mesh(ParallelConfig(**pc_kw), world, rank)
    eng = build_engine_for_mesh(model, mesh, fused=False)
    g = torch.Generator().manual_seed(1)
    ids_c = torch.randint(0, cfg.vocab_size, (1, 16), generator=g)
    ids_u = torch.randint(0, cfg.vocab_size, (1, 16), generator=g)
    st = eng.make_state(ids_c, ids_u, (3, 8, 8))
    sc = SamplingConfig(num_steps=steps, guidance=5.0, shift=3.0, seed=2)
    pipe = Cosmos3OmniPipeline(model, None, None, None, engine=eng)
    x = pipe.begin(st, sc)
    for i in range(steps):
        x = pipe.step(x, i)
    return pipe.gather_tokens(x, st)


def _single(steps):
    from cosmos_b200.config import ParallelConfig
    return _gen_worker(0, 1, {}, steps)


@pytest.mark.parametrize("world,pc", [(2, dict(cp=2)), (2, dict(cfgp=2)), (4, dict(cfgp=2, cp=2)),
                                      (2, dict(cp=2, cp_mode="ring")), (2, dict(tp=2)), (4, dict(cfgp=2, tp=2))])
def test_generator_parallel_matches_single(world, pc):
    want = _single(2)
    outs = run_ranks(_gen_worker, world, pc, 2)
    for o in outs:
        assert o.shape == want.shape
        assert torch.allclose(o, want, atol=2e-5), (o - want).abs().max()


def test_mesh_layout_and_presets():
    from cosmos_b200.config import ParallelConfig, preset_parallelism
    from cosmos_b200.parallel.mesh import Mesh

    m = Mesh(ParallelConfig(dp_shard=2, cp=2, tp=2), 8, 5, create_groups=False)
    assert m.coords["dp_shard"] == 1 and m.coords["cp"] == 0 and m.coords["tp"] == 1
    assert m.group_ranks["tp"] == [4, 5] and m.group_ranks["cp"] == [5, 7] and m.group_ranks["dp_shard"] == [1, 5]
    with pytest.raises(ValueError):
        ParallelConfig(cp=3).validate(8)
    lat = preset_parallelism("latency", 8)
    assert (lat.cfgp, lat.cp, lat.cp_mode) == (2, 4, "ulysses")
    thr = preset_parallelism("throughput", 4)
    assert thr.dp_replicate == 4 and thr.world == 4
    assert preset_parallelism("latency", 1).world == 1
