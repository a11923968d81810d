"""Paged-KV batched decoder on CPU (tp = 1) against the contiguous-cache Reasoner engine."""
import torch

from cosmos_b200.config import tiny_config
from cosmos_b200.models.mot import MoTModel
from cosmos_b200.models.reasoner import ReasonerEngine
from cosmos_b200.serve.decoder import TPDecoder
from cosmos_b200.serve.paged import PagedKVCache, make_allocator


def test_allocator_tables_and_slots():
    alloc = make_allocator(10, 4, 5)
    assert alloc.extend(7, 9) and alloc.length(7) == 9 and len(alloc.blocks(7)) == 3
    assert alloc.extend(8, 4) and alloc.num_free() == 6
    assert not alloc.extend(8, 100)           # exceeds the per-sequence table
    alloc.release(7)
    assert alloc.num_free() == 9
    cache = PagedKVCache(1, 2, 8, 12, 4, 6, torch.float32, "cpu")
    assert cache.reserve(0, 10) and cache.reserve(1, 3)
    table, lens = cache.tables([0, 1])
    assert lens.tolist() == [10, 3] and (table[0, :3] >= 0).all() and table[0, 3] == -1
    pos = torch.tensor([[0, 5, 9]])
    slots = PagedKVCache.slots(table[:1], pos, 4)
    assert slots[0, 1] == table[0, 1] * 4 + 1 and slots[0, 2] == table[0, 2] * 4 + 1


def test_paged_decoder_matches_contiguous_cache_logits():
    """Teacher-forced: at every step the paged decoder's logits equal the contiguous-cache engine's."""
    torch.manual_seed(0)
    cfg = tiny_config(n_layers=2, vocab_size=300, max_text_len=16)
    model = MoTModel(cfg, towers=("ar",))
    model.init_weights(seed=4)
    ids = torch.randint(0, cfg.vocab_size, (2, 11))
    forced = torch.randint(0, cfg.vocab_size, (2, 7))
    eng = ReasonerEngine(model)
    dec = TPDecoder(cfg, 1, 0, None, "cpu", page_size=4, max_batch=2, max_len=32, dtype=torch.float32)
    dec.load_from(model)
    dec.prefill(model, ids, None, new_tokens=8)
    from cosmos_b200.models import rope
    kvs = []
    for b in range(2):
        _, kv = eng.prefill(model.embed_tokens(ids[b:b + 1]), rope.text_positions(11))
        kvs.append(kv)
    for step in range(7):
        dec.tokens.copy_(forced[:, step])
        dec.step()
        for b in range(2):
            want, kvs[b] = eng.decode_one(forced[b:b + 1, step], 11 + step, kvs[b])
            got = dec.last_logits[b, :cfg.vocab_size]
            assert torch.allclose(got, want[0], atol=2e-4), (step, b, (got - want[0]).abs().max())
    assert dec.lens.tolist() == [18, 18]
