"""The Hugging Face style front end of the Reasoner."""
import torch


def test_generate_and_auto_registration():
    from cosmos_b200 import hf

    m = hf.Cosmos3ReasonerForConditionalGeneration.from_pretrained(
        "tiny", config_overrides=dict(n_layers=1, vocab_size=300))
    ids = torch.tensor([[3, 4, 5, 6]])
    out = m.generate(ids, max_new_tokens=5)
    assert out.shape == (1, 9) and torch.equal(out[:, :4], ids)
    logits = m(ids)
    assert logits.shape == (1, 4, 300)
    assert int(logits[0, -1].argmax()) == int(out[0, 4])           # greedy continuation matches the forward pass
    # an image fills the positions that hold the image token
    pix = torch.rand(1, 3, 64, 64) * 2 - 1
    _, grid = m.visual(pix)
    n = grid[0] * grid[1] * grid[2]
    out2 = m.generate([7] + [299] * n + [8], pixel_values=pix, image_token_id=299, max_new_tokens=3)
    assert out2.shape[1] == n + 2 + 3
    if hf.register():
        from transformers import AutoConfig
        cfg = AutoConfig.for_model("cosmos3_reasoner", arch="tiny")
        assert isinstance(cfg, hf.Cosmos3ReasonerConfig) and hf.register()
