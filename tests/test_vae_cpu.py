"""Host-side logic of the tokenizer's channels-last paths (no GPU needed)."""
def test_chunked_temporal_stride_keeps_the_even_frames():
    """Frame bookkeeping of the channels-last encoder's temporal down-sampling: whatever the chunking, the frames
    kept over all chunks are the even indices of the level's timeline, in order, and the next level's indices are
    consecutive. (The strided causal convolution's output j reads frames 2j - 2 .. 2j.)"""
    from cosmos_b200.models.vae_cuda import even_frames
    for total, chunk in ((17, 8), (33, 4), (9, 8), (1, 8), (41, 12)):
        starts = [0] + list(range(1, total, chunk))
        sizes = [1] + [min(chunk, total - s) for s in starts[1:]]
        kept, nxt = [], []
        for s, n in zip(starts, sizes):
            first, count, t_next = even_frames(s, n)
            idx = list(range(s + first, s + n, 2))
            assert len(idx) == count
            kept += idx
            nxt += list(range(t_next, t_next + count))
        assert kept == list(range(0, total, 2))
        assert nxt == list(range(len(kept)))
