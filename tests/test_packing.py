import torch

from sensenova_u1_b200.config import tiny_mot
from sensenova_u1_b200.data.batch import Sample, Segment
from sensenova_u1_b200.data.packing import PackedDataset, RestartableLoader, sample_tokens, split_text_tail


def _text(n, loss=True):
    return Segment("text", ids=torch.arange(8, 8 + n), loss=loss)


def _img(cfg, tok_side, kind="und_image"):
    px = tok_side * cfg.token_pixels
    return Segment(kind, pixels=torch.zeros(3, px, px))


def test_best_fit_fills_sequences_and_respects_budgets():
    cfg = tiny_mot()
    samples = [Sample([_text(300)]), Sample([_text(200)]), Sample([_img(cfg, 4), _text(100)]),
               Sample([_text(60), _img(cfg, 8, "gen_image")]), Sample([_text(500)]), Sample([_text(90)])]
    ds = PackedDataset(samples, cfg, max_packed_tokens=640, num_images_expected=1, max_buffer_size=2)
    out = list(ds)
    assert sum(b.n_samples for b in out) == len(samples)
    for b in out:
        assert b.S == 640
        n_img = int((b.meta[:, 2] > 0).sum() > 0)
        assert len(set(b.meta[b.meta[:, 2] > 0, 2].tolist())) <= 1          # image budget
    total = sum(sample_tokens(s, cfg)["gen"] + sample_tokens(s, cfg)["und"] for s in samples)
    assert sum(b.n_tokens for b in out) == total


def test_oversized_sample_is_split_at_a_text_boundary():
    cfg = tiny_mot()
    s = Sample([_text(700), _img(cfg, 4), _text(50)])
    head, tail = split_text_tail(s, 300)
    assert sample_tokens(head, cfg)["und"] == 300 and tail.segments[0].ids.numel() == 400
    assert tail.segments[1].kind == "und_image"
    ds = PackedDataset([s], cfg, max_packed_tokens=640)
    out = list(ds)
    assert sum(b.n_tokens for b in out) == sample_tokens(s, cfg)["und"]


def test_state_roundtrip_keeps_open_buffers():
    cfg = tiny_mot()
    ds = PackedDataset([], cfg, max_packed_tokens=1024)
    ds._place(Sample([_text(100)])); ds._place(Sample([_text(50)]))
    sd = ds.state_dict()
    ds2 = PackedDataset([], cfg, max_packed_tokens=1024)
    ds2.load_state_dict(sd)
    assert len(ds2.buffers) == 1 and ds2.buffers[0].und == 150


def test_loader_restarts_a_dead_worker():
    calls = {"n": 0}

    def make():
        calls["n"] += 1
        def gen():
            yield 1
            if calls["n"] == 1:
                raise RuntimeError("worker died")
            yield 2
        return gen()
    got = list(RestartableLoader(make, backoff_s=0.0))
    assert got == [1, 1, 2] and calls["n"] == 2


def test_context_parallel_split_covers_the_batch_once():
    import torch
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.data.batch import context_parallel_tiles, split_context_parallel
    from sensenova_u1_b200.data.synthetic import tiny_batch
    cfg = tiny_mot()
    b = tiny_batch(cfg, seed=3, n_text=500, image_px=128, with_und_image=True, seq_len=1024)
    W = 2
    assert sorted(torch.cat([context_parallel_tiles(8, W, r) for r in range(W)]).tolist()) == list(range(8))
    parts = [split_context_parallel(b, W, r, cfg) for r in range(W)]
    assert all(p.S == b.S // W for p in parts)
    assert sum(p.n_tokens for p in parts) == b.n_tokens and sum(p.n_label for p in parts) == b.n_label
    assert abs(sum(p.ce_weight_sum for p in parts) - b.ce_weight_sum) < 1e-4
    assert abs(sum(p.gen_weight_sum for p in parts) - b.gen_weight_sum) < 1e-5
    assert sum(p.gen_x16.shape[0] for p in parts) == b.gen_x16.shape[0]
    assert sum(p.und_patches.shape[0] for p in parts) == b.und_patches.shape[0]
    for p in parts:
        # local layout is again [generation | understanding | padding], tile aligned
        assert bool((p.kind[: p.n_gen_pad][p.kind[: p.n_gen_pad] != 0] == 3).all())
        assert p.gen_rows.numel() * cfg.merge_size ** 2 == p.gen_x16.shape[0]
        assert int(p.group_range[1, 1]) == p.n_gen_pad
        # every generation token kept its own pixels: compare through the global row ids
    ids = torch.cat([p.ids for p in parts])
    assert sorted(ids.tolist()) == sorted(b.ids.tolist())
