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


def test_tokenized_text_dataset_and_storage(tmp_path):
    import numpy as np
    import torch
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.data.tokenized import PackedTokenDataset, RandomTokens
    from sensenova_u1_b200.utils import storage
    cfg = tiny_mot()
    toks = np.arange(10, 10 + 1000, dtype=np.uint16) % 900 + 8
    toks[[99, 350, 777]] = 2                                   # end-of-document ids
    toks[:500].tofile(tmp_path / "a.bin"); toks[500:].tofile(tmp_path / "b.bin")
    ds = PackedTokenDataset([str(tmp_path / "a.bin"), str(tmp_path / "b.bin")], cfg, 256, eod_id=2, repeat=False)
    batches = list(ds)
    assert len(batches) == 3                                   # 1000 // 256
    b = batches[1]                                             # tokens 256..511: spans both files, one separator at 350
    real = b.kind == 1
    assert int(real.sum()) == 256 and int(b.meta[real, 0].unique().numel()) == 2
    assert torch.equal(b.ids[real].long(), torch.from_numpy(toks[256:512].astype(np.int64)))
    # labels never cross a document boundary
    last_of_doc0 = int((b.meta[:, 0] == b.meta[real, 0].min()).nonzero().max())
    assert int(b.labels[last_of_doc0]) == -100
    r0 = PackedTokenDataset([str(tmp_path / "a.bin")], cfg, 128, eod_id=2, rank=1, world=2, repeat=False)
    assert len(list(r0)) == 1 and r0.state_dict()["next"] == 3   # sequences 1 (and would-be 3) of 3
    assert next(iter(RandomTokens(cfg, 300))).n_tokens == 300
    # storage: url schemes, atomic local writes, async writer, pluggable remote back-end
    storage.llm_save(f"local:{tmp_path}/ck/x.pt", {"a": torch.ones(3)})
    assert torch.equal(storage.llm_load(f"local:{tmp_path}/ck/x.pt")["a"], torch.ones(3))
    w = storage.AsyncWriter()
    w.save({"b": 2}, f"{tmp_path}/ck/y.pt"); w.wait(); w.close()
    assert storage.llm_load(f"{tmp_path}/ck/y.pt")["b"] == 2 and len(storage.md5_of(f"{tmp_path}/ck/y.pt")) == 32

    class Mem:
        def __init__(self): self.blobs = {}
        def upload(self, lp, rp): self.blobs[rp] = open(lp, "rb").read()
        def download(self, rp, lp): open(lp, "wb").write(self.blobs[rp])
        def exists(self, rp): return rp in self.blobs
        def listdir(self, rp): return sorted(self.blobs)
    mem = Mem()
    storage.register_backend("mem", mem)
    storage.llm_save("mem:bucket/z.pt", [1, 2])
    assert storage.llm_load("mem:bucket/z.pt") == [1, 2] and mem.exists("bucket/z.pt")
    import pytest
    with pytest.raises(KeyError):
        storage.split_url("nosuch:bucket/x")


def test_jsonl_token_files_pack_by_cut_and_by_pad(tmp_path):
    import json
    import numpy as np
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.data.tokenized import JsonlTokenFile, PackedDocumentDataset
    cfg = tiny_mot()
    docs = [list(range(10, 10 + n)) for n in (300, 40, 700, 5, 128)]
    docs[1] = [-t if i < 10 else t for i, t in enumerate(docs[1])]          # a prompt without loss, then the answer
    f = tmp_path / "a.jsonl"
    offs, off = [], 0
    with open(f, "wb") as fh:
        for d in docs:
            line = (json.dumps({"tokens": d}) + "\n").encode()
            offs.append((off, len(d)))
            fh.write(line)
            off += len(line)
    src = JsonlTokenFile(str(f), min_length=8)
    assert len(src) == 4 and src.lengths().tolist() == [300, 40, 700, 128]   # the 5-token document is filtered out
    np.save(str(f) + ".meta.npy", np.asarray(offs, dtype=np.int64))
    (tmp_path / "a.jsonl.meta.npy").rename(tmp_path / "a.jsonl.meta")
    assert JsonlTokenFile(str(f), min_length=8).tokens(2)[:3].tolist() == [10, 11, 12]      # offsets from the .meta file

    cut = PackedDocumentDataset([src], cfg, seq_len=256, mode="cut", seed=3)
    assert len(cut) == (300 + 40 + 700 + 128) // 256                          # the last partial row is dropped
    rows = [cut.row_samples(r) for r in range(len(cut))]
    assert all(sum(sum(seg.ids.numel() for seg in s.segments) for s in row) == 256 for row in rows)
    b = next(iter(cut))
    assert b.n_tokens == 256
    whole = PackedDocumentDataset([src], cfg, seq_len=2048, mode="pad", seed=3)
    segs = [seg for smp in whole.row_samples(0) for seg in smp.segments]
    no_loss = [seg for seg in segs if not seg.loss]
    assert len(no_loss) == 1 and no_loss[0].ids.tolist() == list(range(10, 20))      # the negative ids: context, no loss

    pad = PackedDocumentDataset([src], cfg, seq_len=512, mode="pad", seed=3, rank=1, world=2, epochs=1)
    plan = pad._plan()
    assert all(sum(e - s for _, s, e in row) <= 512 for row in plan) and sorted(d for row in plan for d, _, _ in row) == [0, 1, 2, 3]
    assert max(e for row in plan for _, _, e in row) == 512                   # the 700-token document is truncated
    got = list(pad)
    assert len(got) == len(plan[1::2])                                        # rank 1 of 2 takes every other row, one epoch
    st = PackedDocumentDataset([src], cfg, seq_len=256, mode="cut", seed=3)
    it = iter(st)
    first = next(it)
    sd = st.state_dict()
    second = next(it)
    again = PackedDocumentDataset([src], cfg, seq_len=256, mode="cut", seed=3)
    again.load_state_dict(sd)
    assert torch.equal(next(iter(again)).ids, second.ids) and not torch.equal(first.ids, second.ids)
