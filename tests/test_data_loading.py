"""Video sampling, the background worker pool with recovery, resumable samplers (CPU)."""
import os
import random

import numpy as np
import pytest
import torch

from sensenova_u1_b200.data.loader import WeightedResumableSampler, WorkerPoolLoader
from sensenova_u1_b200.data.video import load_frames, sample_frame_indices, video_record_to_sample


def test_frame_sampling_is_segment_wise():
    assert sample_frame_indices(100, 4, 8) == [6, 18, 31, 43, 56, 68, 81, 93]
    assert sample_frame_indices(3, 4, 8) == [0, 1, 2]                       # fewer frames than the minimum
    rng = random.Random(0)
    idx = sample_frame_indices(240, 4, 24, rng)
    assert 4 <= len(idx) <= 24 and idx == sorted(idx) and len(set(idx)) == len(idx)
    clip = sample_frame_indices(300, 4, 4, None, clip=(10.0, 20.0), fps=10.0)
    assert all(100 <= i <= 200 for i in clip)


def test_video_record_becomes_a_run_of_understanding_images(tmp_path):
    frames = (np.random.default_rng(0).random((12, 64, 64, 3)) * 255).astype("uint8")
    np.save(tmp_path / "clip.npy", frames)
    assert load_frames(str(tmp_path / "clip.npy"), [0, 5]).shape == (2, 3, 64, 64)
    rec = {"video": "clip.npy", "conversations": [{"from": "human", "value": "<video>\nWhat happens?"},
                                                  {"from": "gpt", "value": "A cat jumps."}]}
    tok = lambda s: list(s.encode())
    prep = lambda fr: fr.float() / 127.5 - 1.0
    s = video_record_to_sample(rec, tok, prep, root=tmp_path, min_num_frame=4, max_num_frame=6)
    kinds = [g.kind for g in s.segments]
    assert kinds.count("und_image") == 6 and s.task == 0
    assert s.segments[-1].loss and not s.segments[0].loss
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.data.batch import build_packed_batch
    b = build_packed_batch([s], tiny_mot(patch_size=16, vocab_size=1024))
    assert b.und_rows.numel() == 6 * 4 and b.gen_rows.numel() == 0


def _stream(wid, n, skip):
    """Worker ``wid`` yields wid, wid + n, wid + 2n, ...; its third item kills it once (marker file)."""
    k = skip
    while k < 6:
        if wid == 1 and k == 2 and not os.path.exists(os.environ["SNU1_TEST_MARK"]):
            open(os.environ["SNU1_TEST_MARK"], "w").close()
            os._exit(3)
        yield torch.tensor([wid + n * k])
        k += 1


def test_worker_pool_survives_a_dead_worker_without_losing_items(tmp_path):
    os.environ["SNU1_TEST_MARK"] = str(tmp_path / "died")
    loader = WorkerPoolLoader(_stream, num_workers=2, prefetch=2, worker_fail_retry_backoff_s=0.05, poll_s=0.1)
    got = [int(t) for t in loader]
    loader.close()
    assert got == list(range(12)) and loader.restarts == 1 and loader.state_dict()["taken"] == [6, 6]


def test_worker_pool_resumes_from_its_state(tmp_path):
    os.environ["SNU1_TEST_MARK"] = str(tmp_path / "never")
    open(os.environ["SNU1_TEST_MARK"], "w").close()
    a = WorkerPoolLoader(_stream, num_workers=2, poll_s=0.1)
    it = iter(a)
    first = [int(next(it)) for _ in range(5)]
    sd = a.state_dict()
    a.close()
    b = WorkerPoolLoader(_stream, num_workers=2, poll_s=0.1)
    b.load_state_dict(sd)
    rest = [int(t) for t in b]
    b.close()
    assert first == [0, 1, 2, 3, 4] and sorted(first + rest) == list(range(12))


def test_sampler_state_continues_the_stream():
    s = WeightedResumableSampler([10, 4, 7], weights=[1, 1, 2], rank=1, world=2, seed=3)
    it = iter(s)
    head = [next(it) for _ in range(25)]
    sd = s.state_dict()
    tail = [next(it) for _ in range(25)]
    s2 = WeightedResumableSampler([10, 4, 7], weights=[1, 1, 2], rank=1, world=2, seed=3)
    s2.load_state_dict(sd)
    it2 = iter(s2)
    assert [next(it2) for _ in range(25)] == tail
    assert all(i % 2 == 1 for _, i in head)                                # this rank's indices only
    seen = {(d, i) for d, i in head + tail if d == 1}
    assert seen == {(1, 1), (1, 3)}
