"""Rank layout of multi-GPU image sampling (pure arithmetic; the groups themselves are exercised on GPUs)."""
import pytest

from sensenova_u1_b200.inference.parallel import SamplingGroups, layout


def test_layout_covers_every_rank_once():
    for world in (2, 4, 8):
        sp = world // 2
        seen_sp, seen_cfg = set(), set()
        for r in range(world):
            b, s, sp_ranks, cfg_ranks = layout(world, r)
            assert r in sp_ranks and r in cfg_ranks and (b, s) == divmod(r, sp)
            assert len(sp_ranks) == sp and len(cfg_ranks) == 2
            assert set(sp_ranks) & set(cfg_ranks) == {r}
            seen_sp.add(tuple(sp_ranks)); seen_cfg.add(tuple(cfg_ranks))
        assert len(seen_sp) == 2 and len(seen_cfg) == sp
    with pytest.raises(ValueError):
        layout(3, 0)
    assert layout(6, 4, branches=3)[:2] == (2, 0)


def test_describe():
    assert SamplingGroups().describe() == "single"
    assert SamplingGroups(world=2, sp=1).describe() == "guidance-parallel x2"
    assert SamplingGroups(world=8, sp=4).describe() == "guidance-parallel x2 x sequence-parallel x4"
