"""Rank grid of the parallel context (no process group needed)."""
import pytest

from sensenova_u1_b200.parallel.context import ParallelConfig, ParallelContext, ParallelMode


def _ctx(rank, world, **kw):
    return ParallelContext(ParallelConfig(**kw), rank=rank, world_size=world, create_groups=False)


def test_dp_only():
    c = _ctx(3, 8)
    assert c.get_world_size(ParallelMode.DATA) == 8 and c.get_ranks_in_group(ParallelMode.ZERO1) == list(range(8))
    assert c.get_world_size(ParallelMode.TENSOR) == 1


def test_isp_weight_parallel_grid():
    # shipped 8B layout: wp=8, tp=1 on 8 GPUs -> zero1 group of size 1
    c = _ctx(5, 8, tensor=1, tensor_mode="isp", weight=8)
    assert c.get_ranks_in_group(ParallelMode.WEIGHT) == list(range(8))
    assert c.get_world_size(ParallelMode.ZERO1) == 1
    # A3B layout on 16 GPUs: wp=8 x tp=2
    c = _ctx(5, 16, tensor=2, tensor_mode="isp", weight=8)
    assert c.get_ranks_in_group(ParallelMode.TENSOR) == [4, 5]
    assert c.get_ranks_in_group(ParallelMode.WEIGHT) == [1, 3, 5, 7, 9, 11, 13, 15]
    assert c.get_world_size(ParallelMode.WEIGHT_DATA) == 1


def test_tp_pp_grid():
    c = _ctx(6, 8, tensor=4, pipeline=2)
    assert c.get_ranks_in_group(ParallelMode.TENSOR) == [4, 5, 6, 7]
    assert c.get_ranks_in_group(ParallelMode.PIPELINE) == [2, 6]
    assert c.is_pipeline_last_stage() and not c.is_pipeline_first_stage()
    assert c.get_world_size(ParallelMode.DATA) == 1


def test_expert_groups_partition_the_stage():
    world = 16
    seen = {m: set() for m in (ParallelMode.EXPERT, ParallelMode.EXPERT_WEIGHT, ParallelMode.EXPERT_DATA)}
    for r in range(world):
        c = _ctx(r, world, expert=4, expert_weight=2, tensor=1, tensor_mode="isp", weight=2)
        assert c.get_world_size(ParallelMode.EXPERT) == 4
        assert c.get_world_size(ParallelMode.EXPERT_WEIGHT) == 2
        assert c.get_world_size(ParallelMode.EXPERT_DATA) == 2
        for m in seen:
            assert r in c.get_ranks_in_group(m)
            seen[m].add(tuple(c.get_ranks_in_group(m)))
    assert len(seen[ParallelMode.EXPERT]) == 4 and len(seen[ParallelMode.EXPERT_WEIGHT]) == 8


def test_invalid_layouts_are_rejected():
    with pytest.raises(ValueError):
        _ctx(0, 8, tensor=3)
    with pytest.raises(ValueError):
        _ctx(0, 8, weight=2, tensor_mode="mtp")
    with pytest.raises(ValueError):
        _ctx(0, 8, zero1=3)


def test_config_from_reference_schema():
    cfg = ParallelConfig.from_dict(dict(zero1=dict(size=-1), tensor=dict(size=2, mode="isp"), pipeline=dict(size=1),
                                        weight=dict(size=4, overlap=True), expert=dict(size=8), expert_weight=2))
    assert (cfg.tensor, cfg.tensor_mode, cfg.weight, cfg.expert, cfg.expert_weight) == (2, "isp", 4, 8, 2)
