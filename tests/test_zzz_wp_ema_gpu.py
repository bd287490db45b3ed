"""EMA shadow in weight-parallel mode: on one GPU (a group of one rank) the shadow of the rank's shard must follow
the plain trainer's shadow of the same weights.  The file sorts last on purpose: it covers a path added after the
other GPU tests were last run together."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_weight_parallel_ema_follows_the_plain_trainers():
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.data.synthetic import tiny_batch
    from sensenova_u1_b200.models.params import ParamStore
    from sensenova_u1_b200.ops import _lib
    from sensenova_u1_b200.parallel.weight_parallel import WeightParallelStore
    from sensenova_u1_b200.train.optimizer import AdamConfig
    from sensenova_u1_b200.train.trainer import Trainer
    cfg = tiny_mot(head_dim=128, patch_size=16, num_layers=3)
    adam = AdamConfig(lr=1e-2, state_dtype="fp32", clip_grad_norm=0.0)
    ref = ParamStore(cfg, device="cuda")
    ref.init_weights(0, std=0.05)
    wp = WeightParallelStore(cfg, "cuda")
    wp.init_weights(0, std=0.05)
    t_ref, t_wp = Trainer(cfg, ref, adam, ema_decay=0.5), Trainer(cfg, wp, adam, ema_decay=0.5)
    def shadows(tr, arena="mat"):
        """Bucket name -> this trainer's fp32 shadow of that bucket (the two stores pad their buckets differently)."""
        return {name: tr.ema[arena][so:so + (mhi - mlo)] for name, lo, hi, mlo, mhi, so in tr.optim.pieces[arena]}

    def distance(arena="mat"):
        a, b = shadows(t_wp, arena), shadows(t_ref, arena)
        assert set(a) == set(b)
        num = den = 0.0
        for k in a:
            m = min(a[k].numel(), b[k].numel())
            num += float((a[k][:m] - b[k][:m]).pow(2).sum())
            den += float(b[k][:m].pow(2).sum())
        return (num / den) ** 0.5

    assert distance() == 0.0                                                      # both start from the weights
    start = {k: v.clone() for k, v in shadows(t_ref).items()}
    for step in range(2):
        b = [tiny_batch(cfg, seed=step, n_text=200, image_px=8 * 32, with_und_image=True).to("cuda")]
        t_ref.step_on_device(b)
        t_wp.step_on_device(b)
        if step == 0:
            # the first step's matrix update agrees in both modes up to the summation order of atomically accumulated
            # gradients (embedding rows), which shows in the last bits of the fp32 master only
            assert distance() < 1e-6
    torch.cuda.synchronize()
    _lib.check_status()
    assert all(torch.isfinite(v).all() for v in shadows(t_wp).values()) and distance() < 2e-3
    assert any(not torch.equal(start[k], v) for k, v in shadows(t_ref).items())  # the shadow moved
    assert distance("vec") < 2e-3
