"""The ``data`` section of a training config as one validated object.

The reference reads its ~60 ``data.*`` keys in many places (training/sensenovavl/data/build_dataloader.py:125-340,
multimodal_dataset.py:60-210 and :718-800, batch_sampler.py:15-60, dataset_interleaved_iterable.py:830-930,
sensenovalm/initialize/launch.py:150-260, sensenovalm/core/trainer.py:67).  Here every key has one home:

* keys that drive this package's pipeline are fields with the reference's defaults and are consumed by
  ``train_sensenovau1.make_batches`` (pixel budgets of understanding and generation images, packing limits, dataset
  mixing weights, batch-size ramp-up, epochs, minimum sample length, loss weighting, logging frequency ...);
* keys of the reference's older fixed-tile image pipeline (``force_image_size``, ``use_thumbnail``, ``pad2square``,
  ``min/max_dynamic_patch`` ...) are accepted and checked: this package implements the native-resolution pipeline the
  shipped configs select (``dynamic_image_size=True, dynamic_image_version="native_resolution"``) and refuses a
  config that asks for the other one instead of silently doing something else;
* keys nothing reads in the reference either (``use_bos``, ``use_eos``, ``split_data_chunk``) are accepted and kept.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

_TRUE = ("1", "true", "yes", "on")


def _as_bool(v) -> bool:
    return v.strip().lower() in _TRUE if isinstance(v, str) else bool(v)


class BatchSkipper:
    """``skipper(batch_count)`` is true for the batch counts named by ``"3,10-12"`` (inclusive ranges, ascending): such a
    batch is drawn from the loader, so the data position moves on, but no step is taken on it (a way around a
    poisoned sample without touching the dataset; core/trainer_builder.py:437-545, utils/common.py:157-180)."""

    def __init__(self, spec: str = ""):
        self.spans: List[int] = []
        for part in str(spec or "").split(","):
            part = part.strip()
            if not part:
                continue
            lo, _, hi = part.partition("-")
            lo, hi = int(lo), int(hi or lo)
            if hi < lo or (self.spans and lo < self.spans[-1]):
                raise ValueError(f"data.skip_batches: ranges must be ascending and non-overlapping, got {spec!r}")
            self.spans += [lo, hi + 1]

    def __call__(self, batch_count: int) -> bool:
        import bisect
        return bisect.bisect_right(self.spans, batch_count) % 2 == 1


@dataclass
class DataOptions:
    # ---- sequence / packing --------------------------------------------------------------------------------------
    seq_len: int = 16384
    micro_num: int = 1
    micro_bsz: int = 1
    max_packed_tokens: Optional[int] = None          # default: seq_len
    num_images_expected: int = 144
    max_buffer_size: int = 10
    packed_buffer_stale_threshold: int = 200
    use_packed_ds: bool = True
    pack_sample_into_one: bool = False
    strict_mode: bool = False
    replacement: bool = False
    allow_overflow: bool = False
    allow_empty_data: bool = False
    min_length: int = 0
    total_epochs: int = -1
    rampup_batch_size: Optional[str] = None          # "start increment every"
    group_by_length: bool = False
    log_freq: int = 1000
    skip_batches: str = ""                           # "3,10-12": batch counts that are loaded but not trained on
    diag_outlier_ratio: float = 1.1
    # ---- datasets and mixing ---------------------------------------------------------------------------------------
    meta_path: Optional[str] = None
    tokenizer_path: Optional[str] = None
    train_folder: Optional[str] = None
    llm_data_config: Optional[Any] = None
    llm_data_weights: float = 0.0
    mm_cc_data_weights: float = 0.0
    mm_plain_pair_data_weights: float = 0.0
    nlp_mm_sampling_fixed_token: bool = False
    num_worker: int = 4
    # ---- text ---------------------------------------------------------------------------------------------------
    conv_style: str = "sensenovalm-v3"
    use_bos: bool = True
    use_eos: bool = True
    loss_reduction: str = "square"
    loss_reduction_all_gather: bool = False
    enabel_und_loss: bool = True                     # the reference's spelling
    # ---- images ---------------------------------------------------------------------------------------------------
    patch_size: int = 16
    down_sample_ratio: float = 0.5
    min_pixels: int = 65536
    max_pixels: int = 4194304
    min_pixels_gen: Optional[int] = None             # default: min_pixels
    max_pixels_gen: Optional[int] = None             # default: max_pixels
    candidate_resolutions_for_gen: Optional[Sequence[Tuple[int, int]]] = None
    dynamic_image_size: bool = True
    dynamic_image_version: str = "native_resolution"
    data_augment: bool = True
    min_num_frame: int = 4
    max_num_frame: int = 24
    # legacy fixed-tile pipeline (accepted, checked, not implemented)
    hf_image_size: Optional[int] = None
    force_image_size: Optional[int] = None
    pad2square: bool = False
    use_thumbnail: bool = False
    min_dynamic_patch: int = 1
    max_dynamic_patch: int = 12
    split_data_chunk: Any = None
    # whatever else the config carried
    extra: Dict[str, Any] = field(default_factory=dict)

    # ------------------------------------------------------------------------------------------------------------
    @classmethod
    def from_config(cls, data: Mapping) -> "DataOptions":
        """Builds the options from a config's ``data`` mapping; unknown keys go to ``extra`` (condition-dropping
        probabilities, cloud paths and the like are read where they are used)."""
        known = {f.name: f for f in fields(cls) if f.name != "extra"}
        kw, extra = {}, {}
        for k, v in dict(data).items():
            if k in known:
                t = known[k].type
                if "bool" in str(t) and v is not None:
                    v = _as_bool(v)
                kw[k] = v
            else:
                extra[k] = v
        o = cls(**kw, extra=extra)
        o.validate()
        return o

    def validate(self) -> None:
        if not self.use_packed_ds:
            raise ValueError("data.use_packed_ds=False: only the packed pipeline exists (the reference raises "
                             "NotImplementedError for it as well)")
        if self.group_by_length:
            raise ValueError("data.group_by_length is not supported (the reference asserts it off)")
        if not self.dynamic_image_size or self.dynamic_image_version != "native_resolution":
            raise ValueError("only the native-resolution image pipeline (dynamic_image_size=True, "
                             "dynamic_image_version='native_resolution') is implemented; fixed-tile options "
                             "(force_image_size / use_thumbnail / pad2square / min,max_dynamic_patch) have no effect")
        if self.strict_mode:
            raise ValueError("data.strict_mode must be off with the native-resolution pipeline")
        if self.loss_reduction not in ("token", "sample", "square"):
            raise ValueError(f"data.loss_reduction must be token, sample or square, got {self.loss_reduction!r}")
        if self.rampup_batch_size:
            self.rampup()                                  # parses or raises
        BatchSkipper(self.skip_batches)                    # parses or raises
        for name in ("llm_data_weights", "mm_cc_data_weights", "mm_plain_pair_data_weights"):
            v = float(getattr(self, name))
            if not 0.0 <= v <= 1.0:
                raise ValueError(f"data.{name} must lie in [0, 1]")
        if self.mm_cc_data_weights + self.mm_plain_pair_data_weights > 1.0:
            raise ValueError("data.mm_cc_data_weights + data.mm_plain_pair_data_weights exceed 1")
        lo, hi = self.pixel_budget(False)
        glo, ghi = self.pixel_budget(True)
        if lo > hi or glo > ghi:
            raise ValueError("min_pixels exceeds max_pixels")

    # ---- derived quantities ------------------------------------------------------------------------------------
    @property
    def token_pixels(self) -> int:
        """Side of one LLM image token in pixels (patch 16 / down-sample 0.5 = 32)."""
        return int(round(self.patch_size / self.down_sample_ratio))

    @property
    def packed_tokens(self) -> int:
        return int(self.max_packed_tokens or self.seq_len)

    def pixel_budget(self, for_generation: bool, num_images: int = 1) -> Tuple[int, int]:
        """(min_pixels, max_pixels) of one image of a sample with ``num_images`` images.  Several images share the
        sequence: each may take ``(packed_tokens - 3072) / num_images`` tokens at most, never less than the minimum
        (multimodal_dataset.py:768-800)."""
        lo = int(self.min_pixels_gen if (for_generation and self.min_pixels_gen is not None) else self.min_pixels)
        hi = int(self.max_pixels_gen if (for_generation and self.max_pixels_gen is not None) else self.max_pixels)
        if num_images > 1:
            tp = self.token_pixels
            share = (self.packed_tokens - 3072) * tp * tp // num_images
            hi = max(min(hi, share), lo)
        return lo, hi

    def rampup(self) -> Tuple[int, int, int]:
        """(start, increment, every) of the batch-size ramp-up string."""
        parts = str(self.rampup_batch_size).split()
        if len(parts) != 3:
            raise ValueError("data.rampup_batch_size is 'start increment every', e.g. '2 2 100'")
        start, inc, every = (int(p) for p in parts)
        if start < 1 or inc < 0 or every < 1:
            raise ValueError("data.rampup_batch_size: start >= 1, increment >= 0, every >= 1")
        return start, inc, every

    def batch_size_at(self, batch_count: int, full: Optional[int] = None) -> int:
        """Micro-batches of step number ``batch_count``: grows from ``start`` by ``increment`` every ``every`` steps
        up to the full size (batch_sampler.py:21-45)."""
        full = int(full if full is not None else self.micro_num)
        if not self.rampup_batch_size:
            return full
        start, inc, every = self.rampup()
        return min((batch_count // every) * inc + start, full)

    def mixing_weights(self, kinds: Sequence[str], lengths: Sequence[int]) -> List[float]:
        """Sampling weight per dataset.  ``kinds[i]`` is "paired" (conversation / generation data), "cc"
        (caption pairs) or "plain_pair"; inside a kind the weight is proportional to the dataset's length; the
        kinds share ``1 - llm_data_weights`` as ``mm_cc_data_weights`` / ``mm_plain_pair_data_weights`` / the rest
        (build_dataloader.py:167-176)."""
        mm_total = 1.0 - float(self.llm_data_weights)
        cc = float(self.mm_cc_data_weights) * mm_total
        plain = float(self.mm_plain_pair_data_weights) * mm_total
        share = {"paired": mm_total - cc - plain, "cc": cc, "plain_pair": plain}
        tot = {k: sum(l for kk, l in zip(kinds, lengths) if kk == k) for k in share}
        present = [k for k in share if tot[k] > 0]
        missing = sum(share[k] for k in share if tot[k] == 0)
        out = []
        for k, l in zip(kinds, lengths):
            if k not in share:
                raise ValueError(f"unknown dataset kind {k!r}")
            w = share[k] + (missing * share[k] / max(1e-12, sum(share[p] for p in present)) if present else 0.0)
            out.append(w * l / tot[k] if tot[k] else 0.0)
        return out

    def loss_weight(self, n_label_tokens: int) -> float:
        """Per-token loss weight of a sample with ``n_label_tokens`` supervised tokens (build_dataloader.py:58-68)."""
        if n_label_tokens <= 0:
            return 0.0
        return {"token": 1.0, "sample": 1.0 / n_label_tokens, "square": 1.0 / math.sqrt(n_label_tokens)}[self.loss_reduction]

    def summary(self) -> Dict[str, Any]:
        keep = ("seq_len", "micro_num", "num_images_expected", "max_buffer_size", "min_length", "total_epochs",
                "rampup_batch_size", "loss_reduction", "loss_reduction_all_gather", "min_pixels", "max_pixels",
                "min_pixels_gen", "max_pixels_gen", "llm_data_weights", "mm_cc_data_weights", "conv_style", "log_freq")
        return {k: getattr(self, k) for k in keep}


def image_loader_from_options(opts: DataOptions):
    """``load(path, for_generation, num_images=1)``: native-resolution resize inside the pixel budget of the sample
    (understanding images ImageNet-normalised, generation targets in [-1, 1])."""
    from ..inference.images import load_image_native

    def load(path: str, for_generation: bool, num_images: int = 1):
        lo, hi = opts.pixel_budget(for_generation, num_images)
        return load_image_native(path, factor=opts.token_pixels, min_pixels=lo, max_pixels=hi,
                                 normalize="pm1" if for_generation else "imagenet")
    return load
