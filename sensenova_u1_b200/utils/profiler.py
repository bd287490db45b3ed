"""Inference profiler: load time, device-synchronised generate time, image tokens per second,
peak allocated / reserved device memory and host RSS
(reference: src/sensenova_u1/utils/profiler.py:91-324)."""
from __future__ import annotations

import time
from contextlib import contextmanager


class InferenceProfiler:
    def __init__(self, enabled: bool = True):
        self.enabled = enabled
        self.load_s = 0.0
        self.runs = []

    def _sync(self):
        import torch
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    @contextmanager
    def time_load(self):
        t0 = time.perf_counter()
        yield
        if self.enabled:
            self._sync()
            self.load_s = time.perf_counter() - t0

    @contextmanager
    def time_generate(self, image_tokens: int = 0):
        import torch
        if self.enabled and torch.cuda.is_available():
            torch.cuda.reset_peak_memory_stats()
            self._sync()
        t0 = time.perf_counter()
        yield
        if self.enabled:
            self._sync()
            dt = time.perf_counter() - t0
            rec = {"seconds": dt, "image_tokens": image_tokens,
                   "tokens_per_s": image_tokens / dt if dt > 0 else 0.0}
            if torch.cuda.is_available():
                rec["peak_alloc_gib"] = torch.cuda.max_memory_allocated() / 2 ** 30
                rec["peak_reserved_gib"] = torch.cuda.max_memory_reserved() / 2 ** 30
            try:
                import psutil
                rec["rss_gib"] = psutil.Process().memory_info().rss / 2 ** 30
            except Exception:
                pass
            self.runs.append(rec)

    def report(self) -> str:
        lines = [f"model load: {self.load_s:.3f} s"]
        for i, r in enumerate(self.runs):
            lines.append(f"generate[{i}]: {r['seconds']:.3f} s, {r['tokens_per_s']:.2f} image-tok/s, "
                         f"peak {r.get('peak_alloc_gib', 0):.2f} GiB alloc / {r.get('peak_reserved_gib', 0):.2f} GiB reserved")
        return "\n".join(lines)
