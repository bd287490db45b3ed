"""Text-only pre-tokenised datasets: flat token files packed into fixed-length sequences.

Counterpart of the reference's language-model data path (training/sensenovalm/data/tokenized/
packed_dataset.py:32-746, batch_sampler.py:24-787, dummy_dataset.py): ``.bin`` files hold token ids
back to back (uint16 / uint32 / int32, documents separated by an end-of-document id); a sequence of
``seq_len`` tokens is cut at a deterministic, resumable position, documents inside it keep their
own positions and attention (``doc`` ids restart at every separator), and every token predicts the
next one of its document.  ``RandomTokens`` is the dummy dataset for smoke runs.
"""
from __future__ import annotations

from pathlib import Path
from typing import Iterator, List, Optional, Sequence

import numpy as np
import torch

from ..config import ModelConfig
from .batch import PackedBatch, Sample, Segment, build_packed_batch


class TokenFile:
    def __init__(self, path: str, dtype: str = "uint16"):
        self.arr = np.memmap(path, dtype=np.dtype(dtype), mode="r")

    def __len__(self):
        return int(self.arr.shape[0])


class PackedTokenDataset:
    """Sequences of ``seq_len`` tokens from one or more token files (concatenated in order).
    Rank r of ``world`` reads sequences r, r + world, ...; ``state_dict`` holds the next index."""

    def __init__(self, files: Sequence[str], cfg: ModelConfig, seq_len: int, eod_id: int, dtype: str = "uint16",
                 rank: int = 0, world: int = 1, repeat: bool = True):
        self.files = [TokenFile(f, dtype) for f in files]
        self.cfg, self.seq_len, self.eod = cfg, seq_len, eod_id
        self.rank, self.world, self.repeat = rank, world, repeat
        self.offsets = np.cumsum([0] + [len(f) for f in self.files])
        self.n_seq = int(self.offsets[-1]) // seq_len
        self.next = rank

    def _tokens(self, start: int, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.int64)
        got = 0
        while got < n:
            fi = int(np.searchsorted(self.offsets, start + got, side="right")) - 1
            lo = start + got - int(self.offsets[fi])
            take = min(n - got, len(self.files[fi]) - lo)
            out[got:got + take] = self.files[fi].arr[lo:lo + take]
            got += take
        return out

    def sample(self, index: int) -> Sample:
        """Sequence ``index`` as documents split at the end-of-document id."""
        toks = self._tokens(index * self.seq_len, self.seq_len)
        cuts = np.flatnonzero(toks == self.eod) + 1
        segs: List[Sample] = []
        docs = np.split(toks, cuts)
        return [Sample([Segment("text", ids=torch.from_numpy(d.copy()), loss=True)]) for d in docs if d.size]

    def __iter__(self) -> Iterator[PackedBatch]:
        while True:
            if self.next >= self.n_seq:
                if not self.repeat:
                    return
                self.next = self.next % max(self.n_seq, 1) if self.n_seq else 0
                if self.n_seq == 0:
                    return
            docs = self.sample(self.next)
            self.next += self.world
            S = (self.seq_len + 127) // 128 * 128
            yield build_packed_batch(docs, self.cfg, seq_len=S)

    def state_dict(self):
        return {"next": self.next}

    def load_state_dict(self, sd):
        self.next = int(sd["next"])


class RandomTokens:
    """Uniform random ids in fixed-length documents: the smoke-run dataset."""

    def __init__(self, cfg: ModelConfig, seq_len: int, doc_len: int = 2048, seed: int = 0):
        self.cfg, self.seq_len, self.doc_len, self.seed, self.i = cfg, seq_len, doc_len, seed, 0

    def __iter__(self) -> Iterator[PackedBatch]:
        while True:
            g = torch.Generator().manual_seed(self.seed + self.i)
            self.i += 1
            docs, left = [], self.seq_len
            while left > 0:
                n = min(self.doc_len, left)
                docs.append(Sample([Segment("text", ids=torch.randint(8, self.cfg.vocab_size, (n,), generator=g), loss=True)]))
                left -= n
            yield build_packed_batch(docs, self.cfg, seq_len=(self.seq_len + 127) // 128 * 128)
