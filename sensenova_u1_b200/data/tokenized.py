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


class JsonlTokenFile:
    """One document per line, ``{"tokens": [ids...]}`` (the format of the reference's ``JsonlDataset``,
    sensenovalm/data/tokenized/single_dataset.py:45-204).  Line offsets come from ``<path>.meta`` when it exists (a
    ``.npy`` array of ``(byte offset, token count)`` rows, as the reference's tokeniser tool writes it), otherwise from
    one scan of the file.  Documents shorter than ``min_length`` tokens are left out; negative ids (the reference
    marks tokens that carry no loss this way) are kept: the packer turns them into context segments without loss."""

    def __init__(self, path: str, min_length: int = 0):
        import json
        self.path, self._json = str(path), json
        meta = Path(self.path + ".meta")
        if meta.exists():
            arr = np.load(meta, allow_pickle=False).reshape(-1, 2)
            rows = [(int(o), int(n)) for o, n in arr]
        else:
            rows, off = [], 0
            with open(self.path, "rb") as f:
                for line in f:
                    if line.strip():
                        rows.append((off, len(json.loads(line)["tokens"])))
                    off += len(line)
        self.rows = [(o, n) for o, n in rows if n >= max(1, min_length)]
        self._fh = None

    def __len__(self):
        return len(self.rows)

    def lengths(self) -> np.ndarray:
        return np.asarray([n for _, n in self.rows], dtype=np.int64)

    def tokens(self, i: int) -> np.ndarray:
        if self._fh is None:
            self._fh = open(self.path, "rb")            # one handle per process (opened after a fork, not before)
        self._fh.seek(self.rows[i][0])
        return np.asarray(self._json.loads(self._fh.readline())["tokens"], dtype=np.int64)


class PackedDocumentDataset:
    """Documents of one or more :class:`JsonlTokenFile` packed into rows of ``seq_len`` tokens.

    * order: a seeded permutation of all documents per epoch (the same on every rank; rank r takes rows r, r + world...);
    * ``mode="cut"``: documents are laid end to end and cut at row boundaries, no padding (the reference's
      ``PackedDatasetWithCut``, packed_dataset.py:268-520); the cut-off tail opens the next row as a document of its own;
    * ``mode="pad"``: only whole documents go into a row (longer ones are truncated to ``seq_len``), the rest of the row is
      padding (``PackedDatasetWithPad``, :522-640);
    * resumable: ``state_dict`` = epoch and next row."""

    def __init__(self, files: Sequence, cfg: ModelConfig, seq_len: int, mode: str = "cut", seed: int = 1024,
                 rank: int = 0, world: int = 1, epochs: int = -1):
        if mode not in ("cut", "pad"):
            raise ValueError("mode is 'cut' or 'pad'")
        self.files = [f if isinstance(f, JsonlTokenFile) else JsonlTokenFile(f) for f in files]
        self.cfg, self.seq_len, self.mode, self.seed = cfg, int(seq_len), mode, int(seed)
        self.rank, self.world, self.epochs = rank, world, epochs
        self.doc_file = np.concatenate([np.full(len(f), i, dtype=np.int64) for i, f in enumerate(self.files)] or [np.zeros(0, np.int64)])
        self.doc_idx = np.concatenate([np.arange(len(f), dtype=np.int64) for f in self.files] or [np.zeros(0, np.int64)])
        self.doc_len = np.concatenate([f.lengths() for f in self.files] or [np.zeros(0, np.int64)])
        if self.doc_len.size == 0:
            raise ValueError("no documents (after the minimum-length filter)")
        self.epoch, self.next = 0, rank
        self._plan_epoch = -1

    def _plan(self):
        """Rows of the current epoch: lists of (document, start, end)."""
        if self._plan_epoch == self.epoch:
            return self._rows
        order = np.random.default_rng(self.seed + self.epoch).permutation(self.doc_len.size)
        rows, cur, room = [], [], self.seq_len
        for d in order:
            n, s = int(self.doc_len[d]), 0
            if self.mode == "pad":
                n = min(n, self.seq_len)
                if n > room:
                    rows.append(cur)
                    cur, room = [], self.seq_len
                cur.append((int(d), 0, n))
                room -= n
                continue
            while s < n:
                take = min(n - s, room)
                cur.append((int(d), s, s + take))
                s, room = s + take, room - take
                if room == 0:
                    rows.append(cur)
                    cur, room = [], self.seq_len
        if cur and self.mode == "pad":
            rows.append(cur)                               # "cut": a last partial row is dropped, as in the reference
        self._rows, self._plan_epoch = rows, self.epoch
        return rows

    def __len__(self):
        return len(self._plan())

    def row_samples(self, r: int) -> List[Sample]:
        out = []
        for d, s, e in self._plan()[r]:
            toks = self.files[int(self.doc_file[d])].tokens(int(self.doc_idx[d]))[s:e]
            # runs of equal sign become segments: negative ids are context without loss
            cuts = np.flatnonzero(np.diff((toks < 0).astype(np.int8))) + 1
            segs = [Segment("text", ids=torch.from_numpy(np.abs(part).copy()), loss=bool(part[0] >= 0))
                    for part in np.split(toks, cuts) if part.size]
            out.append(Sample(segs))
        return out

    def __iter__(self) -> Iterator[PackedBatch]:
        S = (self.seq_len + 127) // 128 * 128
        while self.epochs < 0 or self.epoch < self.epochs:
            rows = self._plan()
            while self.next < len(rows):
                r = self.next
                self.next += self.world
                yield build_packed_batch(self.row_samples(r), self.cfg, seq_len=S)
            self.epoch += 1
            self.next = self.rank

    def state_dict(self):
        return {"epoch": self.epoch, "next": self.next}

    def load_state_dict(self, sd):
        self.epoch, self.next = int(sd["epoch"]), int(sd["next"])
