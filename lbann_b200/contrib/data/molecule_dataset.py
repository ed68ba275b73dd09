"""Molecular text data sets for the Python-dataset reader
(python/lbann/contrib/data/molecule_dataset.py): one molecule per line, tokenized, aligned to
a fixed sequence length and masked for masked-language-model training.

A sample is ``[input ids | labels]`` (each ``seqlen`` long; with ``attn_mask`` a third block of
0/1 attention weights): BERT-style masking picks ``mlm_probability`` of the real tokens; of
those 80 % become ``[MASK]``, 10 % a random vocabulary entry, 10 % stay; labels are the original
ids at the picked positions and -100 (ignored) elsewhere.
"""
from __future__ import annotations

from typing import List, Sequence, Union

import numpy as np

from ...util.data import Dataset, Sample, SampleDims
from .chem_tokenizers import TOKENIZERS, ChemTokenType, SPECIAL

IGNORE = -100


class TextDataset:
    """All non-empty lines of one or more text files, in memory."""

    def __init__(self, file_or_files: Union[str, Sequence[str]]):
        files = [file_or_files] if isinstance(file_or_files, str) else list(file_or_files)
        self.lines: List[str] = []
        for name in files:
            with open(name) as f:
                self.lines.extend(line.strip() for line in f if line.strip())

    def __len__(self):
        return len(self.lines)

    def __getitem__(self, i: int) -> str:
        return self.lines[i]


class TextDatasetWithOffsets:
    """Lines read on demand: ``<file>.offsets`` holds, as uint64, the byte position of the
    newline that ends each line (written by ``write_offsets``); nothing is kept in memory, so
    the object pickles small and data sets larger than memory work."""

    def __init__(self, file_or_files: Union[str, Sequence[str]]):
        self.files = [file_or_files] if isinstance(file_or_files, str) else list(file_or_files)
        counts = [np.memmap(f + ".offsets", dtype=np.uint64, mode="r").shape[0] for f in self.files]
        self.cum = np.cumsum(np.asarray(counts, dtype=np.int64))
        self._maps = None

    @staticmethod
    def write_offsets(path: str) -> int:
        ends, pos = [], 0
        with open(path, "rb") as f:
            for line in f:
                pos += len(line)
                ends.append(pos - 1 if line.endswith(b"\n") else pos)
        np.asarray(ends, dtype=np.uint64).tofile(path + ".offsets")
        return len(ends)

    def __len__(self):
        return int(self.cum[-1]) if len(self.cum) else 0

    def __getstate__(self):
        st = dict(self.__dict__)
        st["_maps"] = None                    # memory maps are reopened in the worker
        return st

    def __getitem__(self, i: int) -> str:
        if self._maps is None:
            self._maps = [(np.memmap(f + ".offsets", dtype=np.uint64, mode="r"),
                           np.memmap(f, dtype=np.uint8, mode="r")) for f in self.files]
        f = int(np.searchsorted(self.cum, i, side="right"))
        local = i - (int(self.cum[f - 1]) if f else 0)
        off, data = self._maps[f]
        start = 0 if local == 0 else int(off[local - 1]) + 1
        return bytes(data[start:int(off[local])]).decode("utf-8").strip()


class ChemTextDataset(Dataset):
    def __init__(self, fname, vocab: str, seqlen: int, tokenizer_type: ChemTokenType = ChemTokenType.SMILES,
                 mlm_probability: float = 0.15, attn_mask: bool = False, input_type: ChemTokenType = None,
                 use_offsets: bool = False, seed: int = 0):
        self.text = TextDatasetWithOffsets(fname) if use_offsets else TextDataset(fname)
        self.tokenizer = TOKENIZERS[tokenizer_type](vocab)
        if input_type not in (None, tokenizer_type):
            raise NotImplementedError("conversion between molecule notations needs the selfies / atomInSmiles packages")
        self.seqlen, self.mlm_probability, self.attn_mask = int(seqlen), float(mlm_probability), bool(attn_mask)
        self.seed = int(seed)
        self.special_ids = {self.tokenizer.vocab[s] for s in SPECIAL}

    def __len__(self) -> int:
        return len(self.text)

    def get_sample_dims(self) -> SampleDims:
        return SampleDims(sample=[self.seqlen * (3 if self.attn_mask else 2)])

    def mask_tokens(self, ids: np.ndarray, rng: np.random.Generator):
        """(masked input, labels) by BERT's rule."""
        ids = ids.copy()
        labels = np.full_like(ids, IGNORE)
        real = np.array([i not in self.special_ids for i in ids])
        pick = real & (rng.random(ids.shape[0]) < self.mlm_probability)
        labels[pick] = ids[pick]
        roll = rng.random(ids.shape[0])
        ids[pick & (roll < 0.8)] = self.tokenizer.mask_token_id
        rand = pick & (roll >= 0.8) & (roll < 0.9)
        ids[rand] = rng.integers(len(SPECIAL), len(self.tokenizer), size=int(rand.sum()))
        return ids, labels

    def __getitem__(self, index: int) -> Sample:
        ids = np.asarray(self.tokenizer.encode(self.text[index], max_length=self.seqlen), dtype=np.int64)
        rng = np.random.default_rng([self.seed, index])          # the same masks every epoch per (seed, index)
        masked, labels = self.mask_tokens(ids, rng)
        parts = [masked, labels]
        if self.attn_mask:
            parts.append((ids != self.tokenizer.pad_token_id).astype(np.int64))
        return Sample(sample=np.concatenate(parts).astype(np.float32))
