"""Named random-number generators of a process (include/lbann/utils/random_number_generators.hpp,
src/utils/random.cpp:40-330).

* ``generator``: model randomness (initialisers, dropout masks); differs per rank.
* ``fast_generator``: the same role for code that trades quality for speed; differs per rank.
* ``data_seq_generator``: the order in which samples are visited; THE SAME on every rank, so
  that all ranks shuffle alike without communicating (``data_order`` draws an epoch's order).
* ``io_generator(thread)``: one per I/O thread (augmentation in the transforms); differs per
  rank and thread.
* ``ltfb_generator``: tournament pairing; the same on every rank of EVERY trainer.

All are NumPy ``Generator`` objects over PCG64, so their full state is a small dictionary
that the checkpoints carry per rank.
"""
from __future__ import annotations

import json
from typing import Dict, List, Optional

import numpy as np


def _gen(*words) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(np.random.SeedSequence([int(w) & 0xFFFFFFFF for w in words])))


def data_order(seed: int, indices: np.ndarray, epoch: int) -> np.ndarray:
    """The visiting order of an epoch: a permutation from a stream of the data-sequence family
    that depends on (seed, epoch) only, so every rank of every trainer draws the same one, and a
    restarted run reproduces it without replaying earlier epochs."""
    order = np.array(indices, copy=True)
    _gen(seed, 3, 1000003 + int(epoch)).shuffle(order)
    return order


class GeneratorBanks:
    def __init__(self):
        self.seed = 0
        self.init(42)

    def init(self, seed: int, rank_in_world: int = 0, rank_in_trainer: int = 0, trainer: int = 0,
             num_io_threads: int = 1):
        self.seed = int(seed)
        self.generator = _gen(seed, 1, rank_in_world)
        self.fast_generator = _gen(seed, 2, rank_in_world)
        self.data_seq_generator = _gen(seed, 3)                   # no rank, no trainer: identical everywhere
        self.ltfb_generator = _gen(seed, 4)                       # identical everywhere
        self._io: List[np.random.Generator] = [_gen(seed, 5, rank_in_world, t) for t in range(max(1, num_io_threads))]
        self._where = (rank_in_world, rank_in_trainer, trainer)

    def io_generator(self, thread: int = 0) -> np.random.Generator:
        while thread >= len(self._io):                            # a pool that grew after init
            self._io.append(_gen(self.seed, 5, self._where[0], len(self._io)))
        return self._io[thread]

    def data_order(self, indices: np.ndarray, epoch: int) -> np.ndarray:
        return data_order(self.seed, indices, epoch)

    # ---- checkpoints
    def state(self) -> Dict[str, object]:
        names = {"generator": self.generator, "fast_generator": self.fast_generator,
                 "data_seq_generator": self.data_seq_generator, "ltfb_generator": self.ltfb_generator}
        out = {k: g.bit_generator.state for k, g in names.items()}
        out["io_generators"] = [g.bit_generator.state for g in self._io]
        out["seed"] = self.seed
        return out

    def load_state(self, st: Dict[str, object]):
        self.seed = int(st.get("seed", self.seed))
        for k in ("generator", "fast_generator", "data_seq_generator", "ltfb_generator"):
            if k in st:
                getattr(self, k).bit_generator.state = st[k]
        for t, s in enumerate(st.get("io_generators", [])):
            self.io_generator(t).bit_generator.state = s

    def dumps(self) -> str:
        return json.dumps(self.state())

    def loads(self, text: str):
        self.load_state(json.loads(text))


_banks: Optional[GeneratorBanks] = None


def banks() -> GeneratorBanks:
    global _banks
    if _banks is None:
        _banks = GeneratorBanks()
    return _banks


def init_random(seed: int, rank_in_world: int = 0, rank_in_trainer: int = 0, trainer: int = 0,
                num_io_threads: int = 1) -> GeneratorBanks:
    b = banks()
    b.init(seed, rank_in_world, rank_in_trainer, trainer, num_io_threads)
    return b


def get_generator(): return banks().generator                     # noqa: E704
def get_fast_generator(): return banks().fast_generator           # noqa: E704
def get_data_seq_generator(): return banks().data_seq_generator   # noqa: E704
def get_ltfb_generator(): return banks().ltfb_generator           # noqa: E704
def get_io_generator(thread: int = 0): return banks().io_generator(thread)   # noqa: E704
