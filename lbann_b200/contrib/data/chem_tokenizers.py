"""Tokenizers for molecules written as text (python/lbann/contrib/data/chem_tokenizers.py).

``SMILESTokenizer`` splits a SMILES string into chemically meaningful tokens (bracket atoms,
two-letter elements, ring-bond labels, bonds); ``CharTokenizer`` takes characters.  Both map
tokens to ids through a vocabulary file with one entry per line, whose special entries are
``[PAD] [UNK] [CLS] [SEP] [MASK]`` (the BERT convention of the reference's vocabularies).
SELFIES and atom-in-SMILES inputs need the ``selfies`` / ``atomInSmiles`` packages, absent here:
asking for them raises with that message.
"""
from __future__ import annotations

import re
from enum import Enum, auto
from typing import Dict, List, Sequence

SPECIAL = ("[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]")
# bracket atoms, %(nnn) and %nn ring labels, two-letter halogens before single letters
_SMILES = re.compile(r"(\%\([0-9]{3}\)|\[[^\]]+]|Br?|Cl?|N|O|S|P|F|I|b|c|n|o|s|p|\||\(|\)|\.|=|#|-|\+|\\|\/|:|~|@|\?|>>?|\*|\$|\%[0-9]{2}|[0-9])")


class ChemTokenType(Enum):
    SMILES = auto()
    SELFIES = auto()
    AIS = auto()


class ChemTokenizer:
    def __init__(self, vocab_file: str = None, vocab: Sequence[str] = None):
        if vocab is None:
            with open(vocab_file) as f:
                vocab = [line.rstrip("\n") for line in f if line.strip()]
        self.vocab: Dict[str, int] = {tok: i for i, tok in enumerate(vocab)}
        missing = [s for s in SPECIAL if s not in self.vocab]
        if missing:
            raise ValueError(f"vocabulary lacks the special tokens {missing}")
        self.ids_to_tokens = {i: t for t, i in self.vocab.items()}
        self.pad_token_id, self.unk_token_id = self.vocab["[PAD]"], self.vocab["[UNK]"]
        self.cls_token_id, self.sep_token_id = self.vocab["[CLS]"], self.vocab["[SEP]"]
        self.mask_token_id = self.vocab["[MASK]"]

    def __len__(self):
        return len(self.vocab)

    def tokenize(self, text: str) -> List[str]:
        raise NotImplementedError

    def encode(self, text: str, max_length: int = None, padding: bool = True) -> List[int]:
        """[CLS] tokens [SEP], truncated and padded to ``max_length``."""
        ids = [self.vocab.get(t, self.unk_token_id) for t in self.tokenize(text)]
        if max_length is not None:
            ids = ids[:max_length - 2]
        ids = [self.cls_token_id] + ids + [self.sep_token_id]
        if max_length is not None and padding:
            ids += [self.pad_token_id] * (max_length - len(ids))
        return ids

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        toks = [self.ids_to_tokens.get(int(i), "[UNK]") for i in ids]
        if skip_special_tokens:
            toks = [t for t in toks if t not in SPECIAL]
        return "".join(toks)

    @staticmethod
    def build_vocab(texts: Sequence[str], tokenize) -> List[str]:
        seen: Dict[str, None] = {}
        for t in texts:
            for tok in tokenize(t):
                seen.setdefault(tok)
        return list(SPECIAL) + sorted(seen)


class SMILESTokenizer(ChemTokenizer):
    def tokenize(self, text: str) -> List[str]:
        text = text[text.find("|") + 1:]                 # "name|SMILES" lines keep the molecule
        return _SMILES.findall(text.strip())


class CharTokenizer(ChemTokenizer):
    def tokenize(self, text: str) -> List[str]:
        return list(text.strip())


def _needs(package):
    def make(*a, **k):
        raise ModuleNotFoundError(f"this tokenizer needs the '{package}' package, which is not installed")
    return make


TOKENIZERS = {ChemTokenType.SMILES: SMILESTokenizer, ChemTokenType.SELFIES: _needs("selfies"),
              ChemTokenType.AIS: _needs("atomInSmiles")}
