"""Token-file datasets for the training examples.

``TokenFileDataset`` serves fixed-length samples from a flat file of token ids (``.npy``, or raw
little-endian ``uint16`` / ``int32`` ``.bin``).  ``build_token_cache`` turns a plain-text corpus
(for instance the WikiText-103 ``wiki.train.tokens`` file) into such a file once and reuses it
afterwards, which is what the reference's loader does with the GPT-2 tokeniser
(examples/wikitext_dataset.py:12-96).  No corpus or tokeniser is downloaded here: pass a local
SentencePiece model (``--spm``) or a local Hugging Face tokeniser directory (``--hf``); without
either the text is encoded as UTF-8 bytes (vocabulary 256 + an end-of-document id), which needs
nothing installed and is enough for smoke runs.

    python examples/text_dataset.py --text wiki.train.tokens --out wiki.train.bin [--spm m.model]
"""
from __future__ import annotations

import argparse
import os
from typing import Callable, Iterable, Optional

import numpy as np
import torch

BYTE_EOD = 256          # end-of-document id of the byte-level fallback


class TokenFileDataset(torch.utils.data.Dataset):
    def __init__(self, path: str, sample_len: int, dtype: str = "uint16"):
        if path.endswith(".npy"):
            self.tokens = np.load(path, mmap_mode="r")
        else:
            self.tokens = np.memmap(path, dtype=dtype, mode="r")
        self.sample_len = sample_len
        self.n = max(0, (len(self.tokens) - 1) // sample_len)
        if self.n == 0:
            raise ValueError(f"{path} holds fewer than {sample_len} tokens")

    def __len__(self) -> int:
        return self.n

    def __getitem__(self, i: int) -> torch.Tensor:
        lo = (i % self.n) * self.sample_len
        return torch.from_numpy(np.asarray(self.tokens[lo:lo + self.sample_len]).astype(np.int64))


def byte_tokenizer(text: str) -> list:
    return list(text.encode("utf-8"))


def load_tokenizer(spm: Optional[str] = None, hf: Optional[str] = None) -> tuple:
    """Returns ``(encode, vocab_size, eod_id)`` from local files only."""
    if spm:
        import sentencepiece as sp
        m = sp.SentencePieceProcessor(model_file=spm)
        eod = m.eos_id() if m.eos_id() >= 0 else m.vocab_size() - 1
        return (lambda t: m.encode(t)), m.vocab_size(), eod
    if hf:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(hf, local_files_only=True)
        eod = tok.eos_token_id if tok.eos_token_id is not None else len(tok) - 1
        return (lambda t: tok.encode(t, add_special_tokens=False)), len(tok), eod
    return byte_tokenizer, 257, BYTE_EOD


def _documents(lines: Iterable[str]) -> Iterable[str]:
    """WikiText layout: a line `` = Title = `` starts an article; blank lines separate paragraphs."""
    doc = []
    for line in lines:
        s = line.strip()
        if s.startswith("= ") and s.endswith(" =") and not s.startswith("= ="):
            if doc:
                yield "\n".join(doc)
            doc = [s]
        elif s:
            doc.append(s)
    if doc:
        yield "\n".join(doc)


def build_token_cache(text_path: str, out_path: str, encode: Callable[[str], list] = byte_tokenizer,
                      vocab_size: int = 257, eod_id: int = BYTE_EOD, force: bool = False) -> str:
    """Tokenise ``text_path`` document by document (an end-of-document id after each) into
    ``out_path`` (``uint16`` when the vocabulary fits, else ``int32``); an existing cache newer than
    the text is kept."""
    if not force and os.path.exists(out_path) and os.path.getmtime(out_path) >= os.path.getmtime(text_path):
        return out_path
    dtype = np.uint16 if vocab_size <= 65536 else np.int32
    with open(text_path, encoding="utf-8") as f, open(out_path + ".tmp", "wb") as out:
        for doc in _documents(f):
            ids = encode(doc) + [eod_id]
            np.asarray(ids, dtype=dtype).tofile(out)
    os.replace(out_path + ".tmp", out_path)
    return out_path


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--text", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--spm", default="")
    ap.add_argument("--hf", default="")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args(argv)
    encode, vocab, eod = load_tokenizer(a.spm or None, a.hf or None)
    path = build_token_cache(a.text, a.out, encode, vocab, eod, a.force)
    n = os.path.getsize(path) // (2 if vocab <= 65536 else 4)
    print(f"{path}: {n} tokens, vocabulary {vocab}, dtype {'uint16' if vocab <= 65536 else 'int32'}")


if __name__ == "__main__":
    main()
