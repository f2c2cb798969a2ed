"""Fixed-length samples from a flat file of token ids (``.npy``, or raw little-endian uint16 /
int32 ``.bin``).  Stands where the reference's WikiText-103 loader stands
(examples/wikitext_dataset.py:12-96); tokenising a corpus needs network access or a local
tokenizer and is left to the user (``sentencepiece`` / ``transformers`` are importable)."""
from __future__ import annotations

import numpy as np
import torch


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
