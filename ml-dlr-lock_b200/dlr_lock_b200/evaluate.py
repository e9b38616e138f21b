"""Perplexity of a locked model with the CUDA library under its DLR-Nets: the consumer of the forward that
the reference's quality evaluation uses first (``evaluate_ppl``, dlr_lock/eval_benchmarks.py:89-100).

The reference draws fixed-length token chunks from a tokenised corpus (dlr_lock/data.py:79-112) and averages
the causal-LM loss over ``n_steps`` batches.  Corpora and tokenisers are not available offline, so the
stream here is synthetic, in the way the reference's own smoke test replaces its corpus loader
(examples/smoke_test.py:40-48): sentences of a small word list, mapped to token ids, cut into chunks and
served in a seeded shuffled order.  ``evaluate_ppl`` itself takes any iterator of ``(batch, seq_len)`` id
tensors, so a real tokenised stream plugs in unchanged.
"""
from __future__ import annotations

import math
import random
from typing import Iterator

import torch


class ChunkStream:
    """Infinite shuffled iterator over fixed-length token chunks (dlr_lock/data.py:79-101)."""

    def __init__(self, chunks: torch.Tensor, batch_size: int, seed: int):
        self.chunks = chunks
        self.batch_size = batch_size
        self._gen = torch.Generator().manual_seed(seed)
        self._order = torch.randperm(len(chunks), generator=self._gen)
        self._pos = 0

    def __iter__(self):
        return self

    def __next__(self) -> torch.Tensor:
        if self._pos + self.batch_size > len(self._order):
            self._order = torch.randperm(len(self.chunks), generator=self._gen)
            self._pos = 0
        idx = self._order[self._pos:self._pos + self.batch_size]
        self._pos += self.batch_size
        return self.chunks[idx]


def synthetic_token_stream(vocab_size: int, seq_len: int, batch_size: int, seed: int = 42, n_sentences: int = 800,
                           words_per_sentence: int = 30, n_words: int = 14) -> ChunkStream:
    """A corpus of ``n_sentences`` sentences over ``n_words`` distinct "words" (each a fixed short run of token
    ids below ``vocab_size``), concatenated and cut into ``seq_len`` chunks."""
    rng = random.Random(1)
    words = [[rng.randrange(vocab_size) for _ in range(rng.randint(1, 3))] for _ in range(n_words)]
    ids = []
    for _ in range(n_sentences):
        for _ in range(words_per_sentence):
            ids.extend(rng.choice(words))
    n_chunks = len(ids) // seq_len
    if n_chunks < batch_size:
        raise ValueError("corpus too short for one batch of this sequence length")
    chunks = torch.tensor(ids[:n_chunks * seq_len], dtype=torch.long).view(n_chunks, seq_len)
    return ChunkStream(chunks, batch_size, seed)


@torch.no_grad()
def evaluate_ppl(model, stream: Iterator[torch.Tensor], n_steps: int, device) -> float:
    """exp(mean causal-LM loss) over ``n_steps`` batches of the stream (dlr_lock/eval_benchmarks.py:89-100)."""
    model.eval()
    total = 0.0
    for _ in range(n_steps):
        ids = next(stream).to(device)
        total += model(input_ids=ids, labels=ids).loss.item()
    return math.exp(total / max(n_steps, 1))
