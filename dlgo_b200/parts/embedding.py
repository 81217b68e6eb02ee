"""Token embedding and the output head.

Embedding: ``x = E[token, :]`` with no scaling for this architecture
(models/llm/forward.go:132-135).  Head: ``logits = O . x`` in fp32, with
``O = E`` when the weights are tied (models/llm/forward.go:193-197,
models/llm/loader.go:74-76).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional

import torch

from ..csrc import kernels as K
from .base import ParamSpec, Part
from .linear import STORE_F32, Linear
from .registry import EMBEDDINGS, HEADS


class TokenEmbedding(Part):
    """``name``: the table's tensor name below the part's prefix."""

    def __init__(self, vocab_size: int, hidden_size: int, name: str = "weight"):
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size, name=name)
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)
        self.name = name
        self.table: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.vocab_size, self.hidden_size))}

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        self.table = runtime.compute_copy(get(self.name)).contiguous()

    def forward(self, token_ids: torch.Tensor, copies: Optional[int] = None) -> torch.Tensor:
        """fp32 rows [T, hidden]; with ``copies`` = s, [T, s, hidden] with every copy equal (residual streams)."""
        return K.embed(token_ids, self.table, copies=copies)


class LinearHead(Part):
    """``tied_to`` names the tensor (absolute name) the head shares, or ``None`` for a weight of its own."""

    def __init__(self, vocab_size: int, hidden_size: int, tied_to: Optional[str] = None, name: str = "weight"):
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size, tied_to=tied_to, name=name)
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)
        self.tied_to = tied_to
        self.name = name
        self.proj: Optional[Linear] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {} if self.tied_to else {self.name: ParamSpec((self.vocab_size, self.hidden_size))}

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        self.proj = Linear(get(self.name), runtime)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj(x, STORE_F32)


EMBEDDINGS.register("token_embedding", TokenEmbedding)
HEADS.register("linear_head", LinearHead)
