"""Low-rank token embedding: ``E = fingerprints[V, r] @ basis[r, d]``.

Parity: ``UniversalAdaptiveEmbedding`` (``triune/model/manifold_embedding.py:8-51``): lookup through the rank-r
fingerprint table, logits computed in the r-dimensional space (``h @ basis^T`` then against the fingerprints), optional
top-k, initialisation from a dense embedding by a randomised range finder + small SVD.
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


class UniversalAdaptiveEmbedding(nn.Module):
    def __init__(self, vocab_size: int = 131072, hidden_dim: int = 1536, rank: int = 64):
        super().__init__()
        self.vocab_size, self.hidden_dim, self.rank = vocab_size, hidden_dim, rank
        self.fingerprints = nn.Embedding(vocab_size, rank)
        self.basis = nn.Linear(rank, hidden_dim, bias=False)
        nn.init.normal_(self.fingerprints.weight, std=1.0 / math.sqrt(rank))
        nn.init.orthogonal_(self.basis.weight)

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.basis(self.fingerprints(input_ids))

    def compute_logits(self, hidden_states: torch.Tensor, top_k: Optional[int] = None):
        """[.., d] -> [.., V] (or ``(values, indices)`` of the top-k): 2*r*(d+V) flops per token instead of 2*d*V."""
        scores = F.linear(hidden_states @ self.basis.weight, self.fingerprints.weight)
        if top_k is None or top_k >= self.vocab_size:
            return scores
        top = torch.topk(scores, k=top_k, dim=-1)
        return top.values, top.indices

    @classmethod
    def from_pretrained_weights(cls, weight: torch.Tensor, rank: int = 64, oversample: int = 8) -> "UniversalAdaptiveEmbedding":
        V, D = weight.shape
        rank = min(rank, V, D)
        w = weight.detach().float()
        q = min(rank + oversample, V, D)
        Q, _ = torch.linalg.qr(w @ torch.randn(D, q, device=w.device))  # range of W
        U, S, Vh = torch.linalg.svd(Q.t() @ w, full_matrices=False)    # small [q, D] problem
        root = S[:rank].sqrt()
        mod = cls(V, D, rank)
        with torch.no_grad():
            mod.fingerprints.weight.copy_(((Q @ U[:, :rank]) * root).to(weight.dtype))
            mod.basis.weight.copy_((root.unsqueeze(1) * Vh[:rank]).t().to(weight.dtype))
        return mod.to(weight.device)
