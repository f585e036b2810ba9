"""Model families: multi-exit MoE ``TriuneTransformer`` and dense ``UniversalTransformer``."""

from .attention import HybridAttention, SoftmaxAttention, VectorisedGLA
from .block import DenseFFN, TransformerBlock
from .moe import MoE_FFN, RoutingResult
from .norms import RMSNorm
from .rotary import RotaryEmbedding
from .router import GumbelSoftmaxRouter
from .transformer import TriuneTransformer

__all__ = [
    "HybridAttention", "SoftmaxAttention", "VectorisedGLA", "DenseFFN", "TransformerBlock", "MoE_FFN",
    "RoutingResult", "RMSNorm", "RotaryEmbedding", "GumbelSoftmaxRouter", "TriuneTransformer",
]
