"""Model families. The framework trains Llama-architecture decoders (SmolLM, Llama-2, Llama-3.x shapes)."""
from .llama import (Attention, DecoderLayer, Embedding, FinalProjection, Linear, Llama, MLP, RMSNorm,
                    lm_head_loss)

__all__ = ["Attention", "DecoderLayer", "Embedding", "FinalProjection", "Linear", "Llama", "MLP", "RMSNorm",
           "lm_head_loss"]
