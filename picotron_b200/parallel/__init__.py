"""Parallelism strategies: tensor (Megatron 1-D), pipeline (AFAB, 1F1B), context (ring attention), data (bucketed)."""
