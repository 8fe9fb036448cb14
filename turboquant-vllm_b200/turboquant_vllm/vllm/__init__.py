"""vLLM plugin: the ``vllm.general_plugins`` entry point is ``register_tq4_backend``
(reference: src/turboquant_vllm/vllm/__init__.py:30-42, pyproject.toml:66-67)."""

from turboquant_vllm.vllm.tq4_backend import (
    TQ4AttentionBackend,
    TQ4AttentionImpl,
    TQ4FullAttentionSpec,
    TQ4MetadataBuilder,
    register_tq4_backend,
)

__all__ = [
    "TQ4AttentionBackend",
    "TQ4AttentionImpl",
    "TQ4FullAttentionSpec",
    "TQ4MetadataBuilder",
    "register_tq4_backend",
]
