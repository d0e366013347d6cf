"""B200-native (sm_100a) int4 decode step for Qwen3.5-4B-shaped models, behind LoveManna/deltaforge's op API.

Importing the package does not load the CUDA library; the first op call or engine construction does,
and raises if ``libdfb200.so`` is missing and cannot be built. There is no CPU path.
"""

from .config import ModelConfig, qwen3_5_4b_config, tiny_config  # noqa: F401

__all__ = ["ModelConfig", "qwen3_5_4b_config", "tiny_config"]
