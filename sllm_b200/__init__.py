"""sllm_b200: a single-GPU inference engine for the Qwen2.5 dense architecture,
written for NVIDIA B200 (sm_100a)."""

__version__ = "0.1.0"
