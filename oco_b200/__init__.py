"""B200-native mixture-of-experts layer behind the expert-layer operator interface of xhjkl/oco.

`oco_b200.synth` (numpy only) builds seeded layers in GGUF block layouts; `oco_b200.moe` drives the
CUDA library through its C ABI and needs PyTorch with a CUDA device. Nothing here computes on the CPU.
"""
__all__ = ["synth"]
