"""B200-native Mamba-2 / Mamba-2-hybrid training and inference framework.

Layout:
  models/    HuggingFace-compatible configs and model classes, presets, decode cache
  ops/       sm_100a CUDA kernels (csrc/), their autograd wrappers, and the PyTorch oracle
  parallel/  TP/SP/ZeRO-1 runtime: process groups, parallel layers, fused comm kernels, checkpoints
  utils/     logging, throughput/MFU, data loading, profiling and debugging helpers
"""
__version__ = "0.1.0"
