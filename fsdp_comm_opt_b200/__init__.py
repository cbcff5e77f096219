"""B200-native compressed collectives for PyTorch FSDP2 training.

Layout:
  ops/       codec front end, fused elementwise / optimizer / attention / GEMM ops (sm_100a kernels
             with a plain PyTorch path for CPU tensors)
  parallel/  FSDP2 comm hooks, AggregatedWork, symmetric-memory channels, wrapping helpers
  models/    Llama-shape and GPT-2-shape decoders built from the ops above
  utils/     timers, metrics, checkpointing, synthetic data, failure detection
  csrc/      C++ / CUDA sources of the two in-tree shared objects
"""
__version__ = "0.1.0"
