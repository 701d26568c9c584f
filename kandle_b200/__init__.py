"""kandle_b200: a B200 (sm_100a) compute backend for the Kandle tensor framework.

Layers, bottom up:
  libkandle_cuda.so   hand-written CUDA kernels behind a flat C ABI (include/kandle_cuda.h)
  lib                 ctypes binding of that ABI
  backend / kernels   `CudaBackend`: Kandle's backend contract (createTensorHandle + operator registry)
  core / nn           the dispatch layer and modules the models are written against
  model_utils         Qwen3 and Whisper-encoder modules issuing the reference's operator sequence
  engine              fused bf16 fast path (tensor-core GEMM / attention, CUDA-graph decode)

Importing the package needs the built library; there is no CPU fallback.
"""
from . import lib  # noqa: F401  (fails loudly when the shared library is missing)
from .backend import CudaBackend, CudaTensorHandle  # noqa: F401
from .core import Tensor, env, functional, init  # noqa: F401
