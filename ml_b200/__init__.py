"""ml_b200 — a Blackwell (sm_100a) native multimodal LLM trainer.

Framework layer: PyTorch (flat parameter buffers, process groups, streams, CUDA graphs).
Hot path: hand-written CUDA kernels (tcgen05/TMEM GEMMs fed by TMA, flash attention,
fused norm / RoPE / SwiGLU / cross-entropy / AdamW, in-kernel NVLink collectives) in
``ml_b200/csrc`` exposed through a C ABI (``ml_b200.ops.native``).
Host runtime (token loader, checkpoint IO, metrics writers, RNG init) is C++ in the same tree.
"""
from .config import Config, VisionConfig, RunConfig  # noqa: F401

__version__ = "0.1.0"
