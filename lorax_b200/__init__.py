"""lorax_b200: a multi-LoRA inference server written for NVIDIA B200 (sm_100a).

One base model is served together with many LoRA adapters that are selected per
request.  The framework layer is PyTorch, the hot operators are hand-written
CUDA kernels for sm_100a (tcgen05 / TMEM / TMA), and tensor parallelism runs as
one process per GPU over NCCL with fused compute+collective kernels on NVLink
peer memory.
"""

__version__ = "0.1.0"
