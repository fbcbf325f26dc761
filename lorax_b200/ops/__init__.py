"""Operator layer.

``get_ops(device, dtype)`` returns the module whose functions implement the operators for that tensor
placement: :mod:`native` (hand-written sm_100a kernels) for bf16 tensors on a CUDA device, and
:mod:`reference` (plain PyTorch) on the CPU, where it doubles as the numerical oracle.  On a CUDA device
the native library is mandatory -- a missing build raises instead of silently running eager PyTorch.
"""

from __future__ import annotations

import torch

from . import reference


def get_ops(device, dtype=torch.bfloat16):
    device = torch.device(device)
    if device.type == "cuda":
        if dtype != torch.bfloat16:
            raise ValueError("the CUDA kernels are bf16; got %s" % dtype)
        from . import native
        native.load()
        return native
    return reference
