"""A single-GPU inference engine for the Qwen2.5 dense architecture on NVIDIA B200 (sm_100a).

Importing the package switches off the reduced-precision float32 matrix mode
(TF32) and reduced-precision bfloat16 reductions of the library matrix product,
so that `dtype="float32"` is a true 32-bit path.
"""

import torch as _torch

_torch.backends.cuda.matmul.allow_tf32 = False
_torch.backends.cudnn.allow_tf32 = False
_torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

__version__ = "0.1.0"

from .engine import LLM, Engine, StepEntry  # noqa: E402
from .sampling import SamplingParams  # noqa: E402

__all__ = ["LLM", "Engine", "StepEntry", "SamplingParams"]
