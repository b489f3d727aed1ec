"""From a model folder (or a configuration and a seed) to a bound model on a device."""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..config import config_from_dict, load_config
from ..models import build_model, declare_tensors
from ..weights import draw, load_weights

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute dtype must be bfloat16 or float32, got {name}")
        return name
    try:
        return DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"unknown dtype {name!r}; one of {sorted(DTYPES)}") from None


def require_cuda(device) -> torch.device:
    """The product runs on a CUDA device only; say so instead of falling back."""
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError(f"neurogrid_b200 runs on a CUDA device (sm_100a); got device {device!r}")
    if not torch.cuda.is_available():
        raise RuntimeError("neurogrid_b200 needs a CUDA device and its hand-written kernels; "
                           "no GPU is visible and there is no CPU path")
    if dev.index is not None:
        torch.cuda.set_device(dev)
    torch.backends.cuda.matmul.allow_tf32 = False     # the float32 path is true 32-bit
    torch.backends.cudnn.allow_tf32 = False
    return dev


def model_from_dir(model_dir: str, *, dtype, device):
    """(config, model) for the folder's config.json and safetensors."""
    dtype = parse_dtype(dtype)
    cfg = load_config(model_dir)
    spec = cfg.model_spec()
    weights = load_weights(model_dir, declare_tensors(spec))
    return cfg, build_model(spec, weights, dtype=dtype, device=device)


def model_from_seed(config: Mapping, seed: int, *, dtype, device):
    """(config, model) with weights drawn on the device from ``seed`` (no folder is written).
    The draw uses the device's generator, so it differs from the folder that
    ``write_random_model`` writes for the same seed."""
    dtype = parse_dtype(dtype)
    cfg = config_from_dict(config)
    spec = cfg.model_spec()
    weights = draw(declare_tensors(spec), seed, dtype=torch.bfloat16, device=device)
    return cfg, build_model(spec, weights, dtype=dtype, device=device)
