"""Seeded synthetic tensors shared by the fixture generator and the parity tests.

numpy's legacy RandomState stream is frozen across numpy versions, so inputs are
regenerated from seeds on any machine instead of being stored in the fixtures.
"""
import zlib

import numpy as np


def randn(seed: int, *shape, scale: float = 1.0) -> np.ndarray:
    return (np.random.RandomState(seed).standard_normal(shape) * scale).astype(np.float32)


def _name_seed(seed: int, name: str) -> int:
    return (seed * 1000003 + zlib.crc32(name.encode())) % (2 ** 31 - 1)


def param_value(seed: int, name: str, shape) -> np.ndarray:
    """Deterministic value for a named module parameter.

    LayerNorm / norm weights are centred on 1, LayerScale gammas on 0.5 (so the attention branch
    is visible in block outputs), everything else ~N(0, 0.08)."""
    r = np.random.RandomState(_name_seed(seed, name)).standard_normal(tuple(shape)).astype(np.float32)
    leaf = name.split(".")[-1]
    if "norm" in name and leaf == "weight":
        return (1.0 + 0.1 * r).astype(np.float32)
    if leaf == "gamma":
        return (0.5 + 0.05 * r).astype(np.float32)
    return (0.08 * r).astype(np.float32)


def fill_module_(module, seed: int) -> None:
    """Overwrite every parameter of a torch module with param_value(seed, name, shape)."""
    import torch
    with torch.no_grad():
        for name, p in module.named_parameters():
            p.copy_(torch.from_numpy(param_value(seed, name, p.shape)))


def model_param_value(seed: int, name: str, shape) -> np.ndarray:
    """Deterministic value for a parameter of a whole model: matrices and convolutions ~N(0, 1/fan_in) so that
    activations keep their scale through many layers, norm weights centred on 1, LayerScale gammas on 0.3,
    other vectors (biases, tokens) ~N(0, 0.02)."""
    r = np.random.RandomState(_name_seed(seed, name)).standard_normal(tuple(shape)).astype(np.float32)
    leaf = name.split(".")[-1]
    if "norm" in name and leaf == "weight":
        return (1.0 + 0.1 * r).astype(np.float32)
    if leaf == "gamma":
        return (0.3 + 0.03 * r).astype(np.float32)
    if len(shape) >= 2 and leaf == "weight":
        fan_in = int(np.prod(shape[1:]))
        return (r / np.sqrt(max(fan_in, 1))).astype(np.float32)
    return (0.02 * r).astype(np.float32)


def fill_model_(module, seed: int) -> None:
    """Overwrite every parameter of a torch module with model_param_value(seed, name, shape)."""
    import torch
    with torch.no_grad():
        for name, p in module.named_parameters():
            p.copy_(torch.from_numpy(model_param_value(seed, name, p.shape)).to(p.dtype))
