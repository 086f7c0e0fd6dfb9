"""Small tensor helpers (src/python/pytorch/recstore/dist_utils.py:6-45)."""
import torch


def toindex(data, dtype=torch.int64):
    return torch.as_tensor(data, dtype=dtype)


def toTensor(index):
    return torch.as_tensor(index)


def attach_grad(t: torch.Tensor) -> torch.Tensor:
    return t.detach().requires_grad_(True)


def boolean_mask(t: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    return t[mask.bool()]


def _prefix(name: str, prefix: str) -> str:
    return f"{prefix}:{name}"


def get_data_name(name: str) -> str:
    return _prefix(name, "data")


def get_emb_name(name: str) -> str:
    return _prefix(name, "emb")
