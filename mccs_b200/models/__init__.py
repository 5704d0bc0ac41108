"""Model zoo of the data-parallel training drivers: ResNet-50, VGG-16 (the networks of the
reference's workload traces) and GPT-2-medium. ResNet-50 and VGG-16 come from torchvision (random
init, no weights are downloaded); GPT-2-medium is defined here."""
from __future__ import annotations

import torch

from .gpt2 import GPT2, GPT2Config, gpt2_medium, gpt2_tiny


def build(name: str) -> torch.nn.Module:
    name = name.lower()
    if name in ("gpt2-medium", "gpt2_medium", "gpt2"):
        return gpt2_medium()
    if name in ("gpt2-tiny", "gpt2_tiny"):
        return gpt2_tiny()
    import torchvision
    if name == "resnet50":
        return torchvision.models.resnet50(weights=None)
    if name == "vgg16":
        return torchvision.models.vgg16(weights=None)
    if name == "resnet18":
        return torchvision.models.resnet18(weights=None)
    raise ValueError(f"unknown model '{name}'")


def is_language_model(name: str) -> bool:
    return name.lower().startswith("gpt2")


__all__ = ["build", "is_language_model", "GPT2", "GPT2Config", "gpt2_medium", "gpt2_tiny"]
