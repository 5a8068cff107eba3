"""Shared by the examples: make the package importable from a source checkout and pick the device."""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch


def device() -> torch.device:
    return torch.device("cuda" if torch.cuda.is_available() else "cpu")
