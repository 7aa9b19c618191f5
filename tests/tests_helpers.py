"""Small helpers shared by the tests."""
import torch

import plain_qwen3 as P


def read_all(path):
    """name -> tensor in its stored dtype, through the plain reader."""
    return P.read_safetensors(path)
