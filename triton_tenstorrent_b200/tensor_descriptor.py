"""Host-side tensor descriptor with the fields of triton.tools.tensor_descriptor.TensorDescriptor,
which the reference's examples build (09-persistent-matmul.ttnn.py:158-161, 06-fused-attention.py:243-246)
and its launcher flattens (backend/driver.py:141-159)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch


@dataclass
class TensorDescriptor:
    base: torch.Tensor
    shape: List[int]
    strides: List[int]
    block_shape: List[int]
    padding: str = "zero"

    def __post_init__(self):
        rank = len(self.shape)
        assert len(self.strides) == rank, f"rank mismatch {len(self.strides)=}, {rank=}"
        assert len(self.block_shape) == rank, f"rank mismatch {len(self.block_shape)=}, {rank=}"
        assert rank > 0, "rank must not be zero"
        assert rank <= 5, "rank cannot be more than 5"
        assert self.base.data_ptr() % 16 == 0, "base must be 16-byte aligned"
        elem_bytes = self.base.element_size()
        for stride in self.strides[:-1]:
            assert (stride * elem_bytes) % 16 == 0, "strides must be 16-byte aligned"
        assert self.strides[-1] == 1, "Last dimension must be contiguous"
        assert self.padding in ("zero", "nan"), "Illegal value for padding"

    @staticmethod
    def from_tensor(tensor: torch.Tensor, block_shape: List[int], padding: str = "zero") -> "TensorDescriptor":
        return TensorDescriptor(tensor, list(tensor.shape), list(tensor.stride()), list(block_shape), padding)
