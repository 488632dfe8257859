"""Mirror of tidal/utils/decode_wrapper.py:13-88 on the native `_kernels` drop-in."""
from __future__ import annotations

from typing import Optional

import torch

from .. import _kernels
from .utils import TensorLayout


def _check_kv_layout(kv_layout: str):
    """Only the layout names TensorLayout defines are accepted."""
    if kv_layout not in TensorLayout.FORMAT2STR.values():
        known = ", ".join(sorted(TensorLayout.FORMAT2STR.values()))
        raise KeyError(f"unknown KV layout name {kv_layout!r} (known: {known})")


class BatchDecodeWithPagedKVCacheWrapper:
    def __init__(self, kv_layout: str = "NHD"):
        _check_kv_layout(kv_layout)
        self.kv_layout = kv_layout
        self._wrapper = _kernels.BatchDecodeWithPagedKVCachePyTorchWrapper(getattr(TensorLayout, kv_layout))

    def begin_forward(self, indptr: torch.Tensor, num_qo_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                      data_type, max_pages: int = 0, device=None):
        """max_pages / device (not in the reference): the longest page list the following forward calls may pass and
        where they run, for callers whose `indptr` lives on the device and is not read back."""
        self._wrapper.begin_forward(indptr, num_qo_heads, num_kv_heads, head_dim, page_size, torch.empty(0, dtype=data_type),
                                    max_pages, device)

    def end_forward(self):
        self._wrapper.end_forward()

    def forward(self, q: torch.Tensor, o: torch.Tensor, paged_kv_data: torch.Tensor, paged_kv_indices: torch.Tensor,
                paged_kv_indptr: torch.Tensor, paged_kv_last_page_len: int, paged_kv_last_page_idx: int,
                qk_product: Optional[torch.Tensor] = None, rope_scale: Optional[float] = None,
                rope_theta: Optional[float] = None):
        rope_scale = 1.0 if rope_scale is None else rope_scale
        rope_theta = 1e4 if rope_theta is None else rope_theta
        qk_product = torch.empty(0) if qk_product is None else qk_product
        self._wrapper.forward(q, o, paged_kv_data, paged_kv_indices, paged_kv_indptr, paged_kv_last_page_len,
                              paged_kv_last_page_idx, qk_product, rope_scale, rope_theta)
