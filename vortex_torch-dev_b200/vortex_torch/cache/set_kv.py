"""Write new tokens into the paged K/V caches (reference: ``cache/triton_kernels/set_kv.py:39-62``).

The caches are ``[num_pages, H, page_size, D]`` (flattened ``[num_pages*H, page_size, D]``): token
slot ``t`` of head ``h`` lands in row ``(t // P) * H + h`` at offset ``t % P``.
"""
from __future__ import annotations

import torch

from .. import _cabi


def set_kv_buffer_launcher(k_cache: torch.Tensor, v_cache: torch.Tensor, new_k: torch.Tensor,
                           new_v: torch.Tensor, loc: torch.Tensor, page_size: int) -> None:
    _cabi.set_kv(k_cache, v_cache, new_k, new_v, loc, page_size)
