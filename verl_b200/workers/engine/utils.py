"""Helpers shared by the training engines.

Parity target: ``verl/workers/engine/utils.py`` (``enable_full_determinism`` :31-63, ``pad_packed_inputs`` :66,
``prepare_micro_batches`` :92-130, ``postprocess_batch_func`` :133).
"""

from __future__ import annotations

import os
import random
from typing import Optional

import numpy as np
import torch

from ...utils.seqlen_balancing import get_seqlen_balanced_partitions

__all__ = ["enable_full_determinism", "pad_packed_inputs", "prepare_micro_batches", "restore_order"]


def enable_full_determinism(seed: int) -> None:
    """Seeds every generator and switches the libraries to their deterministic code paths. The native kernels have no
    atomically-accumulated outputs on the default training path (wgrad accumulates in a fixed K order, the MoE combine and
    the fused collectives sum in rank order), so this is sufficient for run-to-run identical losses."""
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    os.environ["VERL_B200_NATIVE_ATTN_BWD"] = "0"  # the tcgen05 attention backward reduces dQ with fp32 atomics
    from ...ops import functional as _F

    _F._ATTN_IMPL["bwd"] = None                    # also when the kernels were selected before this call
    _F.DETERMINISTIC_ATTENTION = True              # the autograd attention backward then runs on the math back-end
    torch.backends.cudnn.deterministic = True
    torch.backends.cudnn.benchmark = False
    try:
        torch.use_deterministic_algorithms(True, warn_only=True)
    except Exception:
        pass


def pad_packed_inputs(input_ids: torch.Tensor, positions: torch.Tensor, cu_seqlens: torch.Tensor, multiple: int, pad_id: int = 0):
    """Append one dummy sequence so that the packed token count is a multiple of ``multiple`` (tile sizes of fused
    kernels, sequence-parallel splits). Returns the padded tensors and the number of padding tokens."""
    T = input_ids.numel()
    pad = (-T) % multiple
    if pad == 0:
        return input_ids, positions, cu_seqlens, 0
    ids = torch.cat([input_ids, input_ids.new_full((pad,), pad_id)])
    pos = torch.cat([positions, torch.arange(pad, dtype=positions.dtype, device=positions.device)])
    cu = torch.cat([cu_seqlens, cu_seqlens.new_tensor([T + pad])])
    return ids, pos, cu, pad


def prepare_micro_batches(seqlens: list[int], micro_batch_size: Optional[int] = None, max_token_len: Optional[int] = None,
                          use_dynamic_bsz: bool = False, min_num_micro_batch: int = 1) -> list[list[int]]:
    """Row indices of each micro-batch: fixed ``micro_batch_size`` rows, or (dynamic) the fewest balanced groups whose token
    sums stay under ``max_token_len``."""
    n = len(seqlens)
    if not use_dynamic_bsz:
        mb = int(micro_batch_size or n)
        return [list(range(i, min(n, i + mb))) for i in range(0, n, mb)]
    assert max_token_len and max(seqlens) <= max_token_len, "max_token_len must cover the longest sequence"
    k = max(min_num_micro_batch, -(-sum(seqlens) // int(max_token_len)))
    k = min(k, n)
    while True:
        parts = get_seqlen_balanced_partitions(seqlens, k, equal_size=False)
        if all(sum(seqlens[i] for i in p) <= max_token_len for p in parts) or k >= n:
            return [sorted(p) for p in parts]
        k += 1


def restore_order(chunks: list[torch.Tensor], index_groups: list[list[int]]) -> torch.Tensor:
    """Concatenate per-micro-batch outputs and undo the micro-batch permutation."""
    cat = torch.cat(chunks, 0)
    idx = torch.tensor([i for g in index_groups for i in g], dtype=torch.long, device=cat.device)
    out = torch.empty_like(cat)
    out[idx] = cat
    return out
