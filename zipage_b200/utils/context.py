"""Per-step launch context shared between the model runner and the attention layers.

Same fields and accessors as the reference's zipage/utils/context.py:5-52, plus
`query_slot_count`: a device int32 [1] with the number of valid rows of `query_slot_mapping`
when that tensor has a fixed capacity (steps built on the device and replayed as a graph).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class Context:
    is_prefill: bool = False
    cu_seqlens_q: torch.Tensor | None = None
    cu_seqlens_k: torch.Tensor | None = None
    max_seqlen_q: int = 0
    max_seqlen_k: int = 0
    slot_mapping: torch.Tensor | None = None
    query_slot_mapping: torch.Tensor | None = None
    context_lens: torch.Tensor | None = None
    block_tables: torch.Tensor | None = None
    query_slot_count: torch.Tensor | None = None


_CONTEXT = Context()


def get_context() -> Context:
    return _CONTEXT


def set_context(is_prefill, cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen_q=0, max_seqlen_k=0,
                slot_mapping=None, query_slot_mapping=None, context_lens=None, block_tables=None,
                query_slot_count=None):
    global _CONTEXT
    _CONTEXT = Context(is_prefill, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                       slot_mapping, query_slot_mapping, context_lens, block_tables, query_slot_count)


def reset_context():
    global _CONTEXT
    _CONTEXT = Context()
