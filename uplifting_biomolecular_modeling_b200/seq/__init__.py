"""Helpers of the sequence-model kits (protein / genomic language models): batch plans under an element ceiling,
resident rotary tables, byte -> row lookup tokenisers, variable-length batches without a host synchronisation,
memory budgets.  Reference: common/opt_core/opt_core/seq/*.py."""
from .backend import pinned_backend, tokens_within
from .plans import BatchPlan, plan_batches
from .rotary import RotaryTable
from .tokenizers import ByteLUT
from .varlen import cu_seqlens, pad_to_multiple

__all__ = ["BatchPlan", "plan_batches", "RotaryTable", "ByteLUT", "cu_seqlens", "pad_to_multiple", "pinned_backend",
           "tokens_within"]
