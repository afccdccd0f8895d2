from .gating import gated_branch_sum
from .index_topk import parallel_nsa_topk, parallel_nsa_topk_grouped_heads, should_use_selection_attention
from .padded_ptr import build_ptr_table, selection_attention_block_store, selection_attention_padded_ptr_fast
from .selection import selection_attention

__all__ = ["parallel_nsa_topk", "parallel_nsa_topk_grouped_heads", "should_use_selection_attention",
           "selection_attention", "gated_branch_sum", "selection_attention_block_store",
           "selection_attention_padded_ptr_fast", "build_ptr_table"]
