from .gating import gated_branch_sum
from .index_topk import parallel_nsa_topk, parallel_nsa_topk_grouped_heads, should_use_selection_attention
from .selection import selection_attention

__all__ = ["parallel_nsa_topk", "parallel_nsa_topk_grouped_heads", "should_use_selection_attention",
           "selection_attention", "gated_branch_sum"]
