"""B200 (sm_100a) implementation of the native-sparse-attention selection path:
block-compressed key scoring, per-query-group top-k block selection, selection attention
forward / backward over a block KV cache, and the LRU block KV cache itself.

    from omnimem_b200.nsa.ops import parallel_nsa_topk, selection_attention   # reference API
    from omnimem_b200.cache import BlockKVCache                                # page pool
    import omnimem_b200.torch_ops                                              # torch.ops.omnimem_nsa.*

The compute lives in ``libomnimem_b200.so`` (C ABI in include/omnimem_b200.h, built by
``python -m omnimem_b200.build``); there is no Python or CPU stand-in for it.
"""
from ._lib import NSABackendError, load as load_library  # noqa: F401

__version__ = "0.1.0"
