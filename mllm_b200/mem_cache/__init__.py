from .base_prefix_cache import (
    BasePrefixCache, EvictResult, InsertResult, MatchResult, RadixKey,
    hash_bytes, hash_to_int64, hash_token_ids,
)
from .chunk_cache import ChunkCache
from .mamba_radix_cache import MambaRadixCache, MambaTreeNode
from .memory_pool import GDNPool, KVPool, ReqToTokenPool, TokenToKVPoolAllocator
from .radix_cache import RadixCache, TreeNode
from .swa_radix_cache import SWARadixCache, SWATreeNode

__all__ = [
    "BasePrefixCache", "EvictResult", "InsertResult", "MatchResult", "RadixKey",
    "hash_bytes", "hash_to_int64", "hash_token_ids", "ChunkCache", "KVPool", "GDNPool",
    "ReqToTokenPool", "TokenToKVPoolAllocator", "RadixCache", "TreeNode", "MambaRadixCache", "MambaTreeNode",
    "SWARadixCache", "SWATreeNode",
]
