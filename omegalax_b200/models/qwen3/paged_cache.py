"""Paged KV cache for decode: fixed-size pages handed out by a free-list allocator, a block
table per sequence, and per-sequence lengths (padding tokens are never stored).  The contiguous
cache in ``cache.py`` keeps the reference's semantics; this one feeds the decode kernels."""
from __future__ import annotations

import torch


class PageAllocator:
    """Host-side free list of physical pages."""

    def __init__(self, num_pages: int):
        self.free = list(range(num_pages - 1, -1, -1))
        self.num_pages = num_pages

    def alloc(self) -> int:
        if not self.free:
            raise RuntimeError("paged KV cache is out of pages")
        return self.free.pop()

    def release(self, pages) -> None:
        self.free.extend(int(p) for p in pages)


class PagedKVCache:
    def __init__(self, cfg, batch_size: int, max_tokens_per_seq: int, *, page_size: int = 64,
                 dtype=torch.bfloat16, device=None, num_pages: int | None = None):
        self.cfg, self.B, self.page_size = cfg, batch_size, page_size
        self.max_blocks = -(-max_tokens_per_seq // page_size)
        self.num_pages = num_pages or batch_size * self.max_blocks
        G, K = cfg.num_kv_heads, cfg.head_dim
        shape = (self.num_pages, page_size, G, K)
        self.k_pages = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(cfg.num_layers)]
        self.v_pages = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(cfg.num_layers)]
        self.allocator = PageAllocator(self.num_pages)
        self.block_table_host = torch.full((batch_size, self.max_blocks), -1, dtype=torch.int32)
        self.block_table = torch.zeros(batch_size, self.max_blocks, dtype=torch.int32, device=device)
        self.seq_lens_host = [0] * batch_size
        self.seq_lens = torch.zeros(batch_size, dtype=torch.int32, device=device)
        self.device = device

    def reserve(self, new_tokens: list[int]) -> None:
        """Make sure every sequence has pages for ``new_tokens[b]`` more tokens."""
        changed = False
        for b, n in enumerate(new_tokens):
            need = -(-(self.seq_lens_host[b] + n) // self.page_size)
            if need > self.max_blocks:
                raise RuntimeError(f"sequence {b} exceeds the cache capacity of {self.max_blocks * self.page_size} tokens")
            have = int((self.block_table_host[b] >= 0).sum())
            for j in range(have, need):
                self.block_table_host[b, j] = self.allocator.alloc()
                changed = True
        if changed:
            self.block_table.copy_(self.block_table_host.clamp_min(0))

    def advance(self, new_tokens: list[int]) -> None:
        for b, n in enumerate(new_tokens):
            self.seq_lens_host[b] += n
        self.seq_lens.copy_(torch.tensor(self.seq_lens_host, dtype=torch.int32))

    def free_sequence(self, b: int) -> None:
        pages = self.block_table_host[b][self.block_table_host[b] >= 0].tolist()
        self.allocator.release(pages)
        self.block_table_host[b] = -1
        self.seq_lens_host[b] = 0
        self.seq_lens.copy_(torch.tensor(self.seq_lens_host, dtype=torch.int32))

    def flat_rows(self, seq_of_token, slot_of_token):
        """Row index into pages.view(-1, G, K) of (sequence, slot) pairs (device tensors)."""
        blk = self.block_table[seq_of_token.long(), (slot_of_token // self.page_size).long()].long()
        return blk * self.page_size + (slot_of_token % self.page_size).long()
