"""Paged KV cache of the Reasoner: fixed-size pages per layer, a native (C++) block allocator
that owns the page tables, and device-side tables that the decode-attention kernel reads.

Layout per layer: k_cache, v_cache [num_pages, Hkv_local, page_size, head_dim] bf16 (the rows of one
(page, head) are contiguous, which is what the decode kernel streams). A sequence
owns a list of pages; token i of the sequence lives in page table[i // page_size] at offset
i % page_size. Pages for the whole generation (prompt + max new tokens) can be reserved up front,
which keeps the block table static during decode (a requirement for CUDA-graph replay).
"""
from __future__ import annotations

from typing import Sequence

import torch

from .. import ops


class _PyAllocator:
    """Pure-Python stand-in with the interface of the C++ `PagedKVAllocator` (used when the
    extension is not built, e.g. CPU-only unit tests)."""

    def __init__(self, num_blocks: int, block_size: int, max_blocks_per_seq: int):
        self.block_size, self.max_blocks = block_size, max_blocks_per_seq
        self.free = list(range(num_blocks - 1, -1, -1))
        self.tables, self.lens = {}, {}

    def num_free(self):
        return len(self.free)

    def can_allocate(self, tokens):
        return (tokens + self.block_size - 1) // self.block_size <= len(self.free)

    def extend(self, seq, tokens):
        tab, n = self.tables.setdefault(seq, []), self.lens.get(seq, 0)
        need = (n + tokens + self.block_size - 1) // self.block_size - len(tab)
        if need > len(self.free) or len(tab) + need > self.max_blocks:
            if not tab and n == 0:
                self.tables.pop(seq, None)
            return False
        for _ in range(need):
            tab.append(self.free.pop())
        self.lens[seq] = n + tokens
        return True

    def release(self, seq):
        self.free.extend(self.tables.pop(seq, []))
        self.lens.pop(seq, None)

    def length(self, seq):
        return self.lens.get(seq, 0)

    def blocks(self, seq):
        return list(self.tables.get(seq, []))

    def fill_tables(self, seqs, table, lens):
        table.fill_(-1)
        for i, s in enumerate(seqs):
            b = self.tables.get(s, [])
            table[i, :len(b)] = torch.tensor(b, dtype=torch.int32)
            lens[i] = self.lens.get(s, 0)


def make_allocator(num_blocks: int, block_size: int, max_blocks_per_seq: int):
    if ops.load_extension(build_if_missing=False):
        return torch.classes.cosmos_b200.PagedKVAllocator(num_blocks, block_size, max_blocks_per_seq)
    return _PyAllocator(num_blocks, block_size, max_blocks_per_seq)


class PagedKVCache:
    def __init__(self, n_layers: int, n_kv_heads: int, head_dim: int, num_pages: int, page_size: int,
                 max_pages_per_seq: int, dtype=torch.bfloat16, device="cuda"):
        self.n_layers, self.page_size, self.max_pages = n_layers, page_size, max_pages_per_seq
        self.alloc = make_allocator(num_pages, page_size, max_pages_per_seq)
        shape = (num_pages, n_kv_heads, page_size, head_dim)
        self.k = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(n_layers)]
        self.v = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(n_layers)]
        self.device = torch.device(device)

    def reserve(self, seq_id: int, tokens: int) -> bool:
        """Reserves pages for `tokens` more tokens of a sequence (False = pool exhausted)."""
        return bool(self.alloc.extend(seq_id, tokens))

    def release(self, seq_id: int) -> None:
        self.alloc.release(seq_id)

    def tables(self, seq_ids: Sequence[int]):
        """(block_table [n, max_pages] int32, reserved lengths [n] int32) on the cache's device."""
        t = torch.empty(len(seq_ids), self.max_pages, dtype=torch.int32)
        l = torch.empty(len(seq_ids), dtype=torch.int32)
        self.alloc.fill_tables(list(seq_ids), t, l)
        return t.to(self.device), l.to(self.device)

    @staticmethod
    def slots(table: torch.Tensor, positions: torch.Tensor, page_size: int) -> torch.Tensor:
        """Flat cache slots (page * page_size + offset) of token `positions` [n, m] of each sequence."""
        page = torch.gather(table.long(), 1, (positions // page_size).long())
        return page * page_size + (positions % page_size).long()

    def write(self, layer: int, k: torch.Tensor, v: torch.Tensor, slots: torch.Tensor) -> None:
        """k, v [N, Hkv, D] -> cache rows `slots` [N]."""
        if k.is_cuda and k.dtype == torch.bfloat16 and ops.load_extension():
            torch.ops.cosmos_b200.kv_cache_write(k.contiguous(), v.contiguous(), slots.contiguous(),
                                                 self.k[layer], self.v[layer])
        else:
            page, off = slots // self.page_size, slots % self.page_size
            self.k[layer][page, :, off] = k
            self.v[layer][page, :, off] = v

    def gather(self, layer: int, table_row: torch.Tensor, n: int):
        """The first n cached tokens of one sequence as contiguous K, V [n, Hkv, D]."""
        pages = table_row[:(n + self.page_size - 1) // self.page_size].long()
        hk, d = self.k[layer].shape[1], self.k[layer].shape[3]
        k = self.k[layer][pages].transpose(1, 2).reshape(-1, hk, d)[:n]
        v = self.v[layer][pages].transpose(1, 2).reshape(-1, hk, d)[:n]
        return k, v
