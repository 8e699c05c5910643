"""Minimal stand-ins for the reference's job and context objects, for tests of the attention
function's metadata. They follow the observable behaviour of
parrot/engine/context/block_context.py:13-124 (one slot per token, a new block every
`block_size` tokens, a parent padded to a block multiple the first time it is forked) and of
parrot/engine/primitive_job.py (Fill carries token_ids, Generate a sampling_config)."""
from __future__ import annotations

from typing import List, Optional


class Pool:
    def __init__(self):
        self.next = 0

    def allocate(self) -> int:
        self.next += 1
        return self.next - 1


class Context:
    def __init__(self, context_id: int, parent: Optional["Context"], pool: Pool, block_size: int):
        self.context_id, self.parent_context, self.pool, self.block_size = context_id, parent, pool, block_size
        self.depth = 0 if parent is None else parent.depth + 1
        self.padded = False
        self.blocks: List[int] = []
        self.slots: List[int] = []
        # the reference's attribute names for the same per-token lists (block_context.py:41-45)
        self.token_kv_block_ids = self.blocks
        self.token_kv_slot_ids = self.slots
        if parent is not None and not parent.padded:
            n = parent.get_this_context_len()
            parent.allocate((n + block_size - 1) // block_size * block_size - n)
            parent.padded = True

    def allocate(self, n: int):
        for _ in range(n):
            if len(self.blocks) % self.block_size == 0:
                b = self.pool.allocate()
                self.blocks.append(b)
                self.slots.append(b * self.block_size)
            else:
                self.blocks.append(self.blocks[-1])
                self.slots.append(self.slots[-1] + 1)

    def get_this_context_len(self) -> int:
        return len(self.blocks)

    def get_context_len(self) -> int:
        return (self.parent_context.get_context_len() if self.parent_context else 0) + len(self.blocks)

    def get_context_block_ids(self) -> List[int]:
        return (self.parent_context.get_context_block_ids() if self.parent_context else []) + self.blocks

    def get_context_slot_ids(self) -> List[int]:
        return (self.parent_context.get_context_slot_ids() if self.parent_context else []) + self.slots


class Generate:
    def __init__(self, context: Context):
        self.context = context
        self.sampling_config = object()


class Fill:
    def __init__(self, context: Context, token_ids: List[int]):
        self.context = context
        self.token_ids = token_ids


class IterationState:
    def __init__(self):
        self.num_fill_tokens: List[int] = []
        self.generation_sampling_config: list = []

    @property
    def num_total_fill_tokens(self) -> int:
        return sum(self.num_fill_tokens)
