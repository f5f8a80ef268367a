"""Address arithmetic of the sparse-attention KV stores, on the host: where logical row `i` of a sequence
lives in a contiguous table, in a paged pool, or in a dual-plane paged pool (raw window rows in one plane,
compressed rows in another), and how the combined ring of the decode path numbers its slots.  The device
kernels take explicit row lists; these resolvers build such lists and check them in tests.

* contiguous: row i of sequence s -> s * stride + i
* paged:      row i -> block_table[s][i // page] * page + i % page
* dual-plane: logical index < window_rows addresses the window plane, the rest the compressed plane; both
              planes are paged with the same block table but different rows per page
* combined ring: the decode selection space is [window ring slots | compressed rows]; ring slot r holds
              position p with p % window == r among the last `window` positions
* recurrent compressor state: `ratio` (or 2 * ratio with overlap) projected rows of width out_dim

Counterpart of crates/ferrule-backend/src/cuda/transformer/sparse_attention.rs:14-640 (layouts + resolvers),
transformer/combined_ring.rs:5-120 and transformer/compressor_recurrent.rs:6-110.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence


class LayoutError(ValueError):
    pass


@dataclass(frozen=True)
class ContiguousLayout:
    stride: int                      # rows reserved per sequence

    def resolve(self, seq: int, row: int) -> int:
        if not 0 <= row < self.stride:
            raise LayoutError(f"row {row} outside the sequence's {self.stride} rows")
        return seq * self.stride + row


@dataclass(frozen=True)
class PagedLayout:
    page_size: int

    def resolve(self, block_table: Sequence[int], row: int) -> int:
        page = row // self.page_size
        if row < 0 or page >= len(block_table) or block_table[page] < 0:
            raise LayoutError(f"row {row} has no page")
        return block_table[page] * self.page_size + row % self.page_size


@dataclass(frozen=True)
class DualPlanePagedLayout:
    """Raw rows and compressed rows of one sequence share pages: a page holds `page_tokens` raw rows in plane 0
    and `page_tokens // ratio` compressed rows in plane 1."""
    page_tokens: int
    ratio: int

    @property
    def compressed_per_page(self) -> int:
        return self.page_tokens // self.ratio

    def resolve_raw(self, block_table: Sequence[int], position: int):
        return 0, PagedLayout(self.page_tokens).resolve(block_table, position)

    def resolve_compressed(self, block_table: Sequence[int], index: int):
        return 1, PagedLayout(self.compressed_per_page).resolve(block_table, index)


@dataclass(frozen=True)
class CombinedRing:
    window: int

    def ring_slot(self, position: int) -> int:
        return position % self.window

    def logical_of_slot(self, slot: int, last_position: int) -> Optional[int]:
        """Position currently held by ring slot `slot` after `last_position` was appended (None: never written)."""
        if not 0 <= slot < self.window:
            raise LayoutError("ring slot out of range")
        p = last_position - ((last_position - slot) % self.window)
        return p if p >= 0 else None

    def selection(self, last_position: int, compressed: Sequence[int]) -> List[int]:
        """Selection list in combined numbering: visible window positions as ring slots (oldest first), then
        compressed rows offset by the window size."""
        lo = max(0, last_position - self.window + 1)
        return [self.ring_slot(p) for p in range(lo, last_position + 1)] + [self.window + c for c in compressed]


@dataclass(frozen=True)
class CompressorStateShape:
    ratio: int
    head_dim: int
    overlap: bool

    @property
    def out_dim(self) -> int:
        return self.head_dim * (2 if self.overlap else 1)

    @property
    def rows(self) -> int:
        return self.ratio * (2 if self.overlap else 1)

    @property
    def state_elems(self) -> int:
        return self.rows * self.out_dim

    def row_of(self, position: int) -> int:
        """State row the projection of `position` is written to (the current group's half when overlapping)."""
        return (self.ratio if self.overlap else 0) + position % self.ratio

    def is_boundary(self, position: int) -> bool:
        return (position + 1) % self.ratio == 0
