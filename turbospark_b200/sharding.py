"""Which part of a routed model a rank holds when the model is spread over the GPUs of one box.

Attention is tensor-parallel over heads, experts are sharded, everything else (embedding, norms, router, head) is
replicated.  Weight rows are verbatim quantized block rows, so a shard is a slice of rows (q, k, v heads; experts) or
of whole 256-column blocks inside every row (the o_proj columns of the rank's heads).  Pure host logic: numpy only.
"""
import numpy as np

from .capi import lib


class HeadShard:
    """The query heads of `rank` and the K/V heads they read.  n_q_heads must divide by world; when world exceeds the
    K/V head count a K/V head is replicated on the ranks whose query heads read it."""

    def __init__(self, n_q_heads, n_kv_heads, head_dim, rank, world):
        if n_q_heads % world:
            raise ValueError("n_q_heads %d does not divide over %d ranks" % (n_q_heads, world))
        self.q_local = n_q_heads // world
        group = n_q_heads // n_kv_heads  # query heads per K/V head
        self.q_lo = rank * self.q_local
        kv_first, kv_last = self.q_lo // group, (self.q_lo + self.q_local - 1) // group
        self.kv_lo, self.kv_local = kv_first, kv_last - kv_first + 1
        if self.q_local % self.kv_local:
            raise ValueError("a rank's query heads must split evenly over the K/V heads it holds")
        if (self.q_local * head_dim) % 256:
            raise ValueError("a rank's heads must cover whole 256-column blocks of o_proj")
        self.head_dim = head_dim

    def q_rows(self):
        return slice(self.q_lo * self.head_dim, (self.q_lo + self.q_local) * self.head_dim)

    def kv_rows(self):
        return slice(self.kv_lo * self.head_dim, (self.kv_lo + self.kv_local) * self.head_dim)

    def o_cols(self):
        return slice(self.q_lo * self.head_dim, (self.q_lo + self.q_local) * self.head_dim)


def expert_range(n_experts, rank, world):
    """(first expert, count) of `rank`: contiguous, equal shares."""
    if n_experts % world:
        raise ValueError("%d experts do not divide over %d ranks" % (n_experts, world))
    n = n_experts // world
    return rank * n, n


def slice_block_columns(blocks, qtype, cols, col_slice):
    """Columns [col_slice) of block rows `blocks` ([rows, row_bytes] uint8): whole blocks of every row."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    rb = int(lib().tsb_row_bytes(qtype, cols))
    per_col_block = 32 if qtype in (2, 4) else 256  # MXFP4 and Q8_0 blocks hold 32 columns, the K formats 256
    lo, hi = col_slice.start, col_slice.stop
    if lo % per_col_block or hi % per_col_block:
        raise ValueError("a column shard must start and end on a block boundary")
    bytes_per_block = rb * per_col_block // cols
    return np.ascontiguousarray(blocks.reshape(blocks.shape[0], rb)[:, lo // per_col_block * bytes_per_block: hi // per_col_block * bytes_per_block])


def slice_experts(stacked, n_experts, expert_lo, n_local):
    """Experts [expert_lo, expert_lo + n_local) of matrices stacked along the rows (`stacked`: [n_experts * rows, row_bytes])."""
    stacked = np.ascontiguousarray(stacked, dtype=np.uint8)
    per = stacked.shape[0] // n_experts
    return np.ascontiguousarray(stacked[expert_lo * per:(expert_lo + n_local) * per])
