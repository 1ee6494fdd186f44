"""Host-side N-sharding of the decode linears (column-parallel, vocab-parallel for lm_head).

Every output row is an independent dot product, so a rank owns a contiguous
block of weight rows, the activation is replicated, and the only exchange is an
all-gather of the bf16 outputs -- plus, on the greedy path, one (value, index)
pair per rank instead of the logits.  No cross-rank reduction of partial sums
exists, which keeps results independent of the number of ranks.
The reference is single-GPU (one device_id, native/include/minicpm_runtime.h:61);
this module has no counterpart there.
"""
from __future__ import annotations


def roundup(a: int, b: int) -> int:
    return (a + b - 1) // b * b


def shard_rows(n: int, world: int, rank: int, mult: int = 8):
    """Rows [lo, hi) of an n-row matrix owned by `rank`, and the uniform shard
    pitch `per` (= rows of every shard but possibly the last, a multiple of
    `mult`).  Trailing ranks may own a short or empty block (vocab 122753)."""
    per = roundup((n + world - 1) // world, mult)
    lo = min(n, rank * per)
    return lo, min(n, lo + per), per


def shard_gate_up(inter: int, world: int, rank: int, mult: int = 8):
    """The fused gate_up tensor [2*inter, K] (rows gate | up) is sharded by
    (gate_j, up_j) PAIRS so that the SwiGLU runs before the gather: returns the
    pair range [lo, hi) and the pitch; the rank's weight holds rows
    gate[lo:hi] and up[lo:hi] interleaved (2*(hi-lo) rows)."""
    return shard_rows(inter, world, rank, mult)


def gathered_view(flat, n: int, world: int, per: int, m: int = 1):
    """View of an all-gathered buffer laid out [world, m, per] as the logical
    [m, n] result (copies only when m > 1).  `flat` is anything reshape-able
    (numpy array or torch tensor)."""
    g = flat.reshape(world, m, per)
    if m == 1:
        return g.reshape(1, world * per)[:, :n]
    return g.transpose(0, 1).reshape(m, world * per)[:, :n] if hasattr(g, "transpose") and not hasattr(g, "swapaxes") \
        else g.swapaxes(0, 1).reshape(m, world * per)[:, :n]


def reduce_argmax_pairs(values, indices):
    """Global greedy token from per-rank (max value, global index) pairs with the
    reference's rule: larger value wins, equal values go to the LOWER index, NaN
    never wins (native/kernels/sm120/sampling.cu:77-83).  Plain Python so that it
    runs on the host after an 8-byte-per-rank gather."""
    best_v, best_i = float("-inf"), 2 ** 31 - 1
    for v, i in zip(values, indices):
        v, i = float(v), int(i)
        if v > best_v or (v == best_v and i < best_i):
            best_v, best_i = v, i
    return best_v, best_i
