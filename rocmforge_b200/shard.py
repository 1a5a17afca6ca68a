"""Output-feature (column) split of a packed weight tensor across the GPUs of one node.

The reference has no multi-GPU path at all (single global backend, one stream:
src/backend/hip_backend/backend.rs:83-105); this is the one distributed component added on top of it. A
projection y[m, n] = x[m, k] * W[n, k]^T shards naturally by rows of W: rank r keeps rows
[r*n/G, (r+1)*n/G), every rank sees the same x, and the only exchange is one all-gather of the [m, n/G]
output slices (no reduction: k is not split). b200q_weight_upload does the same slicing internally when
given shard_rank / shard_count; these helpers are for hosts that want to cut the bytes themselves (for
example to read only their part of a file) and for putting the gathered slices back in [m, n] order.
"""
from . import synth


def shard_rows(n, rank, count):
    """(first row, row count) of a rank; n must divide evenly."""
    if count < 1 or not 0 <= rank < count:
        raise ValueError(f"shard {rank} of {count}")
    if n % count:
        raise ValueError(f"n={n} does not divide into {count} shards")
    per = n // count
    return rank * per, per


def shard_bytes(data, qtype, layout, n, k, rank, count):
    """The packed bytes of a rank's rows of an [n, k] NK tensor (a view, no copy)."""
    row0, rows = shard_rows(n, rank, count)
    be, bb = synth.block_elems(qtype), synth.block_bytes(qtype, layout)
    if (rows * k) % be:
        raise ValueError(f"a shard of {rows} rows x {k} does not end on a {be}-weight block")
    b0 = row0 * k // be
    return data[b0 * bb:(b0 + rows * k // be) * bb]


def gathered_to_matrix(y_all):
    """all_gather_into_tensor output [G, m, n/G] -> [m, n] (column blocks side by side)."""
    g, m, per = y_all.shape
    return y_all.permute(1, 0, 2).reshape(m, g * per)
