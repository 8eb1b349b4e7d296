"""Sharding of the batch axis over ranks (one process a GPU) and the exchanges of a sharded run: the final
loss of a forward pass, calibration's magnitudes, and a training step's gradient.

Every launch of a forward pass carries `batch` as an outer parallel axis with disjoint
outputs (presk-kernel/src/ir.rs:345-375), so a rank runs the whole model on its own rows
with no data-path collective. The loss of the whole batch is the mean over all rows; each
rank holds the mean over its rows, and the means are combined weighted by their row counts
with one all-reduce (a declared two-level order of the sum: rows within a shard, then shards
in rank order).
"""
import torch
import torch.distributed as dist


def shard_rows(n_rows, rank, world):
    """The contiguous slice [lo, hi) of `n_rows` batch rows that `rank` of `world` owns."""
    base, extra = divmod(n_rows, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def combine_mean(local_mean, local_count, device="cpu", group=None):
    """The mean over all ranks' rows from each rank's mean and row count."""
    t = torch.tensor([float(local_mean) * float(local_count), float(local_count)], dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return float(t[0] / t[1])


def max_over_ranks(value, device="cpu", group=None):
    """A timing taken on every rank, as the slowest rank saw it."""
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t[0])


def combine_envelopes(envelope, device="cpu", group=None):
    """`presk calibrate` over a sharded batch: each rank's {site: (max |x|, least non-zero |x|, lo, hi)}
    merged into the whole batch's with ONE max-reduction (the minima travel negated). Every rank
    runs the same program, so the sites and their order are the same everywhere."""
    sites = sorted(envelope)
    t = torch.tensor([[envelope[s][0], -envelope[s][1], -envelope[s][2], envelope[s][3]] for s in sites], dtype=torch.float64, device=device).reshape(-1, 4)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    t = t.cpu()
    return {s: (float(t[i, 0]), float(-t[i, 1]), float(-t[i, 2]), float(t[i, 3])) for i, s in enumerate(sites)}


def combine_gradients(leaves, local_count, device="cpu", group=None):
    """A training step over a sharded batch: each rank holds the gradient of the mean loss over its own rows; the
    gradient of the mean over all rows is the row-weighted mean of those, one all-reduce a leaf. `leaves` maps a
    parameter's path to a float array; every rank passes the same paths. Returns the combined leaves, which the
    caller hands back to the host (`Host.set_result`) before `adamw_step`: every rank then takes the same step."""
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    n = torch.tensor([float(local_count)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(n, op=dist.ReduceOp.SUM, group=group)
    out = {}
    for path in sorted(leaves):
        t = torch.as_tensor(leaves[path], dtype=torch.float64, device=device) * float(local_count)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
        out[path] = (t / n).cpu().numpy()
    return out
