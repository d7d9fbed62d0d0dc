"""Record sharding across the GPUs of one box: the path has no exchange step, so every rank
works on its own records.  The split is aeon's multi-node manifest split
(src/manifest_file.cpp:278-295): interleaved batch-sized slices, then an evenly divided tail."""


def shard_indices(n_records, batch_size, rank, world):
    """Indices (into the unsharded record list) that rank `rank` of `world` processes."""
    if world <= 1:
        return list(range(n_records))
    count = n_records // world
    batches = count // batch_size
    out = []
    for i in range(batches * batch_size):
        b, k = divmod(i, batch_size)
        out.append(b * batch_size * world + batch_size * rank + k)
    tail = count - batches * batch_size
    src = batches * batch_size * world + tail * rank
    out.extend(range(src, src + tail))
    return out


def max_over_ranks(value, group=None):
    """Largest `value` over the ranks of the default (or given) process group; identity when not initialised."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
