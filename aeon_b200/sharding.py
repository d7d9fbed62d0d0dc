"""Record sharding across the GPUs of one box: the path has no exchange step, so every rank
works on its own records.  The split is aeon's multi-node manifest split
(src/manifest_file.cpp:278-295): interleaved batch-sized slices, then an evenly divided tail."""


def shard_indices(n_records, batch_size, rank, world):
    """Indices (into the unsharded record list) that rank `rank` of `world` processes: the library's own node split
    (aeonb_node_record_indices), so python and the C++ loader cannot drift apart."""
    import ctypes as C
    from . import _lib as L
    lib = L.load()
    n = int(L.check(lib.aeonb_node_record_indices(n_records, rank, world, batch_size, None)))
    out = (C.c_int64 * max(n, 1))()
    L.check(lib.aeonb_node_record_indices(n_records, rank, world, batch_size, out))
    return list(out[:n])


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
