"""Sharding of the NSA hot path over the GPUs of one node.

Every branch is independent per (batch element, KV head): the G query heads of
a KV head stay together because they share the selection and every fetched
key/value block.  Ranks therefore own contiguous runs of (batch, KV head) units
-- batch first, then KV-head groups -- and attention itself needs no exchange.
The only collective is the all-gather that reassembles the output."""
import torch
import torch.distributed as dist


def unit_range(num_units, world, rank):
    """Half-open range of units owned by `rank` when `num_units` are dealt out in contiguous, near-equal runs."""
    base, extra = divmod(num_units, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def plan(batch, kv_heads, world):
    """How `world` ranks split a [batch, kv_heads] grid: ('batch', ranks) when the batch alone can feed every rank,
    else ('heads', ranks_per_batch_element) with each batch element's KV heads split over a sub-group of ranks."""
    if world <= 1:
        return 'batch', 1
    if batch % world == 0:
        return 'batch', world
    if world % batch == 0 and kv_heads % (world // batch) == 0:
        return 'heads', world // batch
    raise ValueError(f'cannot split batch {batch} x kv_heads {kv_heads} evenly over {world} ranks')


def local_slices(batch, kv_heads, world, rank):
    """(batch slice, kv-head slice) owned by `rank`."""
    kind, n = plan(batch, kv_heads, world)
    if kind == 'batch':
        b0, b1 = unit_range(batch, world, rank)
        return slice(b0, b1), slice(0, kv_heads)
    b = rank // n
    h0, h1 = unit_range(kv_heads, n, rank % n)
    return slice(b, b + 1), slice(h0, h1)


def shard_heads(t, kv_slice, group_size):
    """Heads of a [B, H, ...] tensor that belong to the KV heads in `kv_slice` (H = kv_heads * group_size)."""
    return t[:, kv_slice.start * group_size: kv_slice.stop * group_size]


def sharded_selected_attend(fq, fk, fv, block_size, idx, fmask, include_block_causal=True, group=None,
                            attend_fn=None):
    """Selected-block attention with the (batch, KV head) units split over the ranks of `group`; every rank passes the
    full tensors and receives the full output.  `attend_fn` defaults to the CUDA operator."""
    if attend_fn is None:
        from .ops import native_sparse_attend
        attend_fn = native_sparse_attend
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    b, hq = fq.shape[:2]
    hkv = fk.shape[1]
    g = hq // hkv
    sel_g = idx.shape[1] // hkv
    bs, hs = local_slices(b, hkv, world, rank)
    out_local = attend_fn(shard_heads(fq[bs], hs, g), fk[bs][:, hs], fv[bs][:, hs], block_size,
                          shard_heads(idx[bs], hs, sel_g), shard_heads(fmask[bs], hs, sel_g),
                          include_block_causal=include_block_causal)
    if world == 1:
        return out_local
    parts = [torch.empty_like(out_local) for _ in range(world)]
    dist.all_gather(parts, out_local.contiguous(), group=group)
    kind, n = plan(b, hkv, world)
    if kind == 'batch':
        return torch.cat(parts, dim=0)
    rows = [torch.cat(parts[i * n:(i + 1) * n], dim=1) for i in range(b)]
    return torch.cat(rows, dim=0)
