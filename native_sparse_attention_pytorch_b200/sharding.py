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


def attend_core(q, qr, kr, v, ck, cv, gates, *, num_mem, stride, block, num_selected, window, causal=True,
                impl='auto', attend_fns=None, combine=None):
    """The hot path between the projections (upstream NSA:621-860) for the heads it is given: compressed attention with
    the importance by-product, block selection, selected-block attention, sliding window, gated combine.

    q: un-rotated queries [B, Hq, N, d]; qr, kr: rotated queries / keys; v: values [B, Hkv, N, d]; ck, cv: compressed
    keys / values with the `num_mem` memory slots in front [B, Hkv, num_mem + ncb, d]; gates [B, Hq, N, 3] (order:
    compressed, selected, sliding).  Returns the merged output [B, N, Hq * d].  `attend_fns` replaces the CUDA operators
    (a dict with the keys used below); the CPU tests pass the oracle's functions.  `combine` replaces the last step
    only (the fused combine + gather of the sharded path) and its result is returned."""
    if attend_fns is None:
        from . import ops
        attend_fns = dict(compressed=ops.compressed_attend, select=ops.select_blocks,
                          selected=ops.native_sparse_attend, sliding=ops.sliding_window_attend,
                          combine=ops.gated_combine)
        kw = dict(impl=impl)
        ckw = dict(impl=impl, pool=block // stride if causal and block % stride == 0 else 0)
    else:
        kw = ckw = {}
    hkv = v.shape[1]
    o_cmp, importance = attend_fns['compressed'](q, ck, cv, num_mem, stride, causal, sel_heads=hkv,
                                                 want_importance=True, **ckw)
    vals, idx = attend_fns['select'](importance, block, stride, num_selected, dtype=q.dtype)
    fmask = vals > 1e-10
    o_sel = attend_fns['selected'](qr, kr, v, block, idx, fmask, include_block_causal=causal, **kw)
    o_swa = attend_fns['sliding'](qr, kr, v, window, causal, **kw)
    return (combine or attend_fns['combine'])(o_cmp, o_sel, o_swa, gates)


def _split_pass(q, qr, kr, v, ck, cv, gates, peer_output, offset, splits, overlap, *, num_mem, stride, block,
                num_selected, window, causal=True, impl='auto', fuse_merge=False):
    """One pass of `sharded_attend_core` over the given KV heads with the query heads of every KV head cut into
    `splits` runs: compressed attention and selection for all heads, then selected + sliding + combine-and-store per
    run.  The features of run r of KV head h sit where the unsplit pass puts them.  With `fuse_merge` the sliding
    branch of a run goes first and the selected branch's last kernel does the combine and the stores
    (`ops.selected_attend_combine_gather`), where the library serves that."""
    from . import ops
    hkv, g, d = v.shape[1], q.shape[1] // v.shape[1], q.shape[-1]
    runs = tuple(splits) if isinstance(splits, (tuple, list)) else (g // splits,) * splits
    if sum(runs) != g or any(r < 1 or r & (r - 1) for r in runs):
        raise ValueError(f'{g} query heads per KV head do not split into runs of {runs} (powers of two that add up)')
    pool = block // stride if causal and block % stride == 0 else 0
    o_cmp, importance = ops.compressed_attend(q, ck, cv, num_mem, stride, causal, sel_heads=hkv, want_importance=True,
                                              impl=impl, pool=pool)
    vals, idx = ops.select_blocks(importance, block, stride, num_selected, dtype=q.dtype)
    fmask = vals > 1e-10
    del importance
    shared = [{} for _ in range(hkv)]      # per KV head: runs of equal size share the index of their selection
    first = 0
    for per in runs:
        for h in range(hkv):
            heads = slice(h * g + first, h * g + first + per)
            kh = slice(h, h + 1)
            at = offset + heads.start * d
            if fuse_merge:
                o_swa = ops.sliding_window_attend(qr[:, heads], kr[:, kh], v[:, kh], window, causal, impl=impl)
                mc = peer_output.multicast_ptr
                if ops.selected_attend_combine_gather(
                        qr[:, heads], kr[:, kh], v[:, kh], block, idx[:, kh], fmask[:, kh], o_cmp[:, heads], o_swa,
                        gates[:, heads], [mc] if mc is not None else peer_output.ptrs, peer_output.features, at,
                        include_block_causal=causal, multicast=mc is not None, impl=impl, index_cache=shared[h]):
                    continue
            else:
                o_swa = None
            o_sel = ops.native_sparse_attend(qr[:, heads], kr[:, kh], v[:, kh], block, idx[:, kh], fmask[:, kh],
                                             include_block_causal=causal, impl=impl, index_cache=shared[h])
            if o_swa is None:
                o_swa = ops.sliding_window_attend(qr[:, heads], kr[:, kh], v[:, kh], window, causal, impl=impl)
            peer_output.store(o_cmp[:, heads], o_sel, o_swa, gates[:, heads], at, overlap)
        first += per


def kv_head_range(kv_heads, world, rank):
    """KV heads owned by `rank` when the heads of one batch element are dealt out over `world` ranks."""
    if kv_heads % world != 0:
        raise ValueError(f'{kv_heads} KV heads do not split evenly over {world} ranks')
    per = kv_heads // world
    return rank * per, (rank + 1) * per


def gather_heads(merged_local, group=None):
    """All-gather of the merged output along the head axis: every rank contributes [B, N, Hl * d] (its own heads, in
    rank order) and receives [B, N, world * Hl * d].  The one collective of the sharded path."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return merged_local
    b, n, f = merged_local.shape
    parts = torch.empty(world * b, n, f, dtype=merged_local.dtype, device=merged_local.device)
    dist.all_gather_into_tensor(parts, merged_local.contiguous(), group=group)
    return parts.view(world, b, n, f).permute(1, 2, 0, 3).reshape(b, n, world * f)


class PeerOutput:
    """The gathered output [B, N, features] of every rank in symmetric memory, so that each rank's combine kernel can
    store its heads straight into all of them (`ops.gated_combine_gather`): the all-gather without a collective call
    and without a local copy of the merged rows.  `begin()` / `end()` order one step against the other ranks: nobody
    stores into a buffer that a peer may still be reading, nobody reads before every peer's stores have landed."""

    def __init__(self, batch, seq, features, dtype, device, group=None, multicast=False):
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.buffer = symm.empty(batch, seq, features, dtype=dtype, device=device)
        self.handle = symm.rendezvous(self.buffer, self.group)
        # the handle's addresses are those of the allocation; the tensor may start inside it
        inside = self.buffer.data_ptr() - int(self.handle.buffer_ptrs[self.rank])
        self.ptrs = [int(p) + inside for p in self.handle.buffer_ptrs]
        self.features = features
        # `multicast`: store through the buffer's NVLink multicast address (one multimem.st per piece, the switch
        # writes every rank's copy) where the symmetric memory has one; plain peer stores otherwise
        mc = int(getattr(self.handle, 'multicast_ptr', 0) or 0) if multicast else 0
        self.multicast_ptr = mc + inside if mc != 0 else None

        self.side = torch.cuda.Stream(device=device)    # the stores of one pass travel while the next pass computes
        self._alive = []

    def begin(self):
        self.handle.barrier(channel=0)

    def store(self, o_cmp, o_sel, o_swa, gates, offset, overlap):
        """Combine the three branch outputs of some heads and store them at feature `offset` of every rank's buffer.
        With `overlap` the kernel runs on the side stream, behind everything the current stream has queued so far, so
        that the NVLink traffic of this piece overlaps whatever the caller launches next."""
        from . import ops
        main = torch.cuda.current_stream(self.buffer.device)
        if overlap:
            self.side.wait_stream(main)
            self._alive.append((o_cmp, o_sel, o_swa, gates))     # until end(): the side stream still reads them
        with torch.cuda.stream(self.side if overlap else main):
            if self.multicast_ptr is not None:
                ops.gated_combine_gather(o_cmp, o_sel, o_swa, gates, [self.multicast_ptr], self.features, offset,
                                         multicast=True)
            else:
                ops.gated_combine_gather(o_cmp, o_sel, o_swa, gates, self.ptrs, self.features, offset)

    def end(self):
        torch.cuda.current_stream(self.buffer.device).wait_stream(self.side)
        self.handle.barrier(channel=1)
        self._alive.clear()     # the barrier is queued behind the stores; the caching allocator frees in stream order
        return self.buffer


class LocalOutput:
    """The interface of `PeerOutput` for one GPU that holds all heads: the merged output [B, N, features] is a plain
    tensor and the only destination, so the forms of `sharded_attend_core` that store per pass (side stream, runs of
    query heads, the selected branch's merge doing the combine) can be used, and measured, without other ranks."""

    def __init__(self, batch, seq, features, dtype, device):
        self.buffer = torch.empty(batch, seq, features, dtype=dtype, device=device)
        self.ptrs = [self.buffer.data_ptr()]
        self.features = features
        self.multicast_ptr = None
        self.side = torch.cuda.Stream(device=device)
        self._alive = []

    def begin(self):
        pass

    store = PeerOutput.store

    def end(self):
        torch.cuda.current_stream(self.buffer.device).wait_stream(self.side)
        self._alive.clear()
        return self.buffer


def sharded_attend_core(q, qr, kr, v, ck, cv, gates, *, group=None, heads_per_pass=1, peer_output=None,
                        overlap=False, head_splits=1, fuse_merge=False, **cfg):
    """`attend_core` with the KV-head groups split over the ranks of `group` (long-context prefill: batch 1, one or a
    few KV heads per GPU).  Every rank passes tensors that hold (at least) its own heads -- either the full tensors or
    already the local slices (`local=True` in cfg) -- and receives the full merged output [B, N, Hq * d].  The local
    heads are processed `heads_per_pass` KV heads at a time to bound the work buffers.

    With a `peer_output`, `overlap` sends each pass's combine + stores to a side stream, so they travel while the next
    pass computes, and `head_splits` (a number of equal runs, or a tuple of run sizes such as (4, 2, 2)) cuts a pass
    once more: compressed attention and the selection run for all query heads of the KV head (the selection is shared
    by them), the selected and the sliding branch then run for one run of query heads at a time, each run stored as
    soon as it is complete; runs of equal size share the index of the selection.  `fuse_merge` lets the selected
    branch's last kernel do the combine and the stores (the sliding branch then runs before it): no separate store
    kernel, and the stores leave from a kernel that is streaming anyway.  Every rank must
    receive the whole output over NVLink whatever the form of the gather (7/8 of it on eight GPUs); only what
    follows the last piece is not hidden behind compute."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    local = cfg.pop('local', False)
    hkv_total = v.shape[1] * (world if local else 1)
    g = q.shape[1] // v.shape[1]
    h0, h1 = (0, v.shape[1]) if local else kv_head_range(hkv_total, world, rank)
    b, _, n, d = q.shape
    if peer_output is not None:
        # fused path: the combine of every pass stores into all ranks' output buffers
        first = (rank * (h1 - h0) if local else h0) * g * d     # first feature of this rank's heads
        peer_output.begin()
        for a in range(h0, h1, heads_per_pass):
            z = min(a + heads_per_pass, h1)
            hs, qs = slice(a, z), slice(a * g, z * g)

            offset = first + (a - h0) * g * d
            if head_splits != 1 or fuse_merge:
                _split_pass(q[:, qs], qr[:, qs], kr[:, hs], v[:, hs], ck[:, hs], cv[:, hs], gates[:, qs], peer_output,
                            offset, head_splits, overlap, fuse_merge=fuse_merge, **cfg)
                continue

            def combine_into_peers(o_cmp, o_sel, o_swa, gts, offset=offset):
                peer_output.store(o_cmp, o_sel, o_swa, gts, offset, overlap)

            attend_core(q[:, qs], qr[:, qs], kr[:, hs], v[:, hs], ck[:, hs], cv[:, hs], gates[:, qs],
                        combine=combine_into_peers, **cfg)
        return peer_output.end()
    merged = torch.empty(b, n, (h1 - h0) * g * d, dtype=q.dtype, device=q.device)
    for a in range(h0, h1, heads_per_pass):
        z = min(a + heads_per_pass, h1)
        hs, qs = slice(a, z), slice(a * g, z * g)
        part = attend_core(q[:, qs], qr[:, qs], kr[:, hs], v[:, hs], ck[:, hs], cv[:, hs], gates[:, qs], **cfg)
        merged[..., (a - h0) * g * d:(z - h0) * g * d] = part
    return gather_heads(merged, group)


class BucketedGradientSum:
    """Data-parallel gradient sum that overlaps the backward: the parameters are grouped into buckets (one per layer, in
    the order the backward reaches them) and a bucket's all-reduce is launched, asynchronously, as soon as the last of
    its gradients has been accumulated; `finish()` waits for all of them and copies the sums back.  The result equals
    one flat all-reduce after the backward (the same element-wise sums over the ranks).  The only collective of the
    training step (NCCL over NVLink on GPUs; the CPU tests run it over gloo)."""

    def __init__(self, buckets, group=None):
        self.group = group
        self.buckets = [[p for p in b if p.requires_grad] for b in buckets]
        self.buckets = [b for b in self.buckets if b]
        self._left = [0] * len(self.buckets)
        self._works = []
        self._fired = [False] * len(self.buckets)
        for bi, bucket in enumerate(self.buckets):
            for p in bucket:
                p.register_post_accumulate_grad_hook(self._make_hook(bi))
        self.start()

    def start(self):
        """Call before every backward."""
        self._left = [len(b) for b in self.buckets]
        self._fired = [False] * len(self.buckets)
        self._works = []

    def _make_hook(self, bi):
        def hook(_param):
            if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
                return      # a CUDA graph of the step is being recorded: its owner sums the gradients after replay
            self._left[bi] -= 1
            if self._left[bi] == 0 and not self._fired[bi]:
                self._launch(bi)
        return hook

    def _launch(self, bi):
        self._fired[bi] = True
        grads = [p.grad for p in self.buckets[bi] if p.grad is not None]
        if not grads:
            return
        flat = torch._utils._flatten_dense_tensors(grads)
        work = dist.all_reduce(flat, group=self.group, async_op=True)
        self._works.append((work, flat, grads))

    def finish(self):
        """Call after the backward: buckets whose parameters did not all receive a gradient are summed now, then every
        sum is awaited (on a GPU: the current stream waits, the host does not) and written back to the gradients."""
        for bi in range(len(self.buckets)):
            if not self._fired[bi]:
                self._launch(bi)
        for work, flat, grads in self._works:
            work.wait()
            for g, f in zip(grads, torch._utils._unflatten_dense_tensors(flat, grads)):
                g.copy_(f)
        self._works = []
