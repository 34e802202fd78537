"""Benchmark of the NSA hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (default): the kernel-level selected-block attention forward+backward
of the baseline's second configuration -- batch 4, 8192 tokens, 32 query
heads over 4 KV heads, dim_head 64, bf16, block 64, 16 selected blocks per
query plus the causal own block, inputs from seeded normal distributions
(synthetic; no dataset is involved).  One step = one forward and one backward
over the whole batch.  The metric is tokens/s = batch*seq / step time, summed
over ranks; with N > 1 every rank runs its own batch of the same shape (the
operator shards over batch and KV-head groups with no exchange), so scaling is
weak and the only collective is the timing reduction.

The printed JSON line also carries:
  roofline     achieved tensor throughput of the dominant kernel (the backward)
               from the algorithmic FLOP count of the selected keys
  e2e          the same metric through the public operator with pinned HOST
               buffers, host<->device copies inside the timed region
  cpu_baseline the CPU oracle (a port of upstream's PyTorch formulation) timed
               on a bounded sample of the same workload on this host's cores
`--impl reference` times that CPU formulation alone, with all host threads.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: batch, seq, q_heads, kv_heads, dim_head, block, nsel
    'sel_fwd_bwd_b4_n8192_h32kv4_d64_blk64_top16': dict(batch=4, seq=8192, q_heads=32, kv_heads=4, dim_head=64,
                                                        block=64, nsel=16),
    'small': dict(batch=1, seq=1024, q_heads=8, kv_heads=2, dim_head=64, block=64, nsel=4),
}
DEFAULT_WORKLOAD = 'sel_fwd_bwd_b4_n8192_h32kv4_d64_blk64_top16'


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the main backward kernel, from an ncu capture of this
# command (profiles/tcgen05_selected_attention_b4_n8192_h32kv4_d64.md, profiles/simt_selected_attention_...md).
NCU_TRAFFIC = {
    (DEFAULT_WORKLOAD, 'auto'): 602.3e6 + 2188.4e6,
    (DEFAULT_WORKLOAD, 'sm100'): 602.3e6 + 2188.4e6,
    (DEFAULT_WORKLOAD, 'simt'): 531.8e6 + 300.4e6,
}


def make_inputs(w, seed, dtype=torch.bfloat16):
    """Seeded host tensors: q,k,v,do ~ N(0,1); block scores ~ N(0,1) with the own and future
    blocks excluded; the top `nsel` scores give the selected blocks, slots with no valid block are masked."""
    g = torch.Generator('cpu').manual_seed(seed)
    b, n, hq, hkv, d, blk, nsel = (w[k] for k in ('batch', 'seq', 'q_heads', 'kv_heads', 'dim_head', 'block', 'nsel'))
    q = torch.randn(b, hq, n, d, generator=g).to(dtype)
    k = torch.randn(b, hkv, n, d, generator=g).to(dtype)
    v = torch.randn(b, hkv, n, d, generator=g).to(dtype)
    nfb = -(-n // blk)
    scores = torch.randn(b, hkv, n, nfb, generator=g)
    own = (torch.arange(n) // blk)[:, None]
    scores.masked_fill_(torch.arange(nfb)[None, :] >= own, float('-inf'))
    vals, idx = scores.topk(min(nsel, nfb), dim=-1)
    mask = torch.isfinite(vals)
    idx = idx.masked_fill(~mask, 0)
    do = torch.randn(b, hq, n, d, generator=g).to(dtype)
    return q, k, v, idx, mask, do


def algorithmic_flops(w, mask):
    """fwd, bwd FLOPs of the attended (query, head, key) pairs: 4*d forward, 10*d backward per pair."""
    n, blk, d, g = w['seq'], w['block'], w['dim_head'], w['q_heads'] // w['kv_heads']
    own = (torch.arange(n) % blk + 1).view(1, 1, n)
    keys = mask.sum(dim=-1) * blk + own          # per (batch, kv head, query)
    pairs = keys.sum().item() * g
    return 4 * d * pairs, 10 * d * pairs


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index):
        self.rows, self.proc = [], None
        self.index = index

    def start(self):
        q = ('clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,'
             'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
             'clocks_event_reasons.sw_power_cap')
        try:
            self.proc = subprocess.Popen(['nvidia-smi', f'--id={self.index}', f'--query-gpu={q}',
                                          '--format=csv,noheader,nounits', '-lms', '100'],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(',')])

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm = [float(r[0]) for r in self.rows if r and r[0].replace('.', '').isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace('.', '').isdigit()]
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        reasons = [nm for j, nm in enumerate(names) if any(len(r) > 3 + j and r[3 + j] == 'Active' for r in self.rows)]
        return {'sm_mhz': statistics.median(sm) if sm else None, 'sm_max_mhz': max(mx) if mx else None,
                'reasons': reasons, 'samples': len(sm)}


def peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        p = json.load(open(path))
        return p['bf16_tflops'], p.get('bf16_tflops_sustained'), 'measured'
    return 1590.0, 1400.0, 'fallback'


def cpu_port_step(w, inputs, rows, heads):
    """One forward+backward of the CPU oracle on `rows` query positions of batch 0 and the first `heads` KV heads."""
    from oracle import nsa_oracle as O
    q, k, v, idx, mask, do = inputs
    g = w['q_heads'] // w['kv_heads']
    qs = q[:1, : heads * g].float().requires_grad_()
    ks = k[:1, :heads].float().requires_grad_()
    vs = v[:1, :heads].float().requires_grad_()
    out = O.selected_attend(qs, ks, vs, w['block'], idx[:1, :heads], mask[:1, :heads], True, rows=rows)
    (out * do[:1, : heads * g][:, :, rows].float()).sum().backward()
    return out


def time_cpu_port(w, inputs, budget_s=15.0):
    """Tokens/s of the CPU port on a bounded sample: `rows` consecutive queries from the middle of the
    sequence, one KV-head group; a token counts 1/kv_heads per head group processed."""
    torch.set_num_threads(os.cpu_count())
    n = w['seq']
    rows_n = min(n, 256)
    start = max(0, n // 2 - rows_n // 2)
    rows = torch.arange(start, start + rows_n)
    cpu_port_step(w, inputs, rows, 1)      # warm-up
    t0, reps = time.perf_counter(), 0
    while True:
        cpu_port_step(w, inputs, rows, 1)
        reps += 1
        el = time.perf_counter() - t0
        if el > budget_s or reps >= 50:
            break
    tokens = reps * rows_n / w['kv_heads']
    return tokens / el, f'{rows_n} queries x 1 of {w["kv_heads"]} KV-head groups of batch element 0, {reps} repetitions'


def run_reference(args, w, name):
    """The reference arm: upstream's PyTorch formulation (CPU oracle port) on the host cores."""
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    inputs = make_inputs(w, seed=0)
    n = w['seq']
    rows_n = min(n, 256)
    start = max(0, n // 2 - rows_n // 2)
    rows = torch.arange(start, start + rows_n)
    torch.set_num_threads(os.cpu_count())
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_port_step(w, inputs, rows, 1)
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        cpu_port_step(w, inputs, rows, 1)
        times.append(time.perf_counter() - t0)
    ms = 1e3 * sum(times) / len(times)
    value = (rows_n / w['kv_heads']) / (ms / 1e3)
    sample = f'each step: {rows_n} queries x 1 of {w["kv_heads"]} KV-head groups of batch element 0'
    print(json.dumps({
        'impl': 'reference', 'metric': 'nsa_selected_attention_fwd_bwd_tokens_per_s', 'value': value,
        'unit': 'tokens/s', 'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': ms,
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': name, **w},
        'cpu_baseline': {'value': value, 'unit': 'tokens/s', 'cores': os.cpu_count(), 'kind': 'port', 'sample': sample},
        'e2e': {'value': value, 'unit': 'tokens/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--workload', default=DEFAULT_WORKLOAD, choices=list(WORKLOADS))
    ap.add_argument('--kernels', default='auto', choices=['auto', 'simt', 'sm100'])
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--rows', action='store_true', help='also time the other kernels of the hot path (N=1 only)')
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if args.impl == 'reference':
        return run_reference(args, w, args.workload)

    import torch.distributed as dist
    import native_sparse_attention_pytorch_b200 as nsa

    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)
    warmup = max(args.warmup, 3)

    host = make_inputs(w, seed=rank)
    pinned = [t.pin_memory() for t in host]
    q, k, v, idx, mask, do = (t.to(dev) for t in host)
    f_fwd, f_bwd = algorithmic_flops(w, host[4])
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)     # > 126 MB of L2

    def step(qd, kd, vd, idxd, maskd, dod, ev=None):
        qd, kd, vd = (t.detach().requires_grad_() for t in (qd, kd, vd))
        if ev:
            ev[0].record()
        out = nsa.native_sparse_attend(qd, kd, vd, w['block'], idxd, maskd, include_block_causal=True,
                                       impl=args.kernels)
        if ev:
            ev[1].record()
        grads = torch.autograd.grad(out, (qd, kd, vd), dod)
        if ev:
            ev[2].record()
        return out, grads

    for _ in range(warmup):
        step(q, k, v, idx, mask, do)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    events = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    for i in range(args.steps):
        flush.fill_(i & 0xff)             # evict L2 between timed iterations (outside the events)
        step(q, k, v, idx, mask, do, events[i])
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    fwd_ms = [e[0].elapsed_time(e[1]) for e in events]
    bwd_ms = [e[1].elapsed_time(e[2]) for e in events]
    total_ms = sum(fwd_ms) + sum(bwd_ms)

    # end to end: every step copies its inputs from pinned host buffers and its results (out, dq, dk, dv) back to
    # the host.  The copies run on their own streams, double buffered, so that step i+1's inputs travel while step i
    # computes and step i-1's results travel back; every step's copies are inside the timed region.
    h_out = [torch.empty_like(t).pin_memory() for t in (host[0], host[0], host[1], host[2])]
    s_in, s_out, s_main = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
    dev_in = [[torch.empty_like(t, device=dev) for t in host] for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]

    def e2e_run(steps):
        for i in range(steps):
            b = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(in_free[b])
                for d, src in zip(dev_in[b], pinned):
                    d.copy_(src, non_blocking=True)
                in_ready[b].record(s_in)
            s_main.wait_event(in_ready[b])
            out, grads = step(*dev_in[b])
            in_free[b].record(s_main)
            done = torch.cuda.Event()
            done.record(s_main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for dst, src in zip(h_out, (out, *grads)):
                    dst.copy_(src, non_blocking=True)
                    src.record_stream(s_out)
        s_main.wait_stream(s_out)

    e2e_run(2)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(3, min(args.steps, 10))
    e0.record()
    e2e_run(e2e_steps)
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1)

    t = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = t.tolist()
    tokens_per_step = w['batch'] * w['seq'] * world
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    ms_per_step = total_ms / args.steps
    value = tokens_per_step / (ms_per_step / 1e3)
    burst, sustained, src = peaks()
    bwd_avg_ms = sum(bwd_ms) / len(bwd_ms)
    fwd_avg_ms = sum(fwd_ms) / len(fwd_ms)
    achieved = f_bwd / (bwd_avg_ms / 1e3) / 1e12
    h2d = sum(t.numel() * t.element_size() for t in pinned)
    d2h = sum(t.numel() * t.element_size() for t in h_out)
    line = {
        'metric': 'nsa_selected_attention_fwd_bwd_tokens_per_s', 'value': value, 'unit': 'tokens/s',
        'n_gpus': world, 'steps': args.steps, 'warmup': warmup, 'ms_per_step': ms_per_step,
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic',
        'config': {'workload': args.workload, **w, 'kernels': args.kernels, 'l2': 'flushed between timed steps',
                   'per_rank': 'each rank runs the full shape on its own seeded batch'},
        'fwd_ms': fwd_avg_ms, 'bwd_ms': bwd_avg_ms,
        'tensor_frac_fwd_bwd': (f_fwd + f_bwd) / (ms_per_step / 1e3) / 1e12 / burst,
        'roofline': {'bound': 'tensor', 'kernel': 'selected-block backward', 'achieved': achieved, 'peak': burst,
                     'unit': 'TFLOP/s', 'frac': achieved / burst, 'peak_source': src, 'peak_sustained': sustained,
                     'flops_per_launch': f_bwd, 'traffic': NCU_TRAFFIC.get((args.workload, args.kernels))},
        'e2e': {'value': tokens_per_step / (e2e_ms / e2e_steps / 1e3), 'unit': 'tokens/s',
                'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h, 'steps': e2e_steps},
        'gpu_launches': None,
        'clocks': clocks,
    }
    from native_sparse_attention_pytorch_b200 import _lib
    line['gpu_launches'] = launches_per_step(args.kernels, w) * args.steps
    if args.rows and world == 1:
        del q, k, v, idx, mask, do
        line['rows'] = measure_rows(dev, flush)
    if not args.no_cpu_baseline and world == 1:
        val, sample = time_cpu_port(w, host)
        line['cpu_baseline'] = {'value': val, 'unit': 'tokens/s', 'cores': os.cpu_count(), 'kind': 'port',
                                'sample': sample}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def measure_rows(dev, flush, iters=5):
    """Times every other kernel of the hot path (compressed attention, block selection, sliding window, gated
    combine, and the selected-block kernels at the layer's head grouping) at the shapes of the full-layer
    configuration: batch 2, 16384 tokens, 16 query / 4 KV heads, dim_head 64, compress stride 16, block 64,
    16 selected blocks, window 512, bf16.  Returns {row: {ms, achieved, unit, peak, frac, bound}}."""
    import native_sparse_attention_pytorch_b200 as nsa
    b, hq, hkv, n, d, st, blk, nsel, win = 2, 16, 4, 16384, 64, 16, 64, 16, 512
    g = hq // hkv
    ncb = n // st
    gen = torch.Generator('cpu').manual_seed(1)
    rnd = lambda *shape: torch.randn(*shape, generator=gen).bfloat16().to(dev)
    q, k, v, do = rnd(b, hq, n, d), rnd(b, hkv, n, d), rnd(b, hkv, n, d), rnd(b, hq, n, d)
    ck, cv = rnd(b, hkv, 1 + ncb, d), rnd(b, hkv, 1 + ncb, d)
    gates = torch.sigmoid(rnd(b, n, hq * 3)).view(b, n, hq, 3).transpose(1, 2)
    tf_peak, _, _ = peaks()
    hbm_peak = json.load(open(os.path.join(ROOT, 'MEASURED_PEAKS.json')))['hbm_gbs'] if os.path.exists(
        os.path.join(ROOT, 'MEASURED_PEAKS.json')) else 6650.0

    def timed(fn):
        for _ in range(2):
            fn()
        evs = []
        for i in range(iters):
            flush.fill_(i)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            evs.append((e0, e1))
        torch.cuda.synchronize()
        return sum(a.elapsed_time(c) for a, c in evs) / iters

    rows = {}

    def add(name, ms, work, bound):
        if bound == 'tensor':
            ach, peak, unit = work / (ms / 1e3) / 1e12, tf_peak, 'TFLOP/s'
        else:
            ach, peak, unit = work / (ms / 1e3) / 1e9, hbm_peak, 'GB/s'
        rows[name] = {'ms': ms, 'achieved': ach, 'unit': unit, 'peak': peak, 'frac': ach / peak, 'bound': bound}

    i = torch.arange(n)
    # compressed attention (+ importance)
    pairs = float(((i // st).clamp(max=ncb) + 1).sum()) * b * hq
    qd, ckd, cvd = (t.detach().requires_grad_() for t in (q, ck, cv))
    holder = {}
    def cmp_fwd():
        holder['o'], holder['imp'] = nsa.compressed_attend(qd, ckd, cvd, 1, st, True)
    add('compressed_fwd', timed(cmp_fwd), 4 * d * pairs, 'tensor')
    add('compressed_bwd', timed(lambda: torch.autograd.grad(holder['o'], (qd, ckd, cvd), do, retain_graph=True)),
        10 * d * pairs, 'tensor')
    imp = holder['imp']
    # block selection
    def select():
        holder['vals'], holder['idx'] = nsa.select_blocks(imp, blk, st, nsel, dtype=torch.bfloat16)
    ms = timed(select)
    add('select', ms, imp.numel() * 4 + b * hkv * n * nsel * 12, 'hbm')
    idx, mask = holder['idx'], holder['vals'] > 1e-10
    # selected-block attention at this head grouping
    keys = (mask.sum(dim=-1).cpu() * blk + (i % blk + 1).view(1, 1, n)).sum().item() * g
    qd2, kd2, vd2 = (t.detach().requires_grad_() for t in (q, k, v))
    def sel_fwd():
        holder['os'] = nsa.native_sparse_attend(qd2, kd2, vd2, blk, idx, mask)
    add('selected_fwd', timed(sel_fwd), 4 * d * keys, 'tensor')
    add('selected_bwd', timed(lambda: torch.autograd.grad(holder['os'], (qd2, kd2, vd2), do, retain_graph=True)),
        10 * d * keys, 'tensor')
    # sliding window
    pairs = float((i.clamp(max=win) + 1).sum()) * b * hq
    qd3, kd3, vd3 = (t.detach().requires_grad_() for t in (q, k, v))
    def swa_fwd():
        holder['ow'] = nsa.sliding_window_attend(qd3, kd3, vd3, win, True)
    add('sliding_fwd', timed(swa_fwd), 4 * d * pairs, 'tensor')
    add('sliding_bwd', timed(lambda: torch.autograd.grad(holder['ow'], (qd3, kd3, vd3), do, retain_graph=True)),
        10 * d * pairs, 'tensor')
    # gated combine
    o1, o2, o3 = (t.detach().requires_grad_() for t in (holder['o'], holder['os'], holder['ow']))
    gd = gates.detach().requires_grad_()
    def comb_fwd():
        holder['m'] = nsa.gated_combine(o1, o2, o3, gd)
    act = b * hq * n * d * 2
    add('combine_fwd', timed(comb_fwd), 4 * act + gates.numel() * 2, 'hbm')
    dm = torch.randn_like(holder['m'])
    add('combine_bwd', timed(lambda: torch.autograd.grad(holder['m'], (o1, o2, o3, gd), dm, retain_graph=True)),
        7 * act + gates.numel() * 6, 'hbm')
    return rows


def launches_per_step(kernels, w):
    """Kernels of this library launched by one forward+backward of the operator."""
    if kernels == 'simt':
        return 2   # one forward kernel, one backward kernel (gradient buffers are cleared by memset)
    # tensor-core family: index pre-pass (4 kernels) + main + merge forward;
    # index pre-pass + delta + main + dq merge backward
    return 6 + 7


if __name__ == '__main__':
    main()
