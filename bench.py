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
  roofline     achieved tensor throughput of the whole step (forward+backward)
               from the algorithmic FLOP count of the selected keys; `kernels`
               below it lists every kernel of the step with its own time
               (CUPTI, a separate untimed pass), work and fraction
  workloads    the full-layer step and the long-context prefill (sharded over
               the ranks by KV-head group, output gathered: strong scaling)
               measured by the same file in child processes, so that one
               record holds all three
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

# Two more workloads of the baseline (not the default line): the full layer forward+backward and the long-context
# prefill that is sharded over the GPUs by KV-head group with the output all-gathered.
LAYER_WORKLOADS = {
    'layer_fwd_bwd_b2_n16384_dim1024_h16kv4_d64': dict(
        batch=2, seq=16384, dim=1024, heads=16, kv_heads=4, dim_head=64, sliding_window_size=512,
        compress_block_size=32, compress_block_sliding_stride=16, selection_block_size=64, num_selected_blocks=16),
    'layer_small': dict(batch=1, seq=1024, dim=256, heads=4, kv_heads=2, dim_head=64, sliding_window_size=128,
                        compress_block_size=32, compress_block_sliding_stride=16, selection_block_size=64,
                        num_selected_blocks=4),
}
LM_WORKLOADS = {
    # the language-model training step of the baseline's fourth configuration: 8 pre-norm blocks of
    # [SparseAttention, feed-forward x4 GELU], byte vocabulary, next-token cross-entropy, forward+backward
    'lm_step_b8_n8192_dim512_depth8': dict(batch=8, seq=8192, vocab=256, dim=512, depth=8, heads=8, kv_heads=4,
                                           dim_head=64, sliding_window_size=512, compress_block_size=32,
                                           compress_block_sliding_stride=16, selection_block_size=64,
                                           num_selected_blocks=16),
    'lm_small': dict(batch=2, seq=1024, vocab=256, dim=256, depth=2, heads=4, kv_heads=2, dim_head=64,
                     sliding_window_size=128, compress_block_size=32, compress_block_sliding_stride=16,
                     selection_block_size=64, num_selected_blocks=4),
}
PREFILL_WORKLOADS = {
    'prefill_b1_n65536_h64kv8_d128': dict(batch=1, seq=65536, q_heads=64, kv_heads=8, dim_head=128,
                                          compress_block_size=32, stride=16, block=64, nsel=16, window=512, num_mem=1),
    'prefill_small': dict(batch=1, seq=4096, q_heads=16, kv_heads=2, dim_head=128, compress_block_size=32, stride=16,
                          block=64, nsel=16, window=512, num_mem=1),
    # the same grouping at a length whose work buffers exceed the L2 but stay under 2 GB: the size for profiler captures
    'prefill_mid': dict(batch=1, seq=16384, q_heads=16, kv_heads=2, dim_head=128, compress_block_size=32, stride=16,
                        block=64, nsel=16, window=512, num_mem=1),
}


# dram__bytes_read.sum + dram__bytes_write.sum per launch, from single-launch ncu captures of this command
# (`ncu --set full -k regex:<kernel> -c 1 python bench.py --steps 2 --warmup 3 --no-cpu-baseline`) at this build.
NCU_DRAM_BYTES = {
    'sel_bwd_ws_kernel': 701.6e6 + 2195.7e6,
    'sel_fwd_kernel': 902.5e6 + 2425.9e6,
    'sel_merge_kernel': 2417.0e6,      # dram__bytes.sum.per_second x gpu__time_duration of a sections-only capture
    'sel_dq_merge_kernel': 2312.0e6,
    'sel_delta_kernel': 276.0e6,
}
# the other workloads whose numbers ride on the default line: (name, timed steps)
EXTRA_WORKLOADS = (('layer_fwd_bwd_b2_n16384_dim1024_h16kv4_d64', 5), ('prefill_b1_n65536_h64kv8_d128', 3),
                   ('lm_step_b8_n8192_dim512_depth8', 3))
CHILD_TIMEOUT_S = 240


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


def emit(line):
    """Rank 0 prints the line of a workload; every rank leaves its process group."""
    import torch.distributed as dist
    if line is not None:
        print(json.dumps(line))
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()


def launch_count():
    from native_sparse_attention_pytorch_b200 import _lib
    return int(_lib.load().nsa_launch_count())


def kernel_breakdown(step_fn, steps=2):
    """Per-kernel device time of `steps` untimed steps, from CUPTI through torch.profiler: {name: (launches per step,
    mean microseconds per launch)}; None when the profiler is not available."""
    try:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(steps):
                step_fn()
            torch.cuda.synchronize()
        rows = {}
        for ev in prof.key_averages():
            us = getattr(ev, 'device_time_total', None)
            if us is None:
                us = getattr(ev, 'cuda_time_total', 0.0)
            if us and ev.count:
                rows[ev.key] = (ev.count / steps, us / ev.count)
        return rows
    except Exception as exc:      # the breakdown is an explanation, never a reason to lose the measurement
        sys.stderr.write(f'kernel breakdown unavailable: {exc}\n')
        return None


def child_workload(name, steps, world, index):
    """Runs `bench.py --workload name` as a child process of this rank (all ranks do, on a rendezvous port of their own)
    and returns rank 0's line in short form.  A child that fails or overruns costs its entry, not the parent's line."""
    # torchrun's own variables must not reach the child: with TORCHELASTIC_USE_AGENT_STORE set a rank 0 would look
    # for the launcher's rendezvous store on the new port instead of opening one, and every child would wait for it
    env = {k: v for k, v in os.environ.items() if not k.startswith('TORCHELASTIC_')}
    if world > 1:
        env['MASTER_PORT'] = str(int(env.get('MASTER_PORT', '29500')) + 1 + index)
    cmd = [sys.executable, os.path.abspath(__file__), '--gpus', str(world), '--steps', str(steps), '--warmup', '3',
           '--workload', name, '--no-cpu-baseline']
    try:
        out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=CHILD_TIMEOUT_S)
    except subprocess.TimeoutExpired:
        return {'error': f'child run exceeded {CHILD_TIMEOUT_S} s'} if int(os.environ.get('RANK', '0')) == 0 else None
    if int(os.environ.get('RANK', '0')) != 0:
        return None
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith('{')]
    if out.returncode != 0 or not lines:
        return {'error': f'child run failed (rc {out.returncode}): ' + out.stderr.strip().splitlines()[-1][:200]
                if out.stderr.strip() else f'child run failed (rc {out.returncode})'}
    full = json.loads(lines[-1])
    keep = ('metric', 'value', 'unit', 'n_gpus', 'steps', 'ms_per_step', 'scaling', 'gpu_launches')
    short = {k: full.get(k) for k in keep}
    short['config'] = {k: v for k, v in full.get('config', {}).items() if k in ('workload', 'sharding', 'parallelism', 'per_rank', 'gather_check', 'step')}
    short['roofline'] = {k: v for k, v in full.get('roofline', {}).items() if k in ('achieved', 'peak', 'unit', 'frac', 'kernel')}
    short['e2e'] = full.get('e2e')
    return short


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--workload', default=DEFAULT_WORKLOAD,
                    choices=list(WORKLOADS) + list(LAYER_WORKLOADS) + list(PREFILL_WORKLOADS) + list(LM_WORKLOADS))
    ap.add_argument('--kernels', default='auto', choices=['auto', 'simt', 'sm100'])
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--gather', default='auto', choices=['auto', 'multimem', 'fused', 'nccl'],
                    help='prefill workloads, N > 1: the combine kernel stores its heads into every rank, through the '
                         'NVLink multicast address with multimem.st (multimem; falls back to fused where the symmetric '
                         'memory has no multicast) or with one peer store per rank (fused); auto times a few untimed '
                         'steps of both and keeps the faster; or an NCCL all-gather')
    ap.add_argument('--overlap', action='store_true', help='prefill, fused gather: stores on a side stream')
    ap.add_argument('--fuse-merge', action='store_true',
                    help="prefill, fused gather: the selected branch's last kernel combines and stores")
    ap.add_argument('--head-splits', type=int, default=1,
                    help='prefill, fused gather: query heads of a KV head in this many runs, each stored when complete')
    ap.add_argument('--no-graph', action='store_true', help='layer and language-model step: issue the kernels one by one instead of replaying a CUDA graph')
    ap.add_argument('--rows', action='store_true', help='also time the other kernels of the hot path (N=1 only)')
    ap.add_argument('--no-workloads', action='store_true', help='default workload: skip the layer and prefill child runs')
    args = ap.parse_args()
    if args.workload in LAYER_WORKLOADS:
        return emit(run_layer(args, LAYER_WORKLOADS[args.workload]))
    if args.workload in PREFILL_WORKLOADS:
        return emit(run_prefill(args, PREFILL_WORKLOADS[args.workload]))
    if args.workload in LM_WORKLOADS:
        return emit(run_lm(args, LM_WORKLOADS[args.workload]))
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
    launches_before = launch_count()
    for i in range(args.steps):
        flush.fill_(i & 0xff)             # evict L2 between timed iterations (outside the events)
        step(q, k, v, idx, mask, do, events[i])
    torch.cuda.synchronize()
    launches = launch_count() - launches_before
    nsa.ops.check_device_status()     # a kernel that gave up on a bounded wait makes the whole measurement void
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
    clocks = sampler.stop() if rank == 0 else None     # sampled over both timed regions (device-resident and end to end)
    breakdown = kernel_breakdown(lambda: step(q, k, v, idx, mask, do)) if rank == 0 else None

    t = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = t.tolist()
    tokens_per_step = w['batch'] * w['seq'] * world

    line = None
    if rank == 0:
        ms_per_step = total_ms / args.steps
        value = tokens_per_step / (ms_per_step / 1e3)
        burst, sustained, src = peaks()
        bwd_avg_ms = sum(bwd_ms) / len(bwd_ms)
        fwd_avg_ms = sum(fwd_ms) / len(fwd_ms)
        achieved = (f_fwd + f_bwd) / (ms_per_step / 1e3) / 1e12
        h2d = sum(t_.numel() * t_.element_size() for t_ in pinned)
        d2h = sum(t_.numel() * t_.element_size() for t_ in h_out)
        line = {
            'metric': 'nsa_selected_attention_fwd_bwd_tokens_per_s', 'value': value, 'unit': 'tokens/s',
            'n_gpus': world, 'steps': args.steps, 'warmup': warmup, 'ms_per_step': ms_per_step,
            'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic',
            'config': {'workload': args.workload, **w, 'kernels': args.kernels, 'l2': 'flushed between timed steps',
                       'per_rank': 'each rank runs the full shape on its own seeded batch'},
            'fwd_ms': fwd_avg_ms, 'bwd_ms': bwd_avg_ms,
            'roofline': {'bound': 'tensor', 'kernel': 'selected-block attention, forward + backward (whole step)',
                         'achieved': achieved, 'peak': burst, 'unit': 'TFLOP/s', 'frac': achieved / burst,
                         'peak_source': src, 'peak_sustained': sustained, 'frac_of_sustained': achieved / sustained,
                         'flops_per_step': f_fwd + f_bwd, 'flops_fwd': f_fwd, 'flops_bwd': f_bwd,
                         'frac_fwd': f_fwd / (fwd_avg_ms / 1e3) / 1e12 / burst,
                         'frac_bwd': f_bwd / (bwd_avg_ms / 1e3) / 1e12 / burst,
                         'traffic': None, 'kernels': kernel_rows(breakdown, w, host[4], f_fwd, f_bwd, burst)},
            'e2e': {'value': tokens_per_step / (e2e_ms / e2e_steps / 1e3), 'unit': 'tokens/s',
                    'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h, 'steps': e2e_steps},
            'gpu_launches': launches,
            'clocks': clocks,
        }
        top = max(line['roofline']['kernels'] or [{'dram_bytes': None, 'ms': 0}], key=lambda r: r['ms'])
        line['roofline']['traffic'] = top.get('dram_bytes')
        if args.rows and world == 1:
            del q, k, v, idx, mask, do
            line['rows'] = measure_rows(dev, flush)
        if not args.no_cpu_baseline and world == 1:
            val, sample = time_cpu_port(w, host)
            line['cpu_baseline'] = {'value': val, 'unit': 'tokens/s', 'cores': os.cpu_count(), 'kind': 'port',
                                    'sample': sample}
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not args.no_workloads and args.workload == DEFAULT_WORKLOAD:
        # the other baseline configurations in child processes of every rank; this process gives its memory back first
        del pinned, h_out, dev_in, flush, events
        q = k = v = idx = mask = do = None
        torch.cuda.empty_cache()
        extra = {}
        for index, (name, steps) in enumerate(EXTRA_WORKLOADS):
            extra[name] = child_workload(name, steps, world, index)
        if line is not None:
            line['workloads'] = extra
    if line is not None:
        print(json.dumps(line))


def kernel_rows(breakdown, w, mask, f_fwd, f_bwd, tensor_peak):
    """The kernels of one step with their own device time: algorithmic work, achieved rate and fraction of the peak
    that bounds them (tensor cores for the two attention kernels, HBM for the rest)."""
    if not breakdown:
        return None
    hbm = hbm_peak()
    b, n, hq, hkv, d = w['batch'], w['seq'], w['q_heads'], w['kv_heads'], w['dim_head']
    slots = int(mask.sum().item()) * (hq // hkv) + b * hq * n          # (row, slot) pairs incl. the own block
    part = slots * (d * 2)                                            # bf16 partial rows
    rows_bytes = b * hq * n * d * 2
    work = {   # kernel name prefix -> (bound, algorithmic FLOPs or bytes per launch)
        'sel_fwd_kernel': ('tensor', f_fwd), 'sel_bwd_ws_kernel': ('tensor', f_bwd), 'sel_bwd_kernel': ('tensor', f_bwd),
        'sel_merge_kernel': ('hbm', part + slots * 8 + rows_bytes), 'sel_dq_merge_kernel': ('hbm', part + rows_bytes),
        'sel_delta_kernel': ('hbm', 2 * rows_bytes + b * hq * n * 4),
        'attend_fwd_kernel': ('tensor', f_fwd), 'attend_bwd_kernel': ('tensor', f_bwd),
    }
    out = []
    for name, (per_step, us) in sorted(breakdown.items(), key=lambda kv: -kv[1][0] * kv[1][1]):
        short = name.split('(')[0].split('::')[-1].replace('void ', '')
        row = {'name': short[:60], 'launches_per_step': per_step, 'ms': us / 1e3, 'share_of_step': None}
        key = next((k_ for k_ in work if short.startswith(k_)), None)
        if key is not None:
            bound, amount = work[key]
            rate = amount / (us / 1e6)
            row.update(bound=bound, work=amount, achieved=rate / (1e12 if bound == 'tensor' else 1e9),
                       unit='TFLOP/s' if bound == 'tensor' else 'GB/s',
                       frac=rate / ((tensor_peak * 1e12) if bound == 'tensor' else (hbm * 1e9)),
                       dram_bytes=NCU_DRAM_BYTES.get(key))
        out.append(row)
    total = sum(r['ms'] * r['launches_per_step'] for r in out)
    for r in out:
        r['share_of_step'] = r['ms'] * r['launches_per_step'] / total if total else None
    return out[:16]


def hbm_peak():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    return json.load(open(path))['hbm_gbs'] if os.path.exists(path) else 6650.0


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
        holder['o'], holder['imp'] = nsa.compressed_attend(qd, ckd, cvd, 1, st, True, pool=blk // st)
    add('compressed_fwd', timed(cmp_fwd), 4 * d * pairs, 'tensor')
    add('compressed_bwd', timed(lambda: torch.autograd.grad(holder['o'], (qd, ckd, cvd), do, retain_graph=True)),
        10 * d * pairs, 'tensor')
    imp = holder['imp']
    # block selection
    def select():
        holder['vals'], holder['idx'] = nsa.select_blocks(imp, blk, st, nsel, dtype=torch.bfloat16)
    ms = timed(select)
    add('select', ms, imp.numel() * imp.element_size() + b * hkv * n * nsel * 12, 'hbm')
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


def _dist_setup():
    import torch.distributed as dist
    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)
    return dist, rank, world, local, dev


def _timed_steps(step, steps, warmup, flush, dist, world, rank, local):
    """`warmup` untimed steps, then `steps` steps timed one by one with CUDA events (L2 flushed outside the events);
    returns (total ms as the max over ranks, clocks of rank 0, kernels of this library launched in the timed region)."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    evs = []
    launches_before = launch_count()
    for i in range(steps):
        flush.fill_(i & 0xff)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        evs.append((e0, e1))
    torch.cuda.synchronize()
    launches = launch_count() - launches_before
    clocks = sampler.stop() if rank == 0 else None
    from native_sparse_attention_pytorch_b200 import ops
    ops.check_device_status()     # a kernel that gave up on a bounded wait makes the whole measurement void
    t = torch.tensor([sum(a.elapsed_time(b) for a, b in evs)], dtype=torch.float64, device=flush.device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item(), clocks, launches


def hot_path_flops(n, d, g, units, stride, ncb, num_mem, block, window, visible_slots):
    """Forward FLOPs (4*d per attended pair) of the three branches for `units` (batch, KV head) pairs of `g` heads;
    `visible_slots` = number of selected blocks summed over all (batch, KV head, query)."""
    i = torch.arange(n, dtype=torch.float64)
    cmp_pairs = (torch.clamp((i // stride), max=ncb) + num_mem).sum().item() * units * g
    swa_pairs = (torch.clamp(i, max=window) + 1).sum().item() * units * g
    sel_pairs = (visible_slots * block + (i % block + 1).sum().item() * units) * g
    return {k: 4 * d * v for k, v in (('compressed', cmp_pairs), ('selected', sel_pairs), ('sliding', swa_pairs))}


def run_layer(args, w):
    """Full SparseAttention layer forward+backward in bf16 (the baseline's third configuration): every rank runs the
    layer on its own batch (weak scaling)."""
    import native_sparse_attention_pytorch_b200 as nsa
    kw = {k: v for k, v in w.items() if k not in ('batch', 'seq')}
    if args.impl == 'reference':
        run_layer_reference(args, w, kw)
        return None
    dist, rank, world, local, dev = _dist_setup()
    warmup = max(args.warmup, 3)
    torch.manual_seed(0)
    layer = nsa.SparseAttention(causal=True, use_triton_kernel=True, **kw).to(dev).bfloat16()
    gen = torch.Generator('cpu').manual_seed(100 + rank)
    x_host = torch.randn(w['batch'], w['seq'], w['dim'], generator=gen).bfloat16().pin_memory()
    g_host = torch.randn(w['batch'], w['seq'], w['dim'], generator=gen).bfloat16().pin_memory()
    x, up = x_host.to(dev).requires_grad_(), g_host.to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def eager_step():
        layer.zero_grad(set_to_none=True)
        x.grad = None
        out = layer(x)
        out.backward(up)
        return out

    # The step is recorded once as a CUDA graph and replayed (--no-graph: issued kernel by kernel); all of it on a
    # stream of its own, since a graph cannot be recorded around gradients first accumulated on the default stream.
    stream = torch.cuda.Stream(device=dev)
    graphed = {'graph': None, 'out': None, 'launches': 0, 'how': 'issued kernel by kernel'}

    def step():
        if graphed['graph'] is None:
            return eager_step()
        graphed['graph'].replay()
        return graphed['out']

    with torch.cuda.stream(stream):
        with torch.no_grad():
            _, mid = layer(x, return_intermediates=True)
        n, d, hkv = w['seq'], w['dim_head'], w['kv_heads']
        st = w['compress_block_sliding_stride']
        flops = hot_path_flops(n, d, w['heads'] // hkv, w['batch'] * hkv, st, n // st, 1, w['selection_block_size'],
                               w['sliding_window_size'], mid['fmask'].sum().item())
        del mid
        for _ in range(2):
            eager_step()
        torch.cuda.synchronize()
        if not args.no_graph:
            try:
                graph = torch.cuda.CUDAGraph()
                before = launch_count()
                with torch.cuda.graph(graph, stream=stream):
                    g_out = eager_step()
                graphed.update(graph=graph, out=g_out, launches=launch_count() - before,
                               how='replayed as one CUDA graph (forward + backward)')
            except Exception as exc:
                graphed['how'] = f'issued kernel by kernel (graph capture failed: {type(exc).__name__})'
                torch.cuda.synchronize()
        total_ms, clocks, launches = _timed_steps(step, args.steps, warmup, flush, dist, world, rank, local)
        if graphed['graph'] is not None:
            launches = graphed['launches'] * args.steps     # a replay launches what the capture recorded

        # end to end: the input arrives from pinned host memory, the output and the input gradient go back
        h_out, h_dx = torch.empty_like(x_host).pin_memory(), torch.empty_like(x_host).pin_memory()
        def e2e_step():
            x.data.copy_(x_host, non_blocking=True)
            up.copy_(g_host, non_blocking=True)
            out = step()
            h_out.copy_(out.detach(), non_blocking=True)
            h_dx.copy_(x.grad, non_blocking=True)
        e2e_step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2e_steps = max(3, min(args.steps, 10))
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e1.record()
        torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank != 0:
        return None
    ms = total_ms / args.steps
    tokens = w['batch'] * w['seq'] * world
    burst, sustained, src = peaks()
    f_step = 3.5 * sum(flops.values())
    line = {
        'metric': 'nsa_layer_fwd_bwd_tokens_per_s', 'value': tokens / (ms / 1e3), 'unit': 'tokens/s', 'n_gpus': world,
        'steps': args.steps, 'warmup': warmup, 'ms_per_step': ms, 'higher_is_better': True, 'scaling': 'weak',
        'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic',
        'config': {'workload': args.workload, **w, 'l2': 'flushed between timed steps',
                   'per_rank': 'each rank runs the layer on its own seeded batch', 'step': graphed['how']},
        'roofline': {'bound': 'tensor', 'kernel': 'whole layer step; FLOPs of the three attention branches only',
                     'achieved': f_step / (ms / 1e3) / 1e12, 'peak': burst, 'unit': 'TFLOP/s',
                     'frac': f_step / (ms / 1e3) / 1e12 / burst, 'peak_source': src, 'peak_sustained': sustained,
                     'flops_per_step': f_step, 'flops_fwd_by_branch': flops, 'traffic': None},
        'e2e': {'value': tokens / (t.item() / e2e_steps / 1e3), 'unit': 'tokens/s',
                'h2d_bytes_per_step': 2 * x_host.numel() * 2, 'd2h_bytes_per_step': 2 * x_host.numel() * 2,
                'steps': e2e_steps},
        'gpu_launches': None, 'clocks': clocks,
    }
    line['gpu_launches'] = launches
    if not args.no_cpu_baseline and world == 1:
        line['cpu_baseline'] = layer_cpu_sample(kw)
    return line


def layer_cpu_sample(kw, n=1024, budget_s=15.0):
    """The CPU oracle of the layer (a port of upstream's PyTorch path), forward+backward in fp32 at a sequence length
    whose gathered keys fit host memory."""
    from oracle import nsa_oracle as O
    torch.set_num_threads(os.cpu_count())
    torch.manual_seed(0)
    layer = O.OracleSparseAttention(causal=True, **kw)
    x = torch.randn(1, n, kw['dim'], generator=torch.Generator('cpu').manual_seed(1)).requires_grad_()
    layer(x).sum().backward()
    t0, reps = time.perf_counter(), 0
    while True:
        layer.zero_grad()
        layer(x).sum().backward()
        reps += 1
        el = time.perf_counter() - t0
        if el > budget_s or reps >= 20:
            break
    return {'value': reps * n / el, 'unit': 'tokens/s', 'cores': os.cpu_count(), 'kind': 'port',
            'sample': f'batch 1, {n} tokens (upstream\'s gather formulation does not fit host memory at the full length), '
                      f'fp32, {reps} repetitions'}


def run_layer_reference(args, w, kw, metric='nsa_layer_fwd_bwd_tokens_per_s', layers=1):
    if int(os.environ.get('RANK', '0')) != 0:
        return
    base = layer_cpu_sample(kw, budget_s=max(5.0, min(60.0, 3.0 * args.steps)))
    if layers > 1:
        base['value'] /= layers
        base['sample'] = f'one of the {layers} attention layers (value = its tokens/s / {layers}): ' + base['sample']
    print(json.dumps({
        'impl': 'reference', 'metric': metric, 'value': base['value'], 'unit': 'tokens/s',
        'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': 1e3 * 1024 / base['value'],
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': args.workload, **w}, 'cpu_baseline': base,
        'e2e': {'value': base['value'], 'unit': 'tokens/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}}))


def prefill_inputs(w, heads, dev, host=False):
    """Seeded inputs of the KV heads in `heads` (a range) and their query heads; the same values whatever the rank
    that asks.  q, k, v ~ N(0,1) bf16; compressed keys / values from the default compress network (a two-layer MLP
    over each window of `compress_block_size` rows, default init) on the un-rotated keys / values; rotary on q and k
    for the selected and sliding branches; gates = sigmoid(N(0,1))."""
    from native_sparse_attention_pytorch_b200.rotary import RotaryEmbedding
    b, n, d, hkv = w['batch'], w['seq'], w['dim_head'], w['kv_heads']
    g = w['q_heads'] // hkv
    cbs, st = w['compress_block_size'], w['stride']
    ncb = n // st
    torch.manual_seed(0)
    mlp = torch.nn.Sequential(torch.nn.Flatten(-2), torch.nn.Linear(cbs * d, cbs * d), torch.nn.ReLU(),
                              torch.nn.Linear(cbs * d, d)).to(dev).bfloat16()
    rot = RotaryEmbedding(d).to(dev)
    outs = {k: [] for k in ('q', 'qr', 'kr', 'v', 'ck', 'cv', 'gates')}
    with torch.no_grad():
        for h in heads:
            gen = torch.Generator(dev).manual_seed(1000 + h)
            q = torch.randn(b, g, n, d, generator=gen, device=dev).bfloat16()
            k = torch.randn(b, 1, n, d, generator=gen, device=dev).bfloat16()
            v = torch.randn(b, 1, n, d, generator=gen, device=dev).bfloat16()
            gates = torch.sigmoid(torch.randn(b, g, n, 3, generator=gen, device=dev)).bfloat16()
            pad = cbs - st
            def compress(t):
                tp = torch.nn.functional.pad(t, (0, 0, pad, 0))[..., : (ncb - 1) * st + cbs, :]
                win = tp.unfold(-2, cbs, st).transpose(-1, -2)          # [b, 1, ncb, cbs, d]
                c = torch.cat([mlp(win[:, :, a:a + 512]) for a in range(0, ncb, 512)], dim=2)
                return torch.cat((c.new_zeros(b, 1, w['num_mem'], d), c), dim=2)
            qr, kr = rot.rotate_queries_with_cached_keys(q, k)
            for name, t in (('q', q), ('qr', qr), ('kr', kr), ('v', v), ('ck', compress(k)), ('cv', compress(v)),
                            ('gates', gates)):
                outs[name].append(t.cpu().pin_memory() if host else t)
    return {k: torch.cat(v, dim=1) for k, v in outs.items()}


def run_prefill(args, w):
    """Long-context prefill (forward only) of the hot path, KV-head groups split over the ranks, output all-gathered
    (the baseline's fifth configuration).  Total work is fixed: strong scaling."""
    from native_sparse_attention_pytorch_b200 import sharding
    if args.impl == 'reference':
        run_prefill_reference(args, w)
        return None
    dist, rank, world, local, dev = _dist_setup()
    warmup = max(args.warmup, 3)
    h0, h1 = sharding.kv_head_range(w['kv_heads'], world, rank)
    t = prefill_inputs(w, range(h0, h1), dev)
    cfg = dict(num_mem=w['num_mem'], stride=w['stride'], block=w['block'], num_selected=w['nsel'], window=w['window'],
               causal=True, impl=args.kernels, local=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    keep = {}
    # one GPU: the same code path with this GPU's output tensor as the only destination (no collective, no peers)
    fused = args.gather in ('auto', 'fused', 'multimem')
    peer = None
    if fused and world > 1:
        peer = sharding.PeerOutput(w['batch'], w['seq'], w['q_heads'] * w['dim_head'], torch.bfloat16, dev,
                                   multicast=args.gather in ('auto', 'multimem'))
    elif fused:
        peer = sharding.LocalOutput(w['batch'], w['seq'], w['q_heads'] * w['dim_head'], torch.bfloat16, dev)
    multimem = peer is not None and peer.multicast_ptr is not None

    # how the fused gather runs: through the multicast address or with per-peer stores; on a side stream or not; the
    # query heads of a KV head in one piece or several (sharding.sharded_attend_core)
    mode = {'multicast': multimem, 'overlap': bool(args.overlap), 'splits': args.head_splits,
            'fuse': bool(args.fuse_merge)}
    mc_ptr = peer.multicast_ptr if peer is not None else None

    def step():
        if peer is not None:
            peer.multicast_ptr = mc_ptr if mode['multicast'] else None
        keep['out'] = sharding.sharded_attend_core(t['q'], t['qr'], t['kr'], t['v'], t['ck'], t['cv'], t['gates'],
                                                   peer_output=peer, overlap=mode['overlap'] and fused,
                                                   head_splits=mode['splits'] if fused else 1,
                                                   fuse_merge=mode['fuse'] and fused, **cfg)

    def quick(n=3):   # device time of n steps, the slowest rank's
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            step()
        b_.record()
        torch.cuda.synchronize()
        tt = torch.tensor([a.elapsed_time(b_) / n], device=dev)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return tt.item()

    gather_check = None
    if fused:
        # Untimed: the plain form (per-peer stores, one piece, same stream) gives the bytes every other form must
        # reproduce on every rank; a form that differs is never timed.  With --gather auto the forms are then tried
        # for three steps each and the fastest is kept.
        g = w['q_heads'] // w['kv_heads']
        forms = [dict(multicast=False, overlap=False, splits=1, fuse=False)]
        if args.gather == 'auto':
            # runs of query heads per KV head: one; two halves; a half and two quarters; ... (the last run's transfer
            # is the one that no compute hides, so the runs get shorter towards the end)
            run_sets = [1] + [r for r in ((g // 2, g // 2), (g // 2, g // 4, g // 4), (g // 2, g // 4, g // 8, g // 8))
                              if min(r) >= 1 and sum(r) == g]
            for mcast in ((False, True) if multimem else (False,)):
                for ov, sp, fu in [(False, 1, False)] + [(True, r, False) for r in (run_sets if world > 1 else [1])] + \
                                  [(False, 1, True)]:
                    f = dict(multicast=mcast, overlap=ov, splits=sp, fuse=fu)
                    if f not in forms and not (mcast and sp != 1):
                        forms.append(f)
        elif mode != forms[0]:
            forms.append(dict(mode))
        mode.update(forms[0])
        step()
        plain = keep['out'].clone()
        notes, best = [], (None, None)
        for f in forms:
            mode.update(f)
            step()
            same = torch.tensor([int(torch.equal(plain, keep['out']))], device=dev)
            if world > 1:
                dist.all_reduce(same, op=dist.ReduceOp.MIN)
            name = ('multicast' if f['multicast'] else 'per-peer') + (', side stream' if f['overlap'] else '') + \
                   (", stored by the selected branch's merge" if f['fuse'] else '') + \
                   (f', head runs {f["splits"]}' if f['splits'] != 1 else '')
            if same.item() != 1:
                notes.append(f'{name}: DIFFERS from the plain form, not used')
                continue
            ms_f = quick() if len(forms) > 1 else 0.0
            notes.append(f'{name}: {ms_f:.3f} ms' if len(forms) > 1 else f'{name}: identical on every rank')
            if args.gather == 'auto':
                if best[0] is None or ms_f < best[0]:
                    best = (ms_f, dict(f))
            else:
                best = (ms_f, dict(f))      # the requested form, if it is correct; else the plain one stays
        mode.update(best[1] if best[1] is not None else forms[0])
        multimem = mode['multicast']
        gather_check = 'every form identical to the plain one unless noted; untimed trial per step: ' + '; '.join(notes)
        del plain
    total_ms, clocks, launches = _timed_steps(step, args.steps, warmup, flush, dist, world, rank, local)

    # end to end: this rank's inputs arrive from pinned host memory every step, rank 0 reads the gathered output back
    host = {k: v.cpu().pin_memory() for k, v in t.items()}
    h_out = torch.empty_like(keep['out'], device='cpu').pin_memory() if rank == 0 else None
    def e2e_step():
        for k in t:
            t[k].copy_(host[k], non_blocking=True)
        step()
        if rank == 0:
            h_out.copy_(keep['out'], non_blocking=True)
    e2e_step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(2, min(args.steps, 5))
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    te = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    # selected blocks actually visible, for the FLOP count (one more untimed pass of the selection on this rank)
    from native_sparse_attention_pytorch_b200 import ops
    vis = 0
    g = w['q_heads'] // w['kv_heads']
    with torch.no_grad():
        for a in range(h1 - h0):
            _, imp = ops.compressed_attend(t['q'][:, a * g:(a + 1) * g], t['ck'][:, a:a + 1], t['cv'][:, a:a + 1],
                                           w['num_mem'], w['stride'], True, sel_heads=1, want_importance=True,
                                           pool=w['block'] // w['stride'])
            vals, _ = ops.select_blocks(imp, w['block'], w['stride'], w['nsel'], dtype=torch.bfloat16)
            vis += int((vals > 1e-10).sum().item())
            del imp
    tv = torch.tensor([float(vis)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
        dist.all_reduce(tv)
    if rank != 0:
        return None
    ms = total_ms / args.steps
    n = w['seq']
    tokens = w['batch'] * n
    flops = hot_path_flops(n, w['dim_head'], g, w['batch'] * w['kv_heads'], w['stride'], n // w['stride'], w['num_mem'],
                           w['block'], w['window'], tv.item())
    f_step = sum(flops.values())
    burst, sustained, src = peaks()
    in_bytes = sum(v.numel() * v.element_size() for v in host.values())
    line = {
        'metric': 'nsa_prefill_tokens_per_s', 'value': tokens / (ms / 1e3), 'unit': 'tokens/s', 'n_gpus': world,
        'steps': args.steps, 'warmup': warmup, 'ms_per_step': ms, 'higher_is_better': True, 'scaling': 'strong',
        'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic',
        'config': {'workload': args.workload, **w, 'kernels': args.kernels, 'l2': 'flushed between timed steps',
                   'sharding': f'{w["kv_heads"] // world} KV-head group(s) per rank, output '
                               + ('gathered by the combine kernel storing once through the NVLink multicast address '
                                  '(multimem.st)' if multimem else
                                  'gathered by the combine kernel storing into every rank' if fused and world > 1
                                  else 'written by the combine kernel of each pass (one GPU holds all heads)'
                                  if world == 1 else 'gathered by an NCCL all-gather')
                               + ((', on a side stream' if mode['overlap'] else '') +
                                  (", from the selected branch's merge kernel" if mode['fuse'] else '') +
                                  (f', query heads in runs {mode["splits"]}' if mode['splits'] != 1 else '') if fused else ''),
                   'gather_check': gather_check},
        'roofline': {'bound': 'tensor', 'kernel': 'whole forward step of all branches (per GPU)',
                     'achieved': f_step / world / (ms / 1e3) / 1e12, 'peak': burst, 'unit': 'TFLOP/s',
                     'frac': f_step / world / (ms / 1e3) / 1e12 / burst, 'peak_source': src,
                     'peak_sustained': sustained, 'flops_per_step': f_step, 'flops_fwd_by_branch': flops,
                     'traffic': None},
        'e2e': {'value': tokens / (te.item() / e2e_steps / 1e3), 'unit': 'tokens/s',
                'h2d_bytes_per_step': in_bytes * world, 'd2h_bytes_per_step': keep['out'].numel() * 2,
                'steps': e2e_steps},
        'gpu_launches': launches, 'clocks': clocks,
    }
    if args.rows and world == 1:
        line['rows'] = prefill_rows(w, t, flush)
    if not args.no_cpu_baseline and world == 1:
        line['cpu_baseline'] = prefill_cpu_sample(w)
    return line


def prefill_rows(w, t, flush, iters=5):
    """The five operators of ONE KV head of the prefill workload, timed one by one (ms, CUDA events, L2 flushed)."""
    from native_sparse_attention_pytorch_b200 import ops
    g = w['q_heads'] // w['kv_heads']
    q, qr, kr, v, ck, cv, gates = (t[k][:, :(g if k in ('q', 'qr', 'gates') else 1)]
                                   for k in ('q', 'qr', 'kr', 'v', 'ck', 'cv', 'gates'))
    h, rows = {}, {}

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
        return sum(a.elapsed_time(b) for a, b in evs) / iters

    def cmp():
        h['o'], h['imp'] = ops.compressed_attend(q, ck, cv, w['num_mem'], w['stride'], True, sel_heads=1,
                                                 want_importance=True, pool=w['block'] // w['stride'])
    rows['compressed_fwd'] = timed(cmp)
    def sel():
        h['vals'], h['idx'] = ops.select_blocks(h['imp'], w['block'], w['stride'], w['nsel'], dtype=torch.bfloat16)
    rows['select'] = timed(sel)
    mask = h['vals'] > 1e-10
    def selected():
        h['os'] = ops.native_sparse_attend(qr, kr, v, w['block'], h['idx'], mask)
    rows['selected_fwd'] = timed(selected)
    def swa():
        h['ow'] = ops.sliding_window_attend(qr, kr, v, w['window'], True)
    rows['sliding_fwd'] = timed(swa)
    rows['combine_fwd'] = timed(lambda: ops.gated_combine(h['o'], h['os'], h['ow'], gates))
    return {k: {'ms': ms} for k, ms in rows.items()}


def oracle_core_fns(num_mem):
    """The CPU oracle's functions behind the argument lists of the CUDA operators (for the CPU baseline only)."""
    from oracle import nsa_oracle as O

    def compressed(q, ck, cv, nm, stride, causal, sel_heads=None, want_importance=True):
        out, csim = O.compressed_attend(q, ck[:, :, nm:], cv[:, :, nm:], ck[0, :, :nm], cv[0, :, :nm], stride, causal)
        return out, (csim, ck.shape[1])

    def select(importance, block, stride, nsel, dtype=None):
        csim, hkv = importance
        return O.select_blocks(O.importance_scores(csim, num_mem, hkv, stride, block), nsel)

    def selected(q, k, v, block, idx, mask, include_block_causal=True):
        return O.selected_attend(q, k, v, block, idx, mask, include_block_causal)

    return dict(compressed=compressed, select=select, selected=selected, sliding=O.sliding_attend, combine=O.combine)


def prefill_cpu_sample(w, n=2048, budget_s=15.0):
    from native_sparse_attention_pytorch_b200 import sharding
    torch.set_num_threads(os.cpu_count())
    ws = dict(w, seq=n)
    t = {k: v.float() for k, v in prefill_inputs(ws, range(1), torch.device('cpu')).items()}
    cfg = dict(num_mem=w['num_mem'], stride=w['stride'], block=w['block'], num_selected=w['nsel'], window=w['window'],
               causal=True, attend_fns=oracle_core_fns(w['num_mem']))
    run = lambda: sharding.attend_core(t['q'], t['qr'], t['kr'], t['v'], t['ck'], t['cv'], t['gates'], **cfg)
    with torch.no_grad():
        run()
        t0, reps = time.perf_counter(), 0
        while True:
            run()
            reps += 1
            el = time.perf_counter() - t0
            if el > budget_s or reps >= 20:
                break
    return {'value': reps * n / w['kv_heads'] / el, 'unit': 'tokens/s', 'cores': os.cpu_count(), 'kind': 'port',
            'sample': f'{n} tokens, 1 of {w["kv_heads"]} KV-head groups (a token counts 1/{w["kv_heads"]} per group), '
                      f'fp32, forward only, {reps} repetitions'}


def run_prefill_reference(args, w):
    if int(os.environ.get('RANK', '0')) != 0:
        return
    base = prefill_cpu_sample(w, budget_s=max(5.0, min(60.0, 3.0 * args.steps)))
    print(json.dumps({
        'impl': 'reference', 'metric': 'nsa_prefill_tokens_per_s', 'value': base['value'], 'unit': 'tokens/s',
        'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': None,
        'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': args.workload, **w}, 'cpu_baseline': base,
        'e2e': {'value': base['value'], 'unit': 'tokens/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}}))


def build_lm(w, dev, dtype=torch.bfloat16, attn_cls=None, norm_cls=None):
    """The language model of upstream's training example around the layer (transformer.py:142-330): token embedding,
    `depth` pre-norm residual blocks of [SparseAttention, RMSNorm -> Linear x4 -> GELU -> Linear], final RMSNorm,
    logits; next-token cross-entropy on ids[:, 1:].  Module names are upstream's (token_emb, layers, norm,
    to_logits), so a state_dict moves across.  It is a harness around the layer, not part of the library; the tests
    check it against stored results of upstream's model.  `attn_cls` / `norm_cls` default to the library's layer and
    RMS norm (the CPU tests pass the oracle's layer and torch's norm)."""
    from torch import nn
    kw = {k: w[k] for k in ('dim', 'dim_head', 'heads', 'kv_heads', 'sliding_window_size', 'compress_block_size',
                            'compress_block_sliding_stride', 'selection_block_size', 'num_selected_blocks')}
    if attn_cls is None:
        import native_sparse_attention_pytorch_b200 as nsa
        from native_sparse_attention_pytorch_b200.norm import RMSNorm
        attn_cls = lambda **k: nsa.SparseAttention(use_triton_kernel=True, **k)
        norm_cls = RMSNorm
    norm_cls = norm_cls or nn.RMSNorm

    class Lm(nn.Module):
        def __init__(self):
            super().__init__()
            dim = w['dim']
            self.token_emb = nn.Embedding(w['vocab'], dim)
            self.layers = nn.ModuleList([nn.ModuleList([
                attn_cls(causal=True, **kw),
                nn.Sequential(norm_cls(dim), nn.Linear(dim, 4 * dim), nn.GELU(), nn.Linear(4 * dim, dim))])
                for _ in range(w['depth'])])
            self.norm = norm_cls(dim)
            self.to_logits = nn.Linear(dim, w['vocab'], bias=False)

        def logits(self, ids):
            x = self.token_emb(ids)
            for attn, ff in self.layers:
                x = attn(x) + x
                x = ff(x) + x
            return self.to_logits(self.norm(x))

        def forward(self, ids):
            ids, labels = ids[:, :-1], ids[:, 1:]
            return torch.nn.functional.cross_entropy(self.logits(ids).flatten(0, 1).float(), labels.flatten())

    torch.manual_seed(0)
    return Lm().to(dev).to(dtype), kw


def run_lm(args, w):
    """Training step (forward, backward, gradient all-reduce over the ranks) of the byte-level language model: the
    batch is split over the ranks (strong scaling), the gradients are summed with one NCCL all-reduce per step."""
    if args.impl == 'reference':
        kw = {k: w[k] for k in ('dim', 'dim_head', 'heads', 'kv_heads', 'sliding_window_size', 'compress_block_size',
                                'compress_block_sliding_stride', 'selection_block_size', 'num_selected_blocks')}
        run_layer_reference(args, w, kw, metric='nsa_lm_train_step_tokens_per_s', layers=w['depth'])
        return None
    dist, rank, world, local, dev = _dist_setup()
    warmup = max(args.warmup, 3)
    if w['batch'] % world:
        raise SystemExit(f'batch {w["batch"]} does not split over {world} ranks')
    per_rank = w['batch'] // world
    model, kw = build_lm(w, dev)
    gen = torch.Generator('cpu').manual_seed(0)
    ids_host = torch.randint(0, w['vocab'], (w['batch'], w['seq'] + 1), generator=gen)[rank * per_rank:(rank + 1) * per_rank]
    ids_host = ids_host.pin_memory()
    ids = ids_host.to(dev)
    params = [p for p in model.parameters()]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    keep = {}

    reducer = None
    if world > 1:
        # data-parallel gradient sum, one bucket per block in the order the backward reaches them: a block's
        # all-reduce travels while the blocks below it are still in their backward
        from native_sparse_attention_pytorch_b200.sharding import BucketedGradientSum
        in_blocks = {id(p) for blk in model.layers for p in blk.parameters()}
        rest = [p for p in params if id(p) not in in_blocks]
        reducer = BucketedGradientSum([rest] + [list(blk.parameters()) for blk in reversed(model.layers)])

    def eager_step():
        model.zero_grad(set_to_none=True)
        if reducer is not None:
            reducer.start()
        loss = model(ids)
        loss.backward()
        if reducer is not None:
            reducer.finish()
        keep['loss'] = loss

    # Forward + backward of the step as one CUDA graph: with the batch split over the ranks the kernels get short
    # (774 launches in 36 ms at four sequences per rank, of which the host needs 31 ms to issue them), so the step
    # is replayed instead of issued; the gradient sum then follows the replay as one flat all-reduce.  Everything
    # runs on a stream of its own: a graph cannot be recorded around a model whose gradients were first accumulated
    # on the default stream.
    stream = torch.cuda.Stream(device=dev)
    graphed = {'graph': None, 'loss': None, 'launches': 0, 'how': 'issued kernel by kernel'}

    def step():
        if graphed['graph'] is None:
            return eager_step()
        graphed['graph'].replay()
        if world > 1:
            grads = [p.grad for p in params if p.grad is not None]
            flat = torch._utils._flatten_dense_tensors(grads)
            dist.all_reduce(flat)
            for g_, f in zip(grads, torch._utils._unflatten_dense_tensors(flat, grads)):
                g_.copy_(f)
        keep['loss'] = graphed['loss']

    with torch.cuda.stream(stream):
        for _ in range(2):
            eager_step()          # builds the per-shape indices and fills the allocator's pools
        torch.cuda.synchronize()
        if not args.no_graph:
            try:
                graph = torch.cuda.CUDAGraph()
                before = launch_count()
                with torch.cuda.graph(graph, stream=stream):
                    model.zero_grad(set_to_none=True)
                    g_loss = model(ids)
                    g_loss.backward()
                graphed.update(graph=graph, loss=g_loss, launches=launch_count() - before,
                               how='replayed as one CUDA graph (forward + backward); gradient sum after the replay')
            except Exception as exc:   # the step still runs, kernel by kernel
                graphed['how'] = f'issued kernel by kernel (graph capture failed: {type(exc).__name__})'
                torch.cuda.synchronize()
        total_ms, clocks, launches = _timed_steps(step, args.steps, warmup, flush, dist, world, rank, local)
        if graphed['graph'] is not None:
            launches = graphed['launches'] * args.steps     # a replay launches what the capture recorded
        h_loss = torch.empty(1, dtype=torch.float32).pin_memory()
        def e2e_step():
            ids.copy_(ids_host, non_blocking=True)
            step()
            h_loss.copy_(keep['loss'].detach().float().view(1), non_blocking=True)
        e2e_step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2e_steps = max(3, min(args.steps, 10))
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e1.record()
        torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank != 0:
        return None
    ms = total_ms / args.steps
    tokens = w['batch'] * w['seq']
    n, st = w['seq'], w['compress_block_sliding_stride']
    g = w['heads'] // w['kv_heads']
    units = w['batch'] * w['kv_heads']
    # selected blocks: every query past its first blocks sees min(nsel, own block index) of them
    i = torch.arange(n)
    visible = torch.clamp(i // w['selection_block_size'], max=w['num_selected_blocks']).sum().item() * units
    flops = hot_path_flops(n, w['dim_head'], g, units, st, n // st, 1, w['selection_block_size'],
                           w['sliding_window_size'], visible)
    f_step = 3.5 * sum(flops.values()) * w['depth']
    burst, sustained, src = peaks()
    n_params = sum(p.numel() for p in params)
    line = {
        'metric': 'nsa_lm_train_step_tokens_per_s', 'value': tokens / (ms / 1e3), 'unit': 'tokens/s', 'n_gpus': world,
        'steps': args.steps, 'warmup': warmup, 'ms_per_step': ms, 'higher_is_better': True, 'scaling': 'strong',
        'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic',
        'config': {'workload': args.workload, **w, 'l2': 'flushed between timed steps', 'parameters': n_params,
                   'parallelism': f'data parallel, {per_rank} sequences per rank, {n_params * 2 / 1e6:.0f} MB of bf16 '
                                  + ('gradients summed by one NCCL all-reduce after the replay'
                                     if graphed['graph'] is not None else
                                     'gradients summed by one NCCL all-reduce per block, launched as the backward '
                                     'leaves the block'),
                   'step': graphed['how']},
        'roofline': {'bound': 'tensor', 'kernel': 'whole training step; FLOPs of the three attention branches only',
                     'achieved': f_step / world / (ms / 1e3) / 1e12, 'peak': burst, 'unit': 'TFLOP/s',
                     'frac': f_step / world / (ms / 1e3) / 1e12 / burst, 'peak_source': src,
                     'peak_sustained': sustained, 'flops_per_step': f_step, 'traffic': None},
        'e2e': {'value': tokens / (t.item() / e2e_steps / 1e3), 'unit': 'tokens/s',
                'h2d_bytes_per_step': ids_host.numel() * 8 * world, 'd2h_bytes_per_step': 4, 'steps': e2e_steps},
        'gpu_launches': launches, 'clocks': clocks,
        'loss': float(keep['loss'].detach()),
    }
    if not args.no_cpu_baseline and world == 1:
        base = layer_cpu_sample(kw)
        base['value'] /= w['depth']
        base['sample'] = f'one of the {w["depth"]} attention layers (value = its tokens/s / {w["depth"]}; feed-forward not timed): ' + base['sample']
        line['cpu_baseline'] = base
    return line


if __name__ == '__main__':
    main()
