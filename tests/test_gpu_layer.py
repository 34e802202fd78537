"""The whole SparseAttention layer on the GPU against the vectors stored from
the unmodified upstream layer (fp32) and against the fp32 oracle (bf16)."""
import pytest
import torch

import recipe
from oracle import nsa_oracle as O
from util import agreeing_queries, assert_close_bf16, assert_close_f32, load_golden, observe, same_selection

from native_sparse_attention_pytorch_b200 import SparseAttention

pytestmark = pytest.mark.gpu
DEV = 'cuda'
LAYER = list(recipe.LAYER_CASES)


def build(name, dtype=torch.float32):
    c = recipe.LAYER_CASES[name]
    attn = SparseAttention(**c['kw'], use_triton_kernel=True)
    recipe.fill_weights(attn, seed=7, rich=c['rich'])
    return attn.to(DEV).to(dtype)


@pytest.mark.parametrize('name', LAYER)
def test_layer_matches_upstream_vectors(name):
    gold = load_golden('layer_' + name)
    attn = build(name)
    x = recipe.layer_input(name).to(DEV).requires_grad_()
    out, mid = attn(x, return_intermediates=True)
    mid['o_sel'].retain_grad()
    mid['gates'].retain_grad()
    (out * recipe.randn(out.shape, 13).to(DEV)).sum().backward()

    if 'idx' in gold:
        assert same_selection(mid['idx'], mid['fmask'], gold['idx'], gold['vals'] > 1e-10)
        assert_close_f32(mid['vals'], gold['vals'], 'selection values', tol=1e-5)
    else:
        assert mid['idx'] is None
    assert_close_f32(mid['o_sel'], gold['o_sel'], 'selected branch')
    for key in ('o_cmp', 'o_swa', 'qr', 'kr'):
        if key in gold:
            assert_close_f32(mid[key], gold[key], key)
    assert_close_f32(out, gold['out'], 'out')
    assert_close_f32(x.grad, gold['x_grad'], 'd input')
    assert_close_f32(mid['gates'].grad, gold['gates_grad'], 'd gates')
    if 'o_sel_grad' in gold:
        assert_close_f32(mid['o_sel'].grad, gold['o_sel_grad'], 'd selected branch')
    for pname, p in attn.named_parameters():
        g = gold.get('pgrad.' + pname)
        if g is None:
            assert p.grad is None or p.grad.abs().sum().item() == 0, pname
            continue
        got = torch.tensor([p.grad.abs().sum().item(), p.grad.pow(2).sum().item()], dtype=torch.float64)
        assert torch.allclose(got, g, rtol=1e-3, atol=1e-6), (pname, got, g)


@pytest.mark.parametrize('name', ['causal_gqa', 'causal_gqa_win', 'noncausal_gqa', 'causal_nsel0'])
def test_layer_bf16_boundary_tensors(name):
    """bf16 run against the fp32 oracle fed the same bf16-rounded weights and
    input.  The selection is compared first; the branch outputs are compared
    on the queries whose selection agrees (bf16 scores tie often, and a tie
    broken differently is a different but equally valid selection)."""
    c = recipe.LAYER_CASES[name]
    attn = build(name, torch.bfloat16)
    ref = O.OracleSparseAttention(**c['kw'])
    ref.load_state_dict({k: v.float().cpu() for k, v in attn.state_dict().items()})
    x = recipe.layer_input(name).to(torch.bfloat16)
    out, mid = attn(x.to(DEV), return_intermediates=True)
    rout, rmid = ref(x.float(), return_intermediates=True)
    assert_close_bf16(mid['o_cmp'], rmid['o_cmp'], 'compressed branch')
    assert_close_bf16(mid['o_swa'], rmid['o_swa'], 'sliding branch')
    if rmid['idx'] is None:
        assert mid['idx'] is None
        assert_close_bf16(mid['o_sel'], rmid['o_sel'], 'selected branch')
        assert_close_bf16(out, rout, 'out', tol=4e-2)
        return
    # the selection first: identical masks, and the share of queries with identical block sets
    assert torch.equal(mid['fmask'].sum(-1).cpu(), rmid['fmask'].sum(-1)), 'number of visible blocks per query'
    same = agreeing_queries(mid['idx'], mid['fmask'], rmid['idx'], rmid['fmask'])          # [B, Hkv, N]
    observe('selection agreement', share=same.float().mean().item())
    assert same.float().mean().item() > 0.5
    # then the selected branch and the output on the queries whose selection agrees
    heads, kv_heads = c['kw']['heads'], c['kw'].get('kv_heads') or c['kw']['heads']
    per_head = same.repeat_interleave(heads // kv_heads, dim=1)                          # [B, Hq, N]
    assert_close_bf16(mid['o_sel'].cpu()[per_head], rmid['o_sel'][per_head], 'selected branch')
    whole = same.all(dim=1)                                                              # every head group of the token
    assert_close_bf16(out.cpu()[whole], rout[whole], 'out', tol=4e-2)


@pytest.mark.parametrize('seq_len', (2, 8, 16))
@pytest.mark.parametrize('num_selected_blocks', (0, 2))
@pytest.mark.parametrize('stride', (2, 4))
@pytest.mark.parametrize('selection_block_size', (8, 16, 20))
def test_decoding_with_cache_equals_parallel_forward(seq_len, num_selected_blocks, stride, selection_block_size):
    """Upstream's own check of its decode path (tests/test_sparse_attn.py:50-86), on the same grid: feeding the tokens
    one by one with the cache gives the parallel forward's output (atol 1e-5 upstream; 2e-5 here, the parallel side
    sums in another order)."""
    torch.manual_seed(0)
    attn = SparseAttention(dim=512, dim_head=64, heads=8, causal=True, sliding_window_size=2, compress_block_size=5,
                           selection_block_size=selection_block_size, num_selected_blocks=num_selected_blocks,
                           compress_block_sliding_stride=stride, use_triton_kernel=True)
    recipe.fill_weights(attn, seed=3, rich=False)      # memory slots zero, as upstream initialises them (see below)
    attn = attn.to(DEV)
    tokens = recipe.randn((2, seq_len, 512), 5).to(DEV)
    with torch.no_grad():
        parallel = attn(tokens)
        cache, steps = None, []
        for i in range(seq_len):
            one, cache = attn(tokens[:, i:i + 1], cache=cache, return_cache=True)
            steps.append(one)
    sequential = torch.cat(steps, dim=1)
    assert (parallel - sequential).abs().max().item() <= 2e-5


def test_decoding_with_grouped_heads_and_memory_slots():
    # Upstream's decode step attends the memory slots only once a compressed block exists (NSA:402-406), its parallel
    # forward always: with non-zero memory slots the two differ for the first `stride` tokens.  This package keeps
    # both behaviours, so the comparison starts where a compressed block exists.
    torch.manual_seed(0)
    attn = SparseAttention(dim=256, dim_head=64, heads=8, kv_heads=2, causal=True, sliding_window_size=5,
                           compress_block_size=8, compress_block_sliding_stride=4, selection_block_size=8,
                           num_selected_blocks=2, num_compressed_mem_kv=2, use_triton_kernel=True)
    recipe.fill_weights(attn, seed=4, rich=True)
    attn = attn.to(DEV)
    tokens = recipe.randn((2, 37, 256), 6).to(DEV)
    with torch.no_grad():
        parallel = attn(tokens)
        cache, steps = None, []
        for i in range(tokens.shape[1]):
            one, cache = attn(tokens[:, i:i + 1], cache=cache, return_cache=True)
            steps.append(one)
    assert (parallel - torch.cat(steps, dim=1))[:, 4:].abs().max().item() <= 2e-5


def test_language_model_harness_matches_upstream_transformer_on_gpu():
    """The language-model training step the benchmark times (bench.build_lm around the library's layer), in fp32 at a
    toy size, against the stored loss, logits and gradient norms of upstream's Transformer (transformer.py:254-330)
    with the same seeded weights and token ids."""
    import bench
    gold = load_golden('lm_toy')
    model, _ = bench.build_lm(recipe.LM_CASE, DEV, dtype=torch.float32)
    recipe.lm_fill_weights(model, seed=9)
    ids = recipe.lm_ids().to(DEV)
    loss = model(ids)
    loss.backward()
    observe('loss', ours=loss.item(), upstream=gold['loss'].item())
    assert abs(loss.item() - gold['loss'].item()) <= 1e-4 * abs(gold['loss'].item())
    with torch.no_grad():
        assert_close_f32(model.logits(ids[:, :-1]), gold['logits'], 'logits')
    for pname, p in model.named_parameters():
        g = gold.get('pgrad.' + pname)
        if g is None:
            assert p.grad is None or p.grad.abs().sum().item() == 0, pname
            continue
        got = torch.tensor([p.grad.abs().sum().item(), p.grad.pow(2).sum().item()], dtype=torch.float64)
        assert torch.allclose(got, g, rtol=1e-3, atol=1e-6), (pname, got, g)


@pytest.mark.parametrize('case', [(2, 8, 2, 64, 1500, 16, 64, 8, 200, torch.float32), (1, 16, 2, 128, 3000, 16, 64, 16, 512, torch.bfloat16),
                                  (1, 4, 4, 64, 70, 4, 4, 3, 9, torch.float32)])
def test_decode_step_kernel_matches_the_restated_step(case):
    """The decode kernel (one launch per token) on caches far longer than upstream's own grid reaches, against the same
    step restated with tensor operations on the host: compressed attention over all compressed blocks with the memory
    slots in front, selection without own-block exclusion, selected blocks plus the own block's past, window + 1 keys,
    gates."""
    import torch.nn.functional as F
    from native_sparse_attention_pytorch_b200 import _lib as L, ops
    b, hq, hkv, d, t, st, sel, nsel, win, dtype = case
    g, ncb, m = hq // hkv, (t - 1) // st, 2
    pos = t - 1
    rnd = lambda shape, seed: recipe.randn(shape, seed).to(dtype)
    q, qr = rnd((b, hq, d), 1), rnd((b, hq, d), 2)
    keys, vals = rnd((b, hkv, t, d), 3), rnd((b, hkv, t, d), 4)
    ck, cv = rnd((b, hkv, ncb, d), 5), rnd((b, hkv, ncb, d), 6)
    mem = rnd((2, hkv, m, d), 7)
    gates = torch.sigmoid(recipe.randn((b, hq, 3), 8)).to(dtype)
    before = L.load().nsa_launch_count()
    got = ops.decode_step(*(x.to(DEV) for x in (q, qr, keys, vals, ck, cv, mem[0], mem[1], gates)), stride=st, block=sel,
                          num_selected=nsel, window=win)
    assert L.load().nsa_launch_count() - before == 1

    f = lambda x: x.float()
    scale = d ** -0.5
    qg, qrg = f(q).view(b, hkv, g, d), f(qr).view(b, hkv, g, d)

    def attend(query, kk, vv):            # query [b,hkv,g,d]; kk, vv [b,hkv,J,d]
        sim = torch.einsum('bhgd,bhjd->bhgj', query, kk) * scale
        return torch.einsum('bhgj,bhjd->bhgd', sim.softmax(dim=-1), vv), sim

    ckm = torch.cat((f(mem[0]).expand(b, -1, -1, -1), f(ck)), dim=2)
    cvm = torch.cat((f(mem[1]).expand(b, -1, -1, -1), f(cv)), dim=2)
    o_cmp, csim = attend(qg, ckm, cvm)
    imp = csim[..., m:]
    cpf = sel // st
    if st != sel:
        cols = ncb // cpf
        imp = imp[..., : cols * cpf].reshape(b, hkv, g, cols, cpf).mean(dim=-1)
    prob = F.pad(imp.mean(dim=2), (1, 0), value=-1e3).softmax(dim=-1)[..., 1:]
    score, idx = prob.topk(min(nsel, prob.shape[-1]), dim=-1)
    own0 = pos // sel * sel
    o_sel = torch.empty(b, hkv, g, d)
    for bi in range(b):
        for h in range(hkv):
            rows = [torch.arange(j * sel, (j + 1) * sel) for j, sc in zip(idx[bi, h].tolist(), score[bi, h].tolist()) if sc > 1e-10]
            rows.append(torch.arange(own0, pos + 1))
            rows = torch.cat(rows)
            o, _ = attend(qrg[bi:bi + 1, h:h + 1], f(keys)[bi:bi + 1, h:h + 1, rows], f(vals)[bi:bi + 1, h:h + 1, rows])
            o_sel[bi, h] = o[0, 0]
    lo = max(0, pos - win)
    o_swa, _ = attend(qrg, f(keys)[:, :, lo:], f(vals)[:, :, lo:])
    gt = f(gates).view(b, hkv, g, 3)
    ref = (gt[..., 0:1] * o_cmp + gt[..., 1:2] * o_sel + gt[..., 2:3] * o_swa).reshape(b, hq * d)
    (assert_close_f32 if dtype == torch.float32 else assert_close_bf16)(got, ref, 'merged row')


@pytest.mark.gpu
def test_layer_step_can_be_recorded_as_a_cuda_graph():
    """Forward + backward of the module recorded once as a CUDA graph and replayed on new inputs gives what issuing the
    kernels one by one gives: nothing on the path synchronises with the host or allocates outside PyTorch's allocator,
    and the module's status poll leaves a capture alone.  (Everything runs on a side stream: a graph cannot be
    recorded around gradients that were first accumulated on the default stream.)"""
    from native_sparse_attention_pytorch_b200 import ops
    kw = dict(dim=256, dim_head=64, heads=8, kv_heads=2, causal=True, sliding_window_size=128, compress_block_size=32,
              compress_block_sliding_stride=16, selection_block_size=64, num_selected_blocks=4)
    attn = SparseAttention(**kw, use_triton_kernel=True, kernel_impl='sm100')
    recipe.fill_weights(attn, seed=7)
    attn = attn.to(DEV).bfloat16()
    x = recipe.randn((1, 700, 256), 11).bfloat16().to(DEV).requires_grad_()
    up = recipe.randn((1, 700, 256), 13).bfloat16().to(DEV)
    x2, up2 = recipe.randn((1, 700, 256), 17).bfloat16().to(DEV), recipe.randn((1, 700, 256), 19).bfloat16().to(DEV)

    def step():
        attn.zero_grad(set_to_none=True)
        x.grad = None
        out = attn(x)
        out.backward(up)
        return out

    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(2):
            step()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            g_out = step()
        with torch.no_grad():
            x.copy_(x2)
            up.copy_(up2)
        graph.replay()
        torch.cuda.synchronize()
        got = (g_out.clone(), x.grad.clone(), attn.to_qkv.weight.grad.clone())
        want_out = step()                       # the same inputs, issued kernel by kernel
        torch.cuda.synchronize()
        ops.check_device_status()
        assert torch.equal(got[0], want_out)
        # dk / dv are sums of atomics (their order is not fixed), everything downstream of them may differ in the last bits
        assert_close_bf16(got[1], x.grad.float().cpu(), 'd input of the replay', roundings=2)
        assert_close_bf16(got[2], attn.to_qkv.weight.grad.float().cpu(), 'd to_qkv.weight of the replay', roundings=2,
                          rel_to_max=2e-3)
    torch.cuda.current_stream().wait_stream(stream)
