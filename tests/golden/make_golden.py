"""Generate the golden vectors under tests/golden/ from the UNMODIFIED upstream
library.  Run in a container that has the upstream checkout:

    python tests/golden/make_golden.py /path/to/upstream/checkout        (all cases)
    python tests/golden/make_golden.py /path/to/upstream/checkout lm     (the language-model case only)

The three third-party packages upstream imports but this image lacks are
replaced by the stand-ins in tests/golden/standins/.  Upstream code is imported,
never copied; intermediates are captured by wrapping functions in its module
namespace while its forward runs.  Outputs: one .npz per case."""
import ast
import os
import sys
from math import ceil

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, 'standins'))
sys.path.insert(0, HERE)
if len(sys.argv) < 2:
    sys.exit('usage: make_golden.py /path/to/upstream/checkout')
upstream = sys.argv[1]
sys.path.insert(0, upstream)

import recipe  # noqa: E402
import native_sparse_attention_pytorch.native_sparse_attention as nsa_mod  # noqa: E402


def np_(t):
    return None if t is None else t.detach().cpu().numpy()


def run_layer_case(name):
    c = recipe.LAYER_CASES[name]
    torch.manual_seed(0)
    attn = nsa_mod.SparseAttention(**c['kw'])
    recipe.fill_weights(attn, seed=7, rich=c['rich'])
    x = recipe.layer_input(name).requires_grad_()
    cap = {}

    # wrap names in upstream's module namespace to observe intermediates
    orig_stack, orig_attend, orig_topk = nsa_mod.stack, nsa_mod.attend, torch.Tensor.topk

    def stack_spy(ts, *a, **k):
        if len(ts) == 3 and 'branches' not in cap:
            for t in ts:
                t.retain_grad()
            cap['branches'] = ts
        return orig_stack(ts, *a, **k)

    def attend_spy(*a, **k):
        r = orig_attend(*a, **k)
        if k.get('return_sim'):
            cap['csim'] = r[1]
        return r

    def topk_spy(self, *a, **k):
        r = orig_topk(self, *a, **k)
        cap['probs'], cap['vals'], cap['idx'] = self, r[0], r[1]
        return r

    hooks = [
        attn.to_qkv.register_forward_hook(lambda m, i, o: (o.retain_grad(), cap.__setitem__('qkv', o))[0] and None),
        attn.k_compress.register_forward_hook(lambda m, i, o: (o.retain_grad(), cap.__setitem__('ck', o))[0] and None),
        attn.v_compress.register_forward_hook(lambda m, i, o: (o.retain_grad(), cap.__setitem__('cv', o))[0] and None),
        attn.to_strategy_combine.register_forward_hook(lambda m, i, o: (o.retain_grad(), cap.__setitem__('gates', o))[0] and None),
    ]
    orig_rot = attn.rotary_emb.rotate_queries_with_cached_keys

    def rot_spy(q, k):
        r = orig_rot(q, k)
        cap['qr'], cap['kr'] = r
        return r

    attn.rotary_emb.rotate_queries_with_cached_keys = rot_spy
    nsa_mod.stack, nsa_mod.attend, torch.Tensor.topk = stack_spy, attend_spy, topk_spy
    try:
        out = attn(x)
    finally:
        nsa_mod.stack, nsa_mod.attend, torch.Tensor.topk = orig_stack, orig_attend, orig_topk
        for h in hooks:
            h.remove()
    up = recipe.randn(out.shape, 13)
    (out * up).sum().backward()

    o_cmp, o_sel, o_swa = cap['branches']
    res = dict(out=np_(out), x_grad=np_(x.grad), qkv=np_(cap['qkv']), qkv_grad=np_(cap['qkv'].grad),
               qr=np_(cap['qr']), kr=np_(cap['kr']), csim=np_(cap['csim']),
               o_cmp=np_(o_cmp), o_sel=np_(o_sel), o_swa=np_(o_swa),
               o_cmp_grad=np_(o_cmp.grad), o_sel_grad=np_(o_sel.grad), o_swa_grad=np_(o_swa.grad),
               gates=np_(cap['gates']), gates_grad=np_(cap['gates'].grad))
    if 'ck' in cap and cap['ck'].grad is not None:
        res.update(ck=np_(cap['ck']), cv=np_(cap['cv']), ck_grad=np_(cap['ck'].grad), cv_grad=np_(cap['cv'].grad))
    if 'idx' in cap:
        res.update(probs=np_(cap['probs']), vals=np_(cap['vals']), idx=np_(cap['idx']))
    for pname, p in attn.named_parameters():
        if p.grad is not None:
            res['pgrad.' + pname] = np.array([p.grad.abs().sum().item(), p.grad.pow(2).sum().item()])
    if name.startswith('readme'):
        # the README-sized case keeps only what is needed, to stay small
        res = {k: v for k, v in res.items() if k in ('out', 'x_grad', 'idx', 'vals', 'probs', 'o_sel', 'gates_grad')
               or k.startswith('pgrad.')}
    np.savez_compressed(os.path.join(HERE, f'layer_{name}.npz'), **{k: v for k, v in res.items() if v is not None})
    print('layer', name, 'out', tuple(out.shape), 'abs mean', out.abs().mean().item())


def load_regular_attend(block):
    """Pull ``regular_attend`` (and the tiny helpers it uses) out of upstream's
    GPU check script without running the script, which asserts CUDA at import."""
    src = open(os.path.join(upstream, 'test_triton_nsa.py')).read()
    tree = ast.parse(src)
    wanted = {'exists', 'default', 'divisible_by', 'regular_attend'}
    body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in wanted]
    import einx
    from einops import rearrange, einsum, repeat
    import torch.nn.functional as F

    def pad_to_multiple(t, mult, *, dim):
        n = t.shape[dim]
        extra = ceil(n / mult) * mult - n
        right = (-dim - 1) if dim < 0 else (t.ndim - dim - 1)
        return F.pad(t, (0, 0) * right + (0, extra))

    def get_at(pattern, blocks, indices):
        assert pattern == 'b h [w] n d, b h i sel -> b h i (sel n) d'
        b, h = indices.shape[:2]
        bi = torch.arange(b)[:, None, None, None]
        hi = torch.arange(h)[None, :, None, None]
        g = blocks[bi, hi, indices]  # b h i sel n d
        return g.flatten(3, 4)

    einx.get_at = get_at
    ns = dict(torch=torch, einx=einx, rearrange=rearrange, einsum=einsum, repeat=repeat, ceil=ceil,
              pad_to_multiple=pad_to_multiple, fine_block_size=block)
    exec(compile(ast.Module(body=body, type_ignores=[]), 'test_triton_nsa.py', 'exec'), ns)
    return ns['regular_attend']


def run_op_case(name):
    c = recipe.OP_CASES[name]
    q, k, v, idx, mask = recipe.op_inputs(name)
    scale = torch.ones(idx.shape)
    q, k, v, scale = (t.clone().requires_grad_() for t in (q, k, v, scale))
    fn = load_regular_attend(c['block'])
    out, lse = fn(q, k, v, idx, mask, block_size=c['block'], sel_scale=scale, return_lse=True)
    up = recipe.randn(out.shape, 29)
    (out * up).sum().backward()
    np.savez_compressed(os.path.join(HERE, f'{name}.npz'), out=np_(out), lse=np_(lse), dq=np_(q.grad),
                        dk=np_(k.grad), dv=np_(v.grad), dscale=np_(scale.grad))
    print('op', name, 'out', tuple(out.shape), 'abs mean', out.abs().mean().item())


def run_lm_case():
    """Upstream's Transformer (pure-PyTorch SparseAttention path) on seeded token ids: loss, logits of the loss's
    inputs, and two norms of every parameter gradient."""
    import native_sparse_attention_pytorch.transformer as tf_mod
    c = recipe.LM_CASE
    torch.manual_seed(0)
    model = tf_mod.Transformer(
        num_tokens=c['vocab'], dim=c['dim'], depth=c['depth'], heads=c['heads'], kv_heads=c['kv_heads'],
        dim_head=c['dim_head'], use_sparse_attn=True, causal=True, use_triton_fine_selection=False,
        sparse_attn_kwargs=dict(sliding_window_size=c['sliding_window_size'], compress_block_size=c['compress_block_size'],
                                compress_block_sliding_stride=c['compress_block_sliding_stride'],
                                selection_block_size=c['selection_block_size'],
                                num_selected_blocks=c['num_selected_blocks']))
    recipe.lm_fill_weights(model, seed=9)
    ids = recipe.lm_ids()
    loss = model(ids, return_loss=True)
    loss.backward()
    with torch.no_grad():
        logits = model(ids[:, :-1])
    res = dict(loss=np.array([loss.item()]), logits=np_(logits))
    for pname, p in model.named_parameters():
        if p.grad is not None:
            res['pgrad.' + pname] = np.array([p.grad.abs().sum().item(), p.grad.pow(2).sum().item()])
    np.savez_compressed(os.path.join(HERE, 'lm_toy.npz'), **res)
    print('lm loss', loss.item(), 'params with grad', sum(1 for k in res if k.startswith('pgrad.')))


if __name__ == '__main__':
    torch.set_num_threads(8)
    if len(sys.argv) > 2 and sys.argv[2] == 'lm':
        run_lm_case()
        sys.exit(0)
    for n in recipe.LAYER_CASES:
        run_layer_case(n)
    for n in recipe.OP_CASES:
        run_op_case(n)
    run_lm_case()
