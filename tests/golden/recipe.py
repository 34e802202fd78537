"""Seeded synthetic tensors and weights shared by the fixture generator and
the tests.  Everything comes from numpy's PCG64 stream, which is stable across
machines, so a fixture only has to store outputs: inputs and weights are
regenerated from the case description."""
import numpy as np
import torch


def randn(shape, seed, scale=1.0, dtype=torch.float32):
    g = np.random.Generator(np.random.PCG64(seed))
    a = g.standard_normal(size=tuple(shape), dtype=np.float64) * scale
    return torch.from_numpy(a.astype(np.float32)).to(dtype)


def randint(low, high, shape, seed):
    g = np.random.Generator(np.random.PCG64(seed))
    return torch.from_numpy(g.integers(low, high, size=tuple(shape), dtype=np.int64))


def fill_weights(module, seed, rich=True):
    """Overwrite every parameter of a SparseAttention-shaped module, visiting
    parameters in sorted-name order.  ``rich`` gives non-zero memory slots,
    intra-block positions and gate weights so every term of the layer matters;
    otherwise those keep upstream's initial values (zeros, gate bias -2,-2,2)."""
    with torch.no_grad():
        for i, (name, p) in enumerate(sorted(module.named_parameters())):
            s = seed * 1000 + i
            if name == 'norm.weight':
                p.copy_(1.0 + randn(p.shape, s, 0.1))
            elif name.startswith('to_strategy_combine'):
                if not rich:
                    continue
                p.copy_(randn(p.shape, s, 0.5 if name.endswith('bias') else p.shape[-1] ** -0.5))
            elif name in ('compress_mem_kv', 'k_intrablock_positions', 'v_intrablock_positions'):
                if rich:
                    p.copy_(randn(p.shape, s, 0.5))
            elif name.endswith('bias'):
                p.copy_(randn(p.shape, s, 0.1))
            else:  # linear weights [out, in]
                p.copy_(randn(p.shape, s, p.shape[-1] ** -0.5))


# ---- layer-level cases: SparseAttention kwargs, batch, seq, weight style ----
_base = dict(dim=64, dim_head=16, heads=4, sliding_window_size=2)
LAYER_CASES = {
    # the README configuration (non-causal, one query head per KV head)
    'readme': dict(kw=dict(dim=512, dim_head=64, heads=8, sliding_window_size=2, compress_block_size=4,
                           compress_block_sliding_stride=2, selection_block_size=4, num_selected_blocks=2),
                   batch=2, seq=31, rich=False),
    'readme_rich': dict(kw=dict(dim=512, dim_head=64, heads=8, sliding_window_size=2, compress_block_size=4,
                                compress_block_sliding_stride=2, selection_block_size=4, num_selected_blocks=2),
                        batch=2, seq=31, rich=True),
    'causal_gqa': dict(kw=dict(_base, kv_heads=2, causal=True, compress_block_size=8, compress_block_sliding_stride=4,
                               selection_block_size=8, num_selected_blocks=2), batch=2, seq=120, rich=True),
    'causal_gqa_win': dict(kw=dict(_base, kv_heads=1, causal=True, compress_block_size=8, compress_block_sliding_stride=4,
                                   selection_block_size=16, num_selected_blocks=3, sliding_window_size=9),
                           batch=1, seq=97, rich=True),
    'causal_stride_eq_sel': dict(kw=dict(_base, kv_heads=2, causal=True, compress_block_size=4, compress_block_sliding_stride=4,
                                         selection_block_size=4, num_selected_blocks=2), batch=2, seq=31, rich=True),
    'noncausal_gqa': dict(kw=dict(_base, kv_heads=2, causal=False, compress_block_size=4, compress_block_sliding_stride=2,
                                  selection_block_size=8, num_selected_blocks=2), batch=2, seq=32, rich=True),
    'causal_nsel0': dict(kw=dict(_base, kv_heads=2, causal=True, compress_block_size=4, compress_block_sliding_stride=2,
                                 selection_block_size=8, num_selected_blocks=0), batch=2, seq=31, rich=True),
    'noncausal_nsel0': dict(kw=dict(_base, kv_heads=4, causal=False, compress_block_size=4, compress_block_sliding_stride=2,
                                    selection_block_size=8, num_selected_blocks=0), batch=2, seq=31, rich=True),
    'causal_short': dict(kw=dict(_base, kv_heads=2, causal=True, compress_block_size=8, compress_block_sliding_stride=4,
                                 selection_block_size=32, num_selected_blocks=2), batch=2, seq=4, rich=True),
    'causal_one_token': dict(kw=dict(_base, kv_heads=2, causal=True, compress_block_size=8, compress_block_sliding_stride=4,
                                     selection_block_size=8, num_selected_blocks=2), batch=2, seq=1, rich=True),
    'causal_per_head_selection': dict(kw=dict(_base, kv_heads=2, causal=True, compress_block_size=8, compress_block_sliding_stride=4,
                                              selection_block_size=8, num_selected_blocks=2, query_heads_share_selected_kv=False),
                                      batch=2, seq=50, rich=True),
    'causal_diff_topk': dict(kw=dict(_base, kv_heads=2, causal=True, compress_block_size=8, compress_block_sliding_stride=4,
                                     selection_block_size=8, num_selected_blocks=2, use_diff_topk=True),
                             batch=2, seq=50, rich=True),
}

# ---- kernel-level cases for the selected-block operator ----
OP_CASES = {
    # shaped like upstream's own GPU check (ragged length, indices in {0,1}, random slot mask)
    'op_ragged': dict(batch=2, seq=107, q_heads=4, kv_heads=2, dim_head=32, block=16, nsel=2, idx_high=2),
    'op_wide': dict(batch=1, seq=200, q_heads=8, kv_heads=1, dim_head=16, block=32, nsel=3, idx_high=7),
    'op_g1': dict(batch=2, seq=64, q_heads=2, kv_heads=2, dim_head=64, block=16, nsel=2, idx_high=4),
}


def layer_input(case, seed=11):
    c = LAYER_CASES[case]
    return randn((c['batch'], c['seq'], c['kw']['dim']), seed)


def op_inputs(case, seed=23):
    c = OP_CASES[case]
    b, n, hq, hkv, d = c['batch'], c['seq'], c['q_heads'], c['kv_heads'], c['dim_head']
    q = randn((b, hq, n, d), seed)
    k = randn((b, hkv, n, d), seed + 1)
    v = randn((b, hkv, n, d), seed + 2)
    idx = randint(0, c['idx_high'], (b, hkv, n, c['nsel']), seed + 3)
    mask = randint(0, 2, (b, hkv, n, c['nsel']), seed + 4).bool()
    return q, k, v, idx, mask


# ---- language-model case: upstream's Transformer around the layer (transformer.py:142-330), toy size ----
LM_CASE = dict(vocab=256, dim=64, depth=2, heads=4, kv_heads=2, dim_head=16, batch=2, seq=64,
               sliding_window_size=8, compress_block_size=8, compress_block_sliding_stride=4, selection_block_size=8,
               num_selected_blocks=2)


def lm_ids(seed=17):
    c = LM_CASE
    return randint(0, c['vocab'], (c['batch'], c['seq'] + 1), seed)


def lm_fill_weights(module, seed):
    """Overwrite every parameter of a Transformer-shaped module (token embedding, blocks of [SparseAttention,
    feed-forward], final norm, logits), visiting parameters in sorted-name order; the rule for a parameter depends on
    the end of its name and its rank only, so upstream's model and a harness with the same names get the same values."""
    with torch.no_grad():
        for i, (name, p) in enumerate(sorted(module.named_parameters())):
            s = seed * 1000 + i
            leaf = name.split('.')[-1]
            if leaf in ('compress_mem_kv', 'k_intrablock_positions', 'v_intrablock_positions'):
                p.copy_(randn(p.shape, s, 0.5))
            elif p.dim() == 1 and leaf == 'weight':          # RMS norm gains
                p.copy_(1.0 + randn(p.shape, s, 0.1))
            elif leaf == 'bias':
                p.copy_(randn(p.shape, s, 0.5 if 'to_strategy_combine' in name else 0.1))
            elif name.startswith('token_emb'):
                p.copy_(randn(p.shape, s, 1.0))
            else:                                            # linear weights [out, in]
                p.copy_(randn(p.shape, s, p.shape[-1] ** -0.5))
