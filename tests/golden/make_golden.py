"""Generate the golden fixtures in this folder by running the reference's own eager PyTorch path on CPU.

Usage (in a container that has the reference project checked out):

    python tests/golden/make_golden.py --reference <path to the reference project root>

The reference ships no golden vectors for its attention path, so parity is pinned to what its code
computes: this script imports ``LlamaNAtSChunkAttentionLayer`` and ``NAtSCache`` from the reference
(with four stub modules for files the reference imports but does not ship, and a stubbed device-capability
query because there is no GPU where this runs), drives them exactly as ``AttentionLayer.forward`` does in
eval mode (prepare_kv -> repeat_kv_values -> multi_head_attention, i.e. cache.update -> generate_mask ->
scaled_dot_product_attention -> cache.post_update), and stores inputs' seeds, role codes, outputs and the
cache state after the prefill and after a run of single-token decode steps.

Inputs are regenerated from the stored seed by ``golden_inputs`` below (imported by the tests); a float64
checksum of every regenerated tensor is stored next to the outputs so that generator drift is detected.
"""
from __future__ import annotations

import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# name -> (B, Hq, Hkv, N, D, C, SW, p_global, p_local, seed, n_decode, special)
CASES = {
    # tiny cases: complete tensors are stored
    'tiny_mha':       dict(B=2, Hq=2, Hkv=2, N=96,  D=16, C=8,  SW=32, pg=0.10, pl=0.30, seed=1, n_decode=20),
    'tiny_gqa':       dict(B=2, Hq=4, Hkv=2, N=128, D=16, C=16, SW=32, pg=0.10, pl=0.30, seed=2, n_decode=40),
    'tiny_ragged':    dict(B=2, Hq=4, Hkv=2, N=200, D=16, C=16, SW=64, pg=0.10, pl=0.30, seed=3, n_decode=30),
    'tiny_short':     dict(B=1, Hq=2, Hkv=2, N=40,  D=16, C=8,  SW=64, pg=0.20, pl=0.30, seed=4, n_decode=20),
    'tiny_sub_chunk': dict(B=1, Hq=2, Hkv=2, N=5,   D=16, C=8,  SW=16, pg=0.20, pl=0.30, seed=5, n_decode=30),
    'all_local':      dict(B=1, Hq=2, Hkv=2, N=64,  D=16, C=8,  SW=16, pg=0.0,  pl=1.0,  seed=6, n_decode=20, special='all_local'),
    'all_sliding':    dict(B=1, Hq=2, Hkv=2, N=64,  D=16, C=8,  SW=16, pg=0.0,  pl=0.0,  seed=7, n_decode=20, special='all_sliding'),
    'all_global':     dict(B=1, Hq=2, Hkv=2, N=64,  D=16, C=8,  SW=16, pg=1.0,  pl=0.0,  seed=8, n_decode=20, special='all_global'),
    'no_global':      dict(B=2, Hq=2, Hkv=2, N=96,  D=16, C=8,  SW=32, pg=0.0,  pl=0.4,  seed=9, n_decode=20, special='no_global'),
    # kernel-sized cases (head_dim 64 / 128): every 5th output row is stored
    'k64_mha':        dict(B=1, Hq=4, Hkv=4, N=512, D=64,  C=64,  SW=256, pg=0.10, pl=0.30, seed=11, n_decode=70),
    'k128_gqa':       dict(B=1, Hq=4, Hkv=1, N=640, D=128, C=128, SW=256, pg=0.10, pl=0.20, seed=12, n_decode=0),
    'k64_ragged':     dict(B=2, Hq=4, Hkv=2, N=300, D=64,  C=16,  SW=64,  pg=0.10, pl=0.30, seed=13, n_decode=40),
    'k128_decode':    dict(B=2, Hq=4, Hkv=2, N=256, D=128, C=32,  SW=64,  pg=0.15, pl=0.30, seed=14, n_decode=70),
    # the reference's own CPU-runnable configuration: one layer, batch 1, 8 heads (MHA), head_dim 64, 2048 tokens, seed 0,
    # window 256, chunk 64, about 10 % global / 30 % local / 60 % sliding chunks
    'cfg1_mha_2048':  dict(B=1, Hq=8, Hkv=8, N=2048, D=64, C=64,  SW=256, pg=0.10, pl=0.30, seed=0, n_decode=0),
}
# multi-token calls over an existing cache: the sequence is fed in the given segments (N = their sum), then decoded.
# Shapes avoid two reference defects: a first segment shorter than one chunk followed by a multi-token call raises
# (nats_chunk_layer_cache.py:676), and a continuation that starts before the window has filled and runs past it hides the
# ring's chunks in reversed order (:670-679).
SEG_CASES = {
    'seg_tiny_aligned':  dict(B=2, Hq=4, Hkv=2, D=16, C=8,  SW=32, segs=[64, 64, 32], pg=0.10, pl=0.30, seed=21, n_decode=20),
    'seg_tiny_ragged':   dict(B=2, Hq=4, Hkv=2, D=16, C=16, SW=32, segs=[48, 100, 60], pg=0.10, pl=0.30, seed=22, n_decode=20),
    'seg_tiny_steps':    dict(B=1, Hq=2, Hkv=2, D=16, C=8,  SW=32, segs=[64, 5, 5, 54], pg=0.15, pl=0.30, seed=29, n_decode=12),
    'seg_tiny_unfilled': dict(B=2, Hq=2, Hkv=2, D=16, C=8,  SW=64, segs=[24, 40, 64], pg=0.10, pl=0.30, seed=24, n_decode=10),
    'seg_tiny_sparse':   dict(B=1, Hq=2, Hkv=2, D=16, C=4,  SW=16, segs=[30, 30, 30, 30], pg=0.03, pl=0.25, seed=25, n_decode=10),
    'seg_k64':           dict(B=1, Hq=4, Hkv=2, D=64,  C=64, SW=128, segs=[512, 384, 200], pg=0.10, pl=0.30, seed=26, n_decode=0),
    'seg_k128':          dict(B=2, Hq=4, Hkv=2, D=128, C=32, SW=64,  segs=[256, 256, 100], pg=0.10, pl=0.30, seed=27, n_decode=40),
}
for _c in SEG_CASES.values():
    _c['N'] = sum(_c['segs'])
# token-granular cache (one role per token, NAtSLayerCache): the prefill call and its eviction.  Its single-token steps
# defer the placement of tokens by up to update_chunk_size = 16 steps, during which a token stays visible past its rule;
# only the state right after the prefill is comparable with an implementation that places every token at once.
TOK_CASES = {
    'tok_tiny':    dict(B=2, Hq=4, Hkv=2, N=48,  D=16, C=1, SW=16, pg=0.10, pl=0.30, seed=41, n_decode=0),
    'tok_long':    dict(B=2, Hq=2, Hkv=2, N=333, D=16, C=1, SW=32, pg=0.05, pl=0.30, seed=42, n_decode=0),
    'tok_k64':     dict(B=1, Hq=4, Hkv=2, N=512, D=64, C=1, SW=64, pg=0.05, pl=0.25, seed=43, n_decode=0),
}
# token-granular cache, single-token steps: the reference places tokens in batches of update_chunk_size = 16, so its
# index-level state is comparable right after each batched update (steps 16, 32, ... after the prefill).
TOKDEC_CASES = {
    'tokdec_tiny': dict(B=2, Hq=4, Hkv=2, N=48, D=16, C=1, SW=16, pg=0.10, pl=0.30, seed=51, n_decode=64),
    'tokdec_k64':  dict(B=2, Hq=4, Hkv=2, N=128, D=64, C=1, SW=32, pg=0.08, pl=0.30, seed=52, n_decode=48),
}
TOK_UPDATE = 16
# role sampling (pooled hidden states -> role head -> argmax): a sequence of calls through the reference layer -- a prefill
# that ends inside a chunk, a multi-token call that starts inside a chunk, single tokens across chunk boundaries, a call
# that completes no chunk.  ``enh`` is the value the layer adds to the global logit (0.1 in the reference's own modules;
# its Hugging Face forward, hf/llama_nats_chunk.py:194-215, is the same computation without it).
ROLE_CASES = {
    'roles_mean':    dict(B=2, Hq=4, Hkv=2, D=16, C=8, SW=32, method='mean', enh=0.1, seed=61, calls=[50, 13] + [1] * 20 + [3, 1, 1, 25, 2, 6]),
    'roles_max':     dict(B=2, Hq=4, Hkv=2, D=16, C=8, SW=32, method='max',  enh=0.1, seed=62, calls=[50, 13] + [1] * 20 + [3, 1, 1, 25, 2, 6]),
    'roles_mean_hf': dict(B=2, Hq=4, Hkv=2, D=16, C=8, SW=32, method='mean', enh=0.0, seed=63, calls=[64, 9] + [1] * 18 + [5, 30]),
    'roles_max_hf':  dict(B=2, Hq=4, Hkv=2, D=16, C=4, SW=16, method='max',  enh=0.0, seed=64, calls=[30, 7] + [1] * 11 + [2, 1, 17]),
}
ROW_STRIDE = 5


def golden_roles(case: dict) -> np.ndarray:
    sys.path.insert(0, os.path.join(HERE, '..', '..'))
    from oracle.nats_oracle import make_roles
    Nc = -(-case['N'] // case['C'])
    sp = case.get('special')
    if sp == 'all_local':
        return np.full((case['B'], case['Hkv'], Nc), 1, np.uint8)
    if sp == 'all_sliding':
        return np.full((case['B'], case['Hkv'], Nc), 2, np.uint8)
    if sp == 'all_global':
        return np.zeros((case['B'], case['Hkv'], Nc), np.uint8)
    roles = make_roles(case['B'], case['Hkv'], Nc, max(case['pg'], 1e-3), max(case['pl'], 1e-3), case['seed'],
                       force_first_global=(sp != 'no_global'))
    if sp == 'no_global':
        roles[roles == 0] = 2
    if case['N'] % case['C']:
        roles[..., -1] = 0        # the layer marks an unfinished last chunk global (nats_chunk_attention.py:92-94)
    return roles


def golden_inputs(case: dict):
    """q [B,Hq,N,D], k, v [B,Hkv,N,D] fp32 and, per decode step, (q1,k1,v1,role codes [B,Hkv])."""
    g = torch.Generator().manual_seed(case['seed'])
    B, Hq, Hkv, N, D = case['B'], case['Hq'], case['Hkv'], case['N'], case['D']
    q = torch.randn(B, Hq, N, D, generator=g)
    k = torch.randn(B, Hkv, N, D, generator=g)
    v = torch.randn(B, Hkv, N, D, generator=g)
    steps = []
    for _ in range(case['n_decode']):
        q1 = torch.randn(B, Hq, 1, D, generator=g)
        k1 = torch.randn(B, Hkv, 1, D, generator=g)
        v1 = torch.randn(B, Hkv, 1, D, generator=g)
        r1 = torch.randn(B, Hkv, 3, generator=g).argmax(-1).to(torch.uint8).numpy()
        sp = case.get('special')
        if sp == 'all_sliding':
            r1[:] = 2
        steps.append((q1, k1, v1, r1))
    return q, k, v, steps


def checksum(*tensors) -> np.ndarray:
    return np.array([float(t.double().sum()) for t in tensors])


def load_reference(root: str):
    def stub(name, **attrs):
        m = types.ModuleType(name)
        m.__path__ = []
        for key, val in attrs.items():
            setattr(m, key, val)
        sys.modules[name] = m
    stub('nats.components.cache.triton')
    stub('nats.components.cache.triton.update_one_step', post_update_one_step=None)
    stub('nats.models.transformer.triton.flashattention_mask_on_chip', nats_attention=None)
    stub('nats.models.transformer.triton.nats_chunk_attention', nats_chunk_attention=None)
    torch.cuda.get_device_capability = lambda *a, **k: (10, 0)
    torch.cuda.empty_cache = lambda *a, **k: None
    import torch._dynamo as dynamo
    dynamo.config.disable = True                 # the reference decorates small helpers with torch.compile; eager is the same math
    sys.path.insert(0, os.path.join(root, 'src'))
    from nats.components.cache.dyn_cache import NAtSCache
    from nats.models.transformer.attention.nats_chunk_attention import LlamaNAtSChunkAttentionLayer
    return NAtSCache, LlamaNAtSChunkAttentionLayer


def state_of(layer_cache) -> dict:
    n_ctx = int(layer_cache.n_ctx_data)
    return dict(
        cache_k=layer_cache.cache_k.detach().numpy().copy(),
        cache_v=layer_cache.cache_v.detach().numpy().copy(),
        valid=layer_cache.valid_tokens.numpy().copy(),
        size_global=layer_cache.size_global_kv.numpy().copy(),
        size_local=layer_cache.size_local_kv.numpy().copy(),
        n_ctx_data=np.int64(n_ctx),
        chunk_fill=np.int64(layer_cache.chunk_fill_size),
        tail=np.int64(layer_cache.sliding_queue_tail),
        seen=np.int64(layer_cache._seen_tokens),
    )


def log2_sum_exp2(q: torch.Tensor, k: torch.Tensor, mask: np.ndarray, tiny: bool) -> np.ndarray:
    """M of the reference's training forward (triton/nats_chunk_attention.py:319-330: ``m_i + log2(l_i)``) = log2 of the
    row's sum of exp2(score * sm_scale * log2 e) over the keys the row sees, evaluated in float64 over the reference's own
    mask.  q and k are rounded to bf16 first, the precision the kernels take them in.  [B,Hq,N] (every ROW_STRIDE-th row
    for the kernel-sized cases)."""
    B, Hq, N, D = q.shape
    Hkv = k.shape[1]
    qd, kd = q.bfloat16().double(), k.bfloat16().double()
    scale = (1.0 / np.sqrt(D)) * 1.4426950408889634
    rows = slice(None) if tiny else slice(None, None, ROW_STRIDE)
    out = []
    for h in range(Hq):
        s = torch.einsum('bnd,bmd->bnm', qd[:, h, rows], kd[:, h // (Hq // Hkv)]) * scale
        s = s.masked_fill(~torch.from_numpy(mask[:, h // (Hq // Hkv), rows]), -float('inf'))
        mx = s.max(-1, keepdim=True)[0]
        out.append((mx.squeeze(-1) + torch.log2(torch.exp2(s - mx).sum(-1))).numpy())
    return np.stack(out, 1)


def run_case(name: str, case: dict, NAtSCache, Layer) -> dict:
    from oracle.nats_oracle import onehot_from_roles
    B, Hq, Hkv, N, D, C, SW = (case[x] for x in ('B', 'Hq', 'Hkv', 'N', 'D', 'C', 'SW'))
    roles = golden_roles(case)
    q, k, v, steps = golden_inputs(case)
    layer = Layer(dim=Hq * D, n_heads=Hq, n_kv_heads=Hkv, layer_id=0, local_seq_max_length=SW, chunk_size=C)
    layer.eval()
    cache = NAtSCache(sliding_window_size=SW, chunk_size=C)
    out = {'roles': roles, 'in_checksum': checksum(q, k, v)}
    with torch.no_grad():
        info = {'token_states_info': onehot_from_roles(roles)}
        keys, values = layer.prepare_kv(q, k, v, 0, cache=cache, kwargs=info)
        mask = cache.generate_mask(0, N).numpy().copy()          # the reference's ground-truth mask
        keys, values = layer.repeat_kv_values(keys, values)
        o = layer.multi_head_attention(q, keys, values, cache=cache, kwargs=info)
        lc = cache.cache_model[0]
        tiny = D < 64
        out['prefill_out'] = o.numpy() if tiny else o[:, :, ::ROW_STRIDE].numpy()
        out['prefill_M'] = log2_sum_exp2(q, k, mask, tiny)
        if tiny:
            out['prefill_mask'] = np.packbits(mask, axis=-1)
        else:
            out['prefill_mask_rows'] = np.packbits(mask[:, :, ::ROW_STRIDE], axis=-1)
        for key, val in state_of(lc).items():
            if tiny or key not in ('cache_k', 'cache_v'):       # kernel-sized cases keep the index-level state only
                out['pre_' + key] = val
        dec_out, dec_nctx, dec_sizes = [], [], []
        fill = int(lc.chunk_fill_size)
        for (q1, k1, v1, r1) in steps:
            fill += 1
            done = fill == C
            role_now = r1 if done else np.zeros_like(r1)          # placeholder one-hot(global), :81-84
            if done:
                fill = 0
            info1 = {'token_states_info': onehot_from_roles(role_now[..., None])}
            keys, values = layer.prepare_kv(q1, k1, v1, 0, cache=cache, kwargs=info1)
            keys, values = layer.repeat_kv_values(keys, values)
            o1 = layer.multi_head_attention(q1, keys, values, cache=cache, kwargs=info1)
            dec_out.append(o1.numpy().copy())
            dec_nctx.append(int(lc.n_ctx_data))
            dec_sizes.append(np.stack([lc.size_global_kv.numpy().copy(), lc.size_local_kv.numpy().copy()]))
        if steps:
            out['dec_out'] = np.stack(dec_out)
            out['dec_nctx'] = np.array(dec_nctx)
            out['dec_sizes'] = np.stack(dec_sizes)
            out['dec_roles'] = np.stack([s[3] for s in steps])
            out['dec_checksum'] = np.array([checksum(*s[:3]) for s in steps])
            for key, val in state_of(lc).items():
                if tiny or key not in ('cache_k', 'cache_v'):
                    out['post_' + key] = val
    return out


def segment_roles(case: dict, roles: np.ndarray, pos: int, fill: int, x_len: int) -> np.ndarray:
    """Role codes a caller passes with a segment: one per chunk from the unfinished chunk on; an unfinished last chunk is
    marked global (nats_chunk_attention.py:92-94), a call that completes no chunk passes the placeholder (:81-84)."""
    C = case['C']
    if fill + x_len < C:
        return np.zeros(roles.shape[:2] + (1,), np.uint8)
    r = roles[..., (pos - fill) // C:-(-(pos + x_len) // C)].copy()
    if (pos + x_len) % C:
        r[..., -1] = 0
    return r


def run_segmented_case(name: str, case: dict, NAtSCache, Layer) -> dict:
    from oracle.nats_oracle import onehot_from_roles, make_roles
    B, Hq, Hkv, N, D, C, SW = (case[x] for x in ('B', 'Hq', 'Hkv', 'N', 'D', 'C', 'SW'))
    roles = make_roles(B, Hkv, -(-N // C), case['pg'], case['pl'], case['seed'], force_first_global=True)
    q, k, v, steps = golden_inputs(case)
    layer = Layer(dim=Hq * D, n_heads=Hq, n_kv_heads=Hkv, layer_id=0, local_seq_max_length=SW, chunk_size=C)
    layer.eval()
    cache = NAtSCache(sliding_window_size=SW, chunk_size=C)
    out = {'roles': roles, 'in_checksum': checksum(q, k, v), 'segs': np.array(case['segs'])}
    tiny = D < 64
    pos = 0
    with torch.no_grad():
        for si, x_len in enumerate(case['segs']):
            fill = cache.get_nats_chunk_fill_size(0)
            r = segment_roles(case, roles, pos, fill, x_len)
            info = {'token_states_info': onehot_from_roles(r)}
            qs, ks, vs = (t[:, :, pos:pos + x_len] for t in (q, k, v))
            keys, values = layer.prepare_kv(qs, ks, vs, pos, cache=cache, kwargs=info)
            mask = cache.generate_mask(0, x_len).numpy().copy()
            keys, values = layer.repeat_kv_values(keys, values)
            o = layer.multi_head_attention(qs, keys, values, cache=cache, kwargs=info)
            lc = cache.cache_model[0]
            out[f's{si}_out'] = o.numpy() if tiny else o[:, :, ::ROW_STRIDE].numpy()
            out[f's{si}_mask'] = np.packbits(mask if tiny else mask[:, :, ::ROW_STRIDE], axis=-1)
            out[f's{si}_mask_cols'] = np.int64(mask.shape[-1])
            for key, val in state_of(lc).items():
                if tiny or key not in ('cache_k', 'cache_v'):
                    out[f's{si}_{key}'] = val
            pos += x_len
        dec_out, dec_nctx, dec_sizes = [], [], []
        fill = int(lc.chunk_fill_size)
        for (q1, k1, v1, r1) in steps:
            fill += 1
            done = fill == C
            role_now = r1 if done else np.zeros_like(r1)
            if done:
                fill = 0
            info1 = {'token_states_info': onehot_from_roles(role_now[..., None])}
            keys, values = layer.prepare_kv(q1, k1, v1, 0, cache=cache, kwargs=info1)
            keys, values = layer.repeat_kv_values(keys, values)
            o1 = layer.multi_head_attention(q1, keys, values, cache=cache, kwargs=info1)
            dec_out.append(o1.numpy().copy())
            dec_nctx.append(int(lc.n_ctx_data))
            dec_sizes.append(np.stack([lc.size_global_kv.numpy().copy(), lc.size_local_kv.numpy().copy()]))
        if steps:
            out['dec_out'] = np.stack(dec_out)
            out['dec_nctx'] = np.array(dec_nctx)
            out['dec_sizes'] = np.stack(dec_sizes)
            out['dec_roles'] = np.stack([s[3] for s in steps])
            out['dec_checksum'] = np.array([checksum(*s[:3]) for s in steps])
            for key, val in state_of(lc).items():
                if tiny or key not in ('cache_k', 'cache_v'):
                    out['post_' + key] = val
    return out


def run_token_case(name: str, case: dict) -> dict:
    """Prefill through the reference's token-granular ``NAtSLayerCache`` driven as its attention layer would
    (update -> generate_mask -> scaled_dot_product_attention -> post_update)."""
    from nats.components.cache.nats_layer_cache import NAtSLayerCache
    from oracle.nats_oracle import onehot_from_roles, make_roles
    B, Hq, Hkv, N, D, SW = (case[x] for x in ('B', 'Hq', 'Hkv', 'N', 'D', 'SW'))
    roles = make_roles(B, Hkv, N, case['pg'], case['pl'], case['seed'], force_first_global=True)
    q, k, v, _ = golden_inputs(case)
    lc = NAtSLayerCache(B, Hkv, SW, device=torch.device('cpu'))
    out = {'roles': roles, 'in_checksum': checksum(q, k, v)}
    with torch.no_grad():
        keys, values = lc.update(k, v, onehot_from_roles(roles))
        mask = lc.generate_mask(N)
        n_rep = Hq // Hkv
        o = torch.nn.functional.scaled_dot_product_attention(q, keys.repeat_interleave(n_rep, 1), values.repeat_interleave(n_rep, 1),
                                                             attn_mask=mask.repeat_interleave(n_rep, 1))
        lc.post_update(N)
    tiny = D < 64
    out['prefill_out'] = o.numpy() if tiny else o[:, :, ::ROW_STRIDE].numpy()
    out['prefill_mask'] = np.packbits(mask.numpy() if tiny else mask[:, :, ::ROW_STRIDE].numpy(), axis=-1)
    out['pre_size_global'] = lc.size_global_kv.numpy().copy()
    out['pre_size_local'] = lc.size_local_kv.numpy().copy()
    out['pre_n_ctx_data'] = np.int64(int(lc.n_ctx_data))
    out['pre_tail'] = np.int64(int(lc.sliding_queue_tail))
    out['pre_valid'] = lc.valid_tokens.numpy().copy()
    out['pre_cache_k'] = lc.cache_k.numpy().copy()
    out['pre_cache_v'] = lc.cache_v.numpy().copy()
    return out


def run_token_decode_case(name: str, case: dict) -> dict:
    """Prefill, then single-token steps through the reference's ``NAtSLayerCache`` (update -> generate_mask(1) ->
    attention -> post_update(1)).  After every step that triggers its batched update the sizes, the extent and the kept
    K / V rows of every head are stored; the output of every step is stored too."""
    from nats.components.cache.nats_layer_cache import NAtSLayerCache
    from oracle.nats_oracle import onehot_from_roles, make_roles
    B, Hq, Hkv, N, D, SW = (case[x] for x in ('B', 'Hq', 'Hkv', 'N', 'D', 'SW'))
    roles = make_roles(B, Hkv, N, case['pg'], case['pl'], case['seed'], force_first_global=True)
    q, k, v, steps = golden_inputs(case)
    q, k, v = q.bfloat16().float(), k.bfloat16().float(), v.bfloat16().float()       # what a bf16 cache holds
    lc = NAtSLayerCache(B, Hkv, SW, update_chunk_size=TOK_UPDATE, device=torch.device('cpu'))
    n_rep = Hq // Hkv
    out = {'roles': roles, 'in_checksum': checksum(*golden_inputs(case)[:3])}
    with torch.no_grad():
        keys, values = lc.update(k, v, onehot_from_roles(roles))
        lc.generate_mask(N)
        lc.post_update(N)
        dec_out, upd_steps = [], []
        for si, (q1, k1, v1, r1) in enumerate(steps):
            q1, k1, v1 = q1.bfloat16().float(), k1.bfloat16().float(), v1.bfloat16().float()
            keys, values = lc.update(k1, v1, onehot_from_roles(r1[..., None]))
            mask = lc.generate_mask(1)
            o1 = torch.nn.functional.scaled_dot_product_attention(
                q1, keys.repeat_interleave(n_rep, 1), values.repeat_interleave(n_rep, 1), attn_mask=mask.repeat_interleave(n_rep, 1))
            fill_before = lc.chunk_fill_size
            lc.post_update(1)
            dec_out.append(o1.numpy().copy())
            if fill_before == TOK_UPDATE and lc.chunk_fill_size == 0:
                j = len(upd_steps)
                upd_steps.append(si)
                sg, sl = lc.size_global_kv.numpy().copy(), lc.size_local_kv.numpy().copy()
                n_ctx = int(lc.n_ctx_data)
                out[f'u{j}_size_global'], out[f'u{j}_size_local'], out[f'u{j}_n_ctx_data'] = sg, sl, np.int64(n_ctx)
                out[f'u{j}_cache_k'] = lc.cache_k[:, :, :n_ctx].numpy().copy()
                out[f'u{j}_cache_v'] = lc.cache_v[:, :, :n_ctx].numpy().copy()
                out[f'u{j}_valid'] = lc.valid_tokens[:, :, :n_ctx].numpy().copy()
        out['update_steps'] = np.array(upd_steps)
        out['dec_out'] = np.stack(dec_out)
        out['dec_roles'] = np.stack([s[3] for s in steps])
        out['dec_checksum'] = np.array([checksum(*s[:3]) for s in steps])
    return out


def role_inputs(case: dict):
    """Hidden states [B, x_len, dim] of every call of a role-sampling case, regenerated from its seed."""
    g = torch.Generator().manual_seed(case['seed'])
    dim = case['Hq'] * case['D']
    return [torch.randn(case['B'], n, dim, generator=g) for n in case['calls']]


def run_role_case(name: str, case: dict, NAtSCache, Layer) -> dict:
    """Drives the reference layer's own forward hooks call by call (prepare_x_values, whose
    ``_sample_for_token_info_values_inference`` makes the roles; prepare_kv and multi_head_attention so that the cache's
    fill state advances as in a real run) and stores the one-hot roles each call produced."""
    B, Hq, Hkv, D, C, SW = (case[x] for x in ('B', 'Hq', 'Hkv', 'D', 'C', 'SW'))
    torch.manual_seed(case['seed'])
    layer = Layer(dim=Hq * D, n_heads=Hq, n_kv_heads=Hkv, layer_id=0, local_seq_max_length=SW, chunk_size=C,
                  chunk_merge_method=case['method'])
    layer.eval()
    layer.global_token_enhanced_value = case['enh']
    cache = NAtSCache(sliding_window_size=SW, chunk_size=C)
    xs = role_inputs(case)
    out = {'proj_weight': layer.proj_layer.weight.detach().numpy().copy(), 'in_checksum': checksum(*xs)}
    pos = 0
    with torch.no_grad():
        for i, x in enumerate(xs):
            x_len = x.shape[1]
            out[f'c{i}_pre_fill'] = np.int64(cache.get_nats_chunk_fill_size(0))
            out[f'c{i}_start_pos'] = np.int64(pos)
            xq, xk, xv, info = layer.prepare_x_values(x, B, x_len, None, start_pos=pos, cache=cache)
            tsi = info['token_states_info']
            assert bool(((tsi == 0) | (tsi == 1)).all()) and bool((tsi.sum(-1) == 1).all())
            out[f'c{i}_info'] = tsi.numpy().astype(np.uint8)           # one-hot [B, Hkv, chunks, 3]
            keys, values = layer.prepare_kv(xq, xk, xv, pos, cache=cache, kwargs=info)
            keys, values = layer.repeat_kv_values(keys, values)
            layer.multi_head_attention(xq, keys, values, cache=cache, kwargs=info)
            pos += x_len
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--reference', required=True)
    ap.add_argument('--only', default='', help='comma-separated case names (default: all)')
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(HERE, '..', '..'))
    NAtSCache, Layer = load_reference(args.reference)
    only = set(filter(None, args.only.split(',')))
    every = list(CASES.items()) + list(SEG_CASES.items()) + list(TOK_CASES.items()) + list(TOKDEC_CASES.items()) + \
        list(ROLE_CASES.items())
    for name, case in every:
        if only and name not in only:
            continue
        if name in TOK_CASES:
            res = run_token_case(name, case)
        elif name in TOKDEC_CASES:
            res = run_token_decode_case(name, case)
        elif name in ROLE_CASES:
            res = run_role_case(name, case, NAtSCache, Layer)
        else:
            res = (run_segmented_case if name in SEG_CASES else run_case)(name, case, NAtSCache, Layer)
        path = os.path.join(HERE, name + '.npz')
        np.savez_compressed(path, **res)
        print(f'{name}: {os.path.getsize(path) / 1024:.1f} KiB')


if __name__ == '__main__':
    main()
