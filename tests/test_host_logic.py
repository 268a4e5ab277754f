"""Host-side logic that needs no GPU: sharding, role conversion, the pooled hidden-state buffer of the cache."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from neuralattentionsearch_b200 import functional as F_
from neuralattentionsearch_b200.cache import NAtSCache
from neuralattentionsearch_b200.sharding import pairs_per_rank, shard_pairs
from oracle import nats_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize('B,H,W', [(1, 8, 1), (1, 8, 2), (1, 8, 8), (64, 8, 8), (2, 8, 4), (3, 5, 4), (1, 2, 8)])
def test_shards_partition_all_pairs(B, H, W):
    seen = []
    for r in range(W):
        for b, h0, h1 in shard_pairs(B, H, W, r):
            assert 0 <= h0 < h1 <= H
            seen += [(b, h) for h in range(h0, h1)]
    assert seen == [(b, h) for b in range(B) for h in range(H)]
    sizes = pairs_per_rank(B, H, W)
    assert max(sizes) - min(sizes) <= 1 and sum(sizes) == B * H


def test_roles_from_end_seqs_matches_oracle_fill():
    roles = orc.make_roles(2, 3, 40, 0.1, 0.3, seed=4)
    fill = torch.from_numpy(orc.next_global_index(roles))
    sliding = torch.from_numpy((roles == 2).astype(np.float32))
    got = F_.roles_from_end_seqs(fill, sliding).numpy()
    # the last chunk counts as global for the next-global index; everything else must round-trip
    exp = roles.copy()
    last = exp[..., -1]
    last[last == 1] = 0
    assert np.array_equal(got, exp)
    onehot = orc.onehot_from_roles(roles)
    assert np.array_equal(F_.roles_from_token_states_info(onehot).numpy(), roles)


@pytest.mark.parametrize('method', ['mean', 'max'])
def test_pooled_hidden_state_buffer(method):
    """Feeding x in arbitrary pieces gives the same per-chunk pooled states as pooling the whole sequence."""
    torch.manual_seed(0)
    C, T, dim = 8, 53, 6
    x = torch.randn(2, T, dim, dtype=torch.float64)
    full = torch.nn.functional.pad(x, (0, 0, 0, (-T) % C)).unflatten(1, (-1, C))
    ref = full.mean(2) if method == 'mean' else None
    if method == 'max':
        xm = torch.nn.functional.pad(x, (0, 0, 0, (-T) % C), value=float('-inf')).unflatten(1, (-1, C))
        ref = xm.max(2)[0]

    class FakeLayer:
        chunk_fill_size = 0
    cache = NAtSCache(sliding_window_size=16, chunk_size=C)
    cache.cache_model = [FakeLayer()]
    pooled = []
    pos = 0
    for piece in (11, 1, 1, 3, 1, 20, 1, 1, 1, 13):
        xs = x[:, pos:pos + piece]
        pre = cache.get_nats_chunk_fill_size(0)
        if pre + piece < C:
            cache.update_nats_cached_x_in_chunk(xs, 0, method)
        else:
            out, pad = cache.update_nats_cached_x_across_chunk(xs, pre, 0, method)
            n_done = (pre + piece) // C
            pooled.append(out[:, :n_done])
        cache.cache_model[0].chunk_fill_size = (pre + piece) % C
        pos += piece
    assert pos == T
    got = torch.cat(pooled, 1)
    n = got.shape[1]
    if method == 'mean':
        torch.testing.assert_close(got, ref[:, :n], rtol=1e-12, atol=1e-12)
    else:
        # an unfinished chunk pooled with zero padding can differ from a -inf padded max only in the last chunk
        torch.testing.assert_close(got[:, :T // C], ref[:, :T // C], rtol=0, atol=0)


def test_two_rank_gloo_shards_cover_the_job(tmp_path):
    """world_size-2 run on CPU: each rank takes its shard, the gathered pair lists form the whole job."""
    code = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["NATS_ROOT"])
from neuralattentionsearch_b200.sharding import shard_pairs
dist.init_process_group("gloo")
r, w = dist.get_rank(), dist.get_world_size()
mine = [(b, h) for b, h0, h1 in shard_pairs(3, 8, w, r) for h in range(h0, h1)]
t = torch.zeros(24, dtype=torch.int64)
for b, h in mine:
    t[b * 8 + h] += 1
dist.all_reduce(t)
assert bool((t == 1).all()), t
out = [None] * w
dist.all_gather_object(out, len(mine))
if r == 0:
    print("PAIRS", out)
dist.destroy_process_group()
'''
    script = tmp_path / 'rank_main.py'
    script.write_text(code)
    env = dict(os.environ, NATS_ROOT=ROOT, MASTER_ADDR='127.0.0.1')
    res = subprocess.run([sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node=2',
                          '--master-addr', '127.0.0.1', '--master-port', '29731', str(script)],
                         capture_output=True, text=True, env=env, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    assert 'PAIRS [12, 12]' in res.stdout


def test_hf_patch_attaches_role_heads_and_samples_roles():
    """The Hugging Face caller on CPU as far as it goes without kernels: module attributes, the attention-implementation
    name that keeps the model from building a dense mask, and the role decisions incl. the pooled-x carry across calls."""
    from transformers import LlamaConfig, LlamaForCausalLM
    from neuralattentionsearch_b200 import NAtSCache
    from neuralattentionsearch_b200.hf import (ATTN_IMPLEMENTATION, TransformerArgs, enable_llama_nats_chunk_eval,
                                               sample_token_states_info)
    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=16, vocab_size=100)
    model = LlamaForCausalLM(cfg).eval()
    enable_llama_nats_chunk_eval(model, TransformerArgs(n_msks=2, chunk_size=4, local_seq_max_length=8))
    assert model.config._attn_implementation == ATTN_IMPLEMENTATION
    att = model.model.layers[1].self_attn
    assert att.proj_layer.weight.shape == (2 * 3, 64) and att.chunk_size == 4 and att.local_seq_max_length == 8
    assert 'model.layers.1.self_attn.proj_layer.weight' in model.state_dict()
    cache = NAtSCache(8, 4)
    x = torch.randn(2, 10, 64)
    info = sample_token_states_info(att, x, cache, start_pos=0)
    assert info.shape == (2, 2, 3, 3) and (info.sum(-1) == 1).all()
    assert (info[:, :, 0, 0] == 1).all() and (info[:, :, -1, 0] == 1).all()       # sink chunk, unfinished chunk
    pooled = x[:, 4:8].mean(1)
    want = att.proj_layer(pooled).view(2, 2, 3).argmax(-1)
    assert torch.equal(info[:, :, 1].argmax(-1), want)
    with pytest.raises(TypeError):
        att(hidden_states=x, position_embeddings=(x, x), past_key_values=None)
