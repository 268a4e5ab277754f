"""Role sampling (pooled hidden states -> role head -> argmax -> one-hot) against fixtures the reference's own layer
produced (tests/golden/make_golden.py: ``run_role_case`` drives ``_sample_for_token_info_values_inference`` of
src/nats/models/transformer/attention/nats_chunk_attention.py:64-95 / nats_attention.py:96-109 with the pooled-x buffer
of src/nats/components/cache/dyn_cache.py:115-171).  CPU, fp32, bit-exact: the one-hot tensors must be equal."""
import types

import numpy as np
import pytest
import torch

from golden_util import ROLE_CASES, load_roles
from neuralattentionsearch_b200 import hf
from neuralattentionsearch_b200.attention import LlamaNAtSChunkAttentionLayer
from neuralattentionsearch_b200.cache import NAtSCache


class _FillCache(NAtSCache):
    """The cache's pooled hidden-state buffer with the fill of the unfinished chunk given by the test (on a GPU it comes
    from the layer cache, which the fixtures' K/V-free calls do not advance)."""
    fill = 0

    def get_nats_chunk_fill_size(self, layer_idx: int = 0):
        return self.fill


def _calls(fx):
    i = 0
    while f'c{i}_info' in fx:
        yield i, int(fx[f'c{i}_pre_fill']), int(fx[f'c{i}_start_pos']), fx[f'c{i}_info']
        i += 1


@pytest.mark.parametrize('name', [n for n, c in ROLE_CASES.items() if c['enh'] != 0.0])
def test_attention_module_roles_match_reference(name):
    case, fx, xs = load_roles(name)
    layer = LlamaNAtSChunkAttentionLayer(dim=case['Hq'] * case['D'], n_heads=case['Hq'], n_kv_heads=case['Hkv'],
                                         local_seq_max_length=case['SW'], chunk_size=case['C'],
                                         chunk_merge_method=case['method']).eval()
    assert layer.global_token_enhanced_value == pytest.approx(case['enh'])
    with torch.no_grad():
        layer.proj_layer.weight.copy_(torch.from_numpy(fx['proj_weight']))
        cache = _FillCache(case['SW'], case['C'])
        n_real = 0
        for i, pre, pos, ref in _calls(fx):
            cache.fill = pre
            info = layer._sample_for_token_info_values_inference(xs[i], pos, cache)
            assert tuple(info.shape) == ref.shape, f'call {i}'
            assert np.array_equal(info.numpy(), ref.astype(np.float32)), f'call {i} (fill {pre}, start {pos})'
            n_real += int(pre + xs[i].shape[1] >= case['C'])
    assert n_real >= 8          # the fixture exercises the role head, not only the placeholder


@pytest.mark.parametrize('name', [n for n, c in ROLE_CASES.items() if c['enh'] == 0.0])
def test_hf_forward_roles_match_reference(name):
    """The Hugging Face forward's sampling (no enhancement of the global logit)."""
    case, fx, xs = load_roles(name)
    dim = case['Hq'] * case['D']
    proj = torch.nn.Linear(dim, case['Hkv'] * 3, bias=False)
    with torch.no_grad():
        proj.weight.copy_(torch.from_numpy(fx['proj_weight']))
        module = types.SimpleNamespace(config=types.SimpleNamespace(num_key_value_heads=case['Hkv']), layer_idx=0,
                                       chunk_size=case['C'], chunk_merge_method=case['method'], n_options=3, proj_layer=proj)
        cache = _FillCache(case['SW'], case['C'])
        for i, pre, pos, ref in _calls(fx):
            cache.fill = pre
            info = hf.sample_token_states_info(module, xs[i], cache, pos)
            assert np.array_equal(info.numpy(), ref.astype(np.float32)), f'call {i} (fill {pre}, start {pos})'


def test_role_head_shared_by_several_kv_heads_is_expanded():
    """n_msks < n_kv_heads: every mask head's role is used by the kv-heads it covers (query heads i use mask
    i // (n_heads // n_msks), transformer/utils.py:35-46); a mask head finer than a kv-head is refused."""
    torch.manual_seed(0)
    layer = LlamaNAtSChunkAttentionLayer(dim=64, n_heads=8, n_kv_heads=4, n_msks=2, local_seq_max_length=32, chunk_size=8).eval()
    cache = _FillCache(32, 8)
    with torch.no_grad():
        info = layer._sample_for_token_info_values_inference(torch.randn(2, 64, 64), 0, cache)
    assert tuple(info.shape) == (2, 4, 8, 3)
    assert torch.equal(info[:, 0], info[:, 1]) and torch.equal(info[:, 2], info[:, 3])
    assert bool((info.sum(-1) == 1).all())
    with pytest.raises(ValueError, match='n_msks'):
        LlamaNAtSChunkAttentionLayer(dim=64, n_heads=8, n_kv_heads=2, n_msks=4)
