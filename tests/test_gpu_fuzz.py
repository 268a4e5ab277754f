"""Seeded random walks through the whole protocol -- first call, multi-token calls, single-token steps in any order, random
shapes and role mixes -- on the GPU cache next to the CPU oracle: outputs within the bf16 tolerance at every call, cache
state bit-exact after every call."""
import numpy as np
import pytest
import torch

from oracle import nats_oracle as orc
from test_gpu_parity import assert_close_attn, bf16_round, compare_cache, dev

pytestmark = pytest.mark.gpu


def random_case(seed):
    rng = np.random.default_rng(seed)
    D = int(rng.choice([64, 128]))
    C = int(rng.choice([1, 4, 8, 16, 32, 64, 128]))
    SW = C * int(rng.choice([1, 2, 4, 8]))
    Hkv = int(rng.choice([1, 2, 3]))
    nrep = int(rng.choice([1, 2, 4, 8] if D == 128 else [1, 2, 4]))
    B = int(rng.choice([1, 2]))
    if B * Hkv == 1:
        B = 2
    mix = [(0.1, 0.3), (0.02, 0.1), (0.3, 0.3), (0.0, 0.5), (0.5, 0.0), (0.0, 0.0)][int(rng.integers(0, 6))]
    calls = [int(rng.integers(max(C, 2), 700))]                       # the first call completes at least one chunk
    for _ in range(int(rng.integers(2, 7))):
        kind = rng.integers(0, 3)
        if kind == 0:
            calls += [1] * int(rng.integers(1, 2 * C + 3))
        elif kind == 1:
            calls.append(int(rng.integers(2, 400)))
        else:
            calls.append(int(rng.integers(2, max(3, C))))          # a call that may complete no chunk
    return dict(B=B, Hq=Hkv * nrep, Hkv=Hkv, D=D, C=C, SW=SW, mix=mix, calls=calls, seed=seed)


@pytest.mark.parametrize('seed', list(range(100, 140)) + [1009])      # 1009: every chunk of a later call local
def test_random_walk_matches_oracle(seed):
    from neuralattentionsearch_b200 import check_status, prefill_attention
    from neuralattentionsearch_b200.cache import NAtSChunkLayerCache
    c = random_case(seed)
    B, Hq, Hkv, D, C, SW = (c[x] for x in ('B', 'Hq', 'Hkv', 'D', 'C', 'SW'))
    N = sum(c['calls'])
    g = torch.Generator().manual_seed(seed)
    q, k, v = (bf16_round(torch.randn(B, h, N, D, generator=g)) for h in (Hq, Hkv, Hkv))
    roles = orc.make_roles(B, Hkv, -(-N // C), max(c['mix'][0], 1e-3), max(c['mix'][1], 1e-3), seed, force_first_global=True)
    if c['mix'][0] == 0.0:
        roles[..., 1:][roles[..., 1:] == 0] = 2
    if c['mix'][1] == 0.0:
        roles[roles == 1] = 2
    lc = NAtSChunkLayerCache(B, Hkv, SW, chunk_size=C, device=dev(), headroom=32)
    st = orc.ChunkCacheOracle(B, Hkv, SW, C)
    pos = 0
    for ci, n in enumerate(c['calls']):
        fill = st.chunk_fill
        if fill + n < C:
            r = np.zeros((B, Hkv, 1), np.uint8)
        else:
            r = roles[..., (pos - fill) // C:-(-(pos + n) // C)].copy()
            if (pos + n) % C:
                r[..., -1] = 0
        qs, ks, vs = (t[:, :, pos:pos + n].contiguous() for t in (q, k, v))
        info = orc.onehot_from_roles(r).to(dev())
        qd, kd, vd = (t.to(dev()).bfloat16() for t in (qs, ks, vs))
        st.update(ks.numpy(), vs.numpy(), r)
        if ci == 0:
            ref = orc.prefill_attention(qs, ks, vs, r, C, SW)
            keys, values = lc.update(kd, vd, info)
            o = prefill_attention(qd, keys, values, torch.from_numpy(r).to(dev()), C, SW)
        elif n == 1:
            ref = orc.decode_attention(qs, st.cache_k, st.cache_v, st.decode_mask())
            lc.update(kd, vd, info, fused=True)
            o = lc.decode_attention(qd)
        else:
            ref = st.prefill_attention_past(qs, n)
            lc.update(kd, vd, info)
            o = lc.prefill_attention(qd)
        st.post_update(n)
        lc.post_update(n)
        check_status(dev())
        assert_close_attn(o, ref, f'{c}: call {ci} ({n} tokens at {pos})')
        compare_cache(lc, st)
        pos += n


@pytest.mark.parametrize('seed', range(300, 330))
def test_random_first_call_shapes(seed):
    """Random shapes of a first call: sequence lengths that are no multiple of anything, every group size up to 8, both
    head dims, chunk sizes from 1 to 256 with windows of 1 to 8 chunks, random role mixes: outputs, kept-tile counts and the
    backward statistics against the oracle."""
    from neuralattentionsearch_b200 import check_status
    from neuralattentionsearch_b200.functional import nats_chunk_attention_fwd
    rng = np.random.default_rng(seed)
    D = int(rng.choice([64, 128]))
    C = int(rng.choice([1, 2, 8, 16, 32, 64, 128, 256]))
    SW = C * int(rng.choice([1, 2, 4, 8]))
    Hkv = int(rng.choice([1, 2]))
    nrep = int(rng.integers(1, 9))
    B = int(rng.choice([1, 2]))
    N = int(rng.integers(1, 1500))
    pg, pl = [(0.1, 0.3), (0.02, 0.1), (0.3, 0.3), (0.6, 0.2), (0.001, 0.001)][int(rng.integers(0, 5))]
    roles = orc.make_roles(B, Hkv, -(-N // C), pg, pl, seed)
    g = torch.Generator().manual_seed(seed)
    q, k, v = (bf16_round(torch.randn(B, h, N, D, generator=g)) for h in (Hkv * nrep, Hkv, Hkv))
    qd, kd, vd = (t.to(dev()).bfloat16() for t in (q, k, v))
    o, lse, cnt = nats_chunk_attention_fwd(qd, kd, vd, orc.onehot_from_roles(roles).to(dev()), None, True, D ** -0.5, C,
                                           n_rep=nrep, local_seq_max_length=SW)
    check_status(dev())
    what = f'B{B} Hq{Hkv * nrep} Hkv{Hkv} N{N} D{D} C{C} SW{SW}'
    assert_close_attn(o, orc.prefill_attention(q, k, v, roles, C, SW), what)
    lse_ref, cnt_ref = orc.prefill_stats(q, k, roles, C, SW)
    assert np.array_equal(cnt.cpu().numpy(), cnt_ref), what
    assert (lse.cpu() - lse_ref).abs().max().item() < 2e-2, what
