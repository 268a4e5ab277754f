"""Pins the CPU oracle against the committed outputs of the reference's own eager path (tests/golden)."""
import numpy as np
import pytest
import torch

from golden_util import CASES, ROW_STRIDE, SEG_CASES, TOK_CASES, TOKDEC_CASES, load, segment_roles
from oracle import nats_oracle as orc

TINY = [n for n, c in CASES.items() if c['D'] < 64]
KERNEL = [n for n, c in CASES.items() if c['D'] >= 64]


def _run_oracle_prefill(case, roles, q, k, v):
    st = orc.ChunkCacheOracle(case['B'], case['Hkv'], case['SW'], case['C'])
    st.update(k.numpy(), v.numpy(), roles)
    out = orc.prefill_attention(q, k, v, roles, case['C'], case['SW'])
    st.post_update(case['N'])
    return st, out


def _check_state(st, fx, prefix, full):
    assert np.array_equal(st.size_global, fx[prefix + 'size_global'])
    assert np.array_equal(st.size_local, fx[prefix + 'size_local'])
    assert st.n_ctx_data == int(fx[prefix + 'n_ctx_data'])
    assert st.chunk_fill == int(fx[prefix + 'chunk_fill'])
    assert st.tail == int(fx[prefix + 'tail'])
    assert st.seen == int(fx[prefix + 'seen'])
    assert np.array_equal(st.valid, fx[prefix + 'valid'])
    if full:        # the whole physical cache, stale regions included: the restatement moves data as the reference does
        assert np.array_equal(st.cache_k, fx[prefix + 'cache_k'])
        assert np.array_equal(st.cache_v, fx[prefix + 'cache_v'])


@pytest.mark.parametrize('name', TINY + KERNEL)
def test_prefill_mask_matches_reference(name):
    case, fx, _ = load(name)
    m = orc.visible_mask(fx['roles'], case['C'], case['SW'], case['N'])
    if 'prefill_mask' in fx:
        ref = np.unpackbits(fx['prefill_mask'], axis=-1)[..., :case['N']].astype(bool)
    else:
        ref = np.unpackbits(fx['prefill_mask_rows'], axis=-1)[..., :case['N']].astype(bool)
        m = m[:, :, ::ROW_STRIDE]
    assert np.array_equal(m, ref)


@pytest.mark.parametrize('name', TINY + KERNEL)
def test_prefill_output_and_eviction_match_reference(name):
    case, fx, (q, k, v, _) = load(name)
    st, out = _run_oracle_prefill(case, fx['roles'], q, k, v)
    ref = fx['prefill_out']
    got = out.numpy() if case['D'] < 64 else out[:, :, ::ROW_STRIDE].numpy()
    np.testing.assert_allclose(got, ref, rtol=1e-4, atol=2e-5)
    _check_state(st, fx, 'pre_', full=case['D'] < 64)


@pytest.mark.parametrize('name', [n for n in TINY + KERNEL if CASES[n]['n_decode'] > 0])
def test_decode_steps_match_reference(name):
    case, fx, (q, k, v, steps) = load(name)
    st, _ = _run_oracle_prefill(case, fx['roles'], q, k, v)
    C = case['C']
    for i, (q1, k1, v1, r1) in enumerate(steps):
        done = st.chunk_fill + 1 == C
        role_now = (r1 if done else np.zeros_like(r1))[..., None]
        st.update(k1.numpy(), v1.numpy(), role_now)
        o = orc.decode_attention(q1, st.cache_k, st.cache_v, st.decode_mask())
        st.post_update(1)
        np.testing.assert_allclose(o.numpy(), fx['dec_out'][i], rtol=1e-4, atol=2e-5, err_msg=f'step {i}')
        assert st.n_ctx_data == int(fx['dec_nctx'][i]), f'step {i}'
        assert np.array_equal(np.stack([st.size_global, st.size_local]), fx['dec_sizes'][i]), f'step {i}'
    # final state; the physical cache is compared over the region the reference defines
    _check_state(st, fx, 'post_', full=False)
    if case['D'] < 64:
        n = st.n_ctx_data
        lens = st.lens()
        t0 = n // C * C
        for b in range(case['B']):
            for h in range(case['Hkv']):
                for sl in (slice(0, lens[b, h]), slice(t0, n)):
                    assert np.array_equal(st.cache_k[b, h, sl], fx['post_cache_k'][b, h, sl])
                    assert np.array_equal(st.cache_v[b, h, sl], fx['post_cache_v'][b, h, sl])


def test_kept_tiles_match_dense_mask():
    roles = orc.make_roles(2, 2, 16, 0.1, 0.3, seed=3)
    C, SW, N = 64, 256, 1024
    m = orc.visible_mask(roles, C, SW, N)
    t = m.reshape(2, 2, 8, 128, 8, 128).any((3, 5)).sum((-1, -2))
    assert np.array_equal(t, orc.kept_tiles(roles, C, SW, N, 128))


def test_decode_equals_one_shot_prefill():
    """prefill + eviction + decode over the compacted cache == dense attention under the prefill mask."""
    B, Hq, Hkv, D, C, SW, N0, steps = 2, 4, 2, 16, 8, 32, 64, 48
    g = torch.Generator().manual_seed(0)
    N = N0 + steps
    q = torch.randn(B, Hq, N, D, generator=g, dtype=torch.float64)
    k = torch.randn(B, Hkv, N, D, generator=g, dtype=torch.float64)
    v = torch.randn(B, Hkv, N, D, generator=g, dtype=torch.float64)
    roles = orc.make_roles(B, Hkv, N // C, 0.15, 0.3, seed=5)
    m = torch.from_numpy(orc.visible_mask(roles, C, SW, N))
    sc = torch.einsum('bgrsd,bgld->bgrsl', q.view(B, Hkv, 2, N, D), k) / D ** 0.5
    sc = sc.masked_fill(~m[:, :, None], float('-inf'))
    full = torch.einsum('bgrsl,bgld->bgrsd', torch.softmax(sc, -1), v).reshape(B, Hq, N, D)
    st = orc.ChunkCacheOracle(B, Hkv, SW, C)
    st.update(k[:, :, :N0].numpy(), v[:, :, :N0].numpy(), roles[..., :N0 // C])
    st.post_update(N0)
    for i in range(steps):
        t = N0 + i
        done = st.chunk_fill + 1 == C
        role_now = roles[..., t // C][..., None] if done else np.zeros((B, Hkv, 1), np.uint8)
        st.update(k[:, :, t:t + 1].numpy(), v[:, :, t:t + 1].numpy(), role_now)
        mask = st.decode_mask()
        kk = torch.from_numpy(st.cache_k[:, :, :mask.shape[-1]].copy())
        vv = torch.from_numpy(st.cache_v[:, :, :mask.shape[-1]].copy())
        s1 = torch.einsum('bgrd,bgld->bgrl', q[:, :, t].view(B, Hkv, 2, D), kk) / D ** 0.5
        s1 = s1.masked_fill(~torch.from_numpy(mask)[:, :, None], float('-inf'))
        o = torch.einsum('bgrl,bgld->bgrd', torch.softmax(s1, -1), vv).reshape(B, Hq, D)
        st.post_update(1)
        assert (o - full[:, :, t]).abs().max() < 1e-12, i


# ---- multi-token calls over an existing cache (segmented prefill) ----------------------------------------------------
def run_oracle_segments(case, roles, q, k, v, on_segment=None):
    """Feeds the sequence to the oracle in the case's segments; on_segment(si, state, mask_or_None, out) after each."""
    st = orc.ChunkCacheOracle(case['B'], case['Hkv'], case['SW'], case['C'])
    pos = 0
    for si, x_len in enumerate(case['segs']):
        r = segment_roles(case, roles, pos, st.chunk_fill, x_len)
        qs, ks, vs = (t[:, :, pos:pos + x_len] for t in (q, k, v))
        st.update(ks.numpy(), vs.numpy(), r)
        if si == 0:
            mask = orc.visible_mask(r, case['C'], case['SW'], x_len)
            out = orc.prefill_attention(qs, ks, vs, r, case['C'], case['SW'])
        else:
            mask = st.prefill_mask_past(x_len)
            out = st.prefill_attention_past(qs, x_len)
        st.post_update(x_len)
        if on_segment is not None:
            on_segment(si, st, mask, out)
        pos += x_len
    return st


@pytest.mark.parametrize('name', list(SEG_CASES))
def test_segmented_prefill_matches_reference(name):
    case, fx, (q, k, v, _) = load(name)
    tiny = case['D'] < 64

    def check(si, st, mask, out):
        cols = int(fx[f's{si}_mask_cols'])
        ref_mask = np.unpackbits(fx[f's{si}_mask'], axis=-1)[..., :cols].astype(bool)
        got_mask = mask if tiny else mask[:, :, ::ROW_STRIDE]
        assert got_mask.shape == ref_mask.shape
        assert np.array_equal(got_mask, ref_mask), f'segment {si}'
        got = out.numpy() if tiny else out[:, :, ::ROW_STRIDE].numpy()
        np.testing.assert_allclose(got, fx[f's{si}_out'], rtol=1e-4, atol=2e-5, err_msg=f'segment {si}')
        _check_state(st, fx, f's{si}_', full=tiny)

    run_oracle_segments(case, fx['roles'], q, k, v, check)


@pytest.mark.parametrize('name', list(SEG_CASES))
def test_segmented_prefill_equals_one_shot(name):
    """The identity that defines a multi-token call over a cache: the outputs are those of one call over everything."""
    case, fx, (q, k, v, _) = load(name)
    outs = []
    run_oracle_segments(case, fx['roles'], q, k, v, lambda si, st, m, o: outs.append(o))
    roles = fx['roles'].copy()
    if case['N'] % case['C']:
        roles[..., -1] = 0
    one = orc.prefill_attention(q, k, v, roles, case['C'], case['SW'])
    np.testing.assert_allclose(torch.cat(outs, 2).numpy(), one.numpy(), rtol=1e-4, atol=2e-5)


@pytest.mark.parametrize('name', [n for n, c in SEG_CASES.items() if c['n_decode'] > 0])
def test_decode_after_segments_matches_reference(name):
    case, fx, (q, k, v, steps) = load(name)
    st = run_oracle_segments(case, fx['roles'], q, k, v)
    C = case['C']
    for i, (q1, k1, v1, r1) in enumerate(steps):
        done = st.chunk_fill + 1 == C
        role_now = (r1 if done else np.zeros_like(r1))[..., None]
        st.update(k1.numpy(), v1.numpy(), role_now)
        o = orc.decode_attention(q1, st.cache_k, st.cache_v, st.decode_mask())
        st.post_update(1)
        np.testing.assert_allclose(o.numpy(), fx['dec_out'][i], rtol=1e-4, atol=2e-5, err_msg=f'step {i}')
        assert np.array_equal(np.stack([st.size_global, st.size_local]), fx['dec_sizes'][i]), f'step {i}'
    _check_state(st, fx, 'post_', full=False)


@pytest.mark.parametrize('name', TINY)
def test_visible_key_counts_match_the_reference_mask(name):
    """The per-row key counts the training forward stores are the row sums of the reference's mask."""
    case, fx, (q, k, v, _) = load(name)
    ref = np.unpackbits(fx['prefill_mask'], axis=-1)[..., :case['N']].astype(bool)
    lse, cnt = orc.prefill_stats(q, k, fx['roles'], case['C'], case['SW'])
    n_rep = case['Hq'] // case['Hkv']
    assert np.array_equal(cnt, np.repeat(ref.sum(-1), n_rep, axis=1))
    # log-sum-exp against a direct evaluation with the reference's mask
    s = torch.einsum('bhqd,bhkd->bhqk', q, k.repeat_interleave(n_rep, 1)) / case['D'] ** 0.5
    s = s.masked_fill(~torch.from_numpy(np.repeat(ref, n_rep, axis=1)), float('-inf'))
    np.testing.assert_allclose(lse.numpy(), (torch.logsumexp(s, -1) / np.log(2.0)).numpy(), rtol=1e-5, atol=1e-5)


# ---- token-granular cache (one role per token) ------------------------------------------------------------------------
def check_token_granular_state(case, fx, size_global, size_local, n_ctx_data, valid, cache_k, cache_v, exact=True):
    """Compares a chunk-size-1 cache after the prefill with the reference's token-granular ``NAtSLayerCache``: sizes, extent,
    the kept tokens of every head, and the ring.  The reference's tail points at the slot written last
    (nats_layer_cache.py:424-462), so the token N - SW + i sits in slot (tail + 1 + i) % SW there and in slot i here; it also
    keeps the K/V of tokens that are not sliding ones with their flag cleared, so ring data is compared where valid."""
    SW, N = case['SW'], case['N']
    assert np.array_equal(size_global, fx['pre_size_global']) and np.array_equal(size_local, fx['pre_size_local'])
    assert n_ctx_data == int(fx['pre_n_ctx_data'])
    lens = size_global + size_local
    for b in range(case['B']):
        for h in range(case['Hkv']):
            n = lens[b, h]
            assert np.array_equal(valid[b, h, SW:n], fx['pre_valid'][b, h, SW:n]) and valid[b, h, SW:n].all()
            assert np.array_equal(cache_k[b, h, SW:n], fx['pre_cache_k'][b, h, SW:n])
            assert np.array_equal(cache_v[b, h, SW:n], fx['pre_cache_v'][b, h, SW:n])
    shift = -(int(fx['pre_tail']) + 1)
    ref_ring_valid = np.roll(fx['pre_valid'][:, :, :SW], shift, axis=2)
    assert np.array_equal(valid[:, :, :SW], ref_ring_valid)
    ref_ring_k = np.roll(fx['pre_cache_k'][:, :, :SW], shift, axis=2)
    ref_ring_v = np.roll(fx['pre_cache_v'][:, :, :SW], shift, axis=2)
    on = valid[:, :, :SW].astype(bool)
    assert np.array_equal(cache_k[:, :, :SW][on], ref_ring_k[on]) and np.array_equal(cache_v[:, :, :SW][on], ref_ring_v[on])


@pytest.mark.parametrize('name', list(TOK_CASES))
def test_token_granular_prefill_matches_reference(name):
    case, fx, (q, k, v, _) = load(name)
    tiny = case['D'] < 64
    m = orc.visible_mask(fx['roles'], 1, case['SW'], case['N'])
    ref_mask = np.unpackbits(fx['prefill_mask'], axis=-1)[..., :case['N']].astype(bool)
    assert np.array_equal(m if tiny else m[:, :, ::ROW_STRIDE], ref_mask)
    st, out = _run_oracle_prefill(case, fx['roles'], q, k, v)
    got = out.numpy() if tiny else out[:, :, ::ROW_STRIDE].numpy()
    np.testing.assert_allclose(got, fx['prefill_out'], rtol=1e-4, atol=2e-5)
    check_token_granular_state(case, fx, st.size_global, st.size_local, st.n_ctx_data, st.valid, st.cache_k, st.cache_v)


@pytest.mark.parametrize('name', TINY + KERNEL)
def test_log2_sum_exp2_matches_reference_mask_evaluation(name):
    """M of the training forward: the oracle's statistic against the float64 evaluation over the reference's own mask
    that the fixture stores (inputs rounded to bf16 on both sides)."""
    case, fx, (q, k, v, _) = load(name)
    bf = lambda t: t.bfloat16().float()
    lse, cnt = orc.prefill_stats(bf(q), bf(k), fx['roles'], case['C'], case['SW'])
    ref = fx['prefill_M']
    got = lse.numpy() if case['D'] < 64 else lse[:, :, ::ROW_STRIDE].numpy()
    np.testing.assert_allclose(got, ref, rtol=0, atol=1e-4)
    key = 'prefill_mask' if 'prefill_mask' in fx else 'prefill_mask_rows'
    ref_cnt = np.unpackbits(fx[key], axis=-1)[..., :case['N']].sum(-1).repeat(case['Hq'] // case['Hkv'], axis=1)
    assert np.array_equal(cnt if case['D'] < 64 else cnt[:, :, ::ROW_STRIDE], ref_cnt)


def check_token_granular_update(case, fx, j, size_global, size_local, n_ctx_data, cache_k, cache_v):
    """Index-level state right after the reference's j-th batched update of single tokens: sizes, extent and the kept
    K / V rows of every head (the ring is laid out differently, see check_token_granular_state)."""
    SW = case['SW']
    sg, sl = fx[f'u{j}_size_global'], fx[f'u{j}_size_local']
    assert np.array_equal(size_global, sg) and np.array_equal(size_local, sl), f'update {j}'
    assert n_ctx_data == int(fx[f'u{j}_n_ctx_data']), f'update {j}'
    for b in range(case['B']):
        for h in range(case['Hkv']):
            n = sg[b, h] + sl[b, h]
            assert np.array_equal(cache_k[b, h, SW:n], fx[f'u{j}_cache_k'][b, h, SW:n]), (j, b, h)
            assert np.array_equal(cache_v[b, h, SW:n], fx[f'u{j}_cache_v'][b, h, SW:n]), (j, b, h)


@pytest.mark.parametrize('name', list(TOKDEC_CASES))
def test_token_granular_decode_state_at_reference_update_points(name):
    """Single tokens through the token-granular cache.  The reference (NAtSLayerCache) places them in batches of 16; here
    every token is placed at once.  Right after each of the reference's batched updates the two agree on sizes, extent and
    kept rows, and the next step's output agrees too; in between the reference's outputs drift (tokens waiting for their
    placement stay visible), which is not reproduced."""
    case, fx, (q, k, v, steps) = load(name)
    bf = lambda t: t.bfloat16().float()
    st = orc.ChunkCacheOracle(case['B'], case['Hkv'], case['SW'], 1)
    st.update(bf(k).numpy(), bf(v).numpy(), fx['roles'])
    st.post_update(case['N'])
    ups = fx['update_steps'].tolist()
    assert len(ups) >= 3
    for si, (q1, k1, v1, r1) in enumerate(steps):
        st.update(bf(k1).numpy(), bf(v1).numpy(), r1[..., None])
        o = orc.decode_attention(bf(q1), st.cache_k, st.cache_v, st.decode_mask())
        st.post_update(1)
        if si == 0 or si - 1 in ups:
            np.testing.assert_allclose(o.numpy(), fx['dec_out'][si], rtol=1e-4, atol=2e-5, err_msg=f'step {si}')
        if si in ups:
            check_token_granular_update(case, fx, ups.index(si), st.size_global, st.size_local, st.n_ctx_data,
                                        st.cache_k, st.cache_v)
