"""Multi-token calls over an existing compacted cache (segmented prefill) on the GPU, through the C-ABI.

Checked against the CPU oracle segment by segment (role metadata and cache state bit-exact, outputs within the bf16
tolerance), against the fixtures made from the reference's eager path, and through the identity that defines the
operation: the outputs and the final cache of a segmented run equal those of one call over the whole sequence.
"""
import numpy as np
import pytest
import torch

from golden_util import ROW_STRIDE, SEG_CASES, load, segment_roles
from oracle import nats_oracle as orc
from test_gpu_parity import assert_close_attn, bf16_round, compare_cache, dev, make_steps

pytestmark = pytest.mark.gpu

NO_LIMIT_GPU = 2 ** 31 - 1


def run_segments(case, roles, q, k, v, on_segment=None):
    """Feeds the sequence in the case's segments to the GPU cache and to the oracle side by side."""
    from neuralattentionsearch_b200 import functional as F_
    from neuralattentionsearch_b200.cache import NAtSChunkLayerCache
    B, Hkv, SW, C = case['B'], case['Hkv'], case['SW'], case['C']
    lc = NAtSChunkLayerCache(B, Hkv, SW, chunk_size=C, device=dev(), headroom=64)
    st = orc.ChunkCacheOracle(B, Hkv, SW, C)
    pos = 0
    outs = []
    attn = case['D'] >= 64            # the attention kernel is built for head_dim 64 / 128; smaller cases check the rest
    for si, x_len in enumerate(case['segs']):
        r = segment_roles(case, roles, pos, st.chunk_fill, x_len)
        qs, ks, vs = (t[:, :, pos:pos + x_len].contiguous() for t in (q, k, v))
        st.update(ks.numpy(), vs.numpy(), r)
        info = orc.onehot_from_roles(r).to(dev())
        keys, values = lc.update(ks.to(dev()).bfloat16(), vs.to(dev()).bfloat16(), info)
        if si == 0:
            ref = orc.prefill_attention(qs, ks, vs, r, C, SW)
            o = F_.prefill_attention(qs.to(dev()).bfloat16(), keys, values, torch.from_numpy(r).to(dev()), C, SW) if attn else ref
            mask_ref = mask = None
        else:
            ref = st.prefill_attention_past(qs, x_len)
            mask_ref = st.prefill_mask_past(x_len)
            # role metadata of the call: bit-exact against the oracle's row limits over the physical layout
            n_ctx = lc.n_ctx_data
            t0 = n_ctx // C * C
            lim = F_.layout_row_limits(lc._roles, lc._buf_valid, lc.size_global_kv, lc.size_local_kv, x_len, t0, n_ctx - t0,
                                       lc.sliding_queue_tail, C, SW).cpu().numpy().astype(np.int64)
            lim_ref = np.minimum(st.layout_row_limit(), NO_LIMIT_GPU)
            assert np.array_equal(lim, lim_ref), f'segment {si}: row limits'
            mask = lc.generate_mask(x_len).cpu().numpy()
            assert np.array_equal(mask, mask_ref), f'segment {si}: mask'
            assert keys.shape[2] == st.n_ctx_data + x_len
            o = lc.prefill_attention(qs.to(dev()).bfloat16()) if attn else ref
        st.post_update(x_len)
        lc.post_update(x_len)
        from neuralattentionsearch_b200 import check_status
        check_status(dev())
        assert_close_attn(o, ref, f'segment {si}')
        compare_cache(lc, st)
        outs.append(o.float().cpu())
        if on_segment is not None:
            on_segment(si, lc, st, mask, o)
        pos += x_len
    return lc, st, torch.cat(outs, 2)


@pytest.mark.parametrize('name', list(SEG_CASES))
def test_segmented_prefill_matches_oracle_and_fixture(name):
    case, fx, (q, k, v, steps) = load(name)
    q, k, v = bf16_round(q), bf16_round(k), bf16_round(v)
    tiny = case['D'] < 64

    def check(si, lc, st, mask, o):
        # the fixture was made from unrounded fp32 inputs: looser output tolerance, exact masks and index-level state
        if mask is not None:
            cols = int(fx[f's{si}_mask_cols'])
            ref_mask = np.unpackbits(fx[f's{si}_mask'], axis=-1)[..., :cols].astype(bool)
            assert np.array_equal(mask if tiny else mask[:, :, ::ROW_STRIDE], ref_mask), f'segment {si}'
        got = o.float().cpu() if tiny else o.float().cpu()[:, :, ::ROW_STRIDE]
        err = (got - torch.from_numpy(fx[f's{si}_out'])).abs()
        assert err.max().item() <= 4e-2 and err.mean().item() <= 2e-2 * np.abs(fx[f's{si}_out']).mean() + 1e-3, f'segment {si}'
        assert np.array_equal(lc.size_global_kv.cpu().numpy(), fx[f's{si}_size_global'])
        assert np.array_equal(lc.size_local_kv.cpu().numpy(), fx[f's{si}_size_local'])
        assert lc.n_ctx_data == int(fx[f's{si}_n_ctx_data'])
        assert lc.sliding_queue_tail == int(fx[f's{si}_tail'])
        assert lc.chunk_fill_size == int(fx[f's{si}_chunk_fill'])

    lc, st, _ = run_segments(case, fx['roles'], q, k, v, check)
    # decode steps on top of the segmented cache
    C = case['C']
    for i, (q1, k1, v1, r1) in enumerate(steps if not tiny else []):
        q1, k1, v1 = bf16_round(q1), bf16_round(k1), bf16_round(v1)
        done = st.chunk_fill + 1 == C
        role_now = (r1 if done else np.zeros_like(r1))[..., None]
        st.update(k1.numpy(), v1.numpy(), role_now)
        ref = orc.decode_attention(q1, st.cache_k, st.cache_v, st.decode_mask())
        st.post_update(1)
        lc.update(k1.to(dev()).bfloat16(), v1.to(dev()).bfloat16(), orc.onehot_from_roles(role_now).to(dev()), fused=True)
        o = lc.decode_attention(q1.to(dev()).bfloat16())
        lc.post_update(1)
        assert_close_attn(o, ref, f'decode step {i}')
        assert np.array_equal(np.stack([lc.size_global_kv.cpu().numpy(), lc.size_local_kv.cpu().numpy()]), fx['dec_sizes'][i])
    if steps and not tiny:
        compare_cache(lc, st)


SEG_SHAPES = [
    # B, Hq, Hkv, D, C, SW, segments, pg, pl, seed
    (1, 8, 2, 128, 128, 1024, [4096, 2048, 2048], 0.05, 0.15, 31),
    (2, 4, 2, 64, 64, 256, [1000, 1500, 300, 777], 0.10, 0.30, 32),           # nothing aligned to chunks or tiles
    (1, 4, 4, 128, 16, 64, [640, 130, 7, 3, 1200], 0.10, 0.30, 33),           # calls that complete no chunk
    (1, 6, 2, 128, 32, 128, [96, 2000], 0.02, 0.10, 34),                      # first call shorter than the window
    (1, 4, 1, 128, 128, 512, [2048, 2048], 0.0, 0.3, 35),                     # no global chunk after the first
    (2, 2, 2, 64, 1, 16, [300, 212], 0.10, 0.30, 36),                         # token-granular roles
]


@pytest.mark.parametrize('B,Hq,Hkv,D,C,SW,segs,pg,pl,seed', SEG_SHAPES)
def test_segmented_equals_one_shot(B, Hq, Hkv, D, C, SW, segs, pg, pl, seed):
    """Size-independent property: segment by segment == one call, for the outputs (bf16 tolerance, both computed by the
    CUDA path, and the oracle on sampled rows) and for the compacted cache (bit-exact)."""
    from neuralattentionsearch_b200 import functional as F_
    from neuralattentionsearch_b200.cache import NAtSChunkLayerCache
    N = sum(segs)
    case = dict(B=B, Hq=Hq, Hkv=Hkv, D=D, C=C, SW=SW, segs=segs, N=N)
    g = torch.Generator().manual_seed(seed)
    q, k, v = (bf16_round(torch.randn(B, h, N, D, generator=g)) for h in (Hq, Hkv, Hkv))
    roles = orc.make_roles(B, Hkv, -(-N // C), max(pg, 1e-3), pl, seed, force_first_global=True)
    if pg == 0.0:
        roles[..., 1:][roles[..., 1:] == 0] = 2
    lc, st, out_seg = run_segments(case, roles, q, k, v)
    one_roles = roles.copy()
    if N % C:
        one_roles[..., -1] = 0
    qd, kd, vd = (t.to(dev()).bfloat16() for t in (q, k, v))
    out_one = F_.prefill_attention(qd, kd, vd, torch.from_numpy(one_roles).to(dev()), C, SW)
    assert_close_attn(out_seg, out_one, 'segmented vs one call')
    lc1 = NAtSChunkLayerCache(B, Hkv, SW, chunk_size=C, device=dev(), headroom=64)
    lc1.update(kd, vd, orc.onehot_from_roles(one_roles).to(dev()))
    lc1.post_update(N)
    torch.cuda.synchronize()
    assert torch.equal(lc.size_global_kv, lc1.size_global_kv) and torch.equal(lc.size_local_kv, lc1.size_local_kv)
    assert (lc.n_ctx_data, lc.chunk_fill_size) == (lc1.n_ctx_data, lc1.chunk_fill_size)
    n = lc.n_ctx_data
    # the ring is a circular queue: where its newest chunk sits depends on the call history, its content in queue order not
    shift = lc1.sliding_queue_tail - lc.sliding_queue_tail

    def aligned(t):
        return torch.cat([torch.roll(t[:, :, :SW], shifts=shift, dims=2), t[:, :, SW:n]], 2)

    assert torch.equal(aligned(lc.valid_tokens), lc1.valid_tokens[:, :, :n])
    assert torch.equal(aligned(lc.cache_k), lc1.cache_k[:, :, :n]) and torch.equal(aligned(lc.cache_v), lc1.cache_v[:, :, :n])


def test_segmented_prefill_at_benchmark_size():
    """The 32k-token benchmark shape fed as two 16k segments: outputs against one call of the kernel over all 32k tokens
    and, on rows of several query tiles of the second segment, against the blocked fp32 oracle; same compacted cache."""
    import bench
    from neuralattentionsearch_b200 import check_status, prefill_attention
    from neuralattentionsearch_b200.cache import NAtSChunkLayerCache
    w = dict(bench.WORKLOAD)
    B, Hq, Hkv, D, C, SW, N = w['B'], w['Hq'], w['Hkv'], w['D'], w['C'], w['SW'], w['N']
    q, k, v, roles = bench.make_prefill_inputs(w, 123)
    qd, kd, vd, rd = (t.to(dev()) for t in (q, k, v, roles))
    one = prefill_attention(qd, kd, vd, rd, C, SW)
    lc1 = NAtSChunkLayerCache(B, Hkv, SW, chunk_size=C, device=dev())
    lc1.update(kd, vd, rd)
    lc1.post_update(N)
    half, hc = N // 2, N // 2 // C
    lc = NAtSChunkLayerCache(B, Hkv, SW, chunk_size=C, device=dev())
    keys, values = lc.update(kd[:, :, :half].contiguous(), vd[:, :, :half].contiguous(), rd[..., :hc].contiguous())
    o_a = prefill_attention(qd[:, :, :half].contiguous(), keys, values, rd[..., :hc].contiguous(), C, SW)
    lc.post_update(half)
    lc.update(kd[:, :, half:].contiguous(), vd[:, :, half:].contiguous(), rd[..., hc:].contiguous())
    o_b = lc.prefill_attention(qd[:, :, half:].contiguous())
    lc.post_update(half)
    check_status(dev())
    assert_close_attn(torch.cat([o_a, o_b], 2), one, 'two segments vs one call')
    roles_np = roles.numpy()
    for lo in (half, half + 5000, N - 128):
        ref = orc.prefill_attention(q.float(), k.float(), v.float(), roles_np, C, SW, rows=(lo, lo + 128))
        assert_close_attn(o_b[:, :, lo - half:lo - half + 128], ref, f'rows {lo}..{lo + 128} vs oracle')
    assert torch.equal(lc.size_global_kv, lc1.size_global_kv) and torch.equal(lc.size_local_kv, lc1.size_local_kv)
    n = lc.n_ctx_data
    assert n == lc1.n_ctx_data and lc.sliding_queue_tail == lc1.sliding_queue_tail
    assert torch.equal(lc.cache_k[:, :, :n], lc1.cache_k[:, :, :n]) and torch.equal(lc.cache_v[:, :, :n], lc1.cache_v[:, :, :n])
    assert torch.equal(lc.valid_tokens[:, :, :n], lc1.valid_tokens[:, :, :n])


def test_reference_named_entry_point_with_past():
    """``nats_prefill`` with the past-information arguments of the reference (hf/llama.py:235-252)."""
    from neuralattentionsearch_b200 import nats_prefill
    from neuralattentionsearch_b200.cache import NAtSChunkLayerCache
    B, Hq, Hkv, D, C, SW = 1, 4, 2, 128, 32, 128
    segs = [512, 300]
    N = sum(segs)
    g = torch.Generator().manual_seed(41)
    q, k, v = (bf16_round(torch.randn(B, h, N, D, generator=g)) for h in (Hq, Hkv, Hkv))
    roles = orc.make_roles(B, Hkv, -(-N // C), 0.1, 0.3, 41, force_first_global=True)
    case = dict(B=B, Hq=Hq, Hkv=Hkv, D=D, C=C, SW=SW, segs=segs, N=N)
    lc = NAtSChunkLayerCache(B, Hkv, SW, chunk_size=C, device=dev(), headroom=64)
    st = orc.ChunkCacheOracle(B, Hkv, SW, C)
    r0 = segment_roles(case, roles, 0, 0, segs[0])
    k0, v0 = k[:, :, :segs[0]].contiguous(), v[:, :, :segs[0]].contiguous()
    st.update(k0.numpy(), v0.numpy(), r0)
    st.post_update(segs[0])
    lc.update(k0.to(dev()).bfloat16(), v0.to(dev()).bfloat16(), orc.onehot_from_roles(r0).to(dev()))
    lc.post_update(segs[0])
    r1 = segment_roles(case, roles, segs[0], st.chunk_fill, segs[1])
    q1, k1, v1 = (t[:, :, segs[0]:].contiguous() for t in (q, k, v))
    st.update(k1.numpy(), v1.numpy(), r1)
    ref = st.prefill_attention_past(q1, segs[1])
    n_ctx, tail = lc.n_ctx_data, lc.sliding_queue_tail
    keys, values = lc.update(k1.to(dev()).bfloat16(), v1.to(dev()).bfloat16(), orc.onehot_from_roles(r1).to(dev()))
    end_seqs = torch.from_numpy(orc.next_global_index(r1)).to(dev())
    sliding = torch.from_numpy((r1 == 2).astype(np.float32)).to(dev())
    o, mask = nats_prefill(q1.to(dev()).bfloat16(), keys, values, end_seqs, sliding, D ** -0.5, nats_chunk_size=C,
                           global_kv_size=lc.size_global_kv, local_kv_size=lc.size_local_kv,
                           valid_sw_tokens=lc.valid_tokens[:, :, :SW].contiguous(), n_ctx_data=n_ctx, sw_token_tails=tail,
                           n_rep=Hq // Hkv, local_seq_max_length=SW, return_masks=True)
    assert_close_attn(o, ref, 'nats_prefill with past')
    assert np.array_equal(mask.cpu().numpy(), st.prefill_mask_past(segs[1]))


def test_attention_layer_segmented_forward_equals_one_call():
    """The nn.Module fed in segments (prefill, two multi-token calls, single tokens) gives the outputs of one forward over
    the whole sequence: same pooled role decisions, same attention, same cache sizes."""
    from neuralattentionsearch_b200 import LlamaNAtSChunkAttentionLayer, NAtSCache, check_status
    torch.manual_seed(1)
    dim, Hq, Hkv, C, SW = 512, 4, 2, 16, 64
    segs = [200, 150, 9, 1, 1, 1, 90]
    N = sum(segs)
    layer = LlamaNAtSChunkAttentionLayer(dim=dim, n_heads=Hq, n_kv_heads=Hkv, layer_id=0, local_seq_max_length=SW,
                                         chunk_size=C).to(dev()).bfloat16().eval()
    x = (torch.randn(2, N, dim) * 0.5).to(dev()).bfloat16()
    with torch.no_grad():
        one_cache = NAtSCache(SW, C)
        y_one = layer(x, None, None, start_pos=0, cache=one_cache)
        cache = NAtSCache(SW, C)
        ys, pos = [], 0
        for n in segs:
            ys.append(layer(x[:, pos:pos + n], None, None, start_pos=pos, cache=cache))
            pos += n
        check_status(dev())
    y_seg = torch.cat(ys, 1)
    err = (y_seg.float() - y_one.float()).abs()
    assert err.max().item() < 3e-2 and err.mean().item() < 2e-3, (err.max().item(), err.mean().item())
    a, b = cache.cache_model[0], one_cache.cache_model[0]
    assert torch.equal(a.size_global_kv, b.size_global_kv) and torch.equal(a.size_local_kv, b.size_local_kv)
    assert (a.n_ctx_data, a.chunk_fill_size, a.get_seq_length()) == (b.n_ctx_data, b.chunk_fill_size, N)
