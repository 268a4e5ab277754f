"""The allocation-free prefill entry point (scratch inside the library) against the regular one.

Some callers cannot give the library a workspace because they may not allocate device memory at all (a serving loop
that must stay off the allocator, a process whose memory pool belongs to another framework).  For them
``nats_b200_prefill_fwd_static`` keeps its role metadata in a 1 MiB array that is part of the library image.  This test
calls it through the C-ABI twice in a row -- the second call with different roles, so stale metadata from the first
would show -- and expects exactly the output of ``nats_b200_prefill_fwd``: both run the same kernels on the same
metadata, so the bar is equality, tighter than the 2e-2 / 1e-2 bars of the parity tests.
This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _roles(B, H, nc, seed):
    g = torch.Generator().manual_seed(seed)
    r = (torch.randn(B, H, nc, 3, generator=g) + torch.tensor([-1.0, 0.0, 0.6])).argmax(-1).to(torch.uint8)
    r[..., 0] = 0
    return r


def test_static_scratch_prefill_equals_regular_prefill_twice():
    from neuralattentionsearch_b200 import _lib, check_status, prefill_attention
    from neuralattentionsearch_b200.functional import status_word
    dev = torch.device('cuda', 0)
    lib = _lib.lib()
    assert lib.nats_b200_prefill_static_scratch_bytes() == 1 << 20
    B, Hq, Hkv, N, D, C, SW = 2, 8, 2, 1000, 128, 8, 64
    g = torch.Generator().manual_seed(0)
    q = (torch.randn(B, Hq, N, D, generator=g) * 0.5).to(dev).bfloat16()
    k = (torch.randn(B, Hkv, N, D, generator=g) * 0.5).to(dev).bfloat16()
    v = (torch.randn(B, Hkv, N, D, generator=g) * 0.5).to(dev).bfloat16()
    nc = -(-N // C)
    # everything the calls touch exists before the memory reading is taken: inputs, outputs, references
    cases = []
    for seed in (1, 2):
        roles = _roles(B, Hkv, nc, seed).to(dev)
        kept_ref = torch.zeros(B, Hkv, dtype=torch.int64, device=dev)
        ref = prefill_attention(q, k, v, roles, C, SW, kept_tiles=kept_ref)
        cases.append((seed, roles, ref, kept_ref, torch.full_like(q, float('nan')), torch.zeros(B, Hkv, dtype=torch.int64, device=dev)))
    status = status_word(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def static_call(roles, o, kept):
        _lib.call('nats_b200_prefill_fwd_static', q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), roles.data_ptr(),
                  B, Hq, Hkv, N, D, C, SW, D ** -0.5, kept.data_ptr(), status.data_ptr(), stream)

    warm = torch.empty_like(q)
    static_call(cases[0][1], warm, torch.zeros(B, Hkv, dtype=torch.int64, device=dev))     # the first call looks up the scratch address
    torch.cuda.synchronize()
    for seed, roles, ref, kept_ref, o, kept in cases:
        free_before = torch.cuda.mem_get_info(dev)[0]
        static_call(roles, o, kept)
        torch.cuda.synchronize()
        # the call allocated nothing on the device, neither from the driver nor through torch
        assert torch.cuda.mem_get_info(dev)[0] == free_before
        check_status(dev)
        assert torch.equal(o, ref), f'seed {seed}: max diff {(o.float() - ref.float()).abs().max().item()}'
        assert torch.equal(kept, kept_ref)


def test_static_scratch_rejects_shapes_beyond_its_size():
    from neuralattentionsearch_b200 import _lib
    dev = torch.device('cuda', 0)
    lib = _lib.lib()
    one = torch.zeros(64, dtype=torch.uint8, device=dev)
    p = one.data_ptr()
    # 64 x 8 heads x 32768 tokens, chunk 16: 64*8*(2048+512)*4 bytes = 5 MiB of metadata > 1 MiB
    rc = lib.nats_b200_prefill_fwd_static(p, p, p, p, p, 64, 32, 8, 32768, 128, 16, 1024, 0.088, None, p, None)
    assert rc == 4
    msg = lib.nats_b200_last_error().decode()
    assert 'built-in scratch' in msg and 'nats_b200_prefill_fwd' in msg
