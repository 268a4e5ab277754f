"""The C-ABI library loads and exports every symbol the header declares; argument checks work without a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope='module')
def lib():
    from neuralattentionsearch_b200 import build, _lib
    build.build()
    return _lib.lib()


def _declared():
    text = open(os.path.join(ROOT, 'include', 'nats_b200.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(nats_b200_\w+)\s*\(', text)))


def test_every_declared_symbol_is_exported(lib):
    from neuralattentionsearch_b200 import _lib
    names = _declared()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), name
        assert name in _lib.SIGNATURES, f'{name} has no ctypes signature'
    assert sorted(_lib.SIGNATURES) == names


def test_build_info_and_sizes(lib):
    assert b'sm_100a' in lib.nats_b200_build_info()
    ws = lib.nats_b200_prefill_workspace_bytes(1, 8, 32768, 128)
    assert ws >= 8 * 256 * 4 * 3 and ws % 256 == 0
    assert lib.nats_b200_prefill_workspace_bytes(0, 8, 32768, 128) == 0
    small = lib.nats_b200_decode_workspace_bytes(2, 8, 2, 128, 1000)
    big = lib.nats_b200_decode_workspace_bytes(2, 8, 2, 128, 100000)
    assert 0 < small < big
    assert lib.nats_b200_decode_workspace_bytes(2, 7, 2, 128, 1000) == 0


def test_argument_errors_do_not_need_a_gpu(lib):
    from neuralattentionsearch_b200 import _lib
    rc = lib.nats_b200_prefill_fwd(None, None, None, None, None, 1, 4, 2, 128, 128, 16, 64, 0.1, None, 0, None, None, None)
    assert rc == 1 and b'null' in lib.nats_b200_last_error()
    one = ctypes.c_void_p(256)          # never dereferenced: the checks fail first
    rc = lib.nats_b200_prefill_fwd(one, one, one, one, one, 1, 4, 2, 128, 128, 16, 60, 0.1, one, 1 << 20, None, one, None)
    assert rc == 1 and b'multiple' in lib.nats_b200_last_error()
    rc = lib.nats_b200_prefill_fwd(one, one, one, one, one, 1, 4, 2, 128, 96, 16, 64, 0.1, one, 1 << 20, None, one, None)
    assert rc == 2 and b'head_dim' in lib.nats_b200_last_error()
    rc = lib.nats_b200_prefill_fwd(one, one, one, one, one, 1, 4, 2, 128, 128, 16, 64, 0.1, one, 16, None, one, None)
    assert rc == 4
    rc = lib.nats_b200_evict_plan(one, 1, 2, 128, 16, 40, one, one, one, one, None)
    assert rc == 1
    rc = lib.nats_b200_decode_fwd(one, one, one, one, one, one, one, 1024, one, one, one, 20, 512, 1, 4, 2, 128, 16, 64, 0.1,
                                  one, 1 << 30, None)
    assert rc == 1 and b'fill' in lib.nats_b200_last_error()
    rc = lib.nats_b200_decode_place(one, one, one, one, 1024, one, one, one, 5, 1, 2, 128, 16, 64, None)
    assert rc == 1
    with pytest.raises(_lib.NatsB200Error):
        _lib.call('nats_b200_role_prep', None, 1, 1, 128, 16, 64, None, None, None, None, None)


def test_product_refuses_cpu_tensors():
    import torch
    from neuralattentionsearch_b200 import _lib, prefill_attention
    q = torch.zeros(1, 2, 64, 64)
    roles = torch.zeros(1, 2, 4, dtype=torch.uint8)
    with pytest.raises(_lib.NatsB200Error):
        prefill_attention(q, q, q, roles, 16, 64)


def test_argument_errors_of_the_multi_token_and_helper_entry_points(lib):
    one, two = ctypes.c_void_p(256), ctypes.c_void_p(512)
    err = lambda: lib.nats_b200_last_error()
    # append: rows must fit the capacity
    assert lib.nats_b200_cache_append(one, one, two, two, two, 1, 2, 100, 128, 1000, 950, None) == 1 and b'fit' in err()
    assert lib.nats_b200_cache_append(one, one, two, two, None, 1, 2, 100, 128, 2000, 950, None) == 1 and b'null' in err()
    # role metadata over a cache: tail offset a chunk multiple behind the window, fill inside a chunk, ring tail aligned
    args = dict(B=1, H=2, x=100, C=16, SW=64, stride=4096)
    call = lambda t0, fill, tail: lib.nats_b200_role_prep_past(one, one, one, one, args['B'], args['H'], args['x'], args['C'], args['SW'],
                                                                 args['stride'], t0, fill, tail, one, one, one, None, None)
    assert call(70, 0, 0) == 1 and b'tail offset' in err()
    assert call(32, 0, 0) == 1
    assert call(128, 16, 0) == 1
    assert call(128, 3, 8) == 1 and b'ring tail' in err()
    # attention over a cache: the new tokens must have been appended (capacity), head_dim as for a first call
    rc = lib.nats_b200_prefill_past_fwd(one, one, one, one, one, one, 4096, one, one, 1, 4, 2, 100, 128, 16, 64, 200, 128, 3, 0, 0.1,
                                        one, 1 << 20, None, one, None)
    assert rc == 1 and b'appended' in err()
    rc = lib.nats_b200_prefill_past_fwd(one, one, one, one, one, one, 4096, one, one, 1, 4, 2, 100, 32, 16, 64, 4096, 128, 3, 0, 0.1,
                                        one, 1 << 20, None, one, None)
    assert rc == 2 and b'head_dim' in err()
    assert lib.nats_b200_prefill_past_workspace_bytes(1, 2, 4096, 16) % 256 == 0
    # compaction over a cache is out of place
    rc = lib.nats_b200_evict_compact_past(one, one, one, 4096, one, one, one, one, one, one, 1, 2, 100, 128, 16, 64, 128, 0,
                                          one, one, one, 4096, None)
    assert rc == 1 and b'out of place' in err()
    rc = lib.nats_b200_evict_compact_past(one, one, one, 200, one, one, one, one, one, one, 1, 2, 100, 128, 16, 64, 128, 0,
                                          two, two, two, 4096, None)
    assert rc == 1 and b'capacity' in err()
    # statistics entry point needs both outputs
    rc = lib.nats_b200_prefill_fwd_stats(one, one, one, one, one, 1, 4, 2, 128, 128, 16, 64, 0.1, one, 1 << 20, None, None, one, one, None)
    assert rc == 1 and b'null' in err()
    # rotary embedding + head split: strides must cover a row of heads and keep 16-byte alignment
    rope = lambda sq, D=128: lib.nats_b200_rope_split_heads(one, one, one, sq, 256, 256, one, one, 0, two, two, two, 1, 10, 4, 2, D, None)
    assert rope(100) == 1 and b'stride' in err()
    assert rope(516) == 1
    assert rope(512, D=24) == 1 and b'head_dim' in err()
