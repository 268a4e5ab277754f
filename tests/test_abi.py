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
    rc = lib.nats_b200_prefill_fwd(one, one, one, one, one, 1, 4, 2, 128, 256, 16, 64, 0.1, one, 1 << 20, None, one, None)
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
