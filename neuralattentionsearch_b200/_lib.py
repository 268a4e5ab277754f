"""ctypes binding of libnats_b200.so.  There is no fallback: if the library is missing or a call fails,
an exception is raised."""
from __future__ import annotations

import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get('NATS_B200_LIB') or os.path.join(_HERE, 'libnats_b200.so')   # override: a differently built library

_c = ctypes
_P, _I, _F, _SZ = _c.c_void_p, _c.c_int, _c.c_float, _c.c_size_t

# name -> (restype, argtypes); mirrors include/nats_b200.h
SIGNATURES = {
    'nats_b200_last_error': (_c.c_char_p, []),
    'nats_b200_build_info': (_c.c_char_p, []),
    'nats_b200_role_prep': (_I, [_P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P]),
    'nats_b200_prefill_workspace_bytes': (_SZ, [_I, _I, _I, _I]),
    'nats_b200_prefill_fwd': (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _P, _SZ, _P, _P, _P]),
    'nats_b200_prefill_fwd_stats': (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _P, _SZ, _P, _P, _P, _P, _P]),
    'nats_b200_visible_counts': (_I, [_P, _I, _I, _I, _I, _I, _P, _P]),
    'nats_b200_prefill_static_scratch_bytes': (_SZ, []),
    'nats_b200_prefill_fwd_static': (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _P, _P, _P]),
    'nats_b200_evict_plan': (_I, [_P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P]),
    'nats_b200_evict_compact': (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P, _P, _I, _P]),
    'nats_b200_cache_append': (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    'nats_b200_role_prep_past': (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P]),
    'nats_b200_prefill_past_workspace_bytes': (_SZ, [_I, _I, _I, _I]),
    'nats_b200_prefill_past_fwd': (_I, [_P, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F,
                                        _P, _SZ, _P, _P, _P]),
    'nats_b200_evict_plan_past': (_I, [_P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P]),
    'nats_b200_evict_compact_past': (_I, [_P, _P, _P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I,
                                          _P, _P, _P, _I, _P]),
    'nats_b200_rope_split_heads': (_I, [_P, _P, _P, _c.c_longlong, _c.c_longlong, _c.c_longlong, _P, _P, _c.c_longlong, _P, _P, _P,
                                        _I, _I, _I, _I, _I, _P]),
    'nats_b200_decode_workspace_bytes': (_SZ, [_I, _I, _I, _I, _I]),
    'nats_b200_decode_fwd': (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P, _SZ, _P]),
    'nats_b200_decode_step_fwd': (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _P, _SZ, _P]),
    'nats_b200_decode_step_place': (_I, [_P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    'nats_b200_decode_place': (_I, [_P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
}

_lock = threading.Lock()
_lib = None


class NatsB200Error(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """The loaded library (loaded once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise NatsB200Error(
                        f'{LIB_PATH} is missing: build it with `python -m neuralattentionsearch_b200.build` '
                        '(there is no CPU or PyTorch fallback for the NAtS kernels)')
                handle = ctypes.CDLL(LIB_PATH)
                for name, (res, args) in SIGNATURES.items():
                    fn = getattr(handle, name)
                    fn.restype, fn.argtypes = res, args
                _lib = handle
    return _lib


def call(name: str, *args) -> None:
    """Calls an int-returning entry point and raises NatsB200Error with the library's message on failure."""
    rc = getattr(lib(), name)(*args)
    if rc != 0:
        msg = lib().nats_b200_last_error().decode()
        raise NatsB200Error(f'{name} failed (code {rc}): {msg}')
