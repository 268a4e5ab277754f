"""Functional entry points of the NAtS attention hot path on B200.

The first three functions keep the names, argument meaning and return conventions of the reference's Triton
entry points, so a caller can switch the import and nothing else:

* ``nats_prefill``          src/nats/models/transformer/triton/nats_flashattn_fwd.py:617-725
* ``nats_chunk_attention``  src/nats/models/transformer/triton/nats_chunk_attention.py:1154-1185   (forward only)
* ``nats_attention``        src/nats/models/transformer/triton/flashattention_mask_on_chip.py:1018-1048 (forward only)

All of them run the same kernel (``nats_b200_prefill_fwd``): the role mask is the one of the reference's eager
path (``NAtSChunkLayerCache.generate_mask``), which the reference's own test treats as ground truth.  The lower
part of the file wraps the remaining C-ABI entry points for the cache classes.  Nothing here computes attention
with PyTorch ops: if the CUDA library is missing the import of ``_lib`` raises.
"""
from __future__ import annotations

import math

import torch

from . import _lib

ROLE_GLOBAL, ROLE_LOCAL, ROLE_SLIDING = 0, 1, 2
PREFILL_HEAD_DIMS = (64, 128, 256)     # head dims the prefill kernel is built for (256: one query head per work item)
PADDED_HEAD_DIMS = (16, 32)            # run zero-padded to 64 (first call only)
REFERENCE_HEAD_DIMS = (16, 32, 64, 128, 256)      # what the reference's Triton entry point accepts (nats_flashattn_fwd.py:633-634)

_status: dict[int, torch.Tensor] = {}
_workspaces: dict[tuple, torch.Tensor] = {}


def _p(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _call(device: torch.device, name: str, *args) -> None:
    """Calls an entry point with ``device`` current: the library reads the current device for the SM count, the
    per-device kernel attributes and its built-in scratch, while the stream belongs to the tensors' device."""
    if device.index is not None and device.index != torch.cuda.current_device():
        with torch.cuda.device(device):
            _lib.call(name, *args)
    else:
        _lib.call(name, *args)


def _need_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise _lib.NatsB200Error('the NAtS B200 kernels need CUDA tensors; there is no CPU path')
        if t.device != dev:
            raise ValueError('all tensors must live on the same device')
    return dev


def _check_head_dim(D: int, padded_ok: bool = True) -> None:
    """One clear error, before anything is launched, for head dims this build does not cover."""
    ok = PREFILL_HEAD_DIMS + (PADDED_HEAD_DIMS if padded_ok else ())
    if D not in ok:
        raise NotImplementedError(
            f'head_dim {D} is not built: the prefill kernel covers {PREFILL_HEAD_DIMS}' +
            (f', {PADDED_HEAD_DIMS} run zero-padded' if padded_ok else ' for calls over an existing cache') +
            f' (the reference accepts {REFERENCE_HEAD_DIMS})')


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 word the prefill kernel raises when one of its bounded waits gives up."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[idx]


def _raise_status(device: torch.device, code: int) -> None:
    status_word(device).zero_()
    raise _lib.NatsB200Error(f'the prefill kernel gave up a bounded wait (code {code}); its output is invalid')


def check_status(device: torch.device | None = None) -> None:
    """Synchronises with the device and raises if a kernel reported a timed-out wait since the last check.  The cache
    classes call this wherever they read a value back from the device anyway; callers of the bare functions call it
    before they trust an output."""
    device = torch.device('cuda', torch.cuda.current_device()) if device is None else device
    code = int(status_word(device).item())
    if code != 0:
        _raise_status(device, code)


def _workspace(kind: str, device: torch.device, nbytes: int, zero: bool = False) -> torch.Tensor:
    key = (kind, device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = (torch.zeros if zero else torch.empty)(max(nbytes, 256), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


class _PinnedWords:
    """A few pinned int32 word pairs per device for small asynchronous read-backs.  Allocating pinned memory per call would
    synchronise the device, so the words are allocated once and handed out again when their reader is done with them."""
    _free: dict = {}
    _lock = __import__('threading').Lock()

    @classmethod
    def take(cls, dev: torch.device) -> torch.Tensor:
        with cls._lock:
            free = cls._free.setdefault(dev, [])
            return free.pop() if free else torch.empty(2, dtype=torch.int32, pin_memory=True)

    @classmethod
    def give_back(cls, dev: torch.device, word: torch.Tensor) -> None:
        with cls._lock:
            cls._free.setdefault(dev, []).append(word)


_side_streams: dict = {}


def _side_stream(device: torch.device) -> torch.cuda.Stream:
    """One extra stream per device for small read-backs that must not sit between two kernels of the caller's stream."""
    st = _side_streams.get(device.index)
    if st is None:
        st = _side_streams[device.index] = torch.cuda.Stream(device)
    return st


class _AsyncWord:
    """An int32 scalar on its way from the device to the host, with the device's prefill status word riding along.
    Calling the object waits for the copy and returns the value (and raises if a kernel that ran before the copy had
    given up a bounded wait); the pinned words go back to the pool when the value has been read or the object is dropped."""

    def __init__(self, src: torch.Tensor):
        self.dev = src.device
        self.word = _PinnedWords.take(self.dev)
        # The two small copies run on a side stream behind what the current stream holds so far: on the current stream they
        # would stand between the kernel that wrote ``src`` and the (long) kernel the caller launches next, ~10 us per step.
        main = torch.cuda.current_stream(self.dev)
        side = _side_stream(self.dev)
        ready = torch.cuda.Event()
        ready.record(main)
        side.wait_event(ready)
        with torch.cuda.stream(side):
            self.word[:1].copy_(src[:1], non_blocking=True)
            self.word[1:].copy_(status_word(self.dev), non_blocking=True)
            self.done = torch.cuda.Event()
            self.done.record(side)
        src.record_stream(side)

    def __call__(self) -> int:
        self.done.synchronize()
        value, code = int(self.word[0]), int(self.word[1])
        self._release()
        if code != 0:
            _raise_status(self.dev, code)
        return value

    def _release(self):
        if self.word is not None:
            self.done.synchronize()          # the copy must not land in a word that somebody else already holds
            _PinnedWords.give_back(self.dev, self.word)
            self.word = None

    def __del__(self):
        try:
            self._release()
        except Exception:
            pass


def read_word_async(src: torch.Tensor) -> _AsyncWord:
    """Starts copying the int32 scalar ``src[0]`` to the host on the current stream; call the result to get the value."""
    return _AsyncWord(src)


def roles_from_token_states_info(token_states_info: torch.Tensor) -> torch.Tensor:
    """uint8 role codes [B,Hkv,Nc] from the one-hot ``token_states_info`` [B,Hkv,Nc,3] (first max wins)."""
    if token_states_info.dtype == torch.uint8 and token_states_info.dim() == 3:
        return token_states_info.contiguous()
    return token_states_info.argmax(-1).to(torch.uint8).contiguous()


def roles_from_end_seqs(end_seqs_idx: torch.Tensor, sliding_tokens: torch.Tensor) -> torch.Tensor:
    """Role codes from what the Triton entry points take: ``end_seqs_idx[c] == c`` marks a global chunk
    (nats_flashattn_fwd.py:96) and ``sliding_tokens`` a sliding one; everything else is local."""
    nc = end_seqs_idx.shape[-1]
    ar = torch.arange(nc, device=end_seqs_idx.device)
    roles = torch.where(end_seqs_idx == ar, ROLE_GLOBAL, ROLE_LOCAL)
    roles = torch.where(sliding_tokens.to(torch.bool), ROLE_SLIDING, roles).to(torch.uint8)
    return roles.contiguous()


def _as_bf16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).contiguous()


def prefill_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, roles: torch.Tensor, chunk_size: int,
                      sliding_window: int, sm_scale: float | None = None,
                      kept_tiles: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Role-masked causal attention of a first prefill call.  q [B,Hq,N,D], k/v [B,Hkv,N,D] (cast to bf16 if
    needed), roles uint8 [B,Hkv,ceil(N/C)].  Returns o [B,Hq,N,D] in q's dtype."""
    dev = _need_cuda(q, k, v, roles)
    B, Hq, N, D = q.shape
    Hkv = k.shape[1]
    if k.shape != (B, Hkv, N, D) or v.shape != k.shape:
        raise ValueError(f'k/v shape {tuple(k.shape)}/{tuple(v.shape)} does not match q {tuple(q.shape)}')
    nc = -(-N // chunk_size)
    if roles.shape != (B, Hkv, nc) or roles.dtype != torch.uint8:
        raise ValueError(f'roles must be uint8 [{B},{Hkv},{nc}], got {roles.dtype} {tuple(roles.shape)}')
    _check_head_dim(D)
    scale = (1.0 / math.sqrt(D)) if sm_scale is None else float(sm_scale)
    qb, kb, vb = _as_bf16(q), _as_bf16(k), _as_bf16(v)
    if D in PADDED_HEAD_DIMS:
        # narrow heads run in the 64-wide kernel on zero-padded copies: the scores are unchanged by zero columns of q and
        # k, the extra output columns are zero and dropped (the scale still comes from the real head_dim)
        if out is not None:
            raise ValueError(f'out= is not supported for head_dim {D}')
        pad = (0, 64 - D)
        qb, kb, vb = (torch.nn.functional.pad(t, pad) for t in (qb, kb, vb))
    if out is not None and (out.shape != qb.shape or out.dtype != torch.bfloat16 or not out.is_contiguous()):
        raise ValueError('out must be a contiguous bf16 tensor shaped like q')
    o = torch.empty_like(qb) if out is None else out
    lib = _lib.lib()
    nbytes = lib.nats_b200_prefill_workspace_bytes(B, Hkv, N, chunk_size)
    ws = _workspace('prefill', dev, nbytes)
    _call(dev, 'nats_b200_prefill_fwd', _p(qb), _p(kb), _p(vb), _p(o), _p(roles.contiguous()), B, Hq, Hkv, N, qb.shape[-1],
              chunk_size, sliding_window, scale, _p(ws), ws.numel(), _p(kept_tiles), _p(status_word(dev)), _stream(dev))
    if D in PADDED_HEAD_DIMS:
        o = o[..., :D].contiguous()
    return o if q.dtype == torch.bfloat16 else o.to(q.dtype)


class HostPrefillPipeline:
    """Prefill for callers whose q/k/v live in (pinned) host memory and who want the output back in host memory.

    The (batch, kv-head) pairs are independent, so the work is cut into one piece per pair and pipelined over three
    streams: host->device copy of piece i+1, the prefill kernel on piece i and the device->host copy of the output of
    piece i-1 run at the same time (PCIe is full duplex).  K, V and the role codes of all pieces stay on the device
    afterwards (``self.k``, ``self.v``, ``self.roles``) because the eviction that follows a prefill needs them.
    Device buffers are allocated once and reused by later calls of the same shape."""

    def __init__(self, B: int, Hq: int, Hkv: int, N: int, D: int, chunk_size: int, sliding_window: int,
                 device: torch.device, n_buffers: int = 3):
        self.shape = (B, Hq, Hkv, N, D)
        self.C, self.SW, self.device = chunk_size, sliding_window, device
        nrep = Hq // Hkv
        self.k = torch.empty(B, Hkv, N, D, dtype=torch.bfloat16, device=device)
        self.v = torch.empty_like(self.k)
        self.roles = torch.empty(B, Hkv, -(-N // chunk_size), dtype=torch.uint8, device=device)
        self.q_buf = [torch.empty(1, nrep, N, D, dtype=torch.bfloat16, device=device) for _ in range(n_buffers)]
        self.o_buf = [torch.empty(1, nrep, N, D, dtype=torch.bfloat16, device=device) for _ in range(n_buffers)]
        self.s_in, self.s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        self.kept = torch.zeros(B, Hkv, dtype=torch.int64, device=device)

    def run(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, roles: torch.Tensor, out: torch.Tensor,
            sm_scale: float | None = None) -> torch.Tensor:
        B, Hq, Hkv, N, D = self.shape
        nrep, nb = Hq // Hkv, len(self.q_buf)
        main = torch.cuda.current_stream(self.device)
        self.s_in.wait_stream(main)
        self.s_out.wait_stream(main)
        with torch.cuda.stream(self.s_in):
            self.roles.copy_(roles, non_blocking=True)
        copied = [None] * (B * Hkv)
        computed = [None] * (B * Hkv)
        drained = [None] * (B * Hkv)
        for i in range(B * Hkv):
            b, h = divmod(i, Hkv)
            slot = i % nb
            with torch.cuda.stream(self.s_in):
                if i >= nb:
                    self.s_in.wait_event(computed[i - nb])            # the kernel that read this q buffer is done
                self.q_buf[slot].copy_(q[b:b + 1, h * nrep:(h + 1) * nrep], non_blocking=True)
                self.k[b, h].copy_(k[b, h], non_blocking=True)
                self.v[b, h].copy_(v[b, h], non_blocking=True)
                copied[i] = torch.cuda.Event()
                copied[i].record(self.s_in)
            main.wait_event(copied[i])
            if i >= nb:
                main.wait_event(drained[i - nb])                      # the output buffer has been copied out
            o = prefill_attention(self.q_buf[slot], self.k[b:b + 1, h:h + 1], self.v[b:b + 1, h:h + 1], self.roles[b:b + 1, h:h + 1],
                                  self.C, self.SW, sm_scale, kept_tiles=self.kept[b:b + 1, h:h + 1], out=self.o_buf[slot])
            computed[i] = torch.cuda.Event()
            computed[i].record(main)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(computed[i])
                out[b:b + 1, h * nrep:(h + 1) * nrep].copy_(o, non_blocking=True)
                drained[i] = torch.cuda.Event()
                drained[i].record(self.s_out)
        main.wait_stream(self.s_out)
        return out


def dense_role_mask(roles: torch.Tensor, chunk_size: int, sliding_window: int, n: int) -> torch.Tensor:
    """bool [B,Hkv,N,N] visibility mask, materialised (debugging aid and the ``return_masks`` option; it is never
    used to compute attention)."""
    dev = roles.device
    B, H, nc = roles.shape
    lim = torch.empty(B, H, nc, dtype=torch.int32, device=dev)
    nt = -(-n // 128)
    tmax = torch.empty(B, H, nt, dtype=torch.int32, device=dev)
    tmin = torch.empty_like(tmax)
    _call(dev, 'nats_b200_role_prep', _p(roles.contiguous()), B, H, n, chunk_size, sliding_window, _p(lim), _p(tmax), _p(tmin),
              None, _stream(dev))
    lim_tok = lim.repeat_interleave(chunk_size, -1)[..., :n].long()
    ar = torch.arange(n, device=dev)
    return (ar[:, None] >= ar[None, :])[None, None] & (ar[None, None, :, None] <= lim_tok[:, :, None, :])


# ------------------------------------------------------------------------------------------------
# reference-named entry points
# ------------------------------------------------------------------------------------------------
def nats_prefill(q, k, v, end_seqs_idx, sliding_tokens, sm_scale,
                 nats_chunk_size: int = 1,
                 global_kv_size=None, local_kv_size=None, valid_sw_tokens=None, n_ctx_data=None, sw_token_tails=None,
                 n_rep: int = 1, n_tokens_in_first_chunk: int = 0, local_seq_max_length: int = 4,
                 return_masks: bool = False, block_n: int = 32):
    """Drop-in for the reference's ``nats_prefill``: returns ``(o, mask_or_None)``.

    ``block_n`` is accepted and ignored (the tile shape is fixed by the tensor-core kernel).

    With ``global_kv_size`` given this is a multi-token call over an existing compacted cache, as the reference's
    HAS_PAST_INFO path (nats_flashattn_fwd.py:693-722; caller hf/llama.py:235-252): ``k``/``v`` are the cache with the new
    tokens already appended (what ``cache.update`` returned), ``n_ctx_data`` the cache's extent before the call,
    ``valid_sw_tokens`` the ring flags [B,Hkv,SW], ``sw_token_tails`` the ring write position, and
    ``end_seqs_idx``/``sliding_tokens`` describe the chunks from the unfinished one on."""
    if global_kv_size is not None:
        assert q.shape[1] == k.shape[1] * n_rep
        C, SW = nats_chunk_size, local_seq_max_length
        n_ctx = int(n_ctx_data)
        t0 = n_ctx // C * C
        fill = n_ctx - t0
        assert n_tokens_in_first_chunk in (0, fill), 'n_tokens_in_first_chunk contradicts n_ctx_data'
        roles = roles_from_end_seqs(end_seqs_idx, sliding_tokens)
        flags = valid_sw_tokens.to(torch.uint8).contiguous()
        o = prefill_attention_past(q, k, v, flags, roles, global_kv_size, local_kv_size, t0, fill, int(sw_token_tails), C, SW,
                                   sm_scale)
        mask = None
        if return_masks:
            x_len = q.shape[2]
            lim = layout_row_limits(roles, flags, global_kv_size, local_kv_size, x_len, t0, fill, int(sw_token_tails), C, SW)
            L = n_ctx + x_len
            lim_tok = lim.repeat_interleave(C, -1)[..., :L].long()
            qpos = torch.arange(n_ctx, L, device=q.device)
            kpos = torch.arange(L, device=q.device)
            mask = (kpos[None, :] <= qpos[:, None])[None, None] & (qpos[None, None, :, None] <= lim_tok[:, :, None, :])
        return o, mask
    assert q.shape[-1] == k.shape[-1] == v.shape[-1]
    assert q.shape[-1] in set(REFERENCE_HEAD_DIMS)
    assert k.shape[2] == q.shape[2]
    assert q.shape[1] == k.shape[1] * n_rep
    roles = roles_from_end_seqs(end_seqs_idx, sliding_tokens)
    o = prefill_attention(q, k, v, roles, nats_chunk_size, local_seq_max_length, sm_scale)
    mask = dense_role_mask(roles, nats_chunk_size, local_seq_max_length, q.shape[2]) if return_masks else None
    return o, mask


def nats_chunk_attention(q, k, v, seq_info, end_seqs_idx, causal, sm_scale, nats_chunk_size: int,
                         n_rep: int = 1, sparse_regularized_value: float = 0., local_seq_max_length: int = 4,
                         compress_on_q: bool = True):
    """Forward of the reference's chunked training attention (no autograd: inference build).  ``seq_info`` is the
    one-hot role tensor [B,Hkv,Nc,3]; returns ``o`` shaped like ``q``."""
    assert causal, 'only causal attention exists on this path'
    roles = roles_from_token_states_info(seq_info)
    return prefill_attention(q, k, v, roles, nats_chunk_size, local_seq_max_length, sm_scale)


def nats_chunk_attention_fwd(q, k, v, seq_info, end_seqs_idx, causal, sm_scale, nats_chunk_size: int, n_rep: int = 1,
                             local_seq_max_length: int = 4):
    """What the forward of the reference's autograd function computes and saves for its backward
    (triton/nats_chunk_attention.py:987-1060): ``(o, M, n_valid_blocks)`` with ``M`` fp32 [B,Hq,N] = log2 of the row's
    sum of exp2(scaled scores) and ``n_valid_blocks`` int32 [B,Hq,N] = visible keys per row.  The backward itself is
    not part of this package."""
    assert causal, 'only causal attention exists on this path'
    roles = roles_from_token_states_info(seq_info)
    dev = _need_cuda(q, k, v, roles)
    B, Hq, N, D = q.shape
    Hkv = k.shape[1]
    _check_head_dim(D, padded_ok=False)
    qb, kb, vb = _as_bf16(q), _as_bf16(k), _as_bf16(v)
    o = torch.empty_like(qb)
    lse = torch.empty(B, Hq, N, dtype=torch.float32, device=dev)
    n_vis = torch.empty(B, Hq, N, dtype=torch.int32, device=dev)
    lib = _lib.lib()
    ws = _workspace('prefill', dev, lib.nats_b200_prefill_workspace_bytes(B, Hkv, N, nats_chunk_size))
    _call(dev, 'nats_b200_prefill_fwd_stats', _p(qb), _p(kb), _p(vb), _p(o), _p(roles), B, Hq, Hkv, N, D, nats_chunk_size,
              local_seq_max_length, float(sm_scale), _p(ws), ws.numel(), None, _p(lse), _p(n_vis), _p(status_word(dev)),
              _stream(dev))
    return (o if q.dtype == torch.bfloat16 else o.to(q.dtype)), lse, n_vis


def nats_attention(q, k, v, seq_info, end_seqs_idx, causal, sm_scale, n_rep: int = 1,
                   sparse_regularized_value: float = 0., local_seq_max_length: int = 4):
    """Token-granular variant (chunk size 1) of ``nats_chunk_attention``."""
    assert causal, 'only causal attention exists on this path'
    roles = roles_from_token_states_info(seq_info)
    return prefill_attention(q, k, v, roles, 1, local_seq_max_length, sm_scale)


def rope_split_heads(q_in: torch.Tensor, k_in: torch.Tensor, v_in: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                     n_heads: int, n_kv_heads: int, head_dim: int):
    """Rotary embedding + head split in one pass.  q_in [B,N,Hq*D], k_in / v_in [B,N,Hkv*D] as the projections leave them
    (rows may be slices of a wider fused projection); cos / sin [B or 1,N,D] (Hugging Face layout).  Returns bf16
    q [B,Hq,N,D], k, v [B,Hkv,N,D], bit-identical to ``apply_rotary_pos_emb`` on the transposed views in bf16."""
    dev = _need_cuda(q_in, k_in, v_in, cos, sin)
    B, N, _ = q_in.shape
    ins = []
    for t, h in ((q_in, n_heads), (k_in, n_kv_heads), (v_in, n_kv_heads)):
        if t.dtype != torch.bfloat16 or t.stride(2) != 1 or t.stride(0) != N * t.stride(1) or t.shape[2] != h * head_dim:
            t = t.to(torch.bfloat16).contiguous()
        ins.append(t)
    cos = cos.to(torch.bfloat16).contiguous()
    sin = sin.to(torch.bfloat16).contiguous()
    if cos.shape[-2:] != (N, head_dim) or cos.shape != sin.shape or cos.numel() not in (N * head_dim, B * N * head_dim):
        raise ValueError(f'cos / sin must be [1 or {B}, {N}, {head_dim}], got {tuple(cos.shape)}')
    q = torch.empty(B, n_heads, N, head_dim, dtype=torch.bfloat16, device=dev)
    k = torch.empty(B, n_kv_heads, N, head_dim, dtype=torch.bfloat16, device=dev)
    v = torch.empty_like(k)
    _call(dev, 'nats_b200_rope_split_heads', _p(ins[0]), _p(ins[1]), _p(ins[2]), ins[0].stride(1), ins[1].stride(1),
              ins[2].stride(1), _p(cos), _p(sin), 0 if cos.numel() == N * head_dim else N * head_dim, _p(q), _p(k), _p(v),
              B, N, n_heads, n_kv_heads, head_dim, _stream(dev))
    return q, k, v


# ------------------------------------------------------------------------------------------------
# thin wrappers of the cache entry points (used by cache.py)
# ------------------------------------------------------------------------------------------------
def evict_plan(roles: torch.Tensor, n: int, chunk_size: int, sliding_window: int, rank: torch.Tensor,
               size_global: torch.Tensor, size_local: torch.Tensor, state: torch.Tensor) -> None:
    B, H, _ = roles.shape
    _call(roles.device, 'nats_b200_evict_plan', _p(roles), B, H, n, chunk_size, sliding_window, _p(rank), _p(size_global),
              _p(size_local), _p(state), _stream(roles.device))


def evict_compact(k: torch.Tensor, v: torch.Tensor, roles: torch.Tensor, rank: torch.Tensor, size_global: torch.Tensor,
                  size_local: torch.Tensor, state: torch.Tensor, chunk_size: int, sliding_window: int,
                  cache_k: torch.Tensor, cache_v: torch.Tensor, valid: torch.Tensor) -> None:
    B, H, N, D = k.shape
    _call(k.device, 'nats_b200_evict_compact', _p(k), _p(v), _p(roles), _p(rank), _p(size_global), _p(size_local), _p(state),
              B, H, N, D, chunk_size, sliding_window, _p(cache_k), _p(cache_v), _p(valid), cache_k.shape[2],
              _stream(k.device))


def cache_append(k_new: torch.Tensor, v_new: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor,
                 valid: torch.Tensor, pos: int) -> None:
    B, H, x_len, D = k_new.shape
    _call(k_new.device, 'nats_b200_cache_append', _p(k_new), _p(v_new), _p(cache_k), _p(cache_v), _p(valid), B, H, x_len, D,
              cache_k.shape[2], pos, _stream(k_new.device))


def prefill_attention_past(q: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor, valid: torch.Tensor,
                           roles_new: torch.Tensor, size_global: torch.Tensor, size_local: torch.Tensor,
                           t0: int, fill: int, tail: int, chunk_size: int, sliding_window: int,
                           sm_scale: float | None = None, kept_tiles: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of x_len new queries over an existing compacted cache to which their K/V have been appended at rows
    [t0+fill, t0+fill+x_len).  q [B,Hq,x_len,D]; cache_k/v [B,Hkv,capacity,D] bf16; valid uint8 [B,Hkv,capacity];
    roles_new uint8 [B,Hkv,ceil((fill+x_len)/C)] (chunks from the unfinished one on).  Returns o like q."""
    dev = _need_cuda(q, cache_k, cache_v, valid, roles_new)
    B, Hq, x_len, D = q.shape
    Hkv = cache_k.shape[1]
    ncn = -(-(fill + x_len) // chunk_size)
    if roles_new.shape != (B, Hkv, ncn) or roles_new.dtype != torch.uint8:
        raise ValueError(f'roles must be uint8 [{B},{Hkv},{ncn}], got {roles_new.dtype} {tuple(roles_new.shape)}')
    # the cache may be a view [:, :, :n] of a longer buffer: rows contiguous, heads `capacity` rows apart
    cap = cache_k.stride(1) // D
    for t in (cache_k, cache_v):
        if t.dtype != torch.bfloat16 or t.stride(3) != 1 or t.stride(2) != D or t.stride(1) != cap * D or \
                t.stride(0) != Hkv * cap * D or t.shape[2] < t0 + fill + x_len:
            raise ValueError('the cache must be bf16 [B,Hkv,>=t0+fill+x_len,D], dense or a [:, :, :n] view of a dense buffer')
    if valid.dtype != torch.uint8 or valid.stride(2) != 1 or valid.stride(0) != Hkv * valid.stride(1):
        raise ValueError('valid must be uint8 [B,Hkv,>=SW] with contiguous rows')
    _check_head_dim(D, padded_ok=False)
    qb = _as_bf16(q)
    o = torch.empty_like(qb)
    lib = _lib.lib()
    nbytes = lib.nats_b200_prefill_past_workspace_bytes(B, Hkv, t0 + fill + x_len, chunk_size)
    ws = _workspace('prefill', dev, nbytes)
    scale = (1.0 / math.sqrt(D)) if sm_scale is None else float(sm_scale)
    _call(dev, 'nats_b200_prefill_past_fwd', _p(qb), _p(cache_k), _p(cache_v), _p(o), _p(roles_new.contiguous()), _p(valid),
              valid.stride(1), _p(size_global), _p(size_local), B, Hq, Hkv, x_len, D, chunk_size, sliding_window, cap, t0, fill,
              tail, scale,
              _p(ws), ws.numel(), _p(kept_tiles), _p(status_word(dev)), _stream(dev))
    return o if q.dtype == torch.bfloat16 else o.to(q.dtype)


def layout_row_limits(roles_new: torch.Tensor, valid: torch.Tensor, size_global: torch.Tensor, size_local: torch.Tensor,
                      x_len: int, t0: int, fill: int, tail: int, chunk_size: int, sliding_window: int) -> torch.Tensor:
    """int32 [B,Hkv,ceil((t0+fill+x_len)/C)]: per chunk of the cache layout + new tokens, the last query position that may
    see it (what the kernel masks with); a debugging aid."""
    dev = _need_cuda(roles_new, valid)
    B, H, _ = roles_new.shape
    n_kv = t0 + fill + x_len
    lim = torch.empty(B, H, -(-n_kv // chunk_size), dtype=torch.int32, device=dev)
    nt = -(-n_kv // 128)
    tmax = torch.empty(B, H, nt, dtype=torch.int32, device=dev)
    tmin = torch.empty_like(tmax)
    _call(dev, 'nats_b200_role_prep_past', _p(roles_new.contiguous()), _p(valid), _p(size_global), _p(size_local), B, H, x_len,
              chunk_size, sliding_window, valid.stride(1), t0, fill, tail, _p(lim), _p(tmax), _p(tmin), None, _stream(dev))
    return lim


def evict_plan_past(roles_new: torch.Tensor, n_tokens: int, chunk_size: int, sliding_window: int, rank: torch.Tensor,
                    base: torch.Tensor, size_global: torch.Tensor, size_local: torch.Tensor, state: torch.Tensor) -> None:
    B, H, _ = roles_new.shape
    _call(roles_new.device, 'nats_b200_evict_plan_past', _p(roles_new), B, H, n_tokens, chunk_size, sliding_window, _p(rank), _p(base),
              _p(size_global), _p(size_local), _p(state), _stream(roles_new.device))


def evict_compact_past(old_k: torch.Tensor, old_v: torch.Tensor, old_valid: torch.Tensor, roles_new: torch.Tensor,
                       rank: torch.Tensor, base: torch.Tensor, size_global: torch.Tensor, size_local: torch.Tensor,
                       state: torch.Tensor, n_tokens: int, chunk_size: int, sliding_window: int, t0_old: int, tail_old: int,
                       cache_k: torch.Tensor, cache_v: torch.Tensor, valid: torch.Tensor) -> None:
    B, H, cap_old, D = old_k.shape
    _call(old_k.device, 'nats_b200_evict_compact_past', _p(old_k), _p(old_v), _p(old_valid), cap_old, _p(roles_new), _p(rank), _p(base),
              _p(size_global), _p(size_local), _p(state), B, H, n_tokens, D, chunk_size, sliding_window, t0_old, tail_old,
              _p(cache_k), _p(cache_v), _p(valid), cache_k.shape[2], _stream(old_k.device))


def decode_workspace_bytes(B: int, Hq: int, Hkv: int, D: int, max_len: int) -> int:
    return _lib.lib().nats_b200_decode_workspace_bytes(B, Hq, Hkv, D, max_len)


def decode_fwd(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, o: torch.Tensor, cache_k: torch.Tensor,
               cache_v: torch.Tensor, valid: torch.Tensor, size_global: torch.Tensor, size_local: torch.Tensor,
               state: torch.Tensor, fill: int, max_len_bound: int, chunk_size: int, sliding_window: int,
               sm_scale: float, workspace: torch.Tensor) -> None:
    B, Hq, _, D = q.shape
    Hkv = k_new.shape[1]
    _call(q.device, 'nats_b200_decode_fwd', _p(q), _p(k_new), _p(v_new), _p(o), _p(cache_k), _p(cache_v), _p(valid),
              cache_k.shape[2], _p(size_global), _p(size_local), _p(state), fill, max_len_bound, B, Hq, Hkv, D,
              chunk_size, sliding_window, float(sm_scale), _p(workspace), workspace.numel(), _stream(q.device))


def decode_step_fwd(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, o: torch.Tensor, cache_k: torch.Tensor,
                    cache_v: torch.Tensor, valid: torch.Tensor, size_global: torch.Tensor, size_local: torch.Tensor,
                    state: torch.Tensor, max_len_bound: int, chunk_size: int, sliding_window: int, sm_scale: float,
                    workspace: torch.Tensor) -> None:
    B, Hq, _, D = q.shape
    Hkv = k_new.shape[1]
    _call(q.device, 'nats_b200_decode_step_fwd', _p(q), _p(k_new), _p(v_new), _p(o), _p(cache_k), _p(cache_v), _p(valid),
              cache_k.shape[2], _p(size_global), _p(size_local), _p(state), max_len_bound, B, Hq, Hkv, D, chunk_size,
              sliding_window, float(sm_scale), _p(workspace), workspace.numel(), _stream(q.device))


def decode_step_place(roles: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor, valid: torch.Tensor,
                      size_global: torch.Tensor, size_local: torch.Tensor, state: torch.Tensor, chunk_size: int,
                      sliding_window: int) -> None:
    B, H, _, D = cache_k.shape
    _call(cache_k.device, 'nats_b200_decode_step_place', _p(roles), _p(cache_k), _p(cache_v), _p(valid), cache_k.shape[2], _p(size_global),
              _p(size_local), _p(state), B, H, D, chunk_size, sliding_window, _stream(cache_k.device))


def decode_place(roles: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor, valid: torch.Tensor,
                 size_global: torch.Tensor, size_local: torch.Tensor, state: torch.Tensor, tail: int, chunk_size: int,
                 sliding_window: int) -> None:
    B, H, _, D = cache_k.shape
    _call(cache_k.device, 'nats_b200_decode_place', _p(roles), _p(cache_k), _p(cache_v), _p(valid), cache_k.shape[2], _p(size_global),
              _p(size_local), _p(state), tail, B, H, D, chunk_size, sliding_window, _stream(cache_k.device))
