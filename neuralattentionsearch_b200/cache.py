"""GPU-resident KV cache of the NAtS attention path, with the reference's cache protocol.

``NAtSChunkLayerCache`` keeps the attribute and method names of the reference's per-layer cache
(src/nats/components/cache/nats_chunk_layer_cache.py:15) and ``NAtSCache`` those of the per-model container
(src/nats/components/cache/dyn_cache.py:66-195), so callers that read ``size_global_kv``, ``size_local_kv``,
``valid_tokens``, ``cache_k`` ... keep working.  What differs is how the state is produced:

* the first prefill call does not build ``[zeros(SW) | K | pad]`` and then shuffle it in place; ``update`` only keeps
  a reference to K/V, and ``post_update`` runs the eviction kernels, which write the compacted layout
  ``[ring | kept chunks | unfinished chunk]`` straight into a buffer sized from the longest head (one small
  device-to-host read, where the reference synchronises several times);
* a decode step is one fused launch (append + attention over ring / kept tokens / unfinished chunk) plus, every
  ``chunk_size`` steps, one placement launch; the common tail offset lives on the device, the host only tracks an
  upper bound, so decode steps never synchronise;
* buffers carry head-room and are reallocated geometrically instead of ``F.pad`` per step.

Regions the reference leaves undefined (between a head's own length and the common tail offset) read as zero here.
"""
from __future__ import annotations

import math
from typing import Any

import torch

from . import functional as F_


def get_pad_size(x_len: int, chunk_size: int) -> int:
    return math.ceil(x_len / chunk_size) * chunk_size - x_len


class NAtSChunkLayerCache:
    def __init__(self, bsz: int, n_msks: int, sliding_window_size: int, layer_id: int = 0, chunk_size: int = 16,
                 device: torch.device = torch.device('cuda'), headroom: int = 1024):
        assert sliding_window_size % chunk_size == 0
        self.layer_id = layer_id
        self.bsz, self.n_msks = bsz, n_msks
        self.chunk_size = chunk_size
        self.sliding_window_size = sliding_window_size
        self.n_chunks_per_sw = sliding_window_size // chunk_size
        self.device = torch.device(device)
        self.headroom = max(headroom, chunk_size)
        self.reset_cache()

    # ------------------------------------------------------------------ state
    def reset_cache(self):
        dev = self.device
        self.size_local_kv = torch.zeros(self.bsz, self.n_msks, device=dev, dtype=torch.long)
        self.size_global_kv = torch.full([self.bsz, self.n_msks], self.sliding_window_size, device=dev, dtype=torch.long)
        self.chunk_fill_size = 0
        self.chunk_fill_size_last = 0
        self.sliding_queue_tail = 0
        self._seen_tokens = 0
        self._tokens_info = None
        self._roles = None
        self._state = torch.zeros(8, dtype=torch.int32, device=dev)      # [0] = common tail offset T0 (max length)
        self._state[:1].fill_(self.sliding_window_size)                 # (a kernel; indexed assignment would synchronise)
        self._t0_bound = self.sliding_window_size                       # host upper bound of T0
        self._t0_exact = self.sliding_window_size                       # exact value, None while unknown
        self._t0_synced = self.sliding_window_size                      # last exact value read back
        self._buf_k = self._buf_v = self._buf_valid = None
        self._pending = None                                            # K/V handed to update(), not yet placed
        self._plan = None                                               # keep-set of the first call, planned in update()
        self._unposted = 0                                              # tokens seen by update() but not by post_update()
        self._dec_ws = None

    def get_seq_length(self):
        return self._seen_tokens

    def get_chunk_fill_size(self):
        return self.chunk_fill_size

    def _t0(self) -> int:
        if self._t0_exact is None:
            self._t0_exact = int(self._state[0].item())
            self._t0_bound = self._t0_synced = self._t0_exact
            F_.check_status(self.device)      # the host waits for the device here anyway: a failed prefill must not go unnoticed
        return self._t0_exact

    @property
    def n_ctx_data(self) -> int:
        """Valid extent of the cache: longest head plus the tokens of the unfinished chunk (host value; reading it
        after a chunk was placed costs one device-to-host read)."""
        return self._t0() + self.chunk_fill_size - self._unposted

    def _view_len(self) -> int:
        n = self.n_ctx_data + self._unposted
        return math.ceil(n / self.chunk_size) * self.chunk_size

    @property
    def cache_k(self):
        return None if self._buf_k is None else self._buf_k[:, :, :self._view_len()]

    @property
    def cache_v(self):
        return None if self._buf_v is None else self._buf_v[:, :, :self._view_len()]

    @property
    def valid_tokens(self):
        return None if self._buf_valid is None else self._buf_valid[:, :, :self._view_len()].view(torch.bool)

    def kv_bytes(self) -> int:
        """Bytes of K and V a decode step has to read (valid ring slots + kept tokens + unfinished chunk)."""
        ring = self._buf_valid[:, :, :self.sliding_window_size].sum().item()
        main = (self.size_global_kv + self.size_local_kv - self.sliding_window_size).sum().item()
        tail = self.chunk_fill_size * self.bsz * self.n_msks
        return int(ring + main + tail) * self._buf_k.shape[-1] * 2 * 2

    def _alloc(self, cap: int, D: int, dtype=torch.bfloat16):
        dev = self.device
        self._buf_k = torch.empty(self.bsz, self.n_msks, cap, D, dtype=dtype, device=dev)
        self._buf_v = torch.empty(self.bsz, self.n_msks, cap, D, dtype=dtype, device=dev)
        self._buf_valid = torch.empty(self.bsz, self.n_msks, cap, dtype=torch.uint8, device=dev)

    def _grow(self, need: int):
        cap = self._buf_k.shape[2]
        if need <= cap:
            return
        new_cap = max(need + self.headroom, cap + cap // 2)
        new_cap = math.ceil(new_cap / self.chunk_size) * self.chunk_size
        old_k, old_v, old_valid = self._buf_k, self._buf_v, self._buf_valid
        dev, D = self.device, old_k.shape[-1]
        self._buf_k = torch.zeros(self.bsz, self.n_msks, new_cap, D, dtype=old_k.dtype, device=dev)
        self._buf_v = torch.zeros(self.bsz, self.n_msks, new_cap, D, dtype=old_k.dtype, device=dev)
        self._buf_valid = torch.zeros(self.bsz, self.n_msks, new_cap, dtype=torch.uint8, device=dev)
        self._buf_k[:, :, :cap] = old_k
        self._buf_v[:, :, :cap] = old_v
        self._buf_valid[:, :, :cap] = old_valid

    # ------------------------------------------------------------------ protocol
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, token_states_info: torch.Tensor | None,
               fused: bool = False):
        """Hands new K/V to the cache.  First call: the tensors are only referenced (the eviction kernels read them in
        ``post_update``) and returned unchanged, like the reference does.  Single-token calls: with ``fused=True`` (what
        the attention layer of this package passes) nothing is written yet -- ``decode_attention`` appends inside its
        kernel; otherwise the token is written now and views of the cache are returned, as the reference does."""
        bsz, nheads, x_len, head_dim = key_states.shape
        self.chunk_fill_size += x_len
        self._unposted = x_len
        if token_states_info is None:
            assert self.chunk_fill_size < self.chunk_size, \
                'a new token_states_info must be given once the cached tokens fill a chunk'
        if x_len == 0:
            return self.cache_k[:, :, :self.n_ctx_data], self.cache_v[:, :, :self.n_ctx_data]
        self._tokens_info = token_states_info
        self._roles = None if token_states_info is None else F_.roles_from_token_states_info(token_states_info)
        if self._buf_k is None and self._pending is None:
            self._pending = (key_states, value_states)
            self._plan_ahead(x_len)
            return key_states, value_states
        kb = key_states.to(torch.bfloat16).contiguous()
        vb = value_states.to(torch.bfloat16).contiguous()
        if x_len != 1:
            # several tokens over an existing cache: they are appended behind the unfinished chunk, as the reference does
            # (:239-256); ``prefill_attention`` then attends over the buffer and ``post_update`` compacts it
            pos = self.n_ctx_data
            self._grow(pos + x_len)
            F_.cache_append(kb, vb, self._buf_k, self._buf_v, self._buf_valid, pos)
            self._pending = None
            self._plan_ahead_past()
            return self._buf_k[:, :, :pos + x_len], self._buf_v[:, :, :pos + x_len]
        self._pending = (kb, vb)
        if fused:
            return kb, vb
        pos = self.n_ctx_data
        self._grow(pos + 1)
        self._buf_k[:, :, pos] = kb[:, :, 0]
        self._buf_v[:, :, pos] = vb[:, :, 0]
        self._buf_valid[:, :, pos].fill_(1)
        return self._buf_k[:, :, :pos + 1], self._buf_v[:, :, :pos + 1]

    def generate_mask(self, x_len: int) -> torch.Tensor:
        """bool mask of the reference's eager path ([B,Hkv,x_len,L]); the kernels never use it."""
        if x_len == 1:
            if self._seen_tokens == 0 and self._buf_k is None:
                return torch.ones(1, 1, 1, 1, dtype=torch.bool, device=self.device)
            n = self.n_ctx_data + 1
            return self._buf_valid[:, :, :n].view(torch.bool).unsqueeze(-2)
        if self._seen_tokens != 0:
            n_ctx = self.n_ctx_data
            t0 = n_ctx // self.chunk_size * self.chunk_size
            lim = F_.layout_row_limits(self._roles, self._buf_valid, self.size_global_kv, self.size_local_kv, x_len, t0,
                                       n_ctx - t0, self.sliding_queue_tail, self.chunk_size, self.sliding_window_size)
            L = n_ctx + x_len
            lim_tok = lim.repeat_interleave(self.chunk_size, -1)[..., :L].long()
            qpos = torch.arange(n_ctx, L, device=self.device)
            kpos = torch.arange(L, device=self.device)
            return (kpos[None, :] <= qpos[:, None])[None, None] & (qpos[None, None, :, None] <= lim_tok[:, :, None, :])
        return F_.dense_role_mask(self._roles, self.chunk_size, self.sliding_window_size, x_len)

    def prefill_attention(self, xq: torch.Tensor, sm_scale: float | None = None,
                          kept_tiles: torch.Tensor | None = None) -> torch.Tensor:
        """Attention of several new tokens over the existing cache; ``update`` must have appended their K/V.
        xq [B,Hq,x_len,D] -> [B,Hq,x_len,D].  The outputs are those one call over the whole sequence would give."""
        x_len = xq.shape[2]
        n_ctx = self.n_ctx_data
        t0 = n_ctx // self.chunk_size * self.chunk_size
        return F_.prefill_attention_past(xq, self._buf_k, self._buf_v, self._buf_valid, self._roles, self.size_global_kv,
                                         self.size_local_kv, t0, n_ctx - t0, self.sliding_queue_tail, self.chunk_size,
                                         self.sliding_window_size, sm_scale, kept_tiles)

    def decode_attention(self, xq: torch.Tensor, sm_scale: float | None = None) -> torch.Tensor:
        """Attention of one new token per sequence over the compacted cache, fused with its append.
        ``update(..., fused=True)`` must have been called with the token's K/V.  xq [B,Hq,1,D] -> [B,Hq,1,D]."""
        kb, vb = self._pending
        B, Hq, _, D = xq.shape
        fill = self.chunk_fill_size - 1
        self._grow(self._t0_bound + self.chunk_size + 1)
        qb = xq.to(torch.bfloat16).contiguous()
        o = torch.empty_like(qb)
        need = F_.decode_workspace_bytes(B, Hq, self.n_msks, D, self._t0_bound + self.chunk_size)
        if self._dec_ws is None or self._dec_ws.numel() < need:
            self._dec_ws = torch.zeros(F_.decode_workspace_bytes(B, Hq, self.n_msks, D, self._buf_k.shape[2] + self.chunk_size),
                                       dtype=torch.uint8, device=self.device)
        scale = (1.0 / math.sqrt(D)) if sm_scale is None else sm_scale
        F_.decode_fwd(qb, kb, vb, o, self._buf_k, self._buf_v, self._buf_valid, self.size_global_kv, self.size_local_kv,
                      self._state, fill, self._t0_bound, self.chunk_size, self.sliding_window_size, scale, self._dec_ws)
        return o if xq.dtype == torch.bfloat16 else o.to(xq.dtype)

    # ------------------------------------------------------------------ decode steps with static launch parameters
    def prepare_static_decode(self, n_steps: int, n_heads: int, head_dim: int) -> None:
        """Gets the cache ready for ``n_steps`` calls of ``decode_step_static`` that neither allocate nor read anything
        back, so that one such step can be recorded in a CUDA graph and replayed: buffers and workspace get room for the
        steps, and the counters the kernels need move into the device state words."""
        C = self.chunk_size
        t0 = self._t0()
        chunks = (self.chunk_fill_size + n_steps) // C + 1
        self._grow(t0 + chunks * C + C + 1)
        self._static_bound = self._buf_k.shape[2] - C
        need = F_.decode_workspace_bytes(self.bsz, n_heads, self.n_msks, head_dim, self._static_bound + C)
        if self._dec_ws is None or self._dec_ws.numel() < need:
            self._dec_ws = torch.zeros(need, dtype=torch.uint8, device=self.device)
        counters = torch.tensor([self.chunk_fill_size, self.sliding_queue_tail], dtype=torch.int32).to(self.device)
        self._state[4:6].copy_(counters)
        self._static_steps_left = n_steps

    def decode_step_static(self, xq: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, roles: torch.Tensor,
                           out: torch.Tensor, sm_scale: float | None = None, recording: bool = False) -> torch.Tensor:
        """One decode step -- append, attention, placement if the token completes a chunk -- as launches whose parameters
        do not change from step to step.  All tensors bf16 and contiguous: xq / out [B,Hq,1,D], k_new / v_new [B,Hkv,1,D];
        roles uint8 [B,Hkv] = role of the chunk this token completes (read on the device only if it does).  The host
        counters advance by one step.  While a graph is being recorded pass ``recording=True`` (the launches are captured, not
        run, so the host counters stay); after replaying the recorded step n times call ``note_static_steps(n)``."""
        D = xq.shape[-1]
        scale = (1.0 / math.sqrt(D)) if sm_scale is None else sm_scale
        F_.decode_step_fwd(xq, k_new, v_new, out, self._buf_k, self._buf_v, self._buf_valid, self.size_global_kv,
                           self.size_local_kv, self._state, self._static_bound, self.chunk_size, self.sliding_window_size,
                           scale, self._dec_ws)
        F_.decode_step_place(roles, self._buf_k, self._buf_v, self._buf_valid, self.size_global_kv, self.size_local_kv,
                             self._state, self.chunk_size, self.sliding_window_size)
        if not recording:
            self.note_static_steps(1)
        return out

    def note_static_steps(self, n: int) -> None:
        """Advances the host's view of the cache by ``n`` decode steps that ran on the device (recorded and replayed)."""
        if n > self._static_steps_left:
            raise RuntimeError('more static decode steps than prepare_static_decode() made room for')
        self._static_steps_left -= n
        C, SW = self.chunk_size, self.sliding_window_size
        done, fill = divmod(self.chunk_fill_size + n, C)
        self.chunk_fill_size = self.chunk_fill_size_last = fill
        self.sliding_queue_tail = (self.sliding_queue_tail + done * C) % SW
        self._seen_tokens += n
        self._unposted = 0
        self._pending = None
        if done:
            self._t0_bound += done * C
            self._t0_exact = None

    def post_update(self, x_len: int):
        self._seen_tokens += x_len
        self._unposted = 0
        if x_len == 0:
            return
        C, SW = self.chunk_size, self.sliding_window_size
        first = self._seen_tokens == x_len
        if first:
            self._evict_after_prefill(x_len)
            return
        if self.chunk_fill_size < C:
            self.chunk_fill_size_last = self.chunk_fill_size
            return
        if x_len != 1:
            self._evict_after_continuation()
            return
        # a chunk has just been completed by single-token steps: ring write + placement
        assert self._roles is not None
        roles = self._roles.reshape(self.bsz, self.n_msks, -1)[..., 0].contiguous()
        F_.decode_place(roles, self._buf_k, self._buf_v, self._buf_valid, self.size_global_kv, self.size_local_kv,
                        self._state, self.sliding_queue_tail, C, SW)
        self.sliding_queue_tail = (self.sliding_queue_tail + C) % SW
        self.chunk_fill_size = 0
        self.chunk_fill_size_last = 0
        self._t0_bound += C
        self._t0_exact = None
        self._pending = None
        if self._t0_bound - self._t0_synced >= max(8 * C, 512):
            self._t0()        # the bound drifts up when chunks are dropped: refresh it now and then (one small read)

    def _evict_after_continuation(self):
        """Compaction after a multi-token call over an existing cache (reference: the general branch of _post_update,
        :331-385).  Out of place: the old buffer, which holds the call's tokens behind the old tail offset, is the source."""
        C, SW = self.chunk_size, self.sliding_window_size
        n_tokens = self.chunk_fill_size                           # unfinished chunk before the call + the new tokens
        n_full, rem = divmod(n_tokens, C)
        B, H, _, D = self._buf_k.shape
        roles = self._roles
        if roles is None or roles.shape != (B, H, -(-n_tokens // C)):
            raise ValueError(f'token_states_info must describe {-(-n_tokens // C)} chunks')
        t0_old = self._t0()
        plan, self._plan = self._plan, None
        if plan is not None and plan[0] == ('past', n_tokens):
            _, rank, base, self.size_global_kv, self.size_local_kv, self._state, wait = plan
            t0 = wait()                                           # planned in update(), read back while the attention ran
            self._t0_exact = self._t0_bound = self._t0_synced = t0
        else:
            rank = torch.empty(B, H, roles.shape[-1], dtype=torch.int32, device=self.device)
            base = torch.empty(B, H, dtype=torch.int32, device=self.device)
            F_.evict_plan_past(roles, n_tokens, C, SW, rank, base, self.size_global_kv, self.size_local_kv, self._state)
            self._t0_exact = None
            t0 = self._t0()                                       # one host read
        old = (self._buf_k, self._buf_v, self._buf_valid)
        self._alloc(math.ceil((t0 + rem) / C) * C + self.headroom, D)
        F_.evict_compact_past(*old, roles, rank, base, self.size_global_kv, self.size_local_kv, self._state, n_tokens, C, SW,
                              t0_old, self.sliding_queue_tail, self._buf_k, self._buf_v, self._buf_valid)
        self.sliding_queue_tail = (self.sliding_queue_tail + min(n_full, self.n_chunks_per_sw) * C) % SW
        self.chunk_fill_size = rem
        self.chunk_fill_size_last = rem
        self._pending = None

    def _plan_ahead_past(self):
        """The same for a multi-token call over an existing cache: the plan works on copies of the size tensors, because
        the attention of this call still reads the sizes as they are."""
        C, SW = self.chunk_size, self.sliding_window_size
        n_tokens = self.chunk_fill_size
        roles = self._roles
        self._plan = None
        if roles is None or n_tokens < C or roles.shape != (self.bsz, self.n_msks, -(-n_tokens // C)):
            return
        self._t0()                                                # the exact tail offset before the plan replaces the state word
        dev = self.device
        rank = torch.empty(self.bsz, self.n_msks, roles.shape[-1], dtype=torch.int32, device=dev)
        base = torch.empty(self.bsz, self.n_msks, dtype=torch.int32, device=dev)
        sg, sl = self.size_global_kv.clone(), self.size_local_kv.clone()
        state = torch.zeros(8, dtype=torch.int32, device=dev)
        F_.evict_plan_past(roles, n_tokens, C, SW, rank, base, sg, sl, state)
        self._plan = (('past', n_tokens), rank, base, sg, sl, state, F_.read_word_async(state))

    def _plan_ahead(self, N: int):
        """The keep-set of a first call depends on the roles only, so it is planned as soon as ``update`` knows them: the
        plan kernel runs in front of the attention kernel and the size of the compacted cache travels to the host while
        the attention runs.  ``post_update`` then finds it there instead of stalling the stream with a read-back.
        The cache's own size tensors change in ``post_update`` only, as in the reference."""
        C, SW = self.chunk_size, self.sliding_window_size
        roles = self._roles
        nc = -(-N // C)
        if roles is None or N < C or not roles.is_cuda or roles.shape != (self.bsz, self.n_msks, nc):
            self._plan = None
            return
        dev = self.device
        rank = torch.empty(self.bsz, self.n_msks, nc, dtype=torch.int32, device=dev)
        sg = torch.empty(self.bsz, self.n_msks, dtype=torch.long, device=dev)
        sl = torch.empty_like(sg)
        state = torch.zeros(8, dtype=torch.int32, device=dev)
        F_.evict_plan(roles, N, C, SW, rank, sg, sl, state)
        self._plan = (N, rank, sg, sl, state, F_.read_word_async(state))

    def _evict_after_prefill(self, x_len: int):
        C, SW = self.chunk_size, self.sliding_window_size
        k, v = self._pending
        self._pending = None
        kb = k.to(torch.bfloat16).contiguous()
        vb = v.to(torch.bfloat16).contiguous()
        B, H, N, D = kb.shape
        rem = N % C
        n_full = N // C
        nc = -(-N // C)
        roles = self._roles
        if roles is None or roles.shape != (B, H, nc):
            raise ValueError(f'token_states_info must describe {nc} chunks')
        if n_full == 0:
            # less than one chunk: nothing is evicted, the tokens wait behind the (empty) ring  (reference :264-268)
            cap = SW + C + self.headroom
            self._alloc(cap, D)
            self._buf_k.zero_(); self._buf_v.zero_(); self._buf_valid.zero_()
            self._buf_k[:, :, SW:SW + N] = kb
            self._buf_v[:, :, SW:SW + N] = vb
            self._buf_valid[:, :, SW:SW + N].fill_(1)
            self.chunk_fill_size_last = self.chunk_fill_size
            return
        plan, self._plan = self._plan, None
        if plan is not None and plan[0] == N:
            _, rank, self.size_global_kv, self.size_local_kv, self._state, wait = plan
            t0 = wait()                                           # the 4 bytes left the device before the attention started
            self._t0_exact = self._t0_bound = self._t0_synced = t0
        else:
            rank = torch.empty(B, H, nc, dtype=torch.int32, device=self.device)
            F_.evict_plan(roles, N, C, SW, rank, self.size_global_kv, self.size_local_kv, self._state)
            self._t0_exact = None
            t0 = self._t0()                                       # one host read
        cap = math.ceil((t0 + rem) / C) * C + self.headroom
        self._alloc(cap, D)
        F_.evict_compact(kb, vb, roles, rank, self.size_global_kv, self.size_local_kv, self._state, C, SW,
                         self._buf_k, self._buf_v, self._buf_valid)
        n_upd = min(n_full, self.n_chunks_per_sw)
        self.sliding_queue_tail = (n_upd * C) % SW
        self.chunk_fill_size = rem
        self.chunk_fill_size_last = rem


class NAtSCache:
    """Per-model container: one ``NAtSChunkLayerCache`` per layer plus the pooled hidden states the role head
    needs across decode steps (reference: dyn_cache.py:66-195).

    ``chunk_size == 1`` is the token-granular cache (one role per token; the reference's ``NAtSLayerCache``,
    nats_layer_cache.py:20): the same layer cache with one-token chunks.  After a prefill its sizes and kept tokens are
    those of the reference.  Single tokens are placed as soon as they arrive, so every output follows the one-call rule
    exactly; the reference defers placement by up to ``update_chunk_size = 16`` steps (:196-223, 300-310), during which
    tokens stay visible past their rule, and agrees with this cache on the step after each of its batched updates."""

    def __init__(self, sliding_window_size: int, chunk_size: int = 1):
        self.cache_model: list[NAtSChunkLayerCache] = []
        self.sliding_window_size = sliding_window_size
        self.chunk_size = chunk_size
        self.cached_x: list[torch.Tensor | None] = []

    def reset_cache(self):
        self.cache_model = []
        self.cached_x = []

    def get_seq_length(self, layer_idx: int = 0) -> int:
        if len(self.cache_model) <= layer_idx:
            return 0
        return self.cache_model[layer_idx]._seen_tokens

    # what a Hugging Face model asks of the object passed as ``past_key_values`` (the reference derives from DynamicCache)
    is_compileable = False

    def get_mask_sizes(self, query_length, layer_idx: int = 0):
        n = query_length.shape[0] if isinstance(query_length, torch.Tensor) else int(query_length)
        return self.get_seq_length(layer_idx) + n, 0

    def generate_mask(self, layer_idx: int, x_len: int):
        return self.cache_model[layer_idx].generate_mask(x_len)

    def get_nats_chunk_fill_size(self, layer_idx: int = 0):
        if len(self.cache_model) <= layer_idx or self.chunk_size == 1:
            return 0
        return self.cache_model[layer_idx].chunk_fill_size

    def get_nats_cached_x_in_chunk(self, layer_idx: int = 0):
        return self.cached_x[layer_idx] if layer_idx < len(self.cached_x) else None

    def _set_cached_x(self, x, layer_idx: int):
        while len(self.cached_x) <= layer_idx:
            self.cached_x.append(None)
        self.cached_x[layer_idx] = x

    @staticmethod
    def merge_new_x_values_in_chunk(x_cache, x_new, chunk_size: int, chunk_merge_method: str = 'mean'):
        """Running pooled hidden state of an unfinished chunk: sum of x / C for 'mean', running max for 'max'."""
        if chunk_merge_method == 'mean':
            part = (x_new / chunk_size).sum(1, keepdim=True)
            return part if x_cache is None else x_cache + part
        if x_cache is None:
            return x_new if x_new.shape[1] == 1 else x_new.max(1, keepdim=True)[0]
        return torch.cat([x_cache, x_new], 1).max(1, keepdim=True)[0]

    def update_nats_cached_x_in_chunk(self, x, layer_idx: int = 0, chunk_merge_method: str = 'mean'):
        cur = self.get_nats_cached_x_in_chunk(layer_idx)
        self._set_cached_x(self.merge_new_x_values_in_chunk(cur, x, self.chunk_size, chunk_merge_method), layer_idx)

    def update_nats_cached_x_across_chunk(self, x, pre_fill_chunk_size: int, layer_idx: int = 0,
                                          chunk_merge_method: str = 'mean'):
        """Pools ``x`` [B,T,dim] per chunk, starting inside an unfinished chunk if there is one.  Returns
        ``(pooled [B,n_chunks,dim], pad_size)``; the pooled state of a trailing unfinished chunk is kept for later."""
        C = self.chunk_size
        pre = self.get_nats_chunk_fill_size(layer_idx)
        T = x.shape[1]

        def pool(t, pad):
            if pad:
                t = torch.nn.functional.pad(t, (0, 0, 0, pad))
            t = t.unflatten(1, (-1, C))
            return t.mean(2) if chunk_merge_method == 'mean' else t.max(2)[0]

        if pre != 0:
            head = C - pre
            first = self.merge_new_x_values_in_chunk(self.get_nats_cached_x_in_chunk(layer_idx), x[:, :head], C,
                                                     chunk_merge_method)
            rest = T - head
            if rest == 0:
                pad, pooled = 0, first
            else:
                pad = get_pad_size(rest, C)
                pooled = torch.cat([first, pool(x[:, head:], pad)], 1)
        else:
            pad = get_pad_size(T, C)
            pooled = pool(x, pad)
        if pad == 0:
            self._set_cached_x(None, layer_idx)
        else:
            last = x[:, pad - C:]
            self._set_cached_x(self.merge_new_x_values_in_chunk(None, last, C, chunk_merge_method), layer_idx)
        return pooled, pad

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs: dict[str, Any] | None = None):
        while len(self.cache_model) <= layer_idx:
            bsz, n_kv_heads = key_states.shape[:2]
            self.cache_model.append(NAtSChunkLayerCache(bsz, n_kv_heads, self.sliding_window_size,
                                                        layer_id=len(self.cache_model), chunk_size=self.chunk_size,
                                                        device=key_states.device))
        return self.cache_model[layer_idx].update(key_states, value_states, **(cache_kwargs or {}))

    def post_update(self, layer_idx: int, x_len=1, **kwargs):
        self.cache_model[layer_idx].post_update(x_len=x_len, **kwargs)
