"""CPU oracle for the NAtS attention hot path.  TEST INFRASTRUCTURE ONLY.

This module is the checker, never the product: only the test-suite, the smoke check and the
CPU-baseline legs of the benchmark may import it.  Nothing in ``neuralattentionsearch_b200``
imports it, and the product path raises when its CUDA library is missing instead of
falling back to anything here.

It restates, in plain numpy/torch on the host, what the reference's *eager PyTorch* path
computes for one attention layer (paths are relative to the reference project root):

* role mask of the chunked prefill     src/nats/components/cache/nats_chunk_layer_cache.py:589-620
                                       src/nats/components/masks/utils.py:81-94
* masked attention                     src/nats/models/transformer/attention/nats_chunk_attention.py:130-149
* cache append                         src/nats/components/cache/nats_chunk_layer_cache.py:171-256
* sliding-window ring fill             src/nats/components/cache/nats_chunk_layer_cache.py:391-437
* keep-set / ranks / compaction        src/nats/components/cache/nats_chunk_layer_cache.py:715-868
                                       src/nats/components/cache/cache_update.py:25-76
* size / validity bookkeeping          src/nats/components/cache/nats_chunk_layer_cache.py:262-385,634-656
* decode mask and decode attention     src/nats/components/cache/nats_chunk_layer_cache.py:622-632
* multi-token call over a cache        src/nats/components/cache/nats_chunk_layer_cache.py:239-256,444-511,658-713 (mask),
                                       :331-385 (eviction); one deviation, marked where it is made: the unfinished chunk
                                       is always moved (:840 leaves it behind in one corner case)
* training-forward statistics          src/nats/models/transformer/triton/nats_chunk_attention.py:131-133,319-330
                                       (the log-sum-exp has no reference output to pin against: Triton only)
* token-granular cache after a prefill src/nats/components/cache/nats_layer_cache.py (the chunk cache with one-token chunks
                                       reproduces its sizes and kept tokens; its deferred single-token updates are not restated)

Parity pin: the reference ships no golden vectors or known-answer tests for this path, so the
oracle is pinned against outputs of the reference's own code, imported and executed on CPU by
``tests/golden/make_golden.py``; the resulting fixtures are committed under ``tests/golden/`` and
checked by ``tests/test_oracle_golden.py`` (first calls + decode steps, segmented calls ``seg_*``,
token-granular prefills ``tok_*``).

Role codes: 0 = global, 1 = local, 2 = sliding window (column order of ``token_states_info``,
nats_chunk_layer_cache.py:188-190).
"""
from __future__ import annotations

import math

import numpy as np
import torch

ROLE_GLOBAL, ROLE_LOCAL, ROLE_SLIDING = 0, 1, 2
NO_LIMIT = np.iinfo(np.int32).max


# --------------------------------------------------------------------------------------------
# synthetic inputs (shared by tests and the benchmark's CPU legs)
# --------------------------------------------------------------------------------------------
def role_bias_for_mix(p_global: float, p_local: float) -> tuple[float, float, float]:
    """Biases b such that argmax(N(0,1)^3 + b) has roughly the requested mix (solved by bisection on
    a fixed 200k-sample Monte-Carlo table, deterministic)."""
    rng = np.random.default_rng(12345)
    z = rng.standard_normal((200_000, 3))
    bg, bl = 0.0, 0.0
    for _ in range(40):
        r = np.argmax(z + np.array([bg, bl, 0.0]), -1)
        bg += 0.5 * (math.log(max(p_global, 1e-6)) - math.log(max((r == 0).mean(), 1e-6)))
        bl += 0.5 * (math.log(max(p_local, 1e-6)) - math.log(max((r == 1).mean(), 1e-6)))
    return float(bg), float(bl), 0.0


def make_roles(B: int, Hkv: int, Nc: int, p_global: float, p_local: float, seed: int,
               force_first_global: bool = True) -> np.ndarray:
    """uint8 role codes [B,Hkv,Nc] from 3-way N(0,1) logits plus a bias, argmax (first max wins)."""
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(B, Hkv, Nc, 3, generator=g)
    logits = logits + torch.tensor(role_bias_for_mix(p_global, p_local))
    roles = logits.argmax(-1).to(torch.uint8).numpy()
    if force_first_global and Nc > 0:
        roles[..., 0] = ROLE_GLOBAL          # nats_attention.py:104-105 (chunk 0 is the sink)
    return roles


def onehot_from_roles(roles: np.ndarray, dtype=torch.float32) -> torch.Tensor:
    return torch.nn.functional.one_hot(torch.from_numpy(roles.astype(np.int64)), 3).to(dtype)


# --------------------------------------------------------------------------------------------
# role mask
# --------------------------------------------------------------------------------------------
def next_global_index(roles: np.ndarray) -> np.ndarray:
    """fill[c] = smallest j >= c whose chunk is global, the last chunk counting as global.

    masks/utils.py:85-87 (``end_seqs_hard[..., -1] = 1`` then a reversed cummax of indices)."""
    roles = np.asarray(roles)
    Nc = roles.shape[-1]
    is_g = roles == ROLE_GLOBAL
    is_g = is_g.copy()
    is_g[..., -1] = True
    idx = np.where(is_g, np.arange(Nc), Nc)           # Nc = "none yet"
    return np.minimum.accumulate(idx[..., ::-1], axis=-1)[..., ::-1].astype(np.int64)


def row_limit(roles: np.ndarray, C: int, SW: int) -> np.ndarray:
    """lim[c] = last query row (token index) that may still see KV chunk c.

    global (or last chunk, unless sliding) -> no limit; sliding -> c*C + SW + C - 1
    (nats_chunk_layer_cache.py:603-611: chunk distance <= SW//C overrides the segment mask wherever
    the chunk is a sliding one); local -> (fill[c]+1)*C - 1 (masks/utils.py:92)."""
    roles = np.asarray(roles)
    Nc = roles.shape[-1]
    fill = next_global_index(roles)
    c = np.arange(Nc, dtype=np.int64)
    lim = (fill + 1) * C - 1
    is_gf = (roles == ROLE_GLOBAL)
    is_gf = is_gf.copy()
    is_gf[..., -1] = True
    lim = np.where(is_gf, NO_LIMIT, lim)
    lim = np.where(roles == ROLE_SLIDING, c * C + SW + C - 1, lim)
    return lim.astype(np.int64)


def visible_mask(roles: np.ndarray, C: int, SW: int, N: int, q_lo: int = 0, q_hi: int | None = None) -> np.ndarray:
    """bool [B,Hkv,q_hi-q_lo,N]: may query row q see key k (first prefill call, no past)."""
    q_hi = N if q_hi is None else q_hi
    lim = row_limit(roles, C, SW)                                  # [B,H,Nc]
    lim_tok = np.repeat(lim, C, axis=-1)[..., :N]                  # [B,H,N]
    q = np.arange(q_lo, q_hi, dtype=np.int64)[:, None]
    k = np.arange(N, dtype=np.int64)[None, :]
    return (q >= k)[None, None] & (q[None, None] <= lim_tok[:, :, None, :])


def kept_tiles(roles: np.ndarray, C: int, SW: int, N: int, tile: int = 128) -> np.ndarray:
    """int64 [B,Hkv]: number of (q tile, kv tile) pairs of size tile x tile holding a visible entry."""
    lim = row_limit(roles, C, SW)
    lim_tok = np.repeat(lim, C, axis=-1)[..., :N]
    nt = (N + tile - 1) // tile
    pad = nt * tile - N
    lim_tok = np.pad(lim_tok, [(0, 0), (0, 0), (0, pad)], constant_values=-1)
    tmax = lim_tok.reshape(*lim_tok.shape[:2], nt, tile).max(-1)   # [B,H,nt]
    t = np.arange(nt)
    keep = (t[None, :] <= t[:, None])[None, None] & (tmax[:, :, None, :] >= (t * tile)[None, None, :, None])
    return keep.sum((-1, -2))


def masked_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor,
                     sm_scale: float | None = None) -> torch.Tensor:
    """softmax(q k^T * s + mask) v in fp32; q [B,Hq,S,D], k/v [B,Hkv,L,D], mask bool [B,Hkv,S,L].

    nats_chunk_attention.py:132-149 (mask repeated per query head of a group, transformer/utils.py:35-46)."""
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    n_rep = Hq // Hkv
    s = (1.0 / math.sqrt(D)) if sm_scale is None else sm_scale
    qf = q.float().view(B, Hkv, n_rep, S, D)
    kf, vf = k.float(), v.float()
    sc = torch.einsum('bgrsd,bgld->bgrsl', qf, kf) * s
    sc = sc.masked_fill(~mask[:, :, None], float('-inf'))
    p = torch.softmax(sc, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    out = torch.einsum('bgrsl,bgld->bgrsd', p, vf)
    return out.reshape(B, Hq, S, D)


def prefill_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, roles: np.ndarray, C: int, SW: int,
                      sm_scale: float | None = None, block: int = 1024,
                      rows: tuple[int, int] | None = None) -> torch.Tensor:
    """Role-masked causal attention of the first prefill call, fp32, evaluated in query-row blocks so
    that the dense [N,N] mask of the reference is never materialised.  ``rows=(lo,hi)`` restricts the
    evaluation to those query rows (used for spot checks at full benchmark sizes)."""
    B, Hq, N, D = q.shape
    lo, hi = (0, N) if rows is None else rows
    outs = []
    for r0 in range(lo, hi, block):
        r1 = min(hi, r0 + block)
        m = torch.from_numpy(visible_mask(roles, C, SW, N, r0, r1)[..., :r1])
        outs.append(masked_attention(q[:, :, r0:r1], k[:, :, :r1], v[:, :, :r1], m, sm_scale))
    return torch.cat(outs, dim=2)


def prefill_stats(q: torch.Tensor, k: torch.Tensor, roles: np.ndarray, C: int, SW: int,
                  sm_scale: float | None = None, block: int = 1024) -> tuple[torch.Tensor, np.ndarray]:
    """The two per-row statistics the reference's training forward stores for its backward
    (triton/nats_chunk_attention.py:131-133, 319-330): ``M = m_i + log2(l_i)`` = log2 of the sum over the visible keys of
    exp2(q.k * sm_scale * log2 e), fp32 [B,Hq,N], and ``N_VALID_BLOCKS`` = number of visible keys per row (the mask summed
    over the computed blocks), int32 [B,Hq,N].  The mask is the eager one, as everywhere in this file."""
    B, Hq, N, D = q.shape
    Hkv = k.shape[1]
    n_rep = Hq // Hkv
    scale = (1.0 / math.sqrt(D) if sm_scale is None else sm_scale) * 1.4426950408889634
    lse, cnt = [], []
    for r0 in range(0, N, block):
        r1 = min(N, r0 + block)
        m = torch.from_numpy(visible_mask(roles, C, SW, N, r0, r1)[..., :r1])            # [B,Hkv,rows,r1]
        s = torch.einsum('bhqd,bhkd->bhqk', q[:, :, r0:r1].float(), k[:, :, :r1].float().repeat_interleave(n_rep, 1)) * scale
        s = s.masked_fill(~m.repeat_interleave(n_rep, 1), float('-inf'))
        lse.append(torch.logsumexp(s * math.log(2.0), -1) / math.log(2.0))
        cnt.append(m.sum(-1).repeat_interleave(n_rep, 1).numpy().astype(np.int32))
    return torch.cat(lse, 2), np.concatenate(cnt, 2)


# --------------------------------------------------------------------------------------------
# per-layer chunk cache state machine
# --------------------------------------------------------------------------------------------
class ChunkCacheOracle:
    """Restatement of ``NAtSChunkLayerCache`` (nats_chunk_layer_cache.py:15) for one first prefill call
    followed by single-token decode steps.  Arrays are numpy; the physical layout is the reference's:
    ``cache_k/v [B,H,L,D] = [ring (SW) | kept chunks | pending tail]``."""

    def __init__(self, B: int, H: int, SW: int, C: int):
        assert SW % C == 0                                        # :47
        self.B, self.H, self.SW, self.C = B, H, SW, C
        self.size_local = np.zeros((B, H), np.int64)              # :31
        self.size_global = np.full((B, H), SW, np.int64)          # :32
        self.chunk_fill = 0
        self.tail = 0                                             # sliding_queue_tail
        self.n_ctx_data = SW                                      # :64
        self.seen = 0
        self.cache_k = self.cache_v = None
        self.valid = None
        self.roles = None
        self.gmin = SW                                            # _n_global_min, :54

    # -- update (append) -- :171-256
    def update(self, k: np.ndarray, v: np.ndarray, roles: np.ndarray | None):
        B, H, x_len, D = k.shape
        self.chunk_fill += x_len
        self.roles = roles
        if self.cache_k is None:                                  # :215-237
            pad = (-x_len) % self.C
            z = np.zeros((B, H, self.SW, D), k.dtype)
            p = np.zeros((B, H, pad, D), k.dtype)
            self.cache_k = np.concatenate([z, k, p], 2)
            self.cache_v = np.concatenate([z, v, p], 2)
            self.valid = np.zeros((B, H, self.SW + x_len + pad), bool)
            self.valid[:, :, self.SW:self.SW + x_len] = True
            return k, v
        fill_start = self.n_ctx_data                              # :243-256
        score = fill_start + x_len
        need = math.ceil(score / self.C) * self.C
        grow = need - self.cache_k.shape[2]
        if grow > 0:
            self.cache_k = np.pad(self.cache_k, [(0, 0), (0, 0), (0, grow), (0, 0)])
            self.cache_v = np.pad(self.cache_v, [(0, 0), (0, 0), (0, grow), (0, 0)])
            self.valid = np.pad(self.valid, [(0, 0), (0, 0), (0, grow)])
        self.cache_k[:, :, fill_start:score] = k
        self.cache_v[:, :, fill_start:score] = v
        self.valid[:, :, fill_start:score] = True
        return self.cache_k[:, :, :score], self.cache_v[:, :, :score]

    # -- decode mask -- :622-632
    def decode_mask(self) -> np.ndarray:
        return self.valid[:, :, :self.n_ctx_data + 1]

    # -- mask of a multi-token call over an existing cache -- :444-511, 589-620, 658-713
    def layout_row_limit(self) -> np.ndarray:
        """Call after ``update`` of a multi-token continuation.  int64 [B,H,T0/C + Nc_new]: for every chunk of the
        physical layout ``[ring | kept | gap | unfinished chunk + new tokens]`` the last cache POSITION of a query that
        may still see it (a query token sits at the position its own K/V was appended to); -1 = never.

        The reference builds the same mask from three pieces: ring slots by their age in the queue
        (``_fit_sliding_queue_masks`` :658-713: a slot written a chunks before the newest stays visible while the
        query's chunk is at most SW/C - 1 - a chunks into the new tokens), kept local chunks until the first global chunk of
        the new tokens (:479-491), kept global chunks always, and the new tokens by the rule of a first call
        (``_generate_local_mask`` :589-620) -- together: the first-call rule applied to the whole logical sequence."""
        C, SW = self.C, self.SW
        W = SW // C
        t0 = self.n_ctx_data // C * C
        n_old = t0 // C
        lim_new = row_limit(self.roles, C, SW)                                  # [B,H,Nc_new], rows counted from t0
        lim_new = np.where(lim_new >= NO_LIMIT, NO_LIMIT, lim_new + t0)
        fill = next_global_index(self.roles)[..., 0]                            # first global (or last) new chunk
        lim_local = t0 + (fill + 1) * C - 1
        lim = np.full((self.B, self.H, n_old), -1, np.int64)
        j = np.arange(n_old)
        sg, sl = self.size_global // C, self.size_local // C
        lim = np.where((j[None, None] >= W) & (j[None, None] < sg[..., None]), NO_LIMIT, lim)
        is_loc = (j[None, None] >= sg[..., None]) & (j[None, None] < (sg + sl)[..., None])
        lim = np.where(is_loc, lim_local[..., None], lim)
        age = (self.tail // C - 1 - np.arange(W)) % W                            # 0 = newest slot
        ring_valid = self.valid[:, :, :SW:C]                                     # a slot holds one chunk
        lim[..., :W] = np.where(ring_valid, t0 + (W - age) * C - 1, -1)
        return np.concatenate([lim, lim_new], -1)

    def prefill_mask_past(self, x_len: int) -> np.ndarray:
        """bool [B,H,x_len,n_ctx_data + x_len] of a multi-token call over an existing cache (after ``update``)."""
        C = self.C
        L = self.n_ctx_data + x_len
        lim = np.repeat(self.layout_row_limit(), C, axis=-1)[..., :L]
        qpos = np.arange(self.n_ctx_data, L, dtype=np.int64)[:, None]
        k = np.arange(L, dtype=np.int64)[None, :]
        return (k <= qpos)[None, None] & (qpos[None, None] <= lim[:, :, None, :])

    def prefill_attention_past(self, q: torch.Tensor, x_len: int, sm_scale: float | None = None) -> torch.Tensor:
        """Attention of the x_len new queries over the cache that ``update`` has just extended
        (nats_chunk_attention.py:131-142 with the mask of :444-511).  q [B,Hq,x_len,D] -> fp32 [B,Hq,x_len,D]."""
        L = self.n_ctx_data + x_len
        mask = torch.from_numpy(self.prefill_mask_past(x_len))
        k = torch.from_numpy(np.ascontiguousarray(self.cache_k[:, :, :L]))
        v = torch.from_numpy(np.ascontiguousarray(self.cache_v[:, :, :L]))
        return masked_attention(q, k, v, mask, sm_scale)

    # -- ring fill -- :391-437
    def _ring_fill(self, n_new_chunks: int, n_rem: int, x_len: int):
        C, SW = self.C, self.SW
        n_upd = min(n_new_chunks, SW // C)
        n_fills = n_upd * C
        if self.seen == x_len:
            idx = np.arange(n_fills)
            self.tail = n_fills % SW
        else:
            idx = (np.arange(n_fills) + self.tail) % SW
            self.tail = (self.tail + n_fills) % SW
        Nc = self.roles.shape[-1]
        last = Nc - 1 if n_rem > 0 else Nc                          # drop the unfinished chunk
        is_sw = (self.roles[..., last - n_upd:last] == ROLE_SLIDING)
        is_sw_tok = np.repeat(is_sw, C, axis=-1)                    # [B,H,n_fills]
        s0 = (self.n_ctx_data // C + (n_new_chunks - n_upd)) * C
        for name in ('cache_k', 'cache_v'):
            cache = getattr(self, name)
            src = cache[:, :, s0:s0 + n_fills].copy()
            cache[:, :, idx] = np.where(is_sw_tok[..., None], src, 0)
        self.valid[:, :, idx] = is_sw_tok

    # -- post_update -- :262-385
    def post_update(self, x_len: int):
        C = self.C
        self.seen += x_len
        if x_len == 0 or self.chunk_fill < C:                       # :264-268
            self.n_ctx_data += x_len
            return
        n_rem = self.chunk_fill % C
        n_new = self.chunk_fill // C
        self._ring_fill(n_new, n_rem, x_len)
        self.chunk_fill = n_rem
        roles = self.roles
        if (roles == ROLE_SLIDING).all():                           # :283-288
            self.n_ctx_data = int((self.size_global + self.size_local).max()) + self.chunk_fill
            return
        size_update_global = 0
        if x_len == 1:                                              # :289-330
            t0 = self.n_ctx_data // C * C
            is_g = roles[..., 0] == ROLE_GLOBAL
            is_s = roles[..., -1] == ROLE_SLIDING
            dst = np.where(is_g, self.size_global, self.size_global + self.size_local)
            for name in ('cache_k', 'cache_v'):
                cache = getattr(self, name)
                new = cache[:, :, t0:t0 + C].copy()
                for b in range(self.B):
                    for h in range(self.H):
                        cache[b, h, dst[b, h]:dst[b, h] + C] = new[b, h]
            upd_local = (self.size_local // C + 1) * is_g + is_s
            self.size_global += is_g * C
            self.size_local -= upd_local * C
        else:                                                       # :331-355, 715-868
            size_update_global = self._compact_prefill(n_rem)
        self.size_local += n_new * C                                # :356
        assert not (self.size_local < 0).any()
        self.n_ctx_data = int((self.size_global + self.size_local).max()) + self.chunk_fill
        self.cache_k[:, :, self.n_ctx_data:] = 0                    # :361-362
        self.cache_v[:, :, self.n_ctx_data:] = 0
        self._mask_invalid()                                        # :364-370
        self.gmin = int(self.size_global.min())                     # :371
        if self.seen == x_len:                                      # :373-378
            keep = math.ceil(self.n_ctx_data / C) * C
            self.cache_k = np.ascontiguousarray(self.cache_k[:, :, :keep])
            self.cache_v = np.ascontiguousarray(self.cache_v[:, :, :keep])
            self.valid = np.ascontiguousarray(self.valid[:, :, :keep])

    def _compact_prefill(self, n_rem: int):
        """get_updated_cache_info (:715-868) + merge_local_to_global_caches (cache_update.py:65-74)."""
        C, B, H = self.C, self.B, self.H
        roles = self.roles
        Nc = roles.shape[-1]
        # The reference returns early when every chunk of every head is local (:747-749): nothing is moved.  That is
        # only right while every head is as long as the longest one (a first call); in a later call a shorter head would
        # keep its new tokens behind the gap.  The early exit is taken where it is right, the general path otherwise.
        if (roles == ROLE_LOCAL).all() and ((self.size_global + self.size_local) == self.n_ctx_data // C * C).all():
            return 0
        is_g = roles == ROLE_GLOBAL
        n_g = is_g.sum(-1)
        g_idx = np.where(is_g, np.arange(Nc), -1)
        if n_rem != 0:                                              # :782-786
            n_g = n_g - 1
            g_idx[..., -1] = -1
        last_g = g_idx.max(-1)                                      # [B,H]
        after = np.arange(Nc)[None, None] > last_g[..., None]
        rem_local = np.where(after, roles == ROLE_LOCAL, False)
        upd_local = np.where(last_g > -1, last_g * C + self.size_local, 0)
        n_sw = Nc - np.maximum(last_g, 0) - rem_local.sum(-1)       # :797
        if n_rem != 0:
            n_sw = n_sw - 1
        upd_local = upd_local + n_sw * C
        keep = is_g | rem_local
        if n_rem != 0:
            keep[..., -1] = False                                   # :809-811
        counts = keep.sum(-1)
        base = np.where(last_g == -1, (self.size_global + self.size_local) // C, self.size_global // C)
        src_base = self.n_ctx_data // C
        # The reference moves the unfinished chunk only if no head kept every completed chunk of the call (:840); that leaves
        # it behind when such a head is not the longest one (multi-token call over an existing cache).  Moving it whenever it
        # exists is the same operation wherever the reference is self-consistent (source == destination there).
        move_tail = n_rem != 0
        tail_dst = int((counts + base).max())
        for name in ('cache_k', 'cache_v'):
            cache = getattr(self, name)
            D = cache.shape[-1]
            view = cache.reshape(B, H, -1, C, D)
            gathered = {}
            for b in range(B):
                for h in range(H):
                    src = np.nonzero(keep[b, h])[0] + src_base
                    gathered[b, h] = view[b, h, src].copy()         # gather everything first (.clone())
                    if move_tail:
                        gathered[b, h, 't'] = view[b, h, Nc - 1 + src_base].copy()
            for b in range(B):
                for h in range(H):
                    n = counts[b, h]
                    view[b, h, base[b, h]:base[b, h] + n] = gathered[b, h]
                    if move_tail:
                        view[b, h, tail_dst] = gathered[b, h, 't']
        self.size_global = self.size_global + n_g * C
        self.size_local = self.size_local - upd_local
        return n_g * C

    def _mask_invalid(self):                                        # :634-656
        gmin = self.gmin
        if self.n_ctx_data == gmin:
            return
        n_last = self.n_ctx_data // self.C * self.C
        idx = np.arange(n_last - gmin)[None, None]
        lens = (self.size_global + self.size_local - gmin)[..., None]
        self.valid[:, :, gmin:n_last] = idx < lens
        self.valid[:, :, n_last:n_last + self.chunk_fill] = True

    # -- canonical view of the defined state, used for comparisons with the CUDA path --
    def lens(self) -> np.ndarray:
        return self.size_global + self.size_local

    def defined_state(self) -> dict:
        """The parts of the state the reference defines (stale regions between a head's own length and
        the common tail offset are excluded)."""
        C = self.C
        t0 = self.n_ctx_data // C * C
        fill = self.n_ctx_data - t0
        return dict(size_global=self.size_global.copy(), size_local=self.size_local.copy(),
                    n_ctx_data=int(self.n_ctx_data), chunk_fill=int(self.chunk_fill), tail=int(self.tail),
                    t0=int(t0), fill=int(fill))


def decode_attention(q: torch.Tensor, cache_k: np.ndarray, cache_v: np.ndarray, mask: np.ndarray,
                     sm_scale: float | None = None) -> torch.Tensor:
    """One-row attention over the padded cache with the validity mask (nats_chunk_attention.py:131-142 with
    x_len == 1).  q [B,Hq,1,D]; cache [B,Hkv,L,D]; mask bool [B,Hkv,L]."""
    L = mask.shape[-1]
    k = torch.from_numpy(np.ascontiguousarray(cache_k[:, :, :L]))
    v = torch.from_numpy(np.ascontiguousarray(cache_v[:, :, :L]))
    return masked_attention(q, k, v, torch.from_numpy(mask[:, :, None, :].copy()), sm_scale)
