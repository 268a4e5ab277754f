"""Attention modules with the reference's constructor, parameter names and ``forward`` contract, running the
B200 kernels of this package.

Mirrors (inference only): ``AttentionLayer.forward`` (src/nats/models/transformer/attention/base_attention.py:259-283),
``BaseNAtSAttentionLayer`` (src/nats/models/transformer/attention/nats_attention.py:14-195) and
``BaseNAtSChunkAttentionLayer`` (src/nats/models/transformer/attention/nats_chunk_attention.py:19-157).
``state_dict`` keys are the reference's (``wq, wk, wv, wo, proj_layer``).  The projections are plain library GEMMs;
everything between them -- role mask, attention, cache append, eviction, decode -- is this package's CUDA.

Differences a caller can see: GQA is handled inside the kernels, so ``repeat_kv_values`` returns K/V unchanged;
``multi_head_attention`` ignores ``mask`` (it never materialises one); training mode raises (no backward here).
"""
from __future__ import annotations

import math

import torch
from torch import nn

from . import functional as F_
from .cache import NAtSCache, get_pad_size


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def apply_rotary_pos_emb(q, k, cos, sin, unsqueeze_dim: int = 1):
    """Rotary embedding in the half-rotation convention of the Llama family (what the reference imports from
    ``transformers.models.llama.modeling_llama``)."""
    cos, sin = cos.unsqueeze(unsqueeze_dim), sin.unsqueeze(unsqueeze_dim)
    return q * cos + rotate_half(q) * sin, k * cos + rotate_half(k) * sin


class BaseNAtSChunkAttentionLayer(nn.Module):
    def __init__(self, dim: int = 4096, n_heads: int = 32, n_kv_heads: int | None = None, layer_id: int = 0,
                 dropout: float = 0.0, use_flash: bool = True, on_ddp: bool = False, n_msks: int | None = None,
                 sparse_regularized_value: float = 0.0, local_seq_max_length: int = 4, n_options: int = 3,
                 chunk_size: int = 8, chunk_merge_method: str = 'mean', compress_on_q: bool = False):
        super().__init__()
        self.n_kv_heads = n_heads if n_kv_heads is None else n_kv_heads
        self.layer_id = layer_id
        self.n_local_heads = n_heads
        self.n_local_kv_heads = self.n_kv_heads
        self.n_rep = n_heads // self.n_kv_heads
        self.head_dim = dim // n_heads
        self.wq = nn.Linear(dim, n_heads * self.head_dim, bias=False)
        self.wk = nn.Linear(dim, self.n_kv_heads * self.head_dim, bias=False)
        self.wv = nn.Linear(dim, self.n_kv_heads * self.head_dim, bias=False)
        self.wo = nn.Linear(n_heads * self.head_dim, dim, bias=False)
        self.use_flash = self._use_flash = use_flash
        self.dropout = dropout
        if n_msks is None:
            n_msks = self.n_kv_heads
        if self.n_kv_heads % n_msks != 0:
            # base reference: mask head m covers n_heads // n_msks query heads (transformer/utils.py:35-46); the kernels
            # share one kept-tile list among the query heads of a kv-head, so a mask head must cover whole kv-heads
            raise ValueError(f'n_msks = {n_msks} must divide n_kv_heads = {self.n_kv_heads}: the kernels take one role per '
                             'kv-head (a role head shared by several kv-heads is expanded, one finer than a kv-head is not built)')
        if n_options != 3:
            raise ValueError('three roles (global, local, sliding window) are supported')
        self.proj_layer = nn.Linear(dim, n_msks * n_options, bias=False)
        self.n_msks, self.n_options = n_msks, n_options
        self.n_rep_msk = n_heads // n_msks
        self.sm_scale = 1 / math.sqrt(self.head_dim)
        self.sparse_regularized_value = sparse_regularized_value
        self.local_seq_max_length = local_seq_max_length
        self.global_token_enhanced_value = 0.1
        if chunk_merge_method not in ('mean', 'max'):
            raise ValueError(f'Unknown chunk merge method: {chunk_merge_method}')
        self.chunk_merge_method = chunk_merge_method
        self.chunk_size = chunk_size
        self.compress_on_q = compress_on_q
        self.executor = None
        self._cache_is_till_updating = None

    # ---- role sampling (reference: nats_chunk_attention.py:64-95, nats_attention.py:96-109) ----
    def _one_hot_global(self, like: torch.Tensor, bsz: int) -> torch.Tensor:
        oh = torch.zeros(bsz, self.n_kv_heads, 1, self.n_options, dtype=like.dtype, device=like.device)
        oh[..., 0].fill_(1)
        return oh

    def _roles_from_pooled(self, x_pooled: torch.Tensor, start_pos: int) -> torch.Tensor:
        logit = self.proj_layer(x_pooled).unflatten(-1, (self.n_msks, self.n_options))
        logit[..., 0] += self.global_token_enhanced_value
        index = logit.max(-1, keepdim=True)[1]
        if start_pos < self.chunk_size:
            index[:, 0].fill_(0)                             # the first chunk is the attention sink
        samples = torch.zeros_like(logit).scatter_(-1, index, 1.0)
        samples = samples.transpose(1, 2)                    # [B, n_msks, Nc, 3]
        if self.n_msks != self.n_kv_heads:                   # a role head shared by several kv-heads: one copy per kv-head
            samples = samples.repeat_interleave(self.n_kv_heads // self.n_msks, 1)
        return samples.contiguous()                          # [B, Hkv, Nc, 3]

    def _sample_for_token_info_values_inference(self, x: torch.Tensor, start_pos: int, cache: NAtSCache) -> torch.Tensor:
        x_len = x.shape[1]
        pre = cache.get_nats_chunk_fill_size(self.layer_id)
        if pre + x_len < self.chunk_size:
            cache.update_nats_cached_x_in_chunk(x, self.layer_id, self.chunk_merge_method)
            return self._one_hot_global(x, x.shape[0])       # placeholder until the chunk is complete
        pooled, pad = cache.update_nats_cached_x_across_chunk(x, pre, self.layer_id, self.chunk_merge_method)
        samples = self._roles_from_pooled(pooled, start_pos)
        if pad != 0:
            samples[:, :, -1] = self._one_hot_global(x, x.shape[0])[:, :, 0]   # unfinished last chunk counts as global
        return samples

    # ---- hooks of the reference's forward ----
    def add_rotary_emb(self, xq, xk, pos_emb):
        if pos_emb is not None:
            cos, sin = pos_emb
            xq, xk = apply_rotary_pos_emb(xq, xk, cos, sin)
        return xq, xk

    def prepare_x_values(self, x, bsz: int, seqlen: int, pos_emb, start_pos: int = 0, cache: NAtSCache | None = None):
        if self.training:
            raise NotImplementedError('this build covers inference; the training path (gumbel roles + backward) is out of scope')
        xq, xk, xv = self.wq(x), self.wk(x), self.wv(x)
        token_states_info = self._sample_for_token_info_values_inference(x, start_pos=start_pos, cache=cache)
        if pos_emb is not None and x.is_cuda and type(self).add_rotary_emb is BaseNAtSChunkAttentionLayer.add_rotary_emb \
                and self.head_dim % 16 == 0:
            # rotary embedding and head split in one pass over the projections (bit-identical to the chain below in bf16)
            xq, xk, xv = F_.rope_split_heads(xq, xk, xv, pos_emb[0], pos_emb[1], self.n_local_heads, self.n_local_kv_heads,
                                             self.head_dim)
            return xq, xk, xv, {'token_states_info': token_states_info}
        xq = xq.view(bsz, seqlen, self.n_local_heads, self.head_dim).transpose(1, 2)
        xk = xk.view(bsz, seqlen, self.n_local_kv_heads, self.head_dim).transpose(1, 2)
        xv = xv.view(bsz, seqlen, self.n_local_kv_heads, self.head_dim).transpose(1, 2)
        xq, xk = self.add_rotary_emb(xq, xk, pos_emb)
        return xq, xk, xv, {'token_states_info': token_states_info}

    def prepare_kv(self, xq, xk, xv, start_pos: int = 0, cache: NAtSCache | None = None, kwargs: dict | None = None):
        if self._cache_is_till_updating is not None:
            self._cache_is_till_updating.result()
            self._cache_is_till_updating = None
        return cache.update(key_states=xk, value_states=xv, layer_idx=self.layer_id,
                            cache_kwargs={**(kwargs or {}), 'fused': True})

    def repeat_kv_values(self, keys, values):
        return keys, values

    def multi_head_attention(self, xq, keys, values, mask=None, cache: NAtSCache | None = None,
                             is_first_module: bool = True, kwargs: dict | None = None):
        assert kwargs is not None and 'token_states_info' in kwargs, 'token_states_info is required'
        layer_cache = cache.cache_model[self.layer_id]
        x_len = xq.shape[-2]
        if layer_cache.get_seq_length() == 0:
            roles = F_.roles_from_token_states_info(kwargs['token_states_info'])
            output = F_.prefill_attention(xq, keys, values, roles, self.chunk_size, self.local_seq_max_length, self.sm_scale)
        elif x_len == 1:
            output = layer_cache.decode_attention(xq, self.sm_scale)
        else:
            output = layer_cache.prefill_attention(xq, self.sm_scale)
        if self.executor is not None:
            self._cache_is_till_updating = self.executor.submit(cache.post_update, layer_idx=self.layer_id, x_len=x_len)
        else:
            cache.post_update(layer_idx=self.layer_id, x_len=x_len)
        return output

    def forward(self, x: torch.Tensor, pos_emb, mask, start_pos: int = 0, cache: NAtSCache | None = None, **kwargs):
        bsz, seqlen, _ = x.shape
        xq, xk, xv, mha_kwargs = self.prepare_x_values(x, bsz=bsz, seqlen=seqlen, pos_emb=pos_emb, start_pos=start_pos,
                                                       cache=cache)
        keys, values = self.prepare_kv(xq, xk, xv, start_pos, cache=cache, kwargs=mha_kwargs)
        keys, values = self.repeat_kv_values(keys, values)
        output = self.multi_head_attention(xq, keys, values, mask=mask, cache=cache, kwargs=mha_kwargs)
        output = output.transpose(1, 2).contiguous().view(bsz, seqlen, -1)
        return self.wo(output)


class GPTNAtSChunkAttentionLayer(BaseNAtSChunkAttentionLayer):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.resid_dropout = nn.Dropout(self.dropout)

    def forward(self, *args, **kwargs):
        return self.resid_dropout(super().forward(*args, **kwargs))


class LlamaNAtSChunkAttentionLayer(BaseNAtSChunkAttentionLayer):
    pass
