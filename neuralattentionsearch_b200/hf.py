"""Hugging Face callers of the NAtS attention path: the evaluation-time patch of ``LlamaAttention`` / ``MistralAttention``.

Mirrors ``enable_llama_nats_chunk_eval`` and ``forward_llama_nats_chunk_one_way`` of the reference
(src/nats/models/transformer/hf/llama_nats_chunk.py:171-331; the Mistral twin hf/mistral_nats_chunk.py has the same
structure): every attention module gets a role head ``proj_layer`` (Linear(hidden, n_kv_heads * 3), no bias) and a forward
that pools the hidden states per chunk, takes the argmax role per (kv-head, chunk), applies RoPE, hands K/V to the
``NAtSCache`` passed as ``past_key_values`` and runs the attention of this package: the role-masked prefill kernel for
the first call, the fused decode kernel for single tokens and the prefill-over-cache kernel for further multi-token calls
(the reference falls back to a dense mask + SDPA there).

Differences from the reference file, all forced by the installed ``transformers`` (5.x) rather than the 4.43 it pins:
the attention forward signature is ``(hidden_states, position_embeddings, attention_mask, past_key_values, **kwargs)`` and
returns two values; head counts come from ``module.config``; the start position is the cache's own token count instead
of ``position_ids[0, 0]`` (no device read-back).  The training forward (gumbel roles + Triton backward) is out of scope.
"""
from __future__ import annotations

import types
from dataclasses import dataclass

import torch
from torch import nn

from . import functional as F_
from .cache import NAtSCache


@dataclass
class TransformerArgs:
    """The fields of the reference's ``TransformerArgs`` (src/nats/models/model_configuration.py:30-83) this patch reads."""
    n_msks: int = 8
    sparse_regularized_value: float = 1e-8
    chunk_size: int = 1
    chunk_merge_method: str = 'mean'
    local_seq_max_length: int = 16


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def apply_rotary_pos_emb(q, k, cos, sin, unsqueeze_dim: int = 1):
    cos, sin = cos.unsqueeze(unsqueeze_dim), sin.unsqueeze(unsqueeze_dim)
    return (q * cos) + (rotate_half(q) * sin), (k * cos) + (rotate_half(k) * sin)


def sample_token_states_info(module, hidden_states: torch.Tensor, cache: NAtSCache, start_pos: int) -> torch.Tensor:
    """One-hot roles [B,Hkv,Nc,3] of the chunks this call touches (llama_nats_chunk.py:194-215): placeholder while the
    unfinished chunk stays unfinished; else argmax of the role head over the pooled hidden states, the first chunk of a
    sequence and an unfinished last chunk forced global."""
    bsz, x_len, _ = hidden_states.shape
    n_kv = module.config.num_key_value_heads
    pre = cache.get_nats_chunk_fill_size(module.layer_idx)
    if pre + x_len < module.chunk_size:
        cache.update_nats_cached_x_in_chunk(hidden_states, module.layer_idx, module.chunk_merge_method)
        oh = torch.zeros(bsz, n_kv, 1, module.n_options, dtype=hidden_states.dtype, device=hidden_states.device)
        oh[..., 0].fill_(1)
        return oh
    pooled, pad = cache.update_nats_cached_x_across_chunk(hidden_states, pre, module.layer_idx, module.chunk_merge_method)
    logit = module.proj_layer(pooled).unflatten(-1, (n_kv, module.n_options))
    index = logit.max(-1, keepdim=True)[1]
    if start_pos < module.chunk_size:
        index[:, 0].fill_(0)
    if pad != 0:
        index[:, -1].fill_(0)
    info = torch.zeros_like(logit).scatter_(-1, index, 1.0)
    return info.transpose(1, 2).contiguous()


def forward_llama_nats_chunk_one_way(self, hidden_states: torch.Tensor, position_embeddings=None, attention_mask=None,
                                     past_key_values: NAtSCache | None = None, **kwargs):
    """Replacement of ``LlamaAttention.forward`` in evaluation (llama_nats_chunk.py:171-292)."""
    cache = past_key_values if past_key_values is not None else kwargs.get('past_key_value')
    if not isinstance(cache, NAtSCache):
        raise TypeError('the NAtS attention patch needs a neuralattentionsearch_b200.NAtSCache as past_key_values')
    bsz, q_len, _ = hidden_states.shape
    cfg = self.config
    hd = self.head_dim
    start_pos = cache.get_seq_length(self.layer_idx)
    info = sample_token_states_info(self, hidden_states, cache, start_pos)
    self.token_states = info
    if position_embeddings is None:
        raise ValueError('position_embeddings (cos, sin) are required')
    cos, sin = position_embeddings
    # projections stay [B, N, H*D]; one kernel rotates q / k and writes the [B, H, N, D] tensors the attention reads
    q, k, v = F_.rope_split_heads(self.q_proj(hidden_states), self.k_proj(hidden_states), self.v_proj(hidden_states), cos, sin,
                                  cfg.num_attention_heads, cfg.num_key_value_heads, hd)
    if self.post_update_is_done is not None:
        self.post_update_is_done.result()
        self.post_update_is_done = None
    keys, values = cache.update(k, v, self.layer_idx, cache_kwargs={'token_states_info': info, 'fused': True})
    layer_cache = cache.cache_model[self.layer_idx]
    scale = hd ** -0.5
    if start_pos == 0:
        out = F_.prefill_attention(q, keys, values, F_.roles_from_token_states_info(info), self.chunk_size,
                                   self.local_seq_max_length, scale)
    elif q_len == 1:
        out = layer_cache.decode_attention(q, scale)
    else:
        out = layer_cache.prefill_attention(q, scale)
    if self.executor is None:
        cache.post_update(layer_idx=self.layer_idx, x_len=q_len)
    else:
        self.post_update_is_done = self.executor.submit(cache.post_update, layer_idx=self.layer_idx, x_len=q_len)
    out = out.to(hidden_states.dtype).transpose(1, 2).reshape(bsz, q_len, -1)
    return self.o_proj(out), None


ATTN_IMPLEMENTATION = 'nats_b200'


def _register_attention_name():
    from transformers import AttentionInterface

    def never_called(*args, **kwargs):
        raise RuntimeError('the NAtS patch replaces the attention forward; the attention interface is not used')

    AttentionInterface.register(ATTN_IMPLEMENTATION, never_called)


def _enable_eval(model, transformer_args, n_options: int = 3, executor=None):
    """Adds the role head and the NAtS forward to every attention module of ``model.model.layers``
    (llama_nats_chunk.py:295-331).  Load trained role heads afterwards with ``load_state_dict`` (key ``...self_attn.proj_layer.weight``)."""
    if transformer_args.chunk_merge_method not in ('mean', 'max'):
        raise NotImplementedError(transformer_args.chunk_merge_method)
    _register_attention_name()
    # a name that has no mask builder: the model then creates no dense causal mask for the (replaced) attention
    model.config._attn_implementation = ATTN_IMPLEMENTATION
    p = next(model.parameters())
    for layer in model.model.layers:
        module = layer.self_attn
        cfg = module.config
        module.proj_layer = nn.Linear(cfg.hidden_size, cfg.num_key_value_heads * n_options, device=p.device, dtype=p.dtype, bias=False)
        module.n_reps = cfg.num_attention_heads // transformer_args.n_msks
        module.sparse_regularized_value = transformer_args.sparse_regularized_value
        module.local_seq_max_length = transformer_args.local_seq_max_length
        module.chunk_merge_method = transformer_args.chunk_merge_method
        module.chunk_size = transformer_args.chunk_size
        module.sparse_size = 0.
        module.n_options = n_options
        module.post_update_is_done = None
        module.token_states = None
        module.att_map = None
        module.executor = executor
        module.forward = types.MethodType(forward_llama_nats_chunk_one_way, module)
    return model


def enable_llama_nats_chunk_eval(model, transformer_args, n_options: int = 3, executor=None):
    return _enable_eval(model, transformer_args, n_options, executor)


def enable_mistral_nats_chunk_eval(model, transformer_args, n_options: int = 3, executor=None):
    """hf/mistral_nats_chunk.py: the Mistral attention module has the same projections and cache hand-over."""
    return _enable_eval(model, transformer_args, n_options, executor)


class GraphedGreedyDecoder:
    """Greedy decoding of a model patched by ``enable_llama_nats_chunk_eval`` / ``enable_mistral_nats_chunk_eval`` with
    every step replayed from ONE CUDA graph.

    A decode step of the patched Hugging Face model is a few hundred small launches (per layer: norms, five projections,
    RoPE + head split, append + attention + placement, MLP) behind as much Python; at batch sizes where the GPU work of a
    step is a few milliseconds the host is the bottleneck.  This class runs the same modules with the same arithmetic
    (the role head pools the layer's normalised hidden states over the chunk exactly as the cache's
    ``update_nats_cached_x_in_chunk`` does, the cache step is ``decode_step_static``) but keeps every step-to-step
    quantity on the device -- token, position, tokens in the unfinished chunk, the pooled hidden states -- so that the
    step has static launch parameters, records it once and replays it.  The reference has no counterpart (its decode loop
    is eager PyTorch: hf_pred.py / eval_efficiency.py).

    Use: prefill through the model as usual (``model(input_ids, past_key_values=cache, ...)``), then
    ``GraphedGreedyDecoder(model, cache, max_steps).generate(first_token, n)``; afterwards the cache is where ``n``
    eager decode steps would have left it and can be used by either path."""

    def __init__(self, model, cache: NAtSCache, max_steps: int):
        core = model.model
        attn0 = core.layers[0].self_attn
        cfg = attn0.config
        if attn0.chunk_merge_method != 'mean':
            raise NotImplementedError('graphed decoding pools the hidden states with "mean" only')
        if len(cache.cache_model) != len(core.layers):
            raise ValueError('prefill the prompt through the model first: the cache has no state for some layers')
        self.model, self.cache = model, cache
        self.C = attn0.chunk_size
        self.n_heads, self.n_kv, self.hd = cfg.num_attention_heads, cfg.num_key_value_heads, attn0.head_dim
        lc0 = cache.cache_model[0]
        start = cache.get_seq_length(0)
        if start < self.C:
            raise ValueError('graphed decoding starts behind the first chunk (the first chunk of a sequence is forced global on the host)')
        dev = next(model.parameters()).device
        dt = core.embed_tokens.weight.dtype
        B = lc0.bsz
        self.device, self.B = dev, B
        self.tok = torch.zeros(B, 1, dtype=torch.long, device=dev)
        self.pos = torch.full((1, 1), start, dtype=torch.long, device=dev)
        self.fill = torch.full((1,), lc0.chunk_fill_size, dtype=torch.int32, device=dev)
        self.acc = []
        for li in range(len(core.layers)):
            cur = cache.get_nats_cached_x_in_chunk(li) if lc0.chunk_fill_size else None
            self.acc.append(torch.zeros(B, 1, cfg.hidden_size, dtype=dt, device=dev) if cur is None else cur.to(dt).clone())
        self.o_buf = torch.empty(B, self.n_heads, 1, self.hd, dtype=torch.bfloat16, device=dev)
        self.logits = None
        for lc in cache.cache_model:
            lc.prepare_static_decode(max_steps, self.n_heads, self.hd)
        self.steps_left = max_steps
        self.graph = None
        self._seen = start                  # tokens the cache must hold when generate() is called

    def _step(self, recording: bool) -> None:
        core, C, B = self.model.model, self.C, self.B
        x = core.embed_tokens(self.tok)
        cos, sin = core.rotary_emb(x, self.pos)
        last = self.fill == C - 1                               # this token completes its chunk (device flag)
        scale = self.hd ** -0.5
        for li, layer in enumerate(core.layers):
            attn = layer.self_attn
            h = layer.input_layernorm(x)
            pooled = self.acc[li] + h / C                       # as NAtSCache.merge_new_x_values_in_chunk
            logit = attn.proj_layer(pooled).unflatten(-1, (self.n_kv, attn.n_options))
            roles = logit.max(-1)[1][:, 0].to(torch.uint8).contiguous()   # [B, n_kv]; read on the device only if `last`
            self.acc[li].copy_(torch.where(last, torch.zeros_like(pooled), pooled))
            q, k, v = F_.rope_split_heads(attn.q_proj(h), attn.k_proj(h), attn.v_proj(h), cos, sin, self.n_heads, self.n_kv, self.hd)
            self.cache.cache_model[li].decode_step_static(q, k, v, roles, self.o_buf, scale, recording=True)
            x = x + attn.o_proj(self.o_buf.transpose(1, 2).reshape(B, 1, -1).to(x.dtype))
            x = x + layer.mlp(layer.post_attention_layernorm(x))
        logits = self.model.lm_head(core.norm(x))
        if self.logits is None:
            self.logits = torch.empty_like(logits)
        self.logits.copy_(logits)
        self.tok.copy_(logits[:, -1].argmax(-1, keepdim=True))
        self.pos.add_(1)
        self.fill.copy_(torch.where(last, torch.zeros_like(self.fill), self.fill + 1))

    @torch.no_grad()
    def generate(self, first_token: torch.Tensor, n_steps: int) -> torch.Tensor:
        """Feeds ``first_token`` [B,1] and decodes ``n_steps`` tokens greedily; returns them as [B, n_steps].  ``self.logits``
        holds the logits of the last step."""
        if n_steps < 1 or n_steps > self.steps_left:
            raise ValueError(f'{n_steps} steps asked for, room for {self.steps_left}')
        if self.cache.get_seq_length(0) != self._seen:
            # token position, chunk fill and pooled hidden states live on the device: they are only right if nobody else
            # has moved the cache since this object last did
            raise RuntimeError('the cache has been used by another path since this decoder was built: build a new GraphedGreedyDecoder')
        out = torch.empty(self.B, n_steps, dtype=torch.long, device=self.device)
        self.tok.copy_(first_token.reshape(self.B, 1))
        done = 0
        if self.graph is None:
            # one step outside the graph on a side stream, as graph capture asks (library workspaces, lazy initialisation)
            side = torch.cuda.Stream(self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                self._step(recording=False)
            torch.cuda.current_stream(self.device).wait_stream(side)
            out[:, 0].copy_(self.tok[:, 0])
            done = 1
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._step(recording=True)                      # captured, not run
        for i in range(done, n_steps):
            self.graph.replay()
            out[:, i].copy_(self.tok[:, 0])
        self._note_steps(n_steps)
        self._seen = self.cache.get_seq_length(0)
        return out

    def _note_steps(self, n: int) -> None:
        """Brings the host's view of the cache to where ``n`` eager decode steps would have left it."""
        self.steps_left -= n
        for lc in self.cache.cache_model:
            lc.note_static_steps(n)
        fill = self.cache.cache_model[0].chunk_fill_size
        for li in range(len(self.acc)):
            self.cache._set_cached_x(self.acc[li].clone() if fill else None, li)
