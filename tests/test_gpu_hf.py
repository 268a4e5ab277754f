"""The Hugging Face caller: a random-init Llama with the NAtS attention patch in every layer, on the GPU.

Per layer, the attention module's output is checked against an fp32 evaluation (module's own projections, RoPE, the
oracle's mask for the roles the module chose).  Across calls, the identity of the path is checked at model level:
feeding the tokens in segments and single steps gives the hidden states of one call.
"""
import numpy as np
import pytest
import torch

from oracle import nats_oracle as orc
from test_gpu_parity import dev

pytestmark = pytest.mark.gpu


def tiny_llama(layers=2, hidden=256, heads=4, kv_heads=2, head_dim=64, seed=0):
    from transformers import LlamaConfig, LlamaForCausalLM
    torch.manual_seed(seed)
    cfg = LlamaConfig(hidden_size=hidden, intermediate_size=2 * hidden, num_hidden_layers=layers, num_attention_heads=heads,
                      num_key_value_heads=kv_heads, head_dim=head_dim, vocab_size=512, max_position_embeddings=8192)
    return LlamaForCausalLM(cfg).to(dev()).bfloat16().eval()


def test_patched_llama_layers_match_oracle_and_segments_match_one_call():
    from neuralattentionsearch_b200 import NAtSCache, check_status
    from neuralattentionsearch_b200.hf import TransformerArgs, apply_rotary_pos_emb, enable_llama_nats_chunk_eval
    C, SW, N = 16, 64, 420
    model = tiny_llama()
    enable_llama_nats_chunk_eval(model, TransformerArgs(n_msks=2, chunk_size=C, local_seq_max_length=SW))
    torch.manual_seed(3)
    for layer in model.model.layers:                          # role heads with a spread of roles
        layer.self_attn.proj_layer.weight.data.normal_(0, 0.5)
    ids = torch.randint(0, 512, (2, N), device=dev())
    captured = []

    def hook(mod, args, kwargs, output):
        captured.append((kwargs['hidden_states'].detach(), kwargs['position_embeddings'], mod.token_states.detach(), output[0].detach()))

    handles = [layer.self_attn.register_forward_hook(hook, with_kwargs=True) for layer in model.model.layers]
    with torch.no_grad():
        cache = NAtSCache(SW, C)
        h_one = model.model(input_ids=ids, past_key_values=cache, use_cache=True).last_hidden_state
    check_status(dev())
    for h in handles:
        h.remove()
    assert len(captured) == 2
    cfg = model.config
    for li, (x, (cos, sin), info, out) in enumerate(captured):
        att = model.model.layers[li].self_attn
        roles = info.argmax(-1).cpu().numpy().astype(np.uint8)
        assert (roles[..., 0] == 0).all() and (roles[..., -1] == 0).all()      # sink chunk and unfinished chunk
        assert len(np.unique(roles)) == 3
        xf = x.float()
        q = (xf @ att.q_proj.weight.float().T).view(2, N, cfg.num_attention_heads, 64).transpose(1, 2)
        k = (xf @ att.k_proj.weight.float().T).view(2, N, cfg.num_key_value_heads, 64).transpose(1, 2)
        v = (xf @ att.v_proj.weight.float().T).view(2, N, cfg.num_key_value_heads, 64).transpose(1, 2)
        q, k = apply_rotary_pos_emb(q, k, cos.float(), sin.float())
        ref = orc.prefill_attention(q.cpu(), k.cpu(), v.cpu(), roles, C, SW)
        ref = ref.transpose(1, 2).reshape(2, N, -1).to(dev()) @ att.o_proj.weight.float().T
        err = (out.float() - ref).abs()
        assert err.max().item() < 5e-2 and err.mean().item() / ref.abs().mean().item() < 2e-2, (li, err.max().item())
        lc = cache.cache_model[li]
        assert lc.get_seq_length() == N and lc.chunk_fill_size == N % C
    # the same tokens in segments and single steps
    with torch.no_grad():
        cache2 = NAtSCache(SW, C)
        outs, pos = [], 0
        for n in [200, 150, 1, 1, 1, 30, 37]:
            outs.append(model.model(input_ids=ids[:, pos:pos + n], past_key_values=cache2, use_cache=True).last_hidden_state)
            pos += n
    check_status(dev())
    h_seg = torch.cat(outs, 1)
    err = (h_seg.float() - h_one.float()).abs()
    assert err.mean().item() / h_one.float().abs().mean().item() < 2e-2, err.mean().item()
    for a, b in zip(cache.cache_model, cache2.cache_model):
        assert torch.equal(a.size_global_kv, b.size_global_kv) and torch.equal(a.size_local_kv, b.size_local_kv)


def test_full_depth_decoder_prefill_and_greedy_decode():
    """A 32-layer decoder with the Llama-3-8B attention shape (32 query / 8 kv heads, head_dim 128) and NAtS attention in
    every layer, hidden size cut to 1024 so that the test stays short: prefill 4096 tokens, then greedy decoding; the
    caches of all layers hold what their sizes say and the retained fraction is far below the sequence length."""
    from neuralattentionsearch_b200 import NAtSCache, check_status
    from neuralattentionsearch_b200.hf import TransformerArgs, enable_llama_nats_chunk_eval
    C, SW, N, steps, B = 128, 1024, 4096, 40, 2
    model = tiny_llama(layers=32, hidden=1024, heads=32, kv_heads=8, head_dim=128, seed=1)
    enable_llama_nats_chunk_eval(model, TransformerArgs(n_msks=8, chunk_size=C, local_seq_max_length=SW))
    torch.manual_seed(5)
    for layer in model.model.layers:
        w = layer.self_attn.proj_layer.weight.data
        w.normal_(0, 0.3)
    ids = torch.randint(0, 512, (B, N), device=dev())
    cache = NAtSCache(SW, C)
    with torch.no_grad():
        out = model(input_ids=ids, past_key_values=cache, use_cache=True, logits_to_keep=1)
        tok = out.logits[:, -1].argmax(-1, keepdim=True)
        for _ in range(steps):
            out = model(input_ids=tok, past_key_values=cache, use_cache=True)
            tok = out.logits[:, -1].argmax(-1, keepdim=True)
    check_status(dev())
    assert torch.isfinite(out.logits.float()).all()
    assert len(cache.cache_model) == 32
    for lc in cache.cache_model:
        assert lc.get_seq_length() == N + steps and lc.chunk_fill_size == steps % C
        kept = (lc.size_global_kv + lc.size_local_kv - SW).float().mean().item()
        assert kept < 0.8 * N
        n = lc.n_ctx_data
        flags = lc.valid_tokens[:, :, SW:n].sum(-1)
        want = lc.size_global_kv + lc.size_local_kv - SW + lc.chunk_fill_size
        assert torch.equal(flags, want)


@pytest.mark.parametrize('B,N,Hq,Hkv,D,fused_qkv,shared', [(2, 300, 4, 2, 64, False, True), (1, 1000, 32, 8, 128, True, True),
                                                          (3, 77, 6, 2, 128, False, False), (2, 1, 8, 8, 16, False, True)])
def test_rope_split_heads_is_bit_identical_to_the_elementwise_chain(B, N, Hq, Hkv, D, fused_qkv, shared):
    from neuralattentionsearch_b200.functional import rope_split_heads
    from neuralattentionsearch_b200.hf import apply_rotary_pos_emb
    g = torch.Generator(device=dev()).manual_seed(N)
    if fused_qkv:
        qkv = torch.randn(B, N, (Hq + 2 * Hkv) * D, generator=g, device=dev()).bfloat16()
        q_in, k_in, v_in = qkv[..., :Hq * D], qkv[..., Hq * D:(Hq + Hkv) * D], qkv[..., (Hq + Hkv) * D:]
    else:
        q_in, k_in, v_in = (torch.randn(B, N, h * D, generator=g, device=dev()).bfloat16() for h in (Hq, Hkv, Hkv))
    pos = torch.arange(N, device=dev()).float()[None] + (0 if shared else torch.arange(B, device=dev()).float()[:, None] * 13)
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device=dev()).float() / D))
    freqs = pos[..., None] * inv
    emb = torch.cat([freqs, freqs], -1)
    cos, sin = emb.cos().bfloat16(), emb.sin().bfloat16()
    q, k, v = rope_split_heads(q_in, k_in, v_in, cos, sin, Hq, Hkv, D)
    q_ref = q_in.reshape(B, N, Hq, D).transpose(1, 2)
    k_ref = k_in.reshape(B, N, Hkv, D).transpose(1, 2)
    q_ref, k_ref = apply_rotary_pos_emb(q_ref, k_ref, cos, sin)
    assert torch.equal(q, q_ref.contiguous()) and torch.equal(k, k_ref.contiguous())
    assert torch.equal(v, v_in.reshape(B, N, Hkv, D).transpose(1, 2).contiguous())


def test_llama3_8b_shaped_decoder_end_to_end():
    """The decoder configuration at its real width: random-init 32 layers, hidden 4096, FFN 14336, 32 query / 8 kv heads,
    vocabulary 128256, bf16, NAtS attention in every layer; prefill of 16384 random token ids for two sequences, then greedy
    decoding.  Checks what can be checked without a second implementation of the whole model: finite logits, the
    protocol state of every layer's cache, flags that agree with the sizes, and a retained fraction far below 1."""
    from transformers import LlamaConfig, LlamaForCausalLM
    from neuralattentionsearch_b200 import NAtSCache, check_status
    from neuralattentionsearch_b200.hf import TransformerArgs, enable_llama_nats_chunk_eval
    C, SW, N, steps, B = 128, 1024, 16384, 8, 2
    cfg = LlamaConfig(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                      num_key_value_heads=8, head_dim=128, vocab_size=128256, max_position_embeddings=32768,
                      rope_theta=500000.0)
    torch.manual_seed(2)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev()):
            model = LlamaForCausalLM(cfg).eval()
    finally:
        torch.set_default_dtype(prev)
    enable_llama_nats_chunk_eval(model, TransformerArgs(n_msks=8, chunk_size=C, local_seq_max_length=SW))
    for layer in model.model.layers:
        layer.self_attn.proj_layer.weight.data.normal_(0, 0.05)
    ids = torch.randint(0, cfg.vocab_size, (B, N), device=dev())
    cache = NAtSCache(SW, C)
    with torch.no_grad():
        out = model(input_ids=ids, past_key_values=cache, use_cache=True, logits_to_keep=1)
        tok = out.logits[:, -1].argmax(-1, keepdim=True)
        for _ in range(steps):
            out = model(input_ids=tok, past_key_values=cache, use_cache=True)
            tok = out.logits[:, -1].argmax(-1, keepdim=True)
    check_status(dev())
    assert out.logits.shape == (B, 1, cfg.vocab_size) and torch.isfinite(out.logits.float()).all()
    assert len(cache.cache_model) == 32
    fractions = []
    for lc in cache.cache_model:
        assert lc.get_seq_length() == N + steps and lc.chunk_fill_size == steps
        want = lc.size_global_kv + lc.size_local_kv - SW + lc.chunk_fill_size
        assert torch.equal(lc.valid_tokens[:, :, SW:lc.n_ctx_data].sum(-1), want)
        fractions.append((lc.size_global_kv + lc.size_local_kv - SW).float().mean().item() / N)
    assert max(fractions) < 0.9 and min(fractions) >= 0.0


def test_patched_mistral_segments_match_one_call():
    """The Mistral patch (hf/mistral_nats_chunk.py: same structure as the Llama one) on a small random-init Mistral:
    the hidden states of one call equal those of the same tokens fed in segments and single steps, every layer's cache holds
    what its sizes say, and greedy decoding on top stays finite."""
    from transformers import MistralConfig, MistralForCausalLM
    from neuralattentionsearch_b200 import NAtSCache, check_status
    from neuralattentionsearch_b200.hf import TransformerArgs, enable_mistral_nats_chunk_eval
    C, SW, N = 16, 64, 300
    torch.manual_seed(4)
    cfg = MistralConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, head_dim=64, vocab_size=512, max_position_embeddings=8192, sliding_window=None)
    model = MistralForCausalLM(cfg).to(dev()).bfloat16().eval()
    enable_mistral_nats_chunk_eval(model, TransformerArgs(n_msks=2, chunk_size=C, local_seq_max_length=SW))
    for layer in model.model.layers:
        layer.self_attn.proj_layer.weight.data.normal_(0, 0.5)
    ids = torch.randint(0, 512, (2, N), device=dev())
    with torch.no_grad():
        cache = NAtSCache(SW, C)
        h_one = model.model(input_ids=ids, past_key_values=cache, use_cache=True).last_hidden_state
        cache2 = NAtSCache(SW, C)
        outs, pos = [], 0
        for n in [130, 100, 1, 1, 68]:
            outs.append(model.model(input_ids=ids[:, pos:pos + n], past_key_values=cache2, use_cache=True).last_hidden_state)
            pos += n
        out = model(input_ids=ids[:, -1:], past_key_values=cache, use_cache=True)
    check_status(dev())
    assert torch.isfinite(out.logits.float()).all()
    h_seg = torch.cat(outs, 1)
    err = (h_seg.float() - h_one.float()).abs()
    assert err.mean().item() / h_one.float().abs().mean().item() < 2e-2, err.mean().item()
    for a, b in zip(cache.cache_model, cache2.cache_model):
        assert torch.equal(a.size_global_kv, b.size_global_kv) and torch.equal(a.size_local_kv, b.size_local_kv)
        roles = model.model.layers[a.layer_id].self_attn.token_states
        assert roles is not None


@pytest.mark.parametrize('N', [64, 61])                      # prompt ends on a chunk boundary / inside a chunk
def test_graphed_greedy_decoder_equals_the_eager_decode_loop(N):
    """Greedy decoding with every step replayed from one CUDA graph: same tokens, same logits and the same cache as the
    eager loop over the patched model, across several chunk completions; afterwards the eager path continues from the
    graphed decoder's cache."""
    from neuralattentionsearch_b200 import NAtSCache, check_status
    from neuralattentionsearch_b200.hf import GraphedGreedyDecoder, TransformerArgs, enable_llama_nats_chunk_eval
    C, SW, steps, more = 8, 32, 29, 5
    model = tiny_llama(seed=5)
    enable_llama_nats_chunk_eval(model, TransformerArgs(n_msks=2, chunk_size=C, local_seq_max_length=SW))
    torch.manual_seed(6)
    for layer in model.model.layers:
        layer.self_attn.proj_layer.weight.data.normal_(0, 0.5)
    ids = torch.randint(0, 512, (3, N), device=dev())
    with torch.no_grad():
        # eager loop
        c1 = NAtSCache(SW, C)
        out = model(input_ids=ids, past_key_values=c1, use_cache=True)
        first = out.logits[:, -1].argmax(-1, keepdim=True)
        tok, eager = first, []
        for _ in range(steps + more):
            out = model(input_ids=tok, past_key_values=c1, use_cache=True)
            tok = out.logits[:, -1].argmax(-1, keepdim=True)
            eager.append(tok)
        eager = torch.cat(eager, 1)
        # graphed loop, then the eager path on the same cache
        c2 = NAtSCache(SW, C)
        out2 = model(input_ids=ids, past_key_values=c2, use_cache=True)
        assert torch.equal(out2.logits[:, -1].argmax(-1, keepdim=True), first)
        dec = GraphedGreedyDecoder(model, c2, max_steps=steps)
        got = dec.generate(first, 10)
        got = torch.cat([got, dec.generate(got[:, -1:], steps - 10)], 1)
        tok = got[:, -1:]
        tail = []
        for _ in range(more):
            out2 = model(input_ids=tok, past_key_values=c2, use_cache=True)
            tok = out2.logits[:, -1].argmax(-1, keepdim=True)
            tail.append(tok)
    check_status(dev())
    assert torch.equal(got, eager[:, :steps])
    assert torch.equal(torch.cat(tail, 1), eager[:, steps:])
    assert torch.equal(out2.logits, out.logits)
    for a, b in zip(c1.cache_model, c2.cache_model):
        assert torch.equal(a.size_global_kv, b.size_global_kv) and torch.equal(a.size_local_kv, b.size_local_kv)
        assert (a.n_ctx_data, a.chunk_fill_size, a.sliding_queue_tail, a.get_seq_length()) == (b.n_ctx_data, b.chunk_fill_size, b.sliding_queue_tail, b.get_seq_length())
    with pytest.raises(ValueError):
        dec.generate(tok, 1)                                   # no room left
    dec2 = GraphedGreedyDecoder(model, c2, max_steps=4)
    with torch.no_grad():
        model(input_ids=tok, past_key_values=c2, use_cache=True)
    with pytest.raises(RuntimeError):
        dec2.generate(tok, 1)                                  # the eager path moved the cache behind the decoder's back
