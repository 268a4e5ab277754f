#!/usr/bin/env python
"""Benchmark of the NAtS attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

A step is one pass of the path over one batch of synthetic input of the 32k-token configuration: role-masked chunked
prefill (B1, 32 query / 8 kv heads, head_dim 128, N 32768, bf16, window 1024, chunk 128, roles ~5 % global / 15 % local /
80 % sliding) followed by the KV eviction.  With N GPUs every rank runs its own sequence (weak scaling; the (batch, kv-head)
pairs are independent, so there is no collective on the data path -- NCCL only gathers outputs after the timed region).
The headline value is TFLOP/s on kept 128x128 tiles (4*128*128*D flop per kept tile and query head).  The same line
carries the decode leg (batch 64 over a compacted ragged cache, 256 single-token steps) and the roofline / CPU-baseline
objects.  One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(name='prefill32k_evict', B=1, Hq=32, Hkv=8, D=128, N=32768, C=128, SW=1024, p_global=0.05, p_local=0.15,
                sigma=0.5, seed=0)
DECODE = dict(B=64, Hq=32, Hkv=8, D=128, C=128, SW=1024, len_lo=2048, len_hi=6144, steps=256, seed=1, ring_p=0.8, sigma=0.5)
METRIC = 'prefill TFLOP/s on kept tiles @32k'
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


def load_peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d['_source'] = 'measured'
        return d
    return dict(FALLBACK_PEAKS, _source='fallback')


def load_traffic():
    """DRAM bytes per launch measured with ncu (profiles/ncu_traffic.json), or None where no capture is recorded."""
    path = os.path.join(ROOT, 'profiles', 'ncu_traffic.json')
    try:
        with open(path) as f:
            d = json.load(f)
        return {k: v.get('bytes_per_launch') for k, v in d.items() if isinstance(v, dict)}
    except (OSError, ValueError):
        return {}


# ---------------------------------------------------------------------------------------------- synthetic inputs
def role_bias(p_global, p_local):
    """Bias of the 3-way N(0,1) role logits that yields the requested global / local share (rest sliding)."""
    rng = np.random.default_rng(12345)
    z = rng.standard_normal((200_000, 3))
    bg = bl = 0.0
    for _ in range(40):
        r = np.argmax(z + np.array([bg, bl, 0.0]), -1)
        bg += 0.5 * (math.log(p_global) - math.log(max((r == 0).mean(), 1e-6)))
        bl += 0.5 * (math.log(p_local) - math.log(max((r == 1).mean(), 1e-6)))
    return bg, bl, 0.0


def make_roles(B, Hkv, Nc, p_global, p_local, seed):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(B, Hkv, Nc, 3, generator=g) + torch.tensor(role_bias(p_global, p_local))
    roles = logits.argmax(-1).to(torch.uint8)
    roles[..., 0] = 0
    return roles


def make_prefill_inputs(w, seed, pin=False):
    g = torch.Generator().manual_seed(seed)
    mk = lambda h: (torch.randn(w['B'], h, w['N'], w['D'], generator=g) * w['sigma']).to(torch.bfloat16)
    q, k, v = mk(w['Hq']), mk(w['Hkv']), mk(w['Hkv'])
    roles = make_roles(w['B'], w['Hkv'], w['N'] // w['C'], w['p_global'], w['p_local'], seed)
    if pin:
        q, k, v, roles = (t.pin_memory() for t in (q, k, v, roles))
    return q, k, v, roles


def bind_to_gpu_numa_node(index):
    """Runs this rank on the CPUs of the NUMA node its GPU hangs off, so that the pinned host buffers of the end-to-end leg
    are allocated in memory local to that GPU's PCIe root (ranks that share one node's memory halve each other's copy
    bandwidth).  Returns the node, or None if the topology cannot be read."""
    try:
        pr = torch.cuda.get_device_properties(index)
        bdf = '%04x:%02x:%02x.0' % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
        node = int(open(f'/sys/bus/pci/devices/{bdf}/numa_node').read())
        if node < 0:
            return None
        cpus = []
        for part in open(f'/sys/devices/system/node/node{node}/cpulist').read().strip().split(','):
            lo, _, hi = part.partition('-')
            cpus += range(int(lo), int(hi or lo) + 1)
        allowed = os.sched_getaffinity(0) & set(cpus)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except Exception:
        return None


# ---------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ('clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
              'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', '-i', str(self.index), f'--query-gpu={self.FIELDS}',
                                          '--format=csv,noheader,nounits', '-lms', '100'],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=['nvidia-smi unavailable'])
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for line in self.lines:
            parts = [p.strip() for p in line.split(',')]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[2:6]):
                if val.lower().startswith('active'):
                    reasons.add(nm)
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


# ---------------------------------------------------------------------------------------------- decode leg
def build_decode_cache(d, device):
    """A compacted ragged cache as eviction leaves it: per (sequence, kv-head) a retained length drawn uniformly from
    [len_lo, len_hi] (multiple of the chunk), each chunk of the ring valid with probability ring_p, random K/V."""
    from neuralattentionsearch_b200.cache import NAtSChunkLayerCache
    B, H, D, C, SW = d['B'], d['Hkv'], d['D'], d['C'], d['SW']
    g = torch.Generator().manual_seed(d['seed'])
    kept = torch.randint(d['len_lo'] // C, d['len_hi'] // C + 1, (B, H), generator=g) * C      # tokens behind the ring
    n_glob = (kept * 0.8).long() // C * C
    lc = NAtSChunkLayerCache(B, H, SW, chunk_size=C, device=device)
    lc.size_global_kv = (SW + n_glob).to(device)
    lc.size_local_kv = (kept - n_glob).to(device)
    t0 = int((SW + kept).max())
    cap = t0 + 4 * C + 2 * d['steps'] + 64
    gd = torch.Generator(device=device).manual_seed(d['seed'])
    lc._buf_k = (torch.randn(B, H, cap, D, generator=gd, device=device) * d['sigma']).to(torch.bfloat16)
    lc._buf_v = (torch.randn(B, H, cap, D, generator=gd, device=device) * d['sigma']).to(torch.bfloat16)
    valid = torch.zeros(B, H, cap, dtype=torch.uint8, device=device)
    # a ring slot holds one chunk and the eviction sets its flags chunk by chunk (all tokens of a sliding chunk valid)
    ring_chunks = (torch.rand(B, H, SW // C, generator=gd, device=device) < d['ring_p']).to(torch.uint8)
    valid[:, :, :SW] = ring_chunks.repeat_interleave(C, -1)
    pos = torch.arange(cap, device=device)[None, None]
    valid |= ((pos >= SW) & (pos < (SW + kept).to(device)[..., None])).to(torch.uint8)
    lc._buf_valid = valid
    lc._state[0] = t0
    lc._t0_bound = lc._t0_exact = lc._t0_synced = t0
    lc._seen_tokens = 32768
    lc.sliding_queue_tail = 0
    return lc


def run_decode_leg(d, device, steps, warmup):
    """Times `steps` single-token decode steps (append + attention fused; chunk placement when a chunk completes)."""
    B, Hq, Hkv, D, C = d['B'], d['Hq'], d['Hkv'], d['D'], d['C']
    lc = build_decode_cache(d, device)
    gd = torch.Generator(device=device).manual_seed(d['seed'] + 1)
    n_in = 8
    qs = [(torch.randn(B, Hq, 1, D, generator=gd, device=device) * d['sigma']).to(torch.bfloat16) for _ in range(n_in)]
    ks = [(torch.randn(B, Hkv, 1, D, generator=gd, device=device) * d['sigma']).to(torch.bfloat16) for _ in range(n_in)]
    vs = [(torch.randn(B, Hkv, 1, D, generator=gd, device=device) * d['sigma']).to(torch.bfloat16) for _ in range(n_in)]
    placeholder = torch.zeros(B, Hkv, 1, dtype=torch.uint8, device=device)
    role_steps = [torch.randn(B, Hkv, 1, 3, generator=gd, device=device).argmax(-1).to(torch.uint8) for _ in range(4)]
    launches = 0
    bytes_total = 0

    def one(i, count=False):
        nonlocal launches, bytes_total
        done = lc.chunk_fill_size + 1 == C
        roles = role_steps[(i // C) % len(role_steps)] if done else placeholder
        lc.update(ks[i % n_in], vs[i % n_in], roles, fused=True)
        o = lc.decode_attention(qs[i % n_in])
        lc.post_update(1)
        if count:
            launches += 2 if done else 1
        return o

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize(device)
    kv_bytes_start = lc.kv_bytes()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        o = one(warmup + i, count=True)
    e1.record()
    torch.cuda.synchronize(device)
    ms = e0.elapsed_time(e1)
    kv_bytes_end = lc.kv_bytes()
    return dict(ms_total=ms, steps=steps, tokens=B * steps, launches=launches,
                kv_bytes_per_step=(kv_bytes_start + kv_bytes_end) / 2, out=o)


# ---------------------------------------------------------------------------------------------- CPU legs
def cpu_sample_blocks(w):
    """Query-row blocks of the CPU sample: four 512-row blocks spread over the sequence, all heads."""
    n = w['N']
    return [(lo, lo + 512) for lo in (0, n // 4, n // 2, n - 512)]


def _kept_tiles_of_rows(w, roles_np, row_blocks, heads=None, n_tokens=None):
    """Kept 128x128 tile pairs (per kv-head) of the given query-row blocks -- the flop the metric counts."""
    from oracle import nats_oracle as orc
    n_tokens = w['N'] if n_tokens is None else n_tokens
    lim = orc.row_limit(roles_np, w['C'], w['SW'])
    lim_tok = np.repeat(lim, w['C'], -1)[..., :n_tokens]
    tmax = lim_tok.reshape(roles_np.shape[0], roles_np.shape[1], -1, 128).max(-1)
    if heads is not None:
        tmax = tmax[:, heads[0]:heads[1]]
    kept = 0
    for lo, hi in row_blocks:
        for t in range(lo // 128, hi // 128):
            kept += int((tmax[:, :, :t + 1] >= t * 128).sum())
    return kept


def _timed(fn, steps, warmup, budget_s):
    """Median seconds per call over `steps` calls (at least one) after `warmup`, cut short when the time box is used up."""
    for _ in range(warmup):
        fn()
    times = []
    t_begin = time.perf_counter()
    for _ in range(max(1, steps)):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_begin > budget_s:
            break
    return float(np.median(times)), len(times)


def run_cpu_port_leg(w, steps, warmup, threads, budget_s=40.0):
    """The reference's eager math (dense mask rows + softmax(QK^T)V in fp32 over every causal key, per query-row block,
    as its CPU path does it) on a bounded sample of the workload, through the oracle port."""
    from oracle import nats_oracle as orc
    torch.set_num_threads(threads)
    q, k, v, roles = make_prefill_inputs(w, w['seed'])
    q, k, v = q.float(), k.float(), v.float()
    roles_np = roles.numpy()
    blocks = cpu_sample_blocks(w)
    flops = 4.0 * 128 * 128 * w['D'] * (w['Hq'] // w['Hkv']) * _kept_tiles_of_rows(w, roles_np, blocks)

    def one():
        for lo, hi in blocks:
            orc.prefill_attention(q, k, v, roles_np, w['C'], w['SW'], rows=(lo, hi), block=hi - lo)

    dt, n = _timed(one, steps, warmup, budget_s)
    return dict(value=flops / dt / 1e12, seconds_per_step=dt, flops=flops, steps=n, kind='port',
                sample=f'{len(blocks)} query blocks of 512 rows (starting at rows {[b[0] for b in blocks]}), all {w["Hq"]} heads, '
                       f'fp32, dense causal keys as the eager path computes them; value counts kept-tile flop only')


REF_SAMPLE = dict(tokens=4096, kv_heads=2)        # bounded sample the reference's own code runs: a prefix of two kv-heads


def run_cpu_reference_leg(w, steps, warmup, threads, budget_s=60.0):
    """The reference's OWN eager attention path (its layer's prepare_kv -> cache.update -> generate_mask ->
    scaled_dot_product_attention -> cache.post_update, fp32, all host threads) on a bounded sample of the workload: the
    first REF_SAMPLE['tokens'] tokens of REF_SAMPLE['kv_heads'] kv-heads with their query heads (the full 32k sequence
    needs a dense [B,Hq,N,N] mask of 34 GB there).  Returns None when the reference copy is not installed."""
    from oracle import fetch_reference
    if not fetch_reference.available():
        return None
    from oracle import nats_oracle as orc
    NAtSCache, Layer = fetch_reference.load_reference()
    torch.set_num_threads(threads)
    n, hk = min(REF_SAMPLE['tokens'], w['N']), min(REF_SAMPLE['kv_heads'], w['Hkv'])
    nrep = w['Hq'] // w['Hkv']
    q, k, v, roles = make_prefill_inputs(w, w['seed'])
    q, k, v = q[:, :hk * nrep, :n].float().contiguous(), k[:, :hk, :n].float().contiguous(), v[:, :hk, :n].float().contiguous()
    roles_np = roles[:, :hk, :n // w['C']].numpy().copy()
    info = {'token_states_info': orc.onehot_from_roles(roles_np)}
    layer = Layer(dim=hk * nrep * w['D'], n_heads=hk * nrep, n_kv_heads=hk, layer_id=0, local_seq_max_length=w['SW'],
                  chunk_size=w['C']).eval()
    flops = 4.0 * 128 * 128 * w['D'] * nrep * _kept_tiles_of_rows(w, roles_np, [(0, n)], n_tokens=n)

    def one():
        cache = NAtSCache(sliding_window_size=w['SW'], chunk_size=w['C'])
        with torch.no_grad():
            keys, values = layer.prepare_kv(q, k, v, 0, cache=cache, kwargs=info)
            keys, values = layer.repeat_kv_values(keys, values)
            layer.multi_head_attention(q, keys, values, cache=cache, kwargs=info)

    dt, cnt = _timed(one, steps, warmup, budget_s)
    return dict(value=flops / dt / 1e12, seconds_per_step=dt, flops=flops, steps=cnt, kind='reference',
                sample=f"the reference's own eager layer path (dense mask + SDPA + eviction, fp32) on the first {n} tokens of "
                       f'{hk} kv-heads ({hk * nrep} query heads) of the workload; value counts kept-tile flop only; median of {cnt} runs')


def run_cpu_leg(w, steps, warmup, threads):
    """The CPU arm: the reference's own code where its copy is installed, else the oracle port."""
    r = run_cpu_reference_leg(w, steps, warmup, threads)
    return r if r is not None else run_cpu_port_leg(w, steps, warmup, threads)


# ---------------------------------------------------------------------------------------------- further legs
def allmax(x, device, world):
    """Max over ranks of a host scalar (the time of a multi-GPU leg is the time of its slowest rank)."""
    if world == 1:
        return float(x)
    import torch.distributed as dist
    t = torch.tensor([x], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_strong_prefill_leg(w, device, rank, world, steps, barrier, full_inputs):
    """ONE fixed job -- the 32k sequence of rank 0, all 8 kv-heads -- split over the ranks by kv-head
    (sharding.shard_pairs): every rank runs cache.update / prefill / eviction on its heads, no collective inside the timed
    region.  Afterwards the outputs and cache sizes are gathered with NCCL and rank 0 checks them against its own run of
    the whole job on one GPU, bit for bit."""
    import torch.distributed as dist
    from neuralattentionsearch_b200 import prefill_attention
    from neuralattentionsearch_b200.cache import NAtSChunkLayerCache
    from neuralattentionsearch_b200.sharding import shard_pairs
    nrep = w['Hq'] // w['Hkv']
    if rank == 0:
        q, k, v, roles = full_inputs
    else:
        q, k, v, roles = (t.to(device) for t in make_prefill_inputs(w, w['seed']))
    (b0, h0, h1), = shard_pairs(w['B'], w['Hkv'], world, rank)          # B = 1 and world <= 8: one slice of heads per rank
    qs, ks, vs = q[:, h0 * nrep:h1 * nrep].contiguous(), k[:, h0:h1].contiguous(), v[:, h0:h1].contiguous()
    rs = roles[:, h0:h1].contiguous()

    def step(qd, kd, vd, rd):
        lc = NAtSChunkLayerCache(kd.shape[0], kd.shape[1], w['SW'], chunk_size=w['C'], device=device)
        lc.update(kd, vd, rd)
        o = prefill_attention(qd, kd, vd, rd, w['C'], w['SW'])
        lc.post_update(w['N'])
        return o, lc

    def timed(args_, n):
        for _ in range(3):
            step(*args_)
        torch.cuda.synchronize(device)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            o, lc = step(*args_)
        b.record()
        torch.cuda.synchronize(device)
        return a.elapsed_time(b) / n, o, lc

    barrier()
    ms, o, lc = timed((qs, ks, vs, rs), steps)
    barrier()
    ms = allmax(ms, device, world)
    res = dict(job='one 32k sequence x 8 kv-heads (rank 0\'s benchmark inputs), kv-heads split over the ranks', kv_heads_per_gpu=h1 - h0,
               ms_per_step=ms)
    if world > 1:
        # the whole job on one GPU (rank 0 alone, the others wait), for the speed-up and as the reference of the check
        ms1 = o1 = lc1 = None
        if rank == 0:
            ms1, o1, lc1 = timed((q, k, v, roles), steps)
        barrier()
        outs = [torch.empty_like(o) for _ in range(world)]
        dist.all_gather(outs, o.contiguous())
        sizes = torch.stack([lc.size_global_kv, lc.size_local_kv]).contiguous()
        gathered = [torch.empty_like(sizes) for _ in range(world)]
        dist.all_gather(gathered, sizes)
        if rank == 0:
            o_all = torch.cat(outs, 1)
            s_all = torch.cat(gathered, 2)
            res.update(ms_one_gpu=ms1, speedup=ms1 / ms,
                       outputs_bit_identical=bool(torch.equal(o_all, o1)),
                       cache_sizes_identical=bool(torch.equal(s_all, torch.stack([lc1.size_global_kv, lc1.size_local_kv]))),
                       note='at one kv-head per GPU a step is launch latency plus one wave of a persistent kernel: the speed-up flattens')
    else:
        res.update(ms_one_gpu=ms, speedup=1.0)
    return res


def slice_decode_cache(lc, b0, b1, device):
    """The cache of sequences [b0, b1) of a decode cache: the shard a rank owns when the batch is split."""
    from neuralattentionsearch_b200.cache import NAtSChunkLayerCache
    part = NAtSChunkLayerCache(b1 - b0, lc.n_msks, lc.sliding_window_size, chunk_size=lc.chunk_size, device=device)
    part.size_global_kv = lc.size_global_kv[b0:b1].clone()
    part.size_local_kv = lc.size_local_kv[b0:b1].clone()
    t0 = int((part.size_global_kv + part.size_local_kv).max())          # the common tail offset is the longest LOCAL head
    part._buf_k, part._buf_v = lc._buf_k[b0:b1].contiguous(), lc._buf_v[b0:b1].contiguous()
    part._buf_valid = lc._buf_valid[b0:b1].contiguous()
    part._state[0] = t0
    part._t0_bound = part._t0_exact = part._t0_synced = t0
    part._seen_tokens = lc._seen_tokens
    part.sliding_queue_tail = lc.sliding_queue_tail
    return part


def run_strong_decode_leg(d, device, rank, world, steps, barrier):
    """ONE fixed decode job (batch 64 over the compacted ragged cache) split over the ranks by batch; outputs of every
    step's last token gathered afterwards and checked against rank 0's run of the whole batch."""
    import torch.distributed as dist
    B, Hq, Hkv, D, C = d['B'], d['Hq'], d['Hkv'], d['D'], d['C']
    per = B // world
    b0, b1 = rank * per, (rank + 1) * per
    gd = torch.Generator(device=device).manual_seed(d['seed'] + 1)
    qs = [(torch.randn(B, Hq, 1, D, generator=gd, device=device) * d['sigma']).to(torch.bfloat16) for _ in range(4)]
    ks = [(torch.randn(B, Hkv, 1, D, generator=gd, device=device) * d['sigma']).to(torch.bfloat16) for _ in range(4)]
    vs = [(torch.randn(B, Hkv, 1, D, generator=gd, device=device) * d['sigma']).to(torch.bfloat16) for _ in range(4)]
    placeholder = torch.zeros(B, Hkv, 1, dtype=torch.uint8, device=device)

    def run(lc, lo, hi, n):
        outs = []
        torch.cuda.synchronize(device)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(n):                                   # fewer steps than a chunk: no placement, the leg times the attention
            lc.update(ks[i % 4][lo:hi].contiguous(), vs[i % 4][lo:hi].contiguous(), placeholder[lo:hi], fused=True)
            outs.append(lc.decode_attention(qs[i % 4][lo:hi].contiguous()))
            lc.post_update(1)
        b.record()
        torch.cuda.synchronize(device)
        return a.elapsed_time(b) / n, outs[-1]

    n = min(steps, C - 4)
    full = build_decode_cache(d, device)
    mine = slice_decode_cache(full, b0, b1, device) if world > 1 else full
    run(mine, b0, b1, 3)                                     # warm-up: buffers and workspace reach their size
    barrier()
    ms, o = run(mine, b0, b1, n)
    barrier()
    ms = allmax(ms, device, world)
    res = dict(job=f'decode batch {B} over the compacted ragged cache, sequences split over the ranks', sequences_per_gpu=per,
               steps=n, ms_per_step=ms, tok_per_s=B / (ms * 1e-3))
    if world > 1:
        ms1 = o1 = None
        if rank == 0:
            whole = build_decode_cache(d, device)
            run(whole, 0, B, 3)
            ms1, o1 = run(whole, 0, B, n)
        barrier()
        outs = [torch.empty_like(o) for _ in range(world)]
        dist.all_gather(outs, o.contiguous())
        if rank == 0:
            res.update(ms_one_gpu=ms1, speedup=ms1 / ms, outputs_bit_identical=bool(torch.equal(torch.cat(outs, 0), o1)))
    else:
        res.update(ms_one_gpu=ms, speedup=1.0)
    return res


def run_sustained_leg(w, device, rank, seconds, q, k, v, roles, peaks):
    """The dominant kernels for seconds instead of milliseconds: back-to-back prefill launches, then decode steps, with the
    SM clock sampled over each region.  A 32-layer prefill of long prompts runs in this regime (power cap, lower clocks)."""
    from neuralattentionsearch_b200 import check_status, prefill_attention
    kept = torch.zeros(w['B'], w['Hkv'], dtype=torch.int64, device=device)
    prefill_attention(q, k, v, roles, w['C'], w['SW'], kept_tiles=kept)
    flops = 4.0 * 128 * 128 * w['D'] * (w['Hq'] // w['Hkv']) * int(kept.sum().item())
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    a.record()
    for _ in range(20):
        prefill_attention(q, k, v, roles, w['C'], w['SW'])
    b.record()
    torch.cuda.synchronize(device)
    n = max(50, int(seconds * 1e3 / (a.elapsed_time(b) / 20)))
    sampler = ClockSampler(device.index)
    sampler.start()
    time.sleep(0.3)
    a.record()
    for _ in range(n):
        prefill_attention(q, k, v, roles, w['C'], w['SW'])
    b.record()
    torch.cuda.synchronize(device)
    clk = sampler.stop()
    check_status(device)
    ms = a.elapsed_time(b) / n
    tf = flops / (ms * 1e-3) / 1e12
    out = dict(prefill=dict(launches=n, seconds=ms * n * 1e-3, ms_per_launch=ms, tflops=tf, peak=peaks['bf16_tflops_sustained'],
                            frac=tf / peaks['bf16_tflops_sustained'], of=peaks['_source'] + ' cuBLAS bf16, sustained',
                            clocks=clk, ms_times_mhz=(ms * clk['sm_mhz']) if clk.get('sm_mhz') else None))
    # decode: steps below one chunk repeat on a fresh cache until the time is used up
    d = DECODE
    steps_per_round = d['C'] - 1
    r = run_decode_leg(d, device, steps_per_round, warmup=3)
    rounds = max(1, int(seconds * 1e3 / r['ms_total']))
    sampler = ClockSampler(device.index)
    sampler.start()
    time.sleep(0.3)
    tot_ms, tot_bytes = 0.0, 0.0
    for _ in range(rounds):
        r = run_decode_leg(d, device, steps_per_round, warmup=0)
        tot_ms += r['ms_total']
        tot_bytes += r['kv_bytes_per_step'] * steps_per_round
    clk = sampler.stop()
    gbs = tot_bytes / (tot_ms * 1e-3) / 1e9
    out['decode'] = dict(steps=rounds * steps_per_round, seconds=tot_ms * 1e-3, ms_per_step=tot_ms / (rounds * steps_per_round),
                         gbs=gbs, peak=peaks['hbm_gbs'], frac=gbs / peaks['hbm_gbs'], of=peaks['_source'] + ' HBM copy',
                         clocks=clk, note='the clock samples include the rebuilding of the synthetic cache between rounds')
    return out


EVICT_LARGE = dict(B=32, Hkv=8, D=128, N=16384, C=128, SW=1024, p_global=0.07, p_local=0.20, seed=5)   # ~10 % of the tokens retained


def run_eviction_large_leg(device, peaks, steps=5):
    """Eviction at a size where bandwidth, not launch latency, decides: the attention shape of the 32-layer decoder
    configuration (8 kv-heads x 16k tokens per sequence, ~10 % of the tokens retained), 32 sequences at once.
    Kernel-only time of the keep-set plan + the compaction (CUDA events around the two launches)."""
    from neuralattentionsearch_b200 import functional as F_
    e = EVICT_LARGE
    B, H, D, N, C, SW = e['B'], e['Hkv'], e['D'], e['N'], e['C'], e['SW']
    g = torch.Generator(device=device).manual_seed(e['seed'])
    k = (torch.randn(B, H, N, D, generator=g, device=device) * 0.5).to(torch.bfloat16)
    v = (torch.randn(B, H, N, D, generator=g, device=device) * 0.5).to(torch.bfloat16)
    roles = make_roles(B, H, N // C, e['p_global'], e['p_local'], e['seed']).to(device)
    rank = torch.empty(B, H, N // C, dtype=torch.int32, device=device)
    sg = torch.empty(B, H, dtype=torch.long, device=device)
    sl = torch.empty_like(sg)
    state = torch.zeros(8, dtype=torch.int32, device=device)
    F_.evict_plan(roles, N, C, SW, rank, sg, sl, state)
    t0 = int(state[0].item())
    cap = -(-t0 // C) * C                          # exactly the longest head: rows behind a shorter head's tokens are zero-filled
    ck = torch.empty(B, H, cap, D, dtype=torch.bfloat16, device=device)
    cv = torch.empty_like(ck)
    valid = torch.empty(B, H, cap, dtype=torch.uint8, device=device)
    times = []
    for i in range(2 + steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(device)
        a.record()
        F_.evict_plan(roles, N, C, SW, rank, sg, sl, state)
        F_.evict_compact(k, v, roles, rank, sg, sl, state, C, SW, ck, cv, valid)
        b.record()
        torch.cuda.synchronize(device)
        if i >= 2:
            times.append(a.elapsed_time(b))
    ms = float(np.median(times))
    tokens = int((sg + sl).sum().item())
    nbytes = 2 * 2 * tokens * D * 2
    gbs = nbytes / (ms * 1e-3) / 1e9
    return dict(shape=f'B{B} x {H} kv-heads x {N} tokens, head_dim {D}, chunk {C}, window {SW}', ms=ms, bytes=nbytes, gbs=gbs,
                retained_frac=(tokens - B * H * SW) / (B * H * N), written_rows_per_head=cap,
                roofline=dict(bound='hbm', achieved=gbs, peak=peaks['hbm_gbs'], unit='GB/s', frac=gbs / peaks['hbm_gbs'],
                              of=peaks['_source'] + ' HBM copy', kernel='evict_plan_kernel + evict_compact_kernel',
                              note='algorithmic bytes: kept tokens and ring, K and V, read + write; inputs (1 GiB) exceed L2'))


def run_copy_floor_leg(hq, hk, hv, ho, device, world, barrier, steps=3):
    """The end-to-end leg's host<->device bytes with no kernel at all, both directions at once on two streams: what the
    PCIe / host-memory side allows at this number of ranks."""
    dq, dk, dv = (torch.empty_like(t, device=device) for t in (hq, hk, hv))
    do = torch.empty(ho.shape, dtype=ho.dtype, device=device)
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def one():
        with torch.cuda.stream(s_in):
            dq.copy_(hq, non_blocking=True); dk.copy_(hk, non_blocking=True); dv.copy_(hv, non_blocking=True)
        with torch.cuda.stream(s_out):
            ho.copy_(do, non_blocking=True)

    one()
    torch.cuda.synchronize(device)
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    torch.cuda.synchronize(device)
    ms = (time.perf_counter() - t0) / steps * 1e3
    barrier()
    ms = allmax(ms, device, world)
    nbytes = sum(t.numel() * t.element_size() for t in (hq, hk, hv, ho))
    return dict(ms_per_step=ms, bytes_per_step=nbytes, gbs_per_gpu=nbytes / (ms * 1e-3) / 1e9)


# ---------------------------------------------------------------------------------------------- 32-layer decoder
DECODER = dict(layers=32, hidden=4096, ffn=14336, Hq=32, Hkv=8, D=128, vocab=128256, C=128, SW=1024, prompt=16384, steps=512,
               batch=128, micro_batch=32, p_global=0.07, p_local=0.20, retained=0.10, eager_steps=8)


def run_decoder_leg(dc, device, rank, world, barrier):
    """The full decoder configuration through the Hugging Face caller of this package: random-init 32-layer
    Llama-3-8B-shaped model, NAtS attention in every layer, prompts of 16384 random token ids, then greedy decoding;
    the batch is split over the ranks (weights replicated) and runs in micro-batches on each."""
    from transformers import LlamaConfig, LlamaForCausalLM
    from neuralattentionsearch_b200 import NAtSCache, check_status
    from neuralattentionsearch_b200.hf import GraphedGreedyDecoder, TransformerArgs, enable_llama_nats_chunk_eval
    cfg = LlamaConfig(hidden_size=dc['hidden'], intermediate_size=dc['ffn'], num_hidden_layers=dc['layers'],
                      num_attention_heads=dc['Hq'], num_key_value_heads=dc['Hkv'], head_dim=dc['D'], vocab_size=dc['vocab'],
                      max_position_embeddings=32768, rope_theta=500000.0)
    torch.manual_seed(2)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(device):
            model = LlamaForCausalLM(cfg).eval()
    finally:
        torch.set_default_dtype(prev)
    enable_llama_nats_chunk_eval(model, TransformerArgs(n_msks=dc['Hkv'], chunk_size=dc['C'], local_seq_max_length=dc['SW']))
    # Role heads: random weights plus a bias.  The role head has no bias term, so the bias rides on a constant feature:
    # every token embedding carries the same value in dimension 0, which the (scale-free) input norm passes on, and
    # column 0 of each role head holds the biases of its three roles.  The biases are fitted per layer on one short pass
    # so that about p_global / p_local of the chunks come out global / local (=> roughly a tenth of the tokens retained).
    noise = 0.05
    with torch.no_grad():
        model.model.embed_tokens.weight[:, 0] = 5 * cfg.initializer_range
        for layer in model.model.layers:
            wgt = layer.self_attn.proj_layer.weight
            wgt.normal_(0, noise)
            wgt[:, 0] = 0
    per_rank = dc['batch'] // world
    mb = min(dc['micro_batch'], per_rank)
    n_mb = per_rank // mb
    g = torch.Generator(device=device).manual_seed(100 + rank)
    gc = torch.Generator(device=device).manual_seed(99)                       # the calibration pass is the same on every rank
    C, SW, N = dc['C'], dc['SW'], dc['prompt']
    mix = torch.tensor([dc['p_global'], dc['p_local']], device=device)

    def fit_bias(module, args_, kwargs_):
        """Runs in front of a layer's attention during the calibration pass: fits the layer's role biases to the chunk
        features that arrive, so that every later layer sees hidden states made under fitted roles.  The logits of a
        (sequence, kv-head) vary little from chunk to chunk in the deeper layers, so the roles of a head are strongly
        correlated and the retained fraction is not what independent chunks with the same mix would give; the share of
        global / local chunks is therefore scaled (bisection) until the RETAINED fraction -- global chunks plus the local
        ones behind the last global chunk -- of the calibration sequences meets the target."""
        x = (kwargs_['hidden_states'] if 'hidden_states' in kwargs_ else args_[0]).float()
        pooled = x.unflatten(1, (-1, C)).mean(2)                                  # [B, chunks, hidden]
        wgt = module.proj_layer.weight
        wv = wgt.view(cfg.num_key_value_heads, 3, -1)
        wv[:, :, 0] = 0
        z = (pooled @ wgt.float().T).unflatten(-1, (cfg.num_key_value_heads, 3))  # [B, chunks, Hkv, 3], no bias column
        f0 = pooled[..., 0].mean()
        idx = torch.arange(z.shape[1], device=device)[None, :, None]

        def fit(target):
            bias = torch.zeros(3, device=device)
            for _ in range(60):
                r = (z + bias).argmax(-1)
                frac = torch.stack([(r == 0).float().mean(), (r == 1).float().mean()]).clamp_min(1e-4)
                bias[:2] += 0.5 * z.std() * (target.log() - frac.log())
            r = (z + bias).argmax(-1)
            r[:, 0] = 0                                                           # the first chunk is always global
            last_g = torch.where(r == 0, idx, -1).amax(1, keepdim=True)
            kept = (r == 0).sum(1) + ((r == 1) & (idx > last_g)).sum(1)
            return bias, (kept.float() / z.shape[1]).mean().item()

        lo, hi = 0.02, 1.0
        for _ in range(7):
            mid = (lo * hi) ** 0.5
            bias, kept = fit(mix * mid)
            lo, hi = (mid, hi) if kept < dc['retained'] else (lo, mid)
        wv[:, 0, 0] = (bias[0] / f0).to(wgt.dtype)
        wv[:, 1, 0] = (bias[1] / f0).to(wgt.dtype)

    with torch.no_grad():
        ids = torch.randint(0, cfg.vocab_size, (2, N), device=device, generator=gc)
        hooks = [layer.self_attn.register_forward_pre_hook(fit_bias, with_kwargs=True) for layer in model.model.layers]
        model(input_ids=ids, past_key_values=NAtSCache(SW, C), use_cache=True, logits_to_keep=1)
        for h in hooks:
            h.remove()
    torch.cuda.synchronize(device)

    pre_ms, dec_ms, replay_ms, eager_ms = 0.0, 0.0, 0.0, 0.0
    fractions = torch.zeros(dc['layers'], device=device)
    role_mix = torch.zeros(dc['layers'], 3, device=device)
    barrier()
    for m in range(n_mb):
        ids = torch.randint(0, cfg.vocab_size, (mb, N), device=device, generator=g)
        cache = NAtSCache(SW, C)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        with torch.no_grad():
            ev[0].record()
            out = model(input_ids=ids, past_key_values=cache, use_cache=True, logits_to_keep=1)
            tok = out.logits[:, -1].argmax(-1, keepdim=True)
            ev[1].record()
            for li, lc in enumerate(cache.cache_model):
                fractions[li] += (lc.size_global_kv + lc.size_local_kv - SW).float().mean() / N / n_mb
                role_mix[li] += model.model.layers[li].self_attn.token_states.float().mean((0, 1, 2)) / n_mb
            # greedy decoding, every step replayed from one CUDA graph (recorded once per micro-batch: the recording and the
            # step that runs in front of it are inside the timed region) ...
            head = min(16, dc['steps'] - 1)
            dec = GraphedGreedyDecoder(model, cache, dc['steps'])
            toks = dec.generate(tok, head)
            ev[3].record()
            toks = dec.generate(toks[:, -1:], dc['steps'] - head)
            ev[2].record()
            # ... and a few steps of the eager loop over the same modules on the same cache, for comparison
            tok = toks[:, -1:]
            for _ in range(dc['eager_steps']):
                out = model(input_ids=tok, past_key_values=cache, use_cache=True)
                tok = out.logits[:, -1].argmax(-1, keepdim=True)
            ev[4].record()
        torch.cuda.synchronize(device)
        pre_ms += ev[0].elapsed_time(ev[1])
        dec_ms += ev[1].elapsed_time(ev[2])
        replay_ms += ev[3].elapsed_time(ev[2])
        eager_ms += ev[2].elapsed_time(ev[4])
        finite = bool(torch.isfinite(out.logits.float()).all() and torch.isfinite(dec.logits.float()).all())
        del cache, out, dec
    check_status(device)
    barrier()
    pre_ms, dec_ms = allmax(pre_ms, device, world), allmax(dec_ms, device, world)
    replay_ms, eager_ms = allmax(replay_ms, device, world), allmax(eager_ms, device, world)
    head = min(16, dc['steps'] - 1)
    fr = fractions.cpu().tolist()
    del model
    torch.cuda.empty_cache()
    return dict(model='random-init Llama-3-8B shape: 32 layers, hidden 4096, FFN 14336, 32q/8kv heads, vocabulary 128256, bf16; '
                      'NAtS attention in every layer (chunk 128, window 1024)',
                batch=dc['batch'], sequences_per_gpu=per_rank, micro_batch=mb, prompt_tokens=N, decode_steps=dc['steps'],
                prefill_tok_per_s=dc['batch'] * N / (pre_ms * 1e-3), decode_tok_per_s=dc['batch'] * dc['steps'] / (dec_ms * 1e-3),
                decode_replay_tok_per_s=dc['batch'] * (dc['steps'] - head) / (replay_ms * 1e-3),
                decode_eager_tok_per_s=dc['batch'] * dc['eager_steps'] / (eager_ms * 1e-3), eager_steps=dc['eager_steps'],
                decode_note='decode_tok_per_s: all steps of hf.GraphedGreedyDecoder including the recording of its CUDA graph (once per '
                            'micro-batch); decode_replay_tok_per_s: the steps after the first 16; decode_eager_tok_per_s: the eager loop over the '
                            'patched Hugging Face model on the same cache (host bound)',
                prefill_s=pre_ms * 1e-3, decode_s=dec_ms * 1e-3, logits_finite=finite,
                retained_frac_per_layer=[round(x, 4) for x in fr], retained_frac_mean=float(np.mean(fr)),
                retained_frac_target=dc['retained'],
                global_local_sliding_share_mean=[round(x, 4) for x in role_mix.mean(0).cpu().tolist()],
                note='sequences of a rank run in micro-batches (prefill and its decode steps per micro-batch); weights replicated; '
                     'no collective')


# ---------------------------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='b200', choices=['b200', 'reference'])
    ap.add_argument('--no-cpu', action='store_true', help='skip the CPU baseline leg')
    ap.add_argument('--no-decode', action='store_true', help='skip the decode leg')
    ap.add_argument('--no-decoder', action='store_true', help='skip the 32-layer decoder leg')
    ap.add_argument('--no-extra', action='store_true', help='skip the strong-scaling, sustained, large-eviction and copy-floor legs')
    ap.add_argument('--decoder-batch', type=int, default=DECODER['batch'], help='sequences of the decoder leg over all GPUs')
    ap.add_argument('--decoder-steps', type=int, default=DECODER['steps'])
    ap.add_argument('--sustained-seconds', type=float, default=2.0)
    ap.add_argument('--case', default='full', choices=['full', 'small', 'long', 'evict'],
                    help="'small' = a quarter of the heads / of the decode batch: the profiling case (inputs still exceed L2); "
                         "'long' = the 131072-token stress configuration (batch 2, window 4096, ~2 % global / 8 % local), "
                         "prefill + eviction only; 'evict' = only the large eviction leg at a quarter of its batch (the profiling "
                         "case of the compaction kernel); none of these lines is the benchmark value")
    args = ap.parse_args()
    if args.case == 'small':
        WORKLOAD.update(Hq=8, Hkv=2)
        DECODE.update(B=16)
    if args.case == 'long':
        WORKLOAD.update(name='prefill131k_evict', B=2, N=131072, SW=4096, p_global=0.02, p_local=0.08)
        args.no_decode = True
        args.no_cpu = True
    if args.case != 'full':
        args.no_decoder = args.no_extra = True

    rank = int(os.environ.get('RANK', 0))
    world = int(os.environ.get('WORLD_SIZE', 1))
    local_rank = int(os.environ.get('LOCAL_RANK', 0))
    w = WORKLOAD
    config = dict(workload='prefill 32k + eviction: B1 x 32q/8kv heads, head_dim 128, N 32768, window 1024, chunk 128, '
                           'roles 5/15/80 % global/local/sliding; one sequence per GPU',
                  l2='inputs larger than L2 (q+k+v+o = 671 MB per step)', sharding='batch x kv-head, no data-path collective')
    if args.case == 'small':
        config = dict(config, workload='PROFILING CASE (not a benchmark value): 8q/2kv heads of the 32k prefill, decode batch 16',
                      l2='inputs larger than L2 (q+k+v+o = 168 MB per step)')
    if args.case == 'long':
        config = dict(config, workload='LONG-CONTEXT STRESS CASE (not the benchmark value): prefill 131072 + eviction, B2 x 32q/8kv heads, '
                                       'head_dim 128, window 4096, chunk 128, roles 2/8/90 % global/local/sliding; two sequences per GPU',
                      l2='inputs larger than L2 (q+k+v+o = 5.4 GB per step)')

    if args.case == 'evict':
        device = torch.device('cuda', local_rank)
        torch.cuda.set_device(device)
        EVICT_LARGE.update(B=8)
        r = run_eviction_large_leg(device, load_peaks(), steps=args.steps)
        print(json.dumps(dict(metric='eviction GB/s (kept tokens and ring, K and V, read + write)', value=r['gbs'], unit='GB/s',
                              n_gpus=1, steps=args.steps, warmup=2, config=dict(workload='PROFILING CASE (not a benchmark value): ' + r['shape'].replace('B32', 'B8')),
                              eviction_large=r)))
        return

    if args.impl == 'reference':
        if rank != 0:
            return
        threads = os.cpu_count() or 1
        # the steps and warm-up asked for, time-boxed; never fewer than 5 timed runs, so that the median means something
        # (`steps_run` says how many ran)
        r = run_cpu_leg(w, max(args.steps, 5), max(1, args.warmup), threads)
        line = dict(metric=METRIC, value=r['value'], unit='TFLOP/s', n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                    ms_per_step=r['seconds_per_step'] * 1e3, higher_is_better=True, scaling='weak', vs_baseline=None,
                    dtype='f32', data='synthetic', config=config, impl='reference', steps_run=r['steps'],
                    cpu_baseline=dict(value=r['value'], unit='TFLOP/s', cores=threads, kind=r['kind'], sample=r['sample']),
                    e2e=dict(value=r['value'], unit='TFLOP/s', h2d_bytes_per_step=0, d2h_bytes_per_step=0))
        if r['kind'] == 'reference':
            p = run_cpu_port_leg(w, 3, 1, threads, budget_s=30.0)
            line['cpu_port'] = dict(value=p['value'], unit='TFLOP/s', cores=threads, kind='port', sample=p['sample'])
        print(json.dumps(line))
        return

    import torch.distributed as dist
    from neuralattentionsearch_b200 import check_status, prefill_attention
    from neuralattentionsearch_b200.cache import NAtSChunkLayerCache
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        dist.init_process_group('nccl', device_id=torch.device('cuda', local_rank))
    device = torch.device('cuda', local_rank)
    torch.cuda.set_device(device)
    numa = bind_to_gpu_numa_node(local_rank) if world > 1 else None
    peaks = load_peaks()
    traffic = load_traffic() if args.case == 'full' else {}

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    # ---- inputs: host (pinned) and device copies ----
    hq, hk, hv, hroles = make_prefill_inputs(w, w['seed'] + rank, pin=True)
    q, k, v, roles = (t.to(device) for t in (hq, hk, hv, hroles))
    kept = torch.zeros(w['B'], w['Hkv'], dtype=torch.int64, device=device)

    def step(qd, kd, vd, evs=None):
        # the reference's call order: cache.update (keeps K/V, plans the keep-set), attention, cache.post_update (compaction)
        lc = NAtSChunkLayerCache(w['B'], w['Hkv'], w['SW'], chunk_size=w['C'], device=device)
        lc.update(kd, vd, roles)
        o = prefill_attention(qd, kd, vd, roles, w['C'], w['SW'], kept_tiles=kept)
        if evs is not None:
            evs[1].record()
        lc.post_update(w['N'])
        return o, lc

    for _ in range(args.warmup):
        o, lc = step(q, k, v)
    check_status(device)
    n_kept = int(kept.sum().item())
    flops = 4.0 * 128 * 128 * w['D'] * (w['Hq'] // w['Hkv']) * n_kept
    n_tiles_causal = w['B'] * w['Hkv'] * (w['N'] // 128) * (w['N'] // 128 + 1) // 2

    # ---- device-resident timing ----
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    barrier()
    for i in range(args.steps):
        evs[i][0].record()
        o, lc = step(q, k, v, evs[i])
        evs[i][2].record()
    barrier()
    ms_total = evs[0][0].elapsed_time(evs[-1][2])
    check_status(device)
    ms_prefill = float(np.mean([e[0].elapsed_time(e[1]) for e in evs]))
    ms_evict = float(np.mean([e[1].elapsed_time(e[2]) for e in evs]))
    t = torch.tensor([ms_total], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    value = flops * world / (ms_step * 1e-3) / 1e12

    # ---- the dominant kernel by itself: launches queued back to back on the current stream, no host sync in between
    # (each call is the role-metadata kernel, ~1 % of the time, followed by the prefill kernel)
    ka, kb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    ka.record()
    n_kernel = max(args.steps, 10)          # enough launches in the queue to hide the host's launch latency
    for _ in range(n_kernel):
        prefill_attention(q, k, v, roles, w['C'], w['SW'])
    kb.record()
    torch.cuda.synchronize(device)
    check_status(device)
    ms_kernel = ka.elapsed_time(kb) / n_kernel

    # eviction bytes: kept tokens and ring, read + write, K and V
    ev_tokens = int((lc.size_global_kv + lc.size_local_kv).sum().item())
    ev_bytes = 2 * 2 * ev_tokens * w['D'] * 2

    # ---- end to end: host buffers in, host result out ----
    ho = torch.empty(w['B'], w['Hq'], w['N'], w['D'], dtype=torch.bfloat16).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hroles))
    d2h = ho.numel() * ho.element_size()
    e2e_steps = max(3, min(args.steps, 5))

    from neuralattentionsearch_b200 import HostPrefillPipeline
    pipe = HostPrefillPipeline(w['B'], w['Hq'], w['Hkv'], w['N'], w['D'], w['C'], w['SW'], device)

    def e2e_step():
        # the call a user with host-resident tensors makes: pinned q/k/v/roles in, pinned output out; pieces of one
        # (batch, kv-head) pair are copied in, computed and copied out concurrently; the eviction follows on the device
        pipe.run(hq, hk, hv, hroles, ho)
        lc = NAtSChunkLayerCache(w['B'], w['Hkv'], w['SW'], chunk_size=w['C'], device=device)
        lc.update(pipe.k, pipe.v, pipe.roles)
        lc.post_update(w['N'])

    e2e_step()
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(e2e_steps):
        e2e_step()
    b.record()
    barrier()
    t = torch.tensor([a.elapsed_time(b)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / e2e_steps
    e2e_value = flops * world / (e2e_ms * 1e-3) / 1e12
    check_status(device)

    # ---- second 32k segment of the same sequence over the compacted cache of the first ----
    continuation = None
    if not args.no_decode:
        q2, k2, v2, roles2 = (t.to(device) for t in make_prefill_inputs(w, w['seed'] + 1000 + rank))
        kept2 = torch.zeros(w['B'], w['Hkv'], dtype=torch.int64, device=device)
        times = []
        for i in range(2 + 3):
            _, lc2 = step(q, k, v)
            ev4 = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            torch.cuda.synchronize(device)
            ev4[0].record()
            lc2.update(k2, v2, roles2)
            ev4[1].record()
            lc2.prefill_attention(q2, kept_tiles=kept2)
            ev4[2].record()
            lc2.post_update(w['N'])
            ev4[3].record()
            torch.cuda.synchronize(device)
            if i >= 2:
                times.append([ev4[j].elapsed_time(ev4[j + 1]) for j in range(3)])
        check_status(device)
        tm = np.array(times).mean(0)
        n_kept2 = int(kept2.sum().item())
        fl2 = 4.0 * 128 * 128 * w['D'] * (w['Hq'] // w['Hkv']) * n_kept2
        continuation = dict(metric='prefill TFLOP/s on kept tiles, second 32k segment over the compacted cache of the first',
                            value=fl2 / (tm[1] * 1e-3) / 1e12, unit='TFLOP/s', kept_tiles=n_kept2,
                            ms_append=float(tm[0]), ms_attention=float(tm[1]), ms_eviction=float(tm[2]),
                            cache_rows_after=int(lc2.n_ctx_data), per_gpu=True)
        del q2, k2, v2, lc2

    # ---- caller-side helper in front of the prefill: rotary embedding + head split of the projections, one pass ----
    rope = None
    if not args.no_decode:
        from neuralattentionsearch_b200.functional import rope_split_heads
        gq = torch.Generator(device=device).manual_seed(7)
        xin = [torch.randn(w['B'], w['N'], h * w['D'], generator=gq, device=device).to(torch.bfloat16) for h in (w['Hq'], w['Hkv'], w['Hkv'])]
        ang = torch.arange(w['N'], device=device).float()[None, :, None] / (500000.0 ** (torch.arange(0, w['D'], 2, device=device).float() / w['D']))
        ang = torch.cat([ang, ang], -1)
        cos_t, sin_t = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
        for _ in range(3):
            rope_split_heads(*xin, cos_t, sin_t, w['Hq'], w['Hkv'], w['D'])
        ra, rb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(device)
        ra.record()
        for _ in range(10):
            rope_split_heads(*xin, cos_t, sin_t, w['Hq'], w['Hkv'], w['D'])
        rb.record()
        torch.cuda.synchronize(device)
        rms = ra.elapsed_time(rb) / 10
        rbytes = 2 * 2 * w['B'] * w['N'] * (w['Hq'] + 2 * w['Hkv']) * w['D']
        rope = dict(metric='RoPE + head split of the q/k/v projections, GB/s (read + write)', value=rbytes / (rms * 1e-3) / 1e9,
                    unit='GB/s', ms=rms, bytes=rbytes, frac_of_hbm=rbytes / (rms * 1e-3) / 1e9 / peaks['hbm_gbs'], per_gpu=True)
        del xin, cos_t, sin_t

    # ---- decode leg ----
    decode = None
    if not args.no_decode:
        dsteps = DECODE['steps']
        r = run_decode_leg(DECODE, device, dsteps, warmup=max(3, args.warmup))
        t = torch.tensor([r['ms_total']], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dms = float(t.item())
        gbs = r['kv_bytes_per_step'] / (r['ms_total'] / dsteps * 1e-3) / 1e9
        decode = dict(metric='decode tok/s @32k compacted KV', value=r['tokens'] * world / (dms * 1e-3), unit='tok/s',
                      ms_per_step=dms / dsteps, steps=dsteps, batch_per_gpu=DECODE['B'], gpu_launches=r['launches'],
                      config='B64 x 32q/8kv heads, head_dim 128, retained 2k-6k per (sequence, kv-head) + 1024-slot ring '
                             '(each of its 8 chunks valid with p = 0.8), chunk 128, one role per completed chunk',
                      roofline=dict(bound='hbm', achieved=gbs, peak=peaks['hbm_gbs'], unit='GB/s', frac=gbs / peaks['hbm_gbs'],
                                    traffic=traffic.get('decode_kernel'), bytes_per_step=r['kv_bytes_per_step'], of=peaks['_source']))
        if world > 1:      # NCCL only here: gather the last step's outputs of all ranks
            outs = [torch.empty_like(r['out']) for _ in range(world)]
            dist.all_gather(outs, r['out'])

    # the clock samples cover every timed GPU leg above (the prefill + eviction steps alone last ~12 ms, less than one
    # sampling interval of nvidia-smi)
    clocks = sampler.stop() if rank == 0 else None

    # ---- token-granular decode: chunk size 1, every step places its token (appends it or evicts) ----
    decode_c1 = None
    if not args.no_decode:
        d1 = dict(DECODE, C=1)
        r = run_decode_leg(d1, device, d1['steps'], warmup=max(3, args.warmup))
        dms = allmax(r['ms_total'], device, world)
        gbs = r['kv_bytes_per_step'] / (r['ms_total'] / d1['steps'] * 1e-3) / 1e9
        decode_c1 = dict(metric='decode tok/s @32k compacted KV, token-granular roles (chunk 1)', value=r['tokens'] * world / (dms * 1e-3),
                         unit='tok/s', ms_per_step=dms / d1['steps'], steps=d1['steps'], batch_per_gpu=d1['B'], gpu_launches=r['launches'],
                         gbs=gbs, frac_of_hbm=gbs / peaks['hbm_gbs'],
                         note='one attention launch and one placement launch per step; the role of each new token decides whether it is '
                              'kept (global: kept, locals in front of it dropped; local: appended) or only enters the ring (sliding)')

    # ---- the partition of ONE job over the ranks (strong scaling), sustained regime, large eviction, copy floor ----
    strong = sustained = evict_large = copy_floor = None
    if not args.no_extra:
        strong = dict(prefill=run_strong_prefill_leg(w, device, rank, world, max(args.steps, 10), barrier, (q, k, v, roles)))
        if not args.no_decode:
            strong['decode'] = run_strong_decode_leg(DECODE, device, rank, world, 64, barrier)
        copy_floor = run_copy_floor_leg(hq, hk, hv, ho, device, world, barrier)
        barrier()
        sustained = run_sustained_leg(w, device, rank, args.sustained_seconds, q, k, v, roles, peaks)
        evict_large = run_eviction_large_leg(device, peaks)
        barrier()

    # ---- the 32-layer decoder configuration ----
    decoder = None
    if not args.no_decoder:
        del q, k, v, o, pipe
        torch.cuda.empty_cache()
        dc = dict(DECODER, batch=args.decoder_batch, steps=args.decoder_steps)
        if dc['batch'] % world == 0:
            decoder = run_decoder_leg(dc, device, rank, world, barrier)

    # ---- CPU baseline (rank 0, single GPU run only) ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        c = run_cpu_leg(w, 5, 1, threads)
        cpu = dict(value=c['value'], unit='TFLOP/s', cores=threads, kind=c['kind'], sample=c['sample'],
                   seconds=c['seconds_per_step'])

    if rank == 0:
        tf = flops / (ms_kernel * 1e-3) / 1e12
        peak = peaks['bf16_tflops_sustained'] if ms_kernel * max(args.steps, 10) > 1000 else peaks['bf16_tflops']
        line = dict(metric=METRIC if args.case != 'long' else 'prefill TFLOP/s on kept tiles @131k', value=value, unit='TFLOP/s', n_gpus=world, steps=args.steps, warmup=args.warmup,
                    ms_per_step=ms_step, higher_is_better=True, scaling='weak', vs_baseline=None, dtype='bf16',
                    data='synthetic', config=config, clocks=clocks,
                    e2e=dict(value=e2e_value, unit='TFLOP/s', h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h, ms_per_step=e2e_ms,
                             note='q, k, v arrive from and o returns to pinned host memory every step (PCIe bound); in the reference\'s '
                                  'callers these tensors are projections of hidden states that already live on the device',
                             **({'numa_node_of_rank0': numa} if numa is not None else {})),
                    gpu_launches=4 * args.steps,          # timed region: role_prep, prefill, evict_plan, evict_compact per step
                    roofline=dict(bound='tensor', achieved=tf, peak=peak, unit='TFLOP/s', frac=tf / peak, traffic=traffic.get('prefill_kernel'),
                                  kernel='prefill_kernel<128>', ms_per_launch=ms_kernel, ms_in_step=ms_prefill,
                                  timing='CUDA events around %d launches queued back to back (role metadata kernel included); '
                                         'ms_in_step is the same call inside a step, after the eviction read-back' % max(args.steps, 10),
                                  of=peaks['_source'] + ' cuBLAS bf16'),
                    kept_tiles=dict(kept=n_kept, causal=n_tiles_causal, skipped_frac=1 - n_kept / n_tiles_causal,
                                    flop_per_step=flops),
                    eviction=dict(ms=ms_evict, bytes=ev_bytes, gbs=ev_bytes / (ms_evict * 1e-3) / 1e9,
                                  retained_frac=(ev_tokens - w['B'] * w['Hkv'] * w['SW']) / (w['B'] * w['Hkv'] * w['N']),
                                  note='compaction only: the keep-set is planned in update(), ahead of the attention, and its size reaches the host while the attention runs; launch-latency bound at this size'),
                    decode=decode, decode_token_granular=decode_c1, continuation=continuation, rope_split_heads=rope,
                    strong=strong, sustained=sustained, eviction_large=evict_large,
                    e2e_copy_floor=(dict(copy_floor, note='same host<->device bytes as the e2e step, no kernel, all ranks at once; '
                                                          'e2e ms_per_step / this = how close the pipeline is to the copy floor')
                                    if copy_floor else None),
                    decoder=decoder, cpu_baseline=cpu)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
