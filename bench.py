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
    cap = t0 + 4 * C + d['steps']
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


def run_cpu_leg(w, steps, warmup, threads):
    """The reference's eager math (dense mask rows + softmax(QK^T)V in fp32 over every causal key, per query-row block,
    as its CPU path does it) on a bounded sample of the workload, through the oracle port."""
    from oracle import nats_oracle as orc
    torch.set_num_threads(threads)
    q, k, v, roles = make_prefill_inputs(w, w['seed'])
    q, k, v = q.float(), k.float(), v.float()
    roles_np = roles.numpy()
    blocks = cpu_sample_blocks(w)
    lim = orc.row_limit(roles_np, w['C'], w['SW'])
    lim_tok = np.repeat(lim, w['C'], -1)
    tmax = lim_tok.reshape(w['B'], w['Hkv'], -1, 128).max(-1)
    kept = 0
    for lo, hi in blocks:
        for t in range(lo // 128, hi // 128):
            kept += int((tmax[:, :, :t + 1] >= t * 128).sum())
    flops = 4.0 * 128 * 128 * w['D'] * (w['Hq'] // w['Hkv']) * kept

    def one():
        for lo, hi in blocks:
            orc.prefill_attention(q, k, v, roles_np, w['C'], w['SW'], rows=(lo, hi), block=hi - lo)

    for _ in range(warmup):
        one()
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    dt = (time.perf_counter() - t0) / steps
    return dict(value=flops / dt / 1e12, seconds_per_step=dt, flops=flops,
                sample=f'{len(blocks)} query blocks of 512 rows (starting at rows {[b[0] for b in blocks]}), all {w["Hq"]} heads, '
                       f'fp32, dense causal keys as the eager path computes them; value counts kept-tile flop only')


# ---------------------------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='b200', choices=['b200', 'reference'])
    ap.add_argument('--no-cpu', action='store_true', help='skip the CPU baseline leg')
    ap.add_argument('--no-decode', action='store_true', help='skip the decode leg')
    ap.add_argument('--case', default='full', choices=['full', 'small', 'long'],
                    help="'small' = a quarter of the heads / of the decode batch: the profiling case (inputs still exceed L2); "
                         "'long' = the 131072-token stress configuration (batch 2, window 4096, ~2 % global / 8 % local), "
                         "prefill + eviction only; neither line is the benchmark value")
    args = ap.parse_args()
    if args.case == 'small':
        WORKLOAD.update(Hq=8, Hkv=2)
        DECODE.update(B=16)
    if args.case == 'long':
        WORKLOAD.update(name='prefill131k_evict', B=2, N=131072, SW=4096, p_global=0.02, p_local=0.08)
        args.no_decode = True
        args.no_cpu = True

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

    if args.impl == 'reference':
        if rank != 0:
            return
        threads = os.cpu_count() or 1
        steps, warmup = max(1, min(args.steps, 3)), max(1, min(args.warmup, 1))
        r = run_cpu_leg(w, steps, warmup, threads)
        line = dict(metric=METRIC, value=r['value'], unit='TFLOP/s', n_gpus=args.gpus, steps=steps, warmup=warmup,
                    ms_per_step=r['seconds_per_step'] * 1e3, higher_is_better=True, scaling='weak', vs_baseline=None,
                    dtype='f32', data='synthetic', config=config, impl='reference',
                    cpu_baseline=dict(value=r['value'], unit='TFLOP/s', cores=threads, kind='port', sample=r['sample']),
                    e2e=dict(value=r['value'], unit='TFLOP/s', h2d_bytes_per_step=0, d2h_bytes_per_step=0))
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
    e2e_value = flops * world / (float(t.item()) / e2e_steps * 1e-3) / 1e12
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

    # ---- CPU baseline (rank 0, single GPU run only) ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        c = run_cpu_leg(w, 1, 1, threads)
        cpu = dict(value=c['value'], unit='TFLOP/s', cores=threads, kind='port', sample=c['sample'],
                   seconds=c['seconds_per_step'])

    if rank == 0:
        tf = flops / (ms_kernel * 1e-3) / 1e12
        peak = peaks['bf16_tflops_sustained'] if ms_kernel * max(args.steps, 10) > 1000 else peaks['bf16_tflops']
        line = dict(metric=METRIC if args.case != 'long' else 'prefill TFLOP/s on kept tiles @131k', value=value, unit='TFLOP/s', n_gpus=world, steps=args.steps, warmup=args.warmup,
                    ms_per_step=ms_step, higher_is_better=True, scaling='weak', vs_baseline=None, dtype='bf16',
                    data='synthetic', config=config, clocks=clocks,
                    e2e=dict(value=e2e_value, unit='TFLOP/s', h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h,
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
                    decode=decode, continuation=continuation, rope_split_heads=rope, cpu_baseline=cpu)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
