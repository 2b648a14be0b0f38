#!/usr/bin/env python
"""Benchmark of the forward-Laplacian hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One JSON line on stdout (rank 0).  A "step" is one pass of the hot path over one batch of
synthetic triplets; `value` is samples (walker-Laplacians) per second over all ranks with the
inputs already in HBM; `e2e` is the same through host buffers (H2D of the inputs and D2H of the
result inside the timed region).  `--impl reference` times the CPU restatement of the reference's
rules (the reference itself is pure Python on JAX, which is not installed on these machines).

Workloads: `operators` (default; the operator microbench: dot_general, tanh, silu, LayerNorm as
single launches on a dense and on a sparse Jacobian), `mlp`, `ferminet`, `psiformer`, `psiformer64`
(whole wavefunctions through the front end with CUDA-graph replay), and the single-kernel profiling
cases `attention`, `slogdet`, `gather`.  Environment switches, all off by default:
FOLX_B200_CHAIN=1 (tanh + silu as one launch), FOLX_B200_NO_GRAPH=1 (no graph replay in the model
workloads), FOLX_B200_E2E_SLICES=n (sample slices of the end-to-end pipeline),
FOLX_B200_MEASURE_TF32=1 (time a library TF32 GEMM beside the run), FOLX_B200_SLOGDET_N=8|16|32
(matrix size of the `slogdet` case; 16 by default).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = 'walker_laplacians_per_sec'
UNIT = 'walker-Laplacians/s'


def load_peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {'hbm_gbs': p['hbm_gbs'], 'bf16_tflops': p['bf16_tflops'], 'source': 'measured'}
    return {'hbm_gbs': 6650.0, 'bf16_tflops': 1590.0, 'source': 'fallback'}


# ------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ('clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,'
              'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
              'clocks_event_reasons.sw_power_cap')

    def __init__(self, index: int):
        self.index = index
        self.samples: list[list[str]] = []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ['nvidia-smi', f'--query-gpu={self.FIELDS}', '--format=csv,noheader,nounits',
                     '-i', str(self.index)], capture_output=True, text=True, timeout=5).stdout
                row = [c.strip() for c in out.strip().split(',')]
                if len(row) == 6:
                    self.samples.append(row)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        if not self.samples:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['unsampled']}
        sm = [float(s[0]) for s in self.samples if s[0].replace('.', '').isdigit()]
        mx = [float(s[1]) for s in self.samples if s[1].replace('.', '').isdigit()]
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith('active') for s in self.samples)]
        return {'sm_mhz': statistics.median(sm) if sm else None, 'sm_max_mhz': max(mx) if mx else None,
                'reasons': reasons, 'samples': len(self.samples)}


# ------------------------------------------------------------------------------------------
# workload: operator microbench (BASELINE.json configs[1])
# ------------------------------------------------------------------------------------------
B, D, F, KS = 4096, 96, 256, 3  # samples, dense Jacobian rows, features, sparse rows per position
# The microbench times SINGLE primitives, so tanh and silu are two launches.  FOLX_B200_CHAIN=1
# evaluates them as one launch (fl_elementwise_chain), which is what the front end does with a run
# of scalar functions inside a traced function; that variant is for comparison only.
FUSE_SCALAR_RUN = bool(os.environ.get('FOLX_B200_CHAIN'))


def make_host_inputs(seed: int, n_samples: int = B):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g)
    return {
        'dense': (mk(n_samples, F), mk(D, n_samples, F), mk(n_samples, F)),
        'sparse': (mk(n_samples, F), mk(KS, n_samples, F), mk(n_samples, F)),
        'W': mk(F, F) / F**0.5,
        'bias': mk(F) * 0.1,
    }


def chain_device(kernels, a, W, bias, timers=None):
    """dot_general(+bias) -> tanh -> silu -> LayerNorm on one triplet; optional per-kernel events."""
    def run(name, fn):
        if timers is None:
            return fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        timers.append((name, e0, e1))
        return out

    tag = 'dense' if a.jacobian.data.shape[0] > KS else 'sparse'
    h = run(f'dot_general/{tag}', lambda: kernels.dot_general(a, W, bias))
    if FUSE_SCALAR_RUN:
        # what the front end does with a run of scalar functions: one pass for silu(tanh(.))
        h = run(f'tanh+silu/{tag}', lambda: kernels.elementwise_chain(['tanh', 'silu'], h))
    else:
        h = run(f'tanh/{tag}', lambda: kernels.elementwise('tanh', h))
        h = run(f'silu/{tag}', lambda: kernels.elementwise('silu', h))
    h = run(f'layernorm/{tag}', lambda: kernels.layernorm(h, None, None, 1e-6))
    return h


def chain_oracle(rules, t, W, bias):
    t = rules.dot_general(t, W, bias)
    t = rules.elementwise('tanh', t)
    t = rules.elementwise('silu', t)
    return rules.layernorm(t, None, None, 1e-6)


def algorithmic(name: str):
    """(bytes, flops) one launch of the named kernel moves / computes (fp32, algorithmic)."""
    kind, tag = name.split('/')
    K = D if tag == 'dense' else KS
    rows = (K + 2) * B
    if kind == 'dot_general':
        return 4 * (rows * (F + F) + F * F + F), 2 * rows * F * F
    return 8 * rows * F, 0


def measure_tf32_peak(device, n: int = 8192):
    """cuBLAS TF32 GEMM throughput on this GPU (a library call used ONLY to measure a ceiling)."""
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a = torch.randn(n, n, device=device)
        b = torch.randn(n, n, device=device)
        best = float('inf')
        for _ in range(6):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b)
            e1.record()
            torch.cuda.synchronize(device)
            best = min(best, e0.elapsed_time(e1))
        return round(2 * n**3 / best / 1e9, 1)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


def run_ours(args, rank, world, device):
    from folx_b200 import kernels, lib

    lib.load()
    host = make_host_inputs(seed=rank, n_samples=B)
    pinned = {k: tuple(t.pin_memory() for t in host[k]) for k in ('dense', 'sparse')}
    W = host['W'].to(device)
    bias = host['bias'].to(device)

    def upload(kind):
        x, J, lap = pinned[kind]
        a = kernels.alloc_triplet(J.shape[0], x.shape, device)
        a.x.copy_(x, non_blocking=True)
        a.jacobian.data.copy_(J, non_blocking=True)
        a.laplacian.copy_(lap, non_blocking=True)
        return a

    dense, sparse = upload('dense'), upload('sparse')
    torch.cuda.synchronize(device)

    def step(timers=None):
        chain_device(kernels, dense, W, bias, timers)
        chain_device(kernels, sparse, W, bias, timers)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(device)

    # ---- device-resident timing ----
    # The clock sampler (a thread that spawns nvidia-smi) starts before the warm-up so that the GPU
    # does not sit idle between the warm-up and the timed steps while the host forks.
    timers: list = []
    with ClockSampler(device.index or 0) as clocks:
        for _ in range(max(args.warmup, 3)):
            step()
        kernels.check_gemm_status(device)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step(timers)
        e1.record()
        barrier()
        # keep sampling long enough for at least a couple of nvidia-smi readings
        total_ms = e0.elapsed_time(e1)
        if total_ms < 800:
            t_end = time.time() + 0.8
            while time.time() < t_end:
                step()
            torch.cuda.synchronize(device)
    kernels.check_gemm_status(device)
    launches = (6 if FUSE_SCALAR_RUN else 8) * args.steps

    # ---- end to end through host buffers ----
    # The samples are independent, so the host buffers are handled in slices of the sample axis:
    # while one slice is being computed the next one is uploaded and the previous result is
    # downloaded (three streams; PCIe is full duplex).  Host data is laid out slice by slice in
    # pinned memory; every byte of every input and output crosses the bus inside the timed region.
    e2e_steps = max(2, min(args.steps, 5))
    # 4 slices measured best (9.9 ms; 8: 10.3, 16: 10.9, 32: 12.5; both directions of the bus busy
    # at once take 9.3 ms for these bytes)
    n_slices = int(os.environ.get('FOLX_B200_E2E_SLICES', 4))
    if n_slices < 1 or B % n_slices != 0 or B < 64:
        n_slices = 1
    sl = B // n_slices

    def slices_of(t3):
        x, J, lap = t3
        return [(x[i * sl:(i + 1) * sl].contiguous().pin_memory(), J[:, i * sl:(i + 1) * sl].contiguous().pin_memory(),
                 lap[i * sl:(i + 1) * sl].contiguous().pin_memory()) for i in range(n_slices)]

    host_slices = {k: slices_of(host[k]) for k in ('dense', 'sparse')}
    out_slices = {k: [tuple(torch.empty_like(t).pin_memory() for t in s) for s in host_slices[k]]
                  for k in ('dense', 'sparse')}
    s_up, s_down = torch.cuda.Stream(device), torch.cuda.Stream(device)
    s_main = torch.cuda.current_stream(device)
    ring = {k: [kernels.alloc_triplet(host_slices[k][0][1].shape[0], host_slices[k][0][0].shape, device)
                for _ in range(3)] for k in ('dense', 'sparse')}

    def e2e_step():
        pending = []
        for kind in ('dense', 'sparse'):
            free_ev = [None, None, None]
            for i in range(n_slices):
                a = ring[kind][i % 3]
                with torch.cuda.stream(s_up):
                    if free_ev[i % 3] is not None:
                        s_up.wait_event(free_ev[i % 3])  # the slice that used this buffer is done
                    hx, hj, hl = host_slices[kind][i]
                    a.x.copy_(hx, non_blocking=True)
                    a.jacobian.data.copy_(hj, non_blocking=True)
                    a.laplacian.copy_(hl, non_blocking=True)
                    up = torch.cuda.Event()
                    up.record(s_up)
                s_main.wait_event(up)
                h = chain_device(kernels, a, W, bias)
                done = torch.cuda.Event()
                done.record(s_main)
                free_ev[i % 3] = done
                with torch.cuda.stream(s_down):
                    s_down.wait_event(done)
                    ox, oj, ol = out_slices[kind][i]
                    ox.copy_(h.x, non_blocking=True)
                    oj.copy_(h.jacobian.data, non_blocking=True)
                    ol.copy_(h.laplacian, non_blocking=True)
                    h.x.record_stream(s_down)  # one buffer holds x, J and lap
                pending.append(h)
        s_main.wait_stream(s_down)
        s_main.wait_stream(s_up)

    e2e_step()
    barrier()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    for _ in range(e2e_steps):
        e2e_step()
    g1.record()
    barrier()
    e2e_ms = g0.elapsed_time(g1) / e2e_steps
    io_bytes = sum(t.numel() * 4 for k in ('dense', 'sparse') for t in host[k])

    if world > 1:
        t = torch.tensor([total_ms, e2e_ms], device=device, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        total_ms, e2e_ms = float(t[0]), float(t[1])

    # ---- per-kernel roofline from the events recorded inside the timed region ----
    per_kernel: dict[str, list[float]] = {}
    for name, a, b in timers:
        per_kernel.setdefault(name, []).append(a.elapsed_time(b))
    peaks = load_peaks()
    tf32_peak = peaks['bf16_tflops'] / 2.0  # dense TF32 is half the bf16 rate
    kern = {}
    for name, ts in per_kernel.items():
        ms = sum(ts) / len(ts)
        nbytes, flops = algorithmic(name)
        kern[name] = {'ms': round(ms, 4), 'share': None, 'GBps': round(nbytes / ms / 1e6, 1),
                      'frac_hbm': round(nbytes / ms / 1e6 / peaks['hbm_gbs'], 3)}
        if flops:
            kern[name]['TFLOPs_fp32_equiv'] = round(flops / ms / 1e9, 1)
    tot = sum(v['ms'] for v in kern.values())
    for v in kern.values():
        v['share'] = round(v['ms'] / tot, 3)
    dominant = max(kern, key=lambda n: kern[n]['ms'])
    nbytes, flops = algorithmic(dominant)
    ms = kern[dominant]['ms']
    if dominant.startswith('dot_general'):
        achieved = flops / ms / 1e9
        # DRAM traffic of this kernel from the committed ncu capture (profiles/gemm_tc_kernel_*):
        # 362.0 MB read + written for 200 704 rows; it grows in proportion to the rows of a launch
        rows = ((D if dominant.endswith('dense') else KS) + 2) * B
        roofline = {'kernel': dominant, 'bound': 'tensor', 'achieved': round(achieved, 1),
                    'peak': round(tf32_peak, 1), 'unit': 'TFLOP/s', 'frac': round(achieved / tf32_peak, 3),
                    'traffic': round(362.0e6 * rows / 200704),
                    'note': 'achieved = fp32-equivalent (algorithmic) flops; the 3xTF32 split executes 3x '
                            'that on the tensor pipe, so the ceiling is peak/3; peak = measured bf16 / 2 '
                            f'({peaks["source"]}); traffic scaled from the ncu capture at 2048 samples',
                    'frac_of_3xtf32_ceiling': round(3 * achieved / tf32_peak, 3),
                    # a library TF32 GEMM timed beside it, only on request (it is not part of any
                    # path; 709-750 TFLOP/s were measured on this pool)
                    'tf32_cublas_tflops_this_run': (measure_tf32_peak(device)
                                                    if os.environ.get('FOLX_B200_MEASURE_TF32') else None),
                    'hbm_frac': kern[dominant]['frac_hbm']}
    else:
        achieved = nbytes / ms / 1e6
        roofline = {'kernel': dominant, 'bound': 'hbm', 'achieved': round(achieved, 1),
                    'peak': peaks['hbm_gbs'], 'unit': 'GB/s', 'frac': round(achieved / peaks['hbm_gbs'], 3),
                    'traffic': None, 'note': f'peak {peaks["source"]}'}

    result = {
        'metric': METRIC, 'value': world * B * args.steps / (total_ms / 1e3), 'unit': UNIT,
        'n_gpus': world, 'steps': args.steps, 'warmup': max(args.warmup, 3),
        'ms_per_step': total_ms / args.steps, 'higher_is_better': True, 'scaling': 'weak',
        'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': 'operator-microbench (BASELINE configs[1]): per step, on B=4096 samples, '
                               'dot_general(256x256)+bias -> tanh -> silu -> LayerNorm on a dense J (d=96) '
                               'and on a sparse J (3 rows per position)'
                               + ('; tanh and silu are evaluated by one fused launch' if FUSE_SCALAR_RUN else ''),
                   'samples_per_gpu': B, 'jac_rows_dense': D, 'jac_rows_sparse': KS, 'features': F,
                   'l2': 'dense triplet is 411 MB per tensor (> 126 MB L2); every kernel streams it'},
        'clocks': clocks.summary(),
        'e2e': {'value': world * B / (e2e_ms / 1e3), 'unit': UNIT, 'h2d_bytes_per_step': io_bytes,
                'd2h_bytes_per_step': io_bytes, 'ms_per_step': e2e_ms},
        'gpu_launches': launches,
        'roofline': roofline,
        'kernels': kern,
    }
    return result


def use_all_host_threads() -> int:
    """The CPU arm runs on every core this process may use.  (A multi-process launcher sets
    OMP_NUM_THREADS=1 for its workers; only rank 0 runs the CPU arm, so it takes the cores back.)"""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    if torch.get_num_threads() != n:
        torch.set_num_threads(n)
    return n


def cpu_baseline(sample: int, repeats: int = 3):
    """Times the CPU restatement (oracle, torch fp32, all host threads) on `sample` samples."""
    from oracle import rules

    use_all_host_threads()
    host = make_host_inputs(seed=0, n_samples=sample)
    W, bias = host['W'], host['bias']
    chain_oracle(rules, host['sparse'], W, bias)  # warm-up
    chain_oracle(rules, host['dense'], W, bias)
    # repeat the step until about ten seconds of CPU work have been timed (at least `repeats` passes)
    times, budget = [], 10.0
    while len(times) < repeats or (sum(times) < budget and len(times) < 60):
        t0 = time.perf_counter()
        chain_oracle(rules, host['dense'], W, bias)
        chain_oracle(rules, host['sparse'], W, bias)
        times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    return {'value': sample / t, 'unit': UNIT, 'cores': torch.get_num_threads(), 'kind': 'port',
            'sample': f'{sample} of {B} samples of the same step (dense d=96 chain + sparse chain), torch-CPU fp32, '
                      f'median of {len(times)} passes ({sum(times):.1f} s of CPU work); host has '
                      f'{os.cpu_count()} logical cores',
            'seconds': t}


def run_reference(args, rank, world):
    if rank != 0:
        return None
    use_all_host_threads()
    if args.workload != 'operators':
        base = cpu_model_baseline(args.workload, walkers=max(1, min(args.steps, 4)))
        return {
            'impl': 'reference', 'metric': METRIC, 'value': base['value'], 'unit': UNIT, 'n_gpus': world,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': 1e3 / base['value'],
            'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32',
            'data': 'synthetic',
            'config': {'workload': MODEL_WORKLOADS[args.workload][3] + '; each step is one walker',
                       'note': 'brute-force automatic differentiation of the same function on the host '
                               '(the reference needs JAX, which is not installed here)'},
            'cpu_baseline': base,
            'e2e': {'value': base['value'], 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
            'gpu_launches': 0,
        }
    times = []
    sample = 256
    from oracle import rules

    host = make_host_inputs(seed=0, n_samples=sample)
    W, bias = host['W'], host['bias']
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        chain_oracle(rules, host['dense'], W, bias)
        chain_oracle(rules, host['sparse'], W, bias)
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    total = sum(times)
    value = sample * args.steps / total
    return {
        'impl': 'reference', 'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': world,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': total / args.steps * 1e3,
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32',
        'data': 'synthetic',
        'config': {'workload': 'operator-microbench (BASELINE configs[1]); each step is a bounded sample of '
                               f'{sample} of the 4096 samples', 'note': 'CPU restatement of the reference rules '
                               '(the reference needs JAX, which is not installed here)'},
        'cpu_baseline': {'value': value, 'unit': UNIT, 'cores': torch.get_num_threads(), 'kind': 'port',
                         'sample': f'{sample} of {B} samples per step'},
        'e2e': {'value': value, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }


# ------------------------------------------------------------------------------------------
# workloads: whole wavefunctions (BASELINE.json configs[0], [2], [3], [4])
# ------------------------------------------------------------------------------------------
MODEL_WORKLOADS = {
    # name: (walkers per GPU, chunk, sparsity threshold, description)
    'mlp': (20, 20, 4, 'README MLP (configs[0]): 10 x (Dense(100)+SiLU) + Dense(1), x (20,100,4), threshold 4'),
    'ferminet': (4096, 2048, 6, 'FermiNet-style (configs[2]): 16 electrons, 4 nuclei, 4 layers 256/32, 16 dets'),
    'psiformer': (4096, 512, 6, 'PsiFormer-style (configs[3]): 32 electrons, 8 nuclei, 4 layers, 4 heads x 64, 16 dets'),
    'psiformer64': (2048, 128, 6, 'scaled PsiFormer (configs[4]): 64 electrons, 16 nuclei, 16 dets of 32x32; '
                                   '16384 walkers over 8 GPUs = 2048 per GPU'),
}


def build_model(name: str, device, dtype=torch.float32):
    from folx_b200 import wavefunctions as wf

    if name == 'mlp':
        p = wf.tree_to(wf.mlp_params(seed=0), device, dtype)
        return (lambda z: wf.mlp(p, z)), (100, 4), None
    if name == 'ferminet':
        cfg = wf.FermiNetConfig()
        p = wf.tree_to(wf.ferminet_params(cfg), device, dtype)
        return (lambda z: wf.ferminet(cfg, p, z)), (cfg.n_elec, 3), (lambda r: wf.coulomb_potential(r, p['nuclei']))
    cfg = wf.PsiFormerConfig() if name == 'psiformer' else wf.PsiFormerConfig(n_elec=64, n_up=32, n_nuc=16)
    p = wf.tree_to(wf.psiformer_params(cfg), device, dtype)
    return (lambda z: wf.psiformer(cfg, p, z)), (cfg.n_elec, 3), (lambda r: wf.coulomb_potential(r, p['nuclei']))


def time_model(name: str, device, rank: int, world: int, steps: int, warmup: int, walkers: int | None = None):
    """Walker-Laplacians/s of a whole wavefunction: device-resident and end to end."""
    from folx_b200 import harness, kernels

    n_walkers, chunk, thr, desc = MODEL_WORKLOADS[name]
    if walkers is not None:
        n_walkers, chunk = walkers, min(chunk, walkers)
    f, shape, pot = build_model(name, device)
    host_r = torch.randn(n_walkers, *shape, generator=torch.Generator().manual_seed(rank)).pin_memory()
    r = host_r.to(device)

    # each chunk is replayed from a CUDA graph after the first calls (the role jax.jit has for the
    # reference); the all-reduce stays outside the graph
    evaluator = harness.EnergyEvaluator(f, pot, sparsity_threshold=thr, chunk=chunk,
                                        graph=not os.environ.get('FOLX_B200_NO_GRAPH'))

    def step(rr):
        e, sums = evaluator(rr)
        mean, var, n = harness.reduce_energy(sums)  # the one exchange: all-reduce of 3 doubles
        return e, mean

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(device)

    for _ in range(max(warmup, 3)):
        step(r)
    kernels.check_gemm_status(device)
    barrier()
    from folx_b200 import lib as _lib

    launches0 = _lib.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step(r)
    e1.record()
    barrier()
    launches = _lib.launches() - launches0
    ms = e0.elapsed_time(e1) / steps
    # end to end: coordinates come from pinned host memory, energies go back to the host
    host_e = torch.empty(n_walkers).pin_memory()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    g0.record()
    for _ in range(max(2, min(steps, 3))):
        e, mean = step(host_r.to(device, non_blocking=True))
        host_e.copy_(e, non_blocking=True)
        mean_host = float(mean)  # device -> host read of the step's result
    g1.record()
    barrier()
    e2e_ms = g0.elapsed_time(g1) / max(2, min(steps, 3))
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=device, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
    kernels.check_gemm_status(device)
    return {'workload': desc, 'walkers_per_gpu': n_walkers, 'chunk': chunk, 'sparsity_threshold': thr,
            'ms_per_step': ms, 'value': world * n_walkers / (ms / 1e3),
            'e2e_ms_per_step': e2e_ms, 'e2e_value': world * n_walkers / (e2e_ms / 1e3),
            'h2d_bytes_per_step': host_r.numel() * 4, 'd2h_bytes_per_step': n_walkers * 4 + 8,
            'mean_energy': mean_host, 'gpu_launches': launches}


def cpu_model_baseline(name: str, walkers: int = 2):
    """Brute-force Laplacian of the same wavefunction on the host (torch.func, fp32)."""
    from oracle import brute

    use_all_host_threads()
    f, shape, _ = build_model(name, 'cpu')
    r = torch.randn(walkers, *shape, generator=torch.Generator().manual_seed(0))
    brute.jac_and_laplacian(f, r[0])
    t0 = time.perf_counter()
    for w in range(walkers):
        brute.jac_and_laplacian(f, r[w])
    t = time.perf_counter() - t0
    return {'value': walkers / t, 'unit': UNIT, 'cores': torch.get_num_threads(), 'kind': 'port',
            'sample': f'{walkers} walkers, Jacobian + Hessian trace by automatic differentiation '
                      f'(torch.func, fp32) of the same function; host has {os.cpu_count()} logical cores',
            'seconds': t}


def run_kernel_case(args, device):
    """Single-kernel cases at BASELINE shapes, for profiling (`--workload attention|slogdet|gather|pair_product`)."""
    from folx_b200 import kernels

    g = torch.Generator(device=device).manual_seed(0)
    walkers = args.walkers or 128

    def rand(K, shape, scale=1.0):
        a = kernels.alloc_triplet(K, shape, device)
        a.x.normal_(generator=g).mul_(scale)
        a.jacobian.data.normal_(generator=g).mul_(scale)
        a.laplacian.normal_(generator=g).mul_(scale)
        return a

    if args.workload == 'attention':  # PsiFormer layer: n = 32, H = 4, d = 64, R = 96
        q, k, v = (rand(96, (walkers, 32, 4, 64), 0.3) for _ in range(3))
        fn = lambda: kernels.mhsa(q, k, v)
        nbytes = 4 * 4 * walkers * 4 * 98 * 32 * 64
        desc = f'attention-Laplacian kernel, {walkers} walkers x 4 heads, n=32, d=64, R=96'
    elif args.workload == 'pair_product':
        # product of two dense triplets, one 16 x 16 x 16 pair per walker and head (attention-like
        # shapes: 32 matrices per walker), K = 48; FOLX_B200_PAIR_N sets the matrix size
        n = int(os.environ.get('FOLX_B200_PAIR_N', '16'))
        K = 48
        a, b = rand(K, (walkers, 32, n, n)), rand(K, (walkers, 32, n, n))
        fn = lambda: kernels.dot_general_pair(a, b)
        nbytes = 4 * walkers * 32 * (K + 2) * 3 * n * n
        desc = f'two-triplet product kernel, {walkers} walkers x 32 pairs of {n}x{n}x{n}, K={K}'
    elif args.workload == 'gather':
        # the sparse Jacobian of the operator microbench (3 rows per position, row r of sample s
        # belongs to electron s mod 32) scattered into its dense frame of 96 rows, and the sum of
        # the dense result over the feature axis (both run on the table-driven gather kernel)
        import numpy as np
        from folx_b200 import rules as dev_rules
        from folx_b200.api import FwdJacobian, FwdLaplArray
        n = args.walkers or 2048
        idx = (3 * (np.arange(n) % 32)[None, :, None] + np.arange(3)[:, None, None]).astype(np.int32)
        a = rand(3, (n, F))
        a = FwdLaplArray(a.x, FwdJacobian(a.jacobian.data, idx), a.laplacian)
        walkers = n

        def fn():
            d = a.jacobian.dense_array          # (96, n, F): 3 rows read, 96 written
            return dev_rules.reduce_sum(FwdLaplArray(a.x, FwdJacobian(d, None), a.laplacian), (1,))
        nbytes = 4 * n * F * (3 + 96) + 4 * n * F * 98 + 4 * n * 98
        desc = f'gather kernel: densify (3 -> 96 rows) + feature sum of the dense triplet, {n} samples x 256'
    else:
        # determinants of the model configs: 32 matrices per walker of 16 x 16 with K = 96
        # (PsiFormer, the default), 8 x 8 with K = 48 (FermiNet) or 32 x 32 with K = 192 (scaled
        # PsiFormer), chosen by FOLX_B200_SLOGDET_N
        n = int(os.environ.get('FOLX_B200_SLOGDET_N', '16'))
        K = 6 * n
        a = rand(K, (walkers, 32, n, n))
        a.x.div_(n ** 0.5).add_(1.5 * torch.eye(n, device=device))
        fn = lambda: kernels.slogdet(a)
        nbytes = 4 * walkers * 32 * (K + 2) * n * n
        desc = f'slogdet kernel, {walkers} walkers x 32 matrices of {n}x{n}, K={K}'
    for _ in range(max(args.warmup, 3)):
        fn()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    torch.cuda.synchronize(device)
    ms = e0.elapsed_time(e1) / args.steps
    peaks = load_peaks()
    return {'metric': METRIC, 'value': walkers / (ms / 1e3), 'unit': UNIT, 'n_gpus': 1, 'steps': args.steps,
            'warmup': max(args.warmup, 3), 'ms_per_step': ms, 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic', 'config': {'workload': desc},
            'gpu_launches': args.steps,
            'roofline': {'bound': 'hbm', 'achieved': round(nbytes / ms / 1e6, 1), 'peak': peaks['hbm_gbs'],
                         'unit': 'GB/s', 'frac': round(nbytes / ms / 1e6 / peaks['hbm_gbs'], 3), 'traffic': None}}


def run_model(args, rank, world, device):
    name = args.workload
    with ClockSampler(device.index or 0) as clocks:
        m = time_model(name, device, rank, world, args.steps, args.warmup, args.walkers)
    return {
        'metric': METRIC, 'value': m['value'], 'unit': UNIT, 'n_gpus': world, 'steps': args.steps,
        'warmup': max(args.warmup, 3), 'ms_per_step': m['ms_per_step'], 'higher_is_better': True,
        'scaling': 'weak',
        # the only published numbers are the README's MLP example: 2.59 ms per 20 Laplacians with
        # sparsity threshold 4 (README.md:70), hardware not stated
        'vs_baseline': (m['value'] / world / (20 / 2.59e-3)) if name == 'mlp' else None,
        'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': m['workload'], 'walkers_per_gpu': m['walkers_per_gpu'], 'chunk': m['chunk'],
                   'sparsity_threshold': m['sparsity_threshold'],
                   'l2': 'Jacobian tensors are GB-sized (>> 126 MB L2) and streamed by every kernel',
                   'exchange': 'one all-reduce of [sum E, sum E^2, n] (3 x f64) per step'},
        'clocks': clocks.summary(),
        'e2e': {'value': m['e2e_value'], 'unit': UNIT, 'h2d_bytes_per_step': m['h2d_bytes_per_step'],
                'd2h_bytes_per_step': m['d2h_bytes_per_step'], 'ms_per_step': m['e2e_ms_per_step']},
        'gpu_launches': m['gpu_launches'], 'mean_energy': m['mean_energy'],
        'roofline': None,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--workload', default='operators', choices=['operators', 'attention', 'slogdet', 'gather', 'pair_product', *MODEL_WORKLOADS])
    ap.add_argument('--walkers', type=int, default=None, help='walkers per GPU (model workloads)')
    ap.add_argument('--no-models', action='store_true', help='skip the short model timings of the default run')
    ap.add_argument('--samples', type=int, default=None,
                    help='samples per GPU of the operator workload (default 4096; smaller values are for profiling)')
    args = ap.parse_args()
    if args.samples is not None:
        global B
        B = args.samples

    rank = int(os.environ.get('RANK', 0))
    world = int(os.environ.get('WORLD_SIZE', 1))
    local = int(os.environ.get('LOCAL_RANK', 0))

    if args.impl == 'reference':
        res = run_reference(args, rank, world)
        if res is not None:
            print(json.dumps(res), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device (there is no CPU fallback for the product path)')
    device = torch.device('cuda', local)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        torch.distributed.init_process_group('nccl', device_id=device)
    if args.workload == 'operators':
        res = run_ours(args, rank, world, device)
        if not args.no_models:
            # short timings of the whole wavefunctions, reported beside the headline workload
            models = {}
            for name, walkers in (('ferminet', 2048), ('psiformer', 512)):
                try:
                    torch.cuda.empty_cache()
                    models[name] = time_model(name, device, rank, world, steps=3, warmup=3, walkers=walkers)
                except Exception as e:  # a model failing must not lose the headline line
                    models[name] = {'error': f'{type(e).__name__}: {e}'}
            res['models'] = models
        if rank == 0:
            res['cpu_baseline'] = cpu_baseline(sample=1024) if world == 1 else None
    elif args.workload in ('attention', 'slogdet', 'gather', 'pair_product'):
        res = run_kernel_case(args, device)
    else:
        res = run_model(args, rank, world, device)
        if rank == 0:
            res['cpu_baseline'] = cpu_model_baseline(args.workload) if world == 1 else None
    if rank == 0:
        print(json.dumps(res), flush=True)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == '__main__':
    main()
