#!/usr/bin/env python
"""Benchmark of the signature hot path: paths*steps/s for forward+backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg5] [--impl ours|reference]

One "step" is one forward + backward pass of the hot path over one batch of seeded synthetic
Brownian paths.  The default workload (``cfg5``) is the depth-4 signature of (4096, 2048, 16)
float32 paths, the largest configuration of the baseline specification that fits one GPU; under
``torchrun`` the 4096 paths are sharded over the ranks (strong scaling, no collective on the
data path).  Every other workload keeps its batch per rank (weak scaling).

The JSON line printed by rank 0 carries: ``value`` (device-timed, inputs resident in HBM),
``e2e`` (same metric through ``pathsig_b200.Signature`` with pinned-host inputs, H2D and D2H
copies inside the timed region), ``roofline`` (FP32 FMA bound kernels: algorithmic FLOP of the
backward operator over its measured duration, against an FFMA peak measured in the same
process), ``roofline_hbm``, ``cpu_baseline`` (the CPU oracle on a bounded, fixed sample),
``clocks``, ``gather`` (at N > 1: the optional all-gather of the sharded output, timed apart from
the step) and ``others`` (the remaining workloads of the baseline specification: median of
several repeats, each with the reference's CUDA operators, the parity of this library against
them on the same tensors, and the CPU oracle on a fixed sample).

``--impl reference`` times the CPU restatement of the reference algorithm (``oracle/``) on the
host cores instead; the reference itself has no CPU implementation.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
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

METRIC = "paths*steps/s, forward+backward"
UNIT = "paths*steps/s"
HEADLINE = "cfg5"

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch of a workload's dominant
# kernel as captured with ncu on a reduced batch; it grows in proportion to the batch, so the bench
# line scales it by (paths of the timed launch / paths of the capture) and says so.
NCU_TRAFFIC = {
    "cfg5": {"kernel": "sig_backward_tiled (d=16, depth 4)", "captured_paths": 256, "dram_bytes": 158.75e6},
    "cfg2": {"kernel": "sig_backward_tiled (d=8, depth 4)", "captured_paths": 128, "dram_bytes": 180.6e6},
}

# Fixed CPU samples (paths of each workload the CPU oracle runs); work is linear in the batch.
CPU_SAMPLE_PATHS = {"cfg1": 32, "cfg2": 16, "cfg3": 64, "cfg4": 64, "cfg5": 8}


# ----------------------------------------------------------------------------------------------
# workloads (the five configurations of the baseline specification)
# ----------------------------------------------------------------------------------------------

def _brownian(B, L, d, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.cumsum(torch.randn(B, L, d, generator=g, dtype=torch.float64) / math.sqrt(L), dim=1)
    return x.to(torch.float32)


def _normal(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(tuple(shape), generator=g, dtype=torch.float32)


def _random_words(n_words, d, min_len, max_len, seed):
    import random
    rng = random.Random(seed)
    seen = set()
    while len(seen) < n_words:
        n = rng.randint(min_len, max_len)
        seen.add(tuple(rng.randrange(d) for _ in range(n)))
    return sorted(seen, key=lambda w: (len(w), w))


def _dense_fma(d, depth):
    return sum((depth - j + 1) * d ** j for j in range(1, depth + 1))


def _closure_fma(words_by_level, d, depth, dense_levels=()):
    """FMAs per path*step of the shared-prefix Horner scheme for a projected state set:
    sum over target degrees k of the number of distinct non-empty prefixes of the degree-k
    state words (requested words and the prefixes of longer requested words)."""
    requested = set()
    for ws in words_by_level.values():
        requested.update(ws)
    total = 0
    for k in range(1, depth + 1):
        if k in dense_levels:
            total += sum(d ** j for j in range(1, k + 1))
            continue
        state_k = {w[:k] for w in requested if len(w) >= k}
        prefixes = set()
        for w in state_k:
            for j in range(1, k + 1):
                prefixes.add(w[:j])
        total += len(prefixes)
    return total


SPECS = {
    "cfg1": dict(kind="sig", B=32, L=128, d=8, depth=4, desc="Signature depth 4, (32,128,8)"),
    "cfg2": dict(kind="sig", B=256, L=1024, d=8, depth=4, windows=(64, 16, 61),
                 desc="Signature depth 4, (256,1024,8), 61 windows [16k,16k+64)"),
    "cfg3": dict(kind="words", B=512, L=512, d=8, depth=6, n_words=200,
                 desc="Signature depth 6, (512,512,8), level 1 + 200 seeded words"),
    "cfg4": dict(kind="loglyndon", B=1024, L=256, d=4, depth=6,
                 desc="LogSignature depth 6, (1024,256,4), Lyndon projection"),
    "cfg5": dict(kind="sig", B=4096, L=2048, d=16, depth=4, desc="Signature depth 4, (4096,2048,16), batch-sharded"),
}


class Workload:
    """One configuration: inputs, module, step functions and work accounting."""

    def __init__(self, name, B=None, seed=0):
        self.name = name
        s = dict(SPECS[name])
        if B is not None:
            s["B"] = B
        self.spec = s
        self.B, self.L, self.d, self.depth = s["B"], s["L"], s["d"], s["depth"]
        self.seed = seed
        self.windows = None
        if "windows" in s:
            length, stride, count = s["windows"]
            self.windows = torch.tensor([[stride * k, stride * k + length] for k in range(count)], dtype=torch.int32)
            self.steps_per_path = count * (length - 1)
        else:
            self.steps_per_path = self.L - 1
        self.units = self.B * self.steps_per_path
        self.words = None
        if s["kind"] == "words":
            self.words = [(a,) for a in range(self.d)] + _random_words(s["n_words"], self.d, 2, self.depth, seed=1234)
            by_level = {}
            for w in self.words:
                by_level.setdefault(len(w), []).append(w)
            self.fma_fwd = _closure_fma(by_level, self.d, self.depth)
        elif s["kind"] == "loglyndon":
            from pathsig_b200.projections import lyndon_words
            top = lyndon_words(self.d, self.depth)
            letters = []
            for c in top:
                w = []
                for _ in range(self.depth):
                    w.append(c % self.d)
                    c //= self.d
                letters.append(tuple(reversed(w)))
            self.fma_fwd = _closure_fma({self.depth: letters}, self.d, self.depth,
                                        dense_levels=tuple(range(1, self.depth)))
        else:
            self.fma_fwd = _dense_fma(self.d, self.depth)

    # ---- host data ----
    def host_path(self):
        return _brownian(self.B, self.L, self.d, self.seed)

    def out_width(self, mod):
        if self.spec["kind"] == "sig":
            return sum(self.d ** k for k in range(1, self.depth + 1))
        return mod.projection.sig_size

    def degree_widths(self):
        """Columns per degree of the module's output (for the per-degree parity metric)."""
        if self.spec["kind"] == "sig":
            return [self.d ** k for k in range(1, self.depth + 1)]
        return [int(s) for s in self.mod.projection.level_sizes[1: self.depth + 1]]

    def flop_fwd_bwd(self):
        return 8.0 * self.fma_fwd * self.units  # forward F FMAs, backward credited 3F

    def flop_bwd(self):
        return 6.0 * self.fma_fwd * self.units

    def flop_fwd(self):
        return 2.0 * self.fma_fwd * self.units

    # ---- device objects ----
    def build(self, device):
        import pathsig_b200 as ps
        kind = self.spec["kind"]
        win = None if self.windows is None else self.windows.to(device)
        if kind == "sig":
            mod = ps.Signature(depth=self.depth, windows=win)
        elif kind == "words":
            proj = ps.projections.words([w for w in self.words if len(w) > 1], self.depth, self.d, full_levels=(1,),
                                        device=device)
            mod = ps.Signature(depth=self.depth, projection=proj)
        else:
            proj = ps.projections.lyndon(self.depth, self.d, device=device)
            mod = ps.LogSignature(depth=self.depth, projection=proj)
        self.mod = mod.to(device)
        self.x = self.host_path().to(device)
        W = () if self.windows is None else (self.windows.shape[0],)
        self.G = _normal((self.B,) + W + (self.out_width(mod),), self.seed + 1).to(device)
        self.bytes_fwd = self.x.numel() * 4 + self.G.numel() * 4
        self.bytes_fwd_bwd = 2 * self.x.numel() * 4 + 2 * self.G.numel() * 4
        return self

    def step_forward(self):
        with torch.no_grad():
            return self.mod(self.x)

    def step_fwd_bwd(self, events=None):
        """Forward + backward with dL/dout = G (the loss is sum(out * G)).  For the dense signature
        modules the two operators are called directly; projected and log-signature modules go through
        the module and autograd (their forward is more than one operator).  Returns (output, grad wrt
        the path)."""
        import pathsig_b200 as ps
        m = self.mod
        if isinstance(m, ps.Signature) and not m.alternative_projection:
            sig = ps.ops.compute_signature(self.x, m.depth, m.alternative_projection, m._encoded_words,
                                           m._level_sizes, m.use_windows, m._windows)
            if events is not None:
                events[0].record()
            gp = ps.ops.signature_backward(self.x, sig, self.G, m.depth, m.alternative_projection,
                                           m._encoded_words, m._level_sizes, m.use_windows, m._windows)
            if events is not None:
                events[1].record()
            return sig, gp
        x = self.x.detach().requires_grad_(True)
        out = m(x)
        if events is not None:
            events[0].record()
        out.backward(self.G)
        if events is not None:
            events[1].record()
        return out.detach(), x.grad

    def step_through(self):
        """How step_fwd_bwd reaches the kernels (kernels_per_step counts this library's launches only)."""
        import pathsig_b200 as ps
        m = self.mod
        if isinstance(m, ps.Signature) and not m.alternative_projection:
            return "the two operators called directly"
        if isinstance(m, ps.Signature):
            closed = m._closure_pays(self.x)
            return ("module + autograd" + ("; evaluated on the prefix closure of the word set, the requested columns "
                    "selected by one torch gather forward and a zero-fill + scatter backward (3 torch kernels, "
                    "not in kernels_per_step)" if closed else ""))
        return "module + autograd"

    def kernels_per_step(self):
        """Kernels of this library launched by one forward + backward step (counted, not assumed)."""
        from pathsig_b200 import _load
        lib = _load.ensure_loaded()
        torch.cuda.synchronize()
        before = lib.psig_kernel_launches()
        self.step_fwd_bwd()
        torch.cuda.synchronize()
        return int(lib.psig_kernel_launches() - before)


# ----------------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------------

class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows = []
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9:
                self.rows.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                smax.append(float(r[2]))
                power.append(float(r[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        busy = [c for c, p in zip(sm, power) if p >= 0.5 * max(power)] if power else sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------------------------
# measurement helpers
# ----------------------------------------------------------------------------------------------

def _dist_setup(n_gpus):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        # plain NCCL rings/trees over NVLink: the optional gather is the only collective, and it need
        # not bind this process's memory to an NVLink multicast object
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    return world, rank, local


def _barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def _max_over_ranks(value, world, device):
    if world == 1:
        return value
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_steps(fn, steps, warmup, world, device):
    """Device time (ms, max over ranks) of exactly `steps` calls of fn after `warmup` calls."""
    for _ in range(warmup):
        fn()
    _barrier(world)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    _barrier(world)
    return _max_over_ranks(start.elapsed_time(end), world, device)


def time_repeats(fn, steps, warmup, repeats, world, device):
    """ms per step of `repeats` timed loops of `steps` calls each: (median, min, max)."""
    per_step = []
    for r in range(repeats):
        per_step.append(time_steps(fn, steps, warmup if r == 0 else 1, world, device) / steps)
    return statistics.median(per_step), min(per_step), max(per_step)


def _probe_lib():
    """The measurement-only probe library built from bench_probe.cu (FP32 FMA peak loops)."""
    lib = ctypes.CDLL(os.path.join(ROOT, "libbench_probe.so"))
    for name in ("psig_probe_fp32_fma", "psig_probe_fp32_fma_packed"):
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int64
        fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    return lib


def measure_fp32_peak(device, packed=False):
    """TFLOP/s of a register-only FFMA loop (psig_probe_fp32_fma[_packed]), best of 5."""
    lib = _probe_lib()
    probe = lib.psig_probe_fp32_fma_packed if packed else lib.psig_probe_fp32_fma
    scratch = torch.zeros(16, device=device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    best = 0.0
    for it in range(6):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fmas = probe(sms * 8, 20000, ctypes.c_void_p(scratch.data_ptr()), stream)
        e.record()
        torch.cuda.synchronize()
        if it > 0:
            best = max(best, 2.0 * fmas / (s.elapsed_time(e) * 1e-3) / 1e12)
    return best


def cpu_baseline(name, threads=None):
    """The CPU oracle (a port of the reference algorithm) on a fixed sample of the workload:
    one forward + backward of CPU_SAMPLE_PATHS[name] paths.  Returns (record, seconds)."""
    from oracle import oracle
    cores = threads or os.cpu_count() or 1
    oracle.set_threads(cores)
    spec = SPECS[name]
    B = min(spec["B"], CPU_SAMPLE_PATHS[name])
    wl = Workload(name, B=B)
    x = wl.host_path()
    win = wl.windows
    kind = spec["kind"]
    t0 = time.perf_counter()
    if kind == "loglyndon":
        from pathsig_b200.projections import projections
        proj = projections.lyndon(wl.depth, wl.d, device="cpu")
        top = proj.encoded_words[sum(proj.level_sizes[k] for k in range(1, wl.depth)
                                     if proj.level_sizes[k] != wl.d ** k):]
        ext = [0] + [wl.d ** k for k in range(1, wl.depth)] + [proj.level_sizes[wl.depth]]
        idx = proj.logsig_indices()
        g = _normal((B, proj.sig_size), 1)
        oracle.logsignature(x, wl.depth, top_words=top, ext_level_sizes=ext, indices=idx, grad_out=g)
    else:
        ew = ls = None
        if kind == "words":
            from pathsig_b200.projections import projections
            proj = projections.words([w for w in wl.words if len(w) > 1], wl.depth, wl.d, full_levels=(1,), device="cpu")
            ew, ls = proj.encoded_words, proj.level_sizes
        sig = oracle.sig_forward(x, wl.depth, ew, ls, win)
        g = _normal(sig.shape, 1)
        oracle.sig_backward(x, sig, g, wl.depth, ew, ls, win)
    dt = time.perf_counter() - t0
    return {"value": wl.units / dt, "unit": UNIT, "cores": cores, "kind": "port", "sample_paths": B,
            "sample": f"{name} with B={B} of {spec['B']} paths (fixed sample), float32, one forward+backward, "
                      f"{dt:.2f} s wall (work is linear in B); port of the reference per-word algorithm, "
                      f"OpenMP over paths"}, dt


def _parity(ours_out, ours_grad, ref_out, ref_grad, widths):
    """Both parity metrics of this library against the reference's CUDA operators on the same tensors:
    whole tensor max|a-b| / max(1, max|b|) and per degree max|a-b| / max|b| for the output; for the
    input gradient max|a-b| / max|b| over the whole (B, L, d) tensor."""
    def maxabs(t):
        return float(t.abs().max().item()) if t.numel() else 0.0

    whole = maxabs(ours_out - ref_out) / max(1.0, maxabs(ref_out))
    per, off = [], 0
    for w in widths:
        if w:
            den = maxabs(ref_out[..., off: off + w]) or 1.0
            per.append(maxabs(ours_out[..., off: off + w] - ref_out[..., off: off + w]) / den)
        off += w
    return {"output_whole": whole, "output_per_degree": per,
            "input_gradient": maxabs(ours_grad - ref_grad) / (maxabs(ref_grad) or 1.0),
            "against": "the reference's CUDA operators, same tensors, float32"}


def reference_cuda_baseline(wl, device, steps=5, warmup=2):
    """The reference's own CUDA operators (built unchanged into oracle/_ref/ by oracle/build_ref.py)
    on the same tensors, as a reported baseline, plus the parity of this library against their
    results (outside every timed region).  Returns None when that library is not there."""
    lib = os.path.join(ROOT, "oracle", "_ref", "libpathsig_ops.so")
    if not os.path.isfile(lib):
        return None
    try:
        torch.ops.load_library(lib)
        ref = torch.ops.pathsig
        m = wl.mod
        if wl.spec["kind"] == "loglyndon":
            # the reference's LogSignature: signature in the hybrid layout -> logarithm -> column selection
            d, ls, tw, idx = wl.d, list(m._ext_level_sizes), m._top_words, m._indices_from_sig
            sargs = (m.depth, m.alternative_projection, tw, ls, m.use_windows, m._windows)
            largs = (m.depth, m.alternative_projection, tw, ls)

            def fwd():
                sig = ref.compute_signature(wl.x, *sargs)
                logsig, cache = ref.sig_to_logsig(sig, m.depth, d, m.alternative_projection, tw, ls)
                return sig, logsig, cache, logsig.index_select(-1, idx)

            def fwd_bwd():
                sig, logsig, cache, out = fwd()
                g_full = torch.zeros_like(logsig).index_add_(-1, idx, wl.G)
                g_sig = ref.logsig_backward(sig, cache, g_full, *largs)
                return out, ref.signature_backward(wl.x, sig, g_sig, *sargs)
        else:
            args = (m.depth, m.alternative_projection, m._encoded_words, list(m._level_sizes), m.use_windows, m._windows)

            def fwd():
                return ref.compute_signature(wl.x, *args)

            def fwd_bwd():
                sig = ref.compute_signature(wl.x, *args)
                return sig, ref.signature_backward(wl.x, sig, wl.G, *args)

        ms_f = time_steps(fwd, steps, warmup, 1, device)
        ms_fb = time_steps(fwd_bwd, steps, warmup, 1, device)
        ref_out, ref_grad = fwd_bwd()
        our_out, our_grad = wl.step_fwd_bwd()
        torch.cuda.synchronize()
        parity = _parity(our_out, our_grad, ref_out, ref_grad, wl.degree_widths())
        del ref_out, ref_grad, our_out, our_grad
        return {"fwd": {"value": wl.units * steps / (ms_f * 1e-3), "ms_per_step": ms_f / steps},
                "fwd_bwd": {"value": wl.units * steps / (ms_fb * 1e-3), "ms_per_step": ms_fb / steps},
                "unit": UNIT, "steps": steps, "parity": parity,
                "what": "reference CUDA operators compiled for sm_100 from its unchanged sources, same tensors, "
                        "device-timed; a reported baseline, not part of the product"}
    except Exception as exc:  # the baseline must never break the benchmark
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}


# ----------------------------------------------------------------------------------------------
# arms
# ----------------------------------------------------------------------------------------------

def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name = args.workload
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_baseline(name)
    t0 = time.perf_counter()
    last = None
    for _ in range(args.steps):
        last, _dt = cpu_baseline(name)
    total = time.perf_counter() - t0
    spec = SPECS[name]
    B = last["sample_paths"]
    units = Workload(name, B=B).units
    value = units * args.steps / total
    last["value"] = value
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "strong" if name == HEADLINE else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{name}: {spec['desc']}; fixed CPU sample of B={B} paths per step "
                               f"(throughput is linear in B)", "timing": "host wall clock"},
        "cpu_baseline": last,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the reference has no CPU implementation (CUDA-only operators); this arm times the CPU "
                "restatement of its algorithm (oracle/) on the host cores",
    }
    emit(line)


def _steps_for(fn, target_s, lo, hi):
    """Number of calls of fn that take about target_s seconds (one synchronised probe of 3 calls)."""
    fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    per = max((time.perf_counter() - t0) / 3, 1e-6)
    return int(max(lo, min(hi, target_s / per)))


def measure_workload(name, steps, warmup, world, device, per_rank_B=None, with_e2e=False, fp32_peak=None,
                     repeats=1, auto_steps=False):
    wl = Workload(name, B=per_rank_B, seed=int(os.environ.get("RANK", "0"))).build(device)
    res = {"workload": name}
    if auto_steps:
        # sub-millisecond workloads: each of the `repeats` timed loops runs for about 0.2 s
        steps = _steps_for(lambda: wl.step_fwd_bwd(), 0.2, steps, 20000)
        if world > 1:
            steps = int(_max_over_ranks(float(steps), world, device))
    # forward only
    f_med, f_min, f_max = time_repeats(wl.step_forward, steps, warmup, repeats, world, device)
    # forward + backward, with the backward operator bracketed by events in the first loop
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    it = iter(pairs)

    def step():
        wl.step_fwd_bwd(next(it, None))

    per_step = []
    for r in range(repeats):
        per_step.append(time_steps(step if r == 0 else wl.step_fwd_bwd, steps, warmup if r == 0 else 1, world,
                                   device) / steps)
    fb_med, fb_min, fb_max = statistics.median(per_step), min(per_step), max(per_step)
    bwd_ms = statistics.mean(a.elapsed_time(b) for a, b in pairs)
    total_units = wl.units * world
    res.update({
        "units_per_step": total_units,
        "fma_per_unit_fwd": wl.fma_fwd,
        "steps": steps, "repeats": repeats,
        "fwd": {"value": total_units / (f_med * 1e-3), "ms_per_step": f_med, "ms_min": f_min, "ms_max": f_max},
        "fwd_bwd": {"value": total_units / (fb_med * 1e-3), "ms_per_step": fb_med, "ms_min": fb_min, "ms_max": fb_max,
                    "timed_s": sum(per_step) * steps * 1e-3},
        "bwd_op_ms": bwd_ms,
        "tflops_fwd": wl.flop_fwd() * world / (f_med * 1e-3) / 1e12,
        "tflops_fwd_bwd": wl.flop_fwd_bwd() * world / (fb_med * 1e-3) / 1e12,
        "hbm_gbs_fwd_bwd": wl.bytes_fwd_bwd * world / (fb_med * 1e-3) / 1e9,
        "kernels_per_step": wl.kernels_per_step(),
        "step_through": wl.step_through(),
    })
    if wl.units < 200000:
        # launch-bound workload: the same forward+backward step captured in a CUDA graph and
        # replayed (the operators enqueue on the current stream only, so capture is legal)
        try:
            side = torch.cuda.Stream(device=device)
            side.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side):
                for _ in range(3):
                    wl.step_fwd_bwd()
            torch.cuda.current_stream(device).wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                wl.step_fwd_bwd()
            g_med, g_min, g_max = time_repeats(graph.replay, steps, warmup, repeats, world, device)
            res["fwd_bwd_cuda_graph"] = {"value": total_units / (g_med * 1e-3), "ms_per_step": g_med,
                                         "ms_min": g_min, "ms_max": g_max}
            del graph
        except Exception as exc:  # reported, never fatal
            res["fwd_bwd_cuda_graph"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:160]}
    if fp32_peak:
        res["frac_fp32_peak_fwd_bwd"] = res["tflops_fwd_bwd"] / (fp32_peak * world)
        res["frac_fp32_peak_fwd"] = res["tflops_fwd"] / (fp32_peak * world)
    res["_wl"] = wl
    if with_e2e:
        xh = wl.host_path().pin_memory()
        gh = torch.empty_like(xh).pin_memory()
        lh = torch.empty(1, dtype=torch.float32).pin_memory()

        # Input pipeline as a training loop would run it: a copy stream moves batch k+1 to the
        # device and the results of batch k-1 back to pinned host memory while batch k computes.
        copy_stream = torch.cuda.Stream(device=device)
        xd = [torch.empty_like(wl.x), torch.empty_like(wl.x)]
        gd = [torch.empty_like(wl.x), torch.empty_like(wl.x)]
        ld = [torch.empty(1, device=device), torch.empty(1, device=device)]
        ev_in = [torch.cuda.Event(), torch.cuda.Event()]
        ev_out = [torch.cuda.Event(), torch.cuda.Event()]
        ev_free = [torch.cuda.Event(), torch.cuda.Event()]
        state = {"k": 0}

        def stage_in(k):
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(ev_free[k % 2])  # the batch that used this buffer has finished
                xd[k % 2].copy_(xh, non_blocking=True)
                ev_in[k % 2].record(copy_stream)

        def e2e_step():
            k = state["k"]
            cur = torch.cuda.current_stream(device)
            if k == 0:
                for e in ev_free:
                    e.record(cur)
                stage_in(0)
            stage_in(k + 1)                      # next batch's H2D overlaps this batch's compute
            cur.wait_event(ev_in[k % 2])
            x = xd[k % 2].detach().requires_grad_(True)
            out = wl.mod(x)
            loss = torch.dot(out.reshape(-1), wl.G.reshape(-1))
            loss.backward()
            gd[k % 2].copy_(x.grad)
            ld[k % 2].copy_(loss.detach().reshape(1))
            ev_out[k % 2].record(cur)
            ev_free[k % 2].record(cur)
            with torch.cuda.stream(copy_stream):  # results of this batch go home on the copy stream
                copy_stream.wait_event(ev_out[k % 2])
                gh.copy_(gd[k % 2], non_blocking=True)
                lh.copy_(ld[k % 2], non_blocking=True)
            state["k"] = k + 1

        def e2e_timed(n):
            for _ in range(n):
                e2e_step()
            torch.cuda.current_stream(device).wait_stream(copy_stream)  # the last D2H is inside the timed region

        for _ in range(warmup):
            e2e_step()
        torch.cuda.current_stream(device).wait_stream(copy_stream)
        _barrier(world)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        e2e_timed(steps)
        end.record()
        _barrier(world)
        ms_e = _max_over_ranks(start.elapsed_time(end), world, device)
        res["e2e"] = {"value": total_units * steps / (ms_e * 1e-3), "unit": UNIT,
                      "h2d_bytes_per_step": xh.numel() * 4 * world, "d2h_bytes_per_step": (gh.numel() + 1) * 4 * world,
                      "ms_per_step": ms_e / steps,
                      "api": "pathsig_b200.Signature(...)(x); torch.dot(out.flatten(), G.flatten()).backward(); every step copies its batch "
                             "from pinned host memory and its grad and loss back, on a copy stream overlapped with "
                             "the neighbouring steps' compute (one extra batch is staged ahead)"}
        del xd, gd, xh, gh
    return res


def measure_gather(wl, world, device, steps=5, warmup=2):
    """The optional gathered output: all ranks' (B/N, D) signatures concatenated on every rank by one
    NCCL all-gather (pathsig_b200.distributed.gather_batch).  Timed on the device apart from the step,
    max over ranks.  Bytes per rank = what a rank receives from its peers."""
    from pathsig_b200.distributed import gather_batch
    out, _ = wl.step_fwd_bwd()
    sizes = [out.shape[0]] * world

    def fn():
        return gather_batch(out, sizes=sizes)

    ms = time_steps(fn, steps, warmup, world, device) / steps
    full = fn()
    ok = bool(full.shape[0] == out.shape[0] * world)
    received = out.numel() * out.element_size() * (world - 1)
    del full
    return {"ms": ms, "bytes_received_per_rank": received, "gbs_per_rank": received / (ms * 1e-3) / 1e9,
            "gathered_shape_ok": ok, "collective": "NCCL all_gather_into_tensor over NVLink (NVLS off), device-timed, "
                                                   "max over ranks; not part of the step"}


def run_ours(args):
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    world, rank, local = _dist_setup(args.gpus)
    device = torch.device("cuda", local if world > 1 else 0)
    import pathsig_b200  # noqa: F401

    if args.profile:
        wl = Workload(args.workload, B=args.batch).build(device)
        for _ in range(args.warmup + args.steps):
            wl.step_fwd_bwd()
        torch.cuda.synchronize()
        emit({"profile_run": args.workload, "batch": wl.B, "passes": args.warmup + args.steps})
        return
    fp32_peak_scalar = measure_fp32_peak(device)
    fp32_peak_packed = measure_fp32_peak(device, packed=True)
    fp32_peak = max(fp32_peak_scalar, fp32_peak_packed)  # the roof is the better of the two issue forms
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except OSError:
        pass
    hbm_peak, hbm_src = (peaks.get("hbm_gbs"), "measured") if peaks.get("hbm_gbs") else (6650.0, "fallback")

    name = args.workload
    strong = name == HEADLINE  # the headline's batch is sharded over the ranks; the others keep theirs per rank
    per_rank_B = args.batch
    if strong and per_rank_B is None:
        per_rank_B = SPECS[name]["B"] // world
    sampler = ClockSampler(local if world > 1 else 0)
    if rank == 0:
        sampler.start()
    t_begin = time.perf_counter()
    short = Workload(name, B=per_rank_B).units < 2_000_000
    main = measure_workload(name, args.steps, args.warmup, world, device, per_rank_B=per_rank_B, with_e2e=True,
                            fp32_peak=fp32_peak, repeats=5 if short else 1)
    wl = main["_wl"]
    # a short workload keeps running until the 100 ms clock sampler has seen it under load
    while time.perf_counter() - t_begin < 2.0:
        for _ in range(20):
            wl.step_fwd_bwd()
        torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["sampled_over"] = "the timed regions of the headline workload"

    gather = None
    if world > 1 and SPECS[name]["kind"] == "sig" and "windows" not in SPECS[name]:
        gather = measure_gather(wl, world, device)

    cpu = None
    ref_cuda = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu, _ = cpu_baseline(name)
        few = wl.units > 2_000_000  # the reference runs for seconds on the large workloads
        ref_cuda = reference_cuda_baseline(wl, device, steps=1 if few else 5, warmup=1 if few else 2)
    main.pop("_wl")
    kernels_per_step = main["kernels_per_step"]
    bwd_flop = wl.flop_bwd()
    bytes_fwd_bwd = wl.bytes_fwd_bwd
    paths_per_launch = wl.B
    del wl
    torch.cuda.empty_cache()

    others = {}
    if not args.no_others:
        for other in SPECS:
            if other == name:
                continue
            big = Workload(other).units > 2_000_000
            B = SPECS[other]["B"] // world if other == HEADLINE else None
            r = measure_workload(other, 5 if big else 20, 3, world, device, per_rank_B=B, fp32_peak=fp32_peak,
                                 repeats=1 if big else 5, auto_steps=not big)
            other_wl = r.pop("_wl")
            if rank == 0 and world == 1 and not args.no_cpu:
                r["reference_cuda"] = reference_cuda_baseline(other_wl, device, steps=1 if big else 5,
                                                              warmup=1 if big else 2)
                r["cpu_baseline"] = cpu_baseline(other)[0]
            del other_wl
            r["scaling"] = "strong" if other == HEADLINE else "weak"
            others[other] = r
            torch.cuda.empty_cache()

    if rank != 0:
        return
    spec = SPECS[name]
    steps = args.steps
    achieved = bwd_flop / (main["bwd_op_ms"] * 1e-3) / 1e12
    traffic = None
    traffic_note = "no ncu capture of this workload's dominant kernel"
    cap = NCU_TRAFFIC.get(name)
    if cap and cap["dram_bytes"]:
        scale = paths_per_launch / cap["captured_paths"]
        traffic = cap["dram_bytes"] * scale
        traffic_note = (f"ncu capture of {cap['kernel']} at {cap['captured_paths']} paths: {cap['dram_bytes']:.4g} B "
                        f"of dram read+write per launch, scaled x{scale:g} to the {paths_per_launch} paths of a timed "
                        f"launch (traffic grows in proportion to the batch)")
    line = {
        "metric": METRIC, "value": main["fwd_bwd"]["value"], "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": args.warmup, "ms_per_step": main["fwd_bwd"]["ms_per_step"], "higher_is_better": True,
        "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{name}: {spec['desc']}", "per_gpu_batch": paths_per_launch,
                   "global_batch": paths_per_launch * world,
                   "units_per_step": main["units_per_step"], "l2": "inputs_larger_than_l2"
                   if bytes_fwd_bwd > 126e6 else "inputs smaller than L2 (latency-bound configuration)",
                   "parallelism": f"batch shards x{world}, no collective"},
        "forward_only": main["fwd"],
        "timed": {"repeats": main["repeats"], "ms_min": main["fwd_bwd"]["ms_min"], "ms_max": main["fwd_bwd"]["ms_max"],
                  "timed_s": main["fwd_bwd"]["timed_s"]},
        "clocks": clocks,
        "e2e": main["e2e"],
        "gpu_launches": steps * kernels_per_step,
        "roofline": {
            "bound": "fp32_fma", "kernel": "signature_backward operator (sig_backward_tiled, preceded by the "
                                           "cudaMemsetAsync of grad_path where blocks share points)",
            "achieved": achieved, "peak": fp32_peak, "unit": "TFLOP/s", "frac": achieved / fp32_peak,
            "peak_source": "register-only FMA loops (psig_probe_fp32_fma / _packed) measured in this process, best of "
                           "the two; MEASURED_PEAKS.json has no FP32 figure",
            "peak_scalar_fma": fp32_peak_scalar, "peak_packed_fma": fp32_peak_packed,
            "flop_per_launch": bwd_flop, "flop_convention": "backward credited 3 x F_fwd FMAs per path*step",
            "traffic": traffic, "traffic_source": traffic_note,
            "whole_step": {"achieved": main["tflops_fwd_bwd"], "frac": main["tflops_fwd_bwd"] / (fp32_peak * world)},
        },
        "roofline_hbm": {"bound": "hbm", "achieved": main["hbm_gbs_fwd_bwd"], "peak": hbm_peak * world if hbm_peak else None,
                         "unit": "GB/s", "frac": main["hbm_gbs_fwd_bwd"] / (hbm_peak * world) if hbm_peak else None,
                         "peak_source": hbm_src, "bytes": "read path + write signature + read grad + write grad_path"},
        "cpu_baseline": cpu,
        "reference_cuda": ref_cuda,
        "gather": gather,
        "others": others,
    }
    emit(line)


_real_stdout = None


def _claim_stdout():
    """Keep stdout for the JSON line only: anything a library prints there (NCCL's version banner,
    for one) goes to stderr instead; emit() writes to the real stdout."""
    global _real_stdout
    if _real_stdout is None:
        _real_stdout = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(obj):
    print(json.dumps(obj), file=_real_stdout or sys.stdout, flush=True)


def main():
    _claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=HEADLINE, choices=sorted(SPECS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-others", action="store_true", help="skip the short runs of the other workloads")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU and reference-CUDA baseline legs")
    ap.add_argument("--batch", type=int, default=None, help="override the per-GPU batch of the workload")
    ap.add_argument("--profile", action="store_true",
                    help="only run warmup+steps forward+backward passes of the workload (for ncu captures)")
    args = ap.parse_args()
    if args.impl == "ours" and not args.profile:
        args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)
        if int(os.environ.get("WORLD_SIZE", "1")) > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
