#!/usr/bin/env python
"""Benchmark of the contraction hot path.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun)
    python bench.py --impl reference ...                     (the CPU path on the host cores)

Default workload `dense`: 'ijkl,klmn->ijmn', f32 through 3xTF32 on the tcgen05 tensor cores,
i=j=m=n=128, k=l=256, N(0,1) entries: M = N = 16384, K = 65536, 2^45 flop and 9 GiB per step.
One step = one such contraction.  On N > 1 GPUs the ranks split that ONE contraction (strong
scaling): `value` is the free-index split (`--shard i`: every rank contracts its slice of A
into its slice of C, B replicated, no communication); the contracted-index split (`--shard k`:
the pair (k,l) split on l, every rank a full-size partial C, then NCCL reduce-scatter) runs in
the same process right after and is nested in the line as `config.shard_k`.  After the timed
regions every rank checks sampled rows of what it owns against a float64 sum on the host.

Other workloads (`--workload`): `chain` (MPS transfer-matrix chain, complex128, 32 sites,
chi = 512: N independent replicas), `grouped` (4096 ragged f32 products, table sharded over the
ranks), `network4` ('ijk,jlm,kmn,lnp->ip', complex64, dim 96), `abc_bcd` ('abc,bcd->ad', f64,
dim 64), `permute` and `reduce` (bandwidth).

The metric is einsum GFLOP/s (algorithmic: 2 flop per real and 8 per complex multiply-add) or
GB/s for the bandwidth workloads.  `value` is measured with inputs resident in HBM; `e2e`
through the public API from pinned host buffers with the host<->device copies inside the timed
region.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

os.environ.setdefault("OPENBLAS_NUM_THREADS", str(os.cpu_count() or 1))
os.environ.setdefault("OMP_NUM_THREADS", str(os.cpu_count() or 1))

import numpy as np  # noqa: E402

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "tenferro-rs_b200"))
sys.path.insert(0, str(ROOT))

CHAIN = "ab,asc,bsd->cd"
CHAIN_METRIC = "einsum GFLOP/s (MPS transfer-matrix chain, complex128)"
DENSE = "ijkl,klmn->ijmn"
DENSE_METRIC = "einsum GFLOP/s ('ijkl,klmn->ijmn', f32 via 3xTF32)"
CHECK_TOL = 1e-5  # relative Frobenius bound of the sampled-row check (f32 contraction)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="dense",
                    choices=["dense", "chain", "grouped", "network4", "abc_bcd", "permute", "reduce"])
    ap.add_argument("--sites", type=int, default=32)
    ap.add_argument("--chi", type=int, default=512)
    ap.add_argument("--phys", type=int, default=2)
    ap.add_argument("--shard", default="both", choices=["both", "i", "k"],
                    help="dense, N > 1: `both` times the free-index split (the line's value) and then the "
                         "contracted-index split (nested as config.shard_k); i or k times that one alone")
    ap.add_argument("--scale", type=float, default=1.0, help="dense/network4/permute: scale the index extents")
    ap.add_argument("--problems", type=int, default=4096, help="grouped: number of problems")
    ap.add_argument("--case", default="transpose2d", help="permute/reduce: which member of the set")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--sustained-seconds", type=float, default=4.0,
                    help="dense/network4: length of the back-to-back TF32 probe (0: skip it)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="target length of the CPU-baseline sample")
    return ap.parse_args()


def load_peaks():
    try:
        return json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except (OSError, ValueError):
        return None


def chain_flops(chi: int, d: int, sites: int) -> float:
    # per site two contractions of chi * chi * (d chi) complex multiply-adds, 8 flop each
    return sites * 2 * 8.0 * chi * chi * (d * chi)


def seeded_normal(seed: int, shape, dtype, scale: float = 1.0) -> np.ndarray:
    """Column-major N(0, scale^2) tensor (real and imaginary parts alike), seed -> default_rng."""
    rng = np.random.default_rng(seed)
    dtype = np.dtype(dtype)
    if dtype.kind == "c":
        real = np.float32 if dtype == np.complex64 else np.float64
        out = np.empty(shape, dtype=dtype, order="F")
        out.real = rng.standard_normal(shape).astype(real) * scale
        out.imag = rng.standard_normal(shape).astype(real) * scale
        return out
    return np.asfortranarray((rng.standard_normal(shape) * scale).astype(dtype))


def grouped_table(seed: int, n_problems: int) -> np.ndarray:
    """(n, 3) table of (i, j, k) drawn uniformly from {16, 32, 64, 128}."""
    return np.random.default_rng(seed).choice(np.array([16, 32, 64, 128]), size=(n_problems, 3))


def site_tensor(seed: int, chi: int, d: int) -> np.ndarray:
    return seeded_normal(seed, (chi, d, chi), np.complex128, scale=(1.0 / chi) ** 0.5)


def dense_extents(scale: float):
    e = lambda x: max(4, int(round(x * scale / 4)) * 4)
    return e(128), e(256)  # i = j = m = n, k = l


def dense_workload_name(ext: int, kext: int) -> str:
    return f"'{DENSE}' f32, i=j=m=n={ext}, k=l={kext}, N(0,1)"


def chain_workload_name(sites: int, chi: int, d: int) -> str:
    return (f"MPS transfer-matrix chain: {sites} sites, chi={chi}, d={d}, complex128, '{CHAIN}' per site via the "
            f"contraction tree")


# ------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi every 100 ms while the timed regions run (a read-only query)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
            # the first sample takes a moment to arrive: do not start a timed region before it
            t0 = time.time()
            while not self.lines and time.time() - t0 < 3.0:
                time.sleep(0.02)
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self) -> int:
        return len(self.lines)

    def summary(self, first: int = 0, last=None):
        sm, smax, power, reasons = [], [], [], set()
        for line in self.lines[first:last]:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower() == "active":
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [s for s, p in zip(sm, power) if p >= 0.6 * max(power)] or sm
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": float(max(smax)), "power_w_max": float(max(power)),
                "samples": len(sm), "reasons": sorted(reasons)}

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()


def visible_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        parts = [p for p in vis.split(",") if p.strip()]
        if local_rank < len(parts) and parts[local_rank].strip().isdigit():
            return int(parts[local_rank])
    return local_rank


# ------------------------------------------------------------------------------------------
# CPU path (the oracle's TTGT restatement on OpenBLAS): baseline leg and --impl reference.
# Each cpu_sample_* returns (one_step, work_per_step, sample_description); one_step() runs a
# bounded sample of the GPU arm's workload on all host cores.
# ------------------------------------------------------------------------------------------
def cpu_chain(env: np.ndarray, sites) -> np.ndarray:
    from oracle import oracle

    for a in sites:
        t = oracle.ttgt_contract([0, 1], env, [0, 2, 3], a, [1, 2, 3])          # ab,asc->bsc
        env = oracle.ttgt_contract([1, 2, 3], t, [1, 2, 4], np.conj(a), [3, 4])  # bsc,bsd->cd
    return env


def cpu_sample_chain(args):
    chi, d, sample_sites = args.chi, args.phys, 2
    sites = [site_tensor(2000 + s, chi, d) for s in range(sample_sites)]
    env = np.eye(chi, dtype=np.complex128)
    return (lambda: cpu_chain(env, sites)), chain_flops(chi, d, sample_sites), \
        f"{sample_sites} of the {args.sites} sites per step (numpy permute + OpenBLAS ZGEMM)"


def cpu_sample_dense(args):
    """A slab of the contracted pair: 4 of the l values (K = 1024 of the 65536 at full size), every
    (i,j) and (m,n): the same GEMM shape per unit of K as the whole contraction."""
    from oracle import oracle

    ext, kext = dense_extents(args.scale)
    ls = min(4, kext)
    a = seeded_normal(5000, (ext, ext, kext, ls), np.float32)
    b = seeded_normal(5001, (kext, ls, ext, ext), np.float32)
    flops = 2.0 * ext ** 4 * kext * ls
    return (lambda: oracle.ttgt_contract([0, 1, 2, 3], a, [2, 3, 4, 5], b, [0, 1, 4, 5])), flops, \
        f"an l-slab of {ls} of the {kext} values of l per step (K = {kext * ls} of {kext * kext}; M = N = {ext * ext}) " \
        f"through numpy permute + OpenBLAS SGEMM"


def cpu_sample_einsum(notation, arrays, flops):
    from oracle import oracle

    ins, out = oracle.parse_notation(notation)
    run = lambda: np.einsum(*[x for pair in zip(arrays, ins) for x in pair], out, optimize=True)
    return run, flops, f"numpy.einsum('{notation}', optimize=True) on OpenBLAS"


def cpu_sample_grouped(args):
    table = grouped_table(3000, args.problems)[:512]
    rng = np.random.default_rng(3001)
    ops = [(rng.uniform(-1, 1, (i, j)).astype(np.float32), rng.uniform(-1, 1, (j, k)).astype(np.float32))
           for (i, j, k) in table]
    flops = float((2.0 * table[:, 0] * table[:, 1] * table[:, 2]).sum())

    def run():
        for a, b in ops:
            a @ b
    return run, flops, f"the first {len(ops)} of the {args.problems} problems per step, one numpy matmul each"


def cpu_sample_for(args):
    wl = args.workload
    if wl == "dense":
        return cpu_sample_dense(args)
    if wl == "chain":
        return cpu_sample_chain(args)
    if wl == "grouped":
        return cpu_sample_grouped(args)
    if wl == "abc_bcd":
        a, b = seeded_normal(1000, (64, 64, 64), np.float64), seeded_normal(1001, (64, 64, 64), np.float64)
        return cpu_sample_einsum("abc,bcd->ad", [a, b], 2.0 * 64 ** 4)
    if wl == "network4":
        # the full network holds two 679 MB intermediates and takes minutes per pass on the host:
        # the sample is the same network with every index 48 (1/32 of the work)
        dim = min(48, max(8, int(round(96 * args.scale))))
        from oracle import oracle

        a0, a1, a2, a3 = (seeded_normal(4000 + t, (dim,) * 3, np.complex64) for t in range(4))

        def run():
            # the tree the optimiser finds: (jlm,kmn), then ijk with it, then lnp  (labels i..p = 0..6)
            t1 = oracle.ttgt_contract([1, 3, 4], a1, [2, 4, 5], a2, [1, 3, 2, 5])   # jlm,kmn->jlkn
            t2 = oracle.ttgt_contract([0, 1, 2], a0, [1, 3, 2, 5], t1, [0, 3, 5])   # ijk,jlkn->iln
            return oracle.ttgt_contract([0, 3, 5], t2, [3, 5, 6], a3, [0, 6])       # iln,lnp->ip
        return run, 8.0 * (2.0 * dim ** 5 + dim ** 4), \
            f"the same network with every index {dim}, pairwise through numpy permute + OpenBLAS CGEMM"
    if wl == "permute":
        dtype, shape, perm = PERMUTE_CASES[args.case]
        shape = tuple(max(2, int(round(s * args.scale))) for s in shape)
        src = np.asfortranarray(np.random.default_rng(7).integers(0, 255, size=shape).astype(dtype))
        return (lambda: np.asfortranarray(np.transpose(src, perm))), 2.0 * src.nbytes, "numpy transpose + copy"
    if wl == "reduce":
        dtype, shape, kept, op = REDUCE_CASES.get(args.case, REDUCE_CASES["sum_axis0"])
        src = np.asfortranarray(np.random.default_rng(8).standard_normal(shape).astype(dtype))
        axes = tuple(ax for ax in range(len(shape)) if ax not in kept)
        fn = np.sum if op == 0 else np.max
        return (lambda: fn(src, axis=axes)), float(src.nbytes), "numpy reduction"
    raise SystemExit(f"no CPU path for workload {wl}")


def cpu_baseline(args):
    """The CPU path on a bounded sample of the workload: repeated until about --cpu-seconds."""
    run, work, what = cpu_sample_for(args)
    run()
    t0 = time.perf_counter()
    run()
    one = time.perf_counter() - t0
    n = int(max(1, min(4096, args.cpu_seconds / max(one, 1e-6))))
    t0 = time.perf_counter()
    for _ in range(n):
        run()
    dt = time.perf_counter() - t0
    unit = "GB/s" if args.workload in ("permute", "reduce") else "GFLOP/s"
    return {"value": work * n / dt / 1e9, "unit": unit, "cores": os.cpu_count() or 1, "kind": "port",
            "sample": f"{n} x ({what}), {dt:.1f} s"}


def workload_identity(args):
    """(metric, unit, dtype, scaling, workload string): what both arms print."""
    wl = args.workload
    if wl == "dense":
        ext, kext = dense_extents(args.scale)
        return DENSE_METRIC, "GFLOP/s", "f32 (3xTF32)", "strong", dense_workload_name(ext, kext)
    if wl == "chain":
        return (CHAIN_METRIC, "GFLOP/s", "c128 (f64 arithmetic)", "weak",
                chain_workload_name(args.sites, args.chi, args.phys))
    if wl == "grouped":
        return ("einsum GFLOP/s (grouped 'bij,bjk->bik', f32, ragged)", "GFLOP/s", "f32", "strong",
                f"{args.problems} problems 'ij,jk->ik', dims drawn from {{16,32,64,128}} (seed 3000), U(-1,1), f32")
    if wl == "network4":
        dim = max(8, int(round(96 * args.scale)))
        return ("einsum GFLOP/s ('ijk,jlm,kmn,lnp->ip', complex64)", "GFLOP/s", "c64 (f32 arithmetic)", "weak",
                f"'ijk,jlm,kmn,lnp->ip' complex64, every index {dim}, N(0,1) parts")
    if wl == "abc_bcd":
        return ("einsum GFLOP/s ('abc,bcd->ad', f64, dims 64)", "GFLOP/s", "f64", "weak",
                "'abc,bcd->ad' f64, a=b=c=d=64, N(0,1)")
    if wl == "permute":
        dtype, shape, perm = PERMUTE_CASES[args.case]
        shape = tuple(max(2, int(round(s * args.scale))) for s in shape)
        return (f"permute GB/s ({args.case})", "GB/s", np.dtype(dtype).name, "weak",
                f"permute {list(shape)} {np.dtype(dtype).name} by {list(perm)}")
    dtype, shape, kept, op = REDUCE_CASES.get(args.case, REDUCE_CASES["sum_axis0"])
    return (f"reduce GB/s ({args.case})", "GB/s", np.dtype(dtype).name, "weak",
            f"reduce {list(shape)} {np.dtype(dtype).name} keeping modes {kept}, op {op}")


def run_reference(args, rank: int):
    """--impl reference: the reference's own CPU implementation cannot be built or run here (no
    Rust toolchain, its bodies are todo!()), so this arm times the oracle's CPU port of the same
    workload, each step a bounded sample of it, on all host cores."""
    if rank != 0:
        return
    metric, unit, dtype, scaling, workload = workload_identity(args)
    run, work, what = cpu_sample_for(args)
    for _ in range(max(args.warmup, 1)):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    dt = time.perf_counter() - t0
    value = work * args.steps / dt / 1e9
    cores = os.cpu_count() or 1
    print(json.dumps({
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": {"workload": workload, "sample_per_step": what,
                   "note": "a rate over the same per-unit work as the GPU arm's full step"},
        "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port",
                         "sample": f"{what}; {cores} threads"},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------------------
# Workloads.  Each returns a dict:
#   step()            enqueue one step on the context's stream (inputs resident)
#   work              algorithmic flops (or bytes) of one step, summed over all ranks' shares
#   e2e_step()        one step from pinned host inputs to a host-visible result (or None)
#   h2d, d2h          bytes copied per e2e step (all ranks together)
#   check()           relative error of (a sample of) this rank's result against the host
#   kernel, per_launch, bound, peak(), peak_source     roofline of the dominant kernel
# ------------------------------------------------------------------------------------------
class Env:
    def __init__(self, args, tb, ctx, rank, local_rank, world, dist, torch):
        self.args, self.tb, self.ctx = args, tb, ctx
        self.rank, self.local_rank, self.world, self.dist, self.torch = rank, local_rank, world, dist, torch
        self.space = tb.LogicalMemorySpace.GpuMemory(local_rank)
        self.peaks = load_peaks()
        self._copy_ctx = None

    @property
    def copy_ctx(self):
        """A second context of the same device: its stream carries the host<->device copies of the
        end-to-end legs beside the kernels of `ctx` (a context is one in-order queue)."""
        if self._copy_ctx is None:
            self._copy_ctx = self.tb.Context(self.local_rank)
        return self._copy_ctx


def pinned(ctx, nbytes, dtype):
    ptr = ctx.host_alloc(nbytes)
    arr = np.ctypeslib.as_array((C.c_char * nbytes).from_address(ptr)).view(dtype)
    return ptr, arr


def staged_e2e(env: Env, inputs, step, outputs):
    """The plain end-to-end leg: copy every input from pinned host memory, run the step, copy
    every output back, wait.  `inputs`/`outputs`: lists of (device pointer, nbytes).  The pinned
    buffers are filled from the device copies once, outside any timed region."""
    ctx = env.ctx
    host_in = [pinned(ctx, n, np.uint8) for (_, n) in inputs]
    host_out = [pinned(ctx, n, np.uint8) for (_, n) in outputs]
    ctx.synchronize()
    for (hp, _), (dp, n) in zip(host_in, inputs):
        ctx.d2h(C.c_void_p(hp), dp, n)
    ctx.synchronize()

    def e2e_step():
        for (hp, _), (dp, n) in zip(host_in, inputs):
            ctx.h2d(dp, C.c_void_p(hp), n)
        step()
        for (hp, _), (dp, n) in zip(host_out, outputs):
            ctx.d2h(C.c_void_p(hp), dp, n)
        ctx.synchronize()

    return e2e_step, sum(n for _, n in inputs), sum(n for _, n in outputs)


def wl_chain(env: Env):
    args, tb, ctx = env.args, env.tb, env.ctx
    chi, d, sites = args.chi, args.phys, args.sites
    site_bytes, env_bytes = chi * d * chi * 16, chi * chi * 16
    # Pinned host copies (end-to-end leg) and resident device tensors.  Each rank (replica) draws
    # its own chain: seed = 2000 + 100 * rank + site.
    hs_ptr, hs = pinned(ctx, site_bytes * sites, np.complex128)
    he_ptr, he = pinned(ctx, env_bytes, np.complex128)
    ho_ptr, ho = pinned(ctx, env_bytes, np.complex128)
    hs = hs.reshape(sites, chi * d * chi)
    for s in range(sites):
        hs[s] = site_tensor(2000 + 100 * env.rank + s, chi, d).reshape(-1, order="F")
    he[:] = np.eye(chi, dtype=np.complex128).reshape(-1, order="F")
    dev_sites = [tb.Tensor.empty([chi, d, chi], np.complex128, env.space) for _ in range(sites)]
    dev_env0 = tb.Tensor.empty([chi, chi], np.complex128, env.space)
    envs = [tb.Tensor.empty([chi, chi], np.complex128, env.space) for _ in range(2)]

    def upload():
        for s in range(sites):
            ctx.h2d(dev_sites[s]._block.ptr, C.c_void_p(hs_ptr + s * site_bytes), site_bytes)
        ctx.h2d(dev_env0._block.ptr, C.c_void_p(he_ptr), env_bytes)

    upload()
    ctx.synchronize()
    tree = tb.ContractionTree.optimize(tb.Subscripts.parse(CHAIN), [[chi, chi], [chi, d, chi], [chi, d, chi]])
    # One prepared call per site: E_{s+1} = einsum(E_s, A_s, conj(A_s)); conj is a view flag folded
    # into the operand loads, nothing is materialised.
    calls = []
    for s in range(sites):
        src = dev_env0 if s == 0 else envs[(s - 1) % 2]
        calls.append(tb.PreparedEinsum(tree, [src, dev_sites[s], dev_sites[s].into_conj()], envs[s % 2]))
    final_env = envs[(sites - 1) % 2]

    def step():
        for c in calls:
            c.run()

    def read_result():
        ctx.d2h(C.c_void_p(ho_ptr), final_env._block.ptr, env_bytes)
        ctx.synchronize()
        return ho.copy()

    def check():
        # the first two sites of this rank's chain against the host's TTGT contraction
        e = cpu_chain(np.eye(chi, dtype=np.complex128),
                      [hs[s].reshape((chi, d, chi), order="F") for s in range(min(2, sites))])
        probe = [tb.Tensor.empty([chi, chi], np.complex128, env.space) for _ in range(2)]
        src = dev_env0
        for s in range(min(2, sites)):
            tb.einsum_with_plan_into(tree, [src, dev_sites[s], dev_sites[s].into_conj()], 1.0, 0.0, probe[s % 2])
            src = probe[s % 2]
        got = src.to_numpy()
        return float(np.linalg.norm(got - e) / np.linalg.norm(e))

    # End to end: the site tensors travel host -> device on the stream of a second context, one
    # event per site, and each site's contraction waits only for its own tensor, so the copies of
    # later sites hide behind the contractions of earlier ones.
    e2e_step = None
    if not args.no_e2e:
        copy_ctx = env.copy_ctx

        def e2e_step():
            copy_ctx.h2d(dev_env0._block.ptr, C.c_void_p(he_ptr), env_bytes)
            events = []
            for s in range(sites):
                copy_ctx.h2d(dev_sites[s]._block.ptr, C.c_void_p(hs_ptr + s * site_bytes), site_bytes)
                events.append(copy_ctx.record_event())
            for s in range(sites):
                ctx.wait_event(events[s])
                calls[s].run()
            ctx.d2h(C.c_void_p(ho_ptr), final_env._block.ptr, env_bytes)
            ctx.synchronize()

    return {
        "step": step, "work": chain_flops(chi, d, sites) * env.world, "read_result": read_result,
        "e2e_step": e2e_step, "h2d": (site_bytes * sites + env_bytes) * env.world, "d2h": env_bytes * env.world,
        "kernel": "contract_dmma", "check": check, "check_tol": 1e-12,
        "kernel_label": "contract_dmma_tma_kernel (complex128, TMA-fed, 64x64x16 tiles, m16n8k8 DMMA, three real "
                        "products per complex one)",
        "per_launch": 8.0 * chi * chi * (d * chi), "bound": "tensor", "peak": ctx.probe_fp64_tflops,
        "peak_source": "measured on this GPU by the library's register-resident DMMA probe "
                       "(MEASURED_PEAKS.json holds no FP64 figure)",
        "extra_kernels": ["contract_dmma_fixup"], "graph_calls": 1,
        # dram__bytes_read + dram__bytes_write per launch, from an ncu capture of this workload
        # (12.6 and 16.8 MB on the two captured launches)
        "traffic": 14.74e6 if (chi, d) == (512, 2) else None,
        "config": {"parallelism": f"{env.world} independent replica(s)",
                   "l2": f"inputs larger than L2: each pass streams {sites * site_bytes >> 20} MiB of site tensors",
                   "tree_pairs": tree.pairs},
    }


def sampled_check(env: Env, a_t, b_t, read_c, i_range, n_range, rows: int = 8, cols: int = 2048):
    """Sampled entries of C = A.B against a float64 sum over all (k,l) on the host.
    a_t: (l,k,j,i), b_t: (n,m,l,k) torch tensors (column-major [i,j,k,l], [k,l,m,n]);
    read_c(ci, cj, cm, cn) -> device tensor [rows, cols] of this rank's computed values;
    i_range / n_range: the half-open ranges of i and of n this rank owns."""
    torch = env.torch
    dev = a_t.device
    L, K, J, I = a_t.shape
    M = b_t.shape[1]
    rng = np.random.default_rng(55 + env.rank)
    ci = torch.tensor(rng.integers(i_range[0], i_range[1], size=rows), device=dev)
    cj = torch.tensor(rng.integers(0, J, size=rows), device=dev)
    cm = torch.tensor(rng.integers(0, M, size=cols), device=dev)
    cn = torch.tensor(rng.integers(n_range[0], n_range[1], size=cols), device=dev)
    a_rows = a_t[:, :, cj, ci].reshape(L * K, rows).cpu().numpy().astype(np.float64)
    b_cols = b_t[cn, cm].reshape(cols, L * K).cpu().numpy().astype(np.float64)
    want = (b_cols @ a_rows).T
    got = read_c(ci, cj, cm, cn).cpu().numpy().astype(np.float64)
    return float(np.linalg.norm(got - want) / np.linalg.norm(want))


def wl_dense(env: Env):
    """'ijkl,klmn->ijmn', f32, N(0,1).  Strong scaling: the ranks split one contraction."""
    from tenferro_b200 import sharding

    args, tb, ctx, torch, dist = env.args, env.tb, env.ctx, env.torch, env.dist
    ext, kext = dense_extents(args.scale)
    i = j = m = n = ext
    k = l = kext
    W, r = env.world, env.rank
    dev = torch.device("cuda", env.local_rank)
    gen = torch.Generator(device=dev)
    gen.manual_seed(5000)
    # Column-major tensors = torch tensors with reversed dims.  Every rank holds the full A and B
    # (same seed, the device's counter-based generator) and contracts strided sub-views of them.
    a_t = torch.randn((l, k, j, i), generator=gen, device=dev, dtype=torch.float32)
    gen.manual_seed(5001)
    b_t = torch.randn((n, m, l, k), generator=gen, device=dev, dtype=torch.float32)
    c_t = torch.zeros((n, m, j, i), device=dev, dtype=torch.float32)
    wrap = lambda t, dims: tb.Tensor.from_device_pointer(t.data_ptr(), t.numel() * 4, dims, np.float32, env.space, t)
    A, B, Cfull = wrap(a_t, [i, j, k, l]), wrap(b_t, [k, l, m, n]), wrap(c_t, [i, j, m, n])
    sub = lambda T, axis, lo, hi: tb.Tensor(T._block, [hi - lo if d == axis else e for d, e in enumerate(T.dims())],
                                            T.strides(), T.offset() + lo * T.strides()[axis], np.float32, env.space)
    shard = lambda T, axis: tb.Tensor(T._block, *sharding.shard_view(T.dims(), T.strides(), 0, axis, W, r),
                                      np.float32, env.space)
    subs = tb.Subscripts.parse(DENSE)
    flops = 2.0 * i * j * m * n * k * l
    modes = {}

    # ---- free-index split: A and C sliced along i, B whole; no collective
    if i % W:
        raise SystemExit("i must divide by the number of GPUs")
    As, Cs = shard(A, 0), shard(Cfull, 0)
    call_i = tb.PreparedEinsum(tb.ContractionTree.optimize(subs, [As.dims(), B.dims()]), [As, B], Cs)
    i_lo, i_hi = sharding.split_range(i, W, r)
    modes["i"] = {
        "step": call_i.run, "result": c_t,
        "mode": f"free index i split {W} ways, no communication" if W > 1 else "one GPU",
        "check": lambda: sampled_check(
            env, a_t, b_t, lambda ci, cj, cm, cn: c_t[cn[None, :], cm[None, :], cj[:, None], ci[:, None]],
            (i_lo, i_hi), (0, n)),
    }

    # ---- contracted-index split: A and B sliced along l, full-size partial C, NCCL reduce-scatter
    if l % W:
        raise SystemExit("l must divide by the number of GPUs")
    l_lo, l_hi = sharding.split_range(l, W, r)
    part_t = out_t = P = None
    if W > 1:
        part_t = torch.zeros((n, m, j, i), device=dev, dtype=torch.float32)
        out_t = torch.zeros((n * m * j * i) // W, device=dev, dtype=torch.float32)
        P = wrap(part_t, [i, j, m, n])
        Al, Bl = shard(A, 3), shard(B, 1)
        call_k = tb.PreparedEinsum(tb.ContractionTree.optimize(subs, [Al.dims(), Bl.dims()]), [Al, Bl], P)
        scatter = lambda: dist.reduce_scatter_tensor(out_t, part_t.view(-1), op=dist.ReduceOp.SUM)

        def step_k():
            call_k.run()
            scatter()

        n_lo, n_hi = sharding.split_range(n, W, r)  # the flat 1/W of C a rank keeps is a range of n
        out_v = out_t.view(n // W, m, j, i)
        modes["k"] = {
            "step": step_k, "compute": call_k.run, "collective": scatter, "result": out_t,
            "mode": f"contracted pair (k,l) split {W} ways on l, partial outputs reduce-scattered over NCCL",
            "check": lambda: sampled_check(
                env, a_t, b_t,
                lambda ci, cj, cm, cn: out_v[(cn - n_lo)[None, :], cm[None, :], cj[:, None], ci[:, None]],
                (0, i), (n_lo, n_hi)),
        }

    # ---- end to end: this rank's l-range of A and B comes from pinned host memory in slabs (the
    # pitched copy of a B slab is a range of l for every (m,n)); slab s is multiplied while slab
    # s+1 travels; C (or, on N > 1 GPUs, this rank's reduce-scattered part of it) goes back.
    e2e_step, h2d, d2h, e2e_note = None, 0, 0, None
    if not args.no_e2e:
        l_r = l_hi - l_lo
        # Slabs of 32 l-values while plenty is left, then halving down to 8: the upload paces the
        # step (PCIe), so what counts at the end is how little work is left once the last slab lands.
        sizes, rem = [], l_r
        while rem > 0:
            sz = 32 if rem >= 64 else (max(8, (rem // 2) // 8 * 8) if rem > 8 else rem)
            sizes.append(sz)
            rem -= sz
        starts = [l_lo + sum(sizes[:q]) for q in range(len(sizes))]
        n_slabs = len(sizes)
        a_bytes, b_bytes = i * j * k * l_r * 4, k * l_r * m * n * 4
        ha_ptr, _ = pinned(ctx, a_bytes, np.float32)
        hb_ptr, _ = pinned(ctx, b_bytes, np.float32)   # host layout [k, l_r, m, n] column-major
        c_keep = c_t if W == 1 else out_t
        hc_ptr, _ = pinned(ctx, c_keep.numel() * 4, np.float32)
        # fill the host buffers from the device tensors (set-up, untimed)
        ctx.synchronize()
        ctx.d2h(C.c_void_p(ha_ptr), a_t.data_ptr() + l_lo * i * j * k * 4, a_bytes)
        ctx.d2h_2d(C.c_void_p(hb_ptr), k * l_r * 4, b_t.data_ptr() + l_lo * k * 4, k * l * 4, k * l_r * 4, m * n)
        ctx.synchronize()
        acc = Cfull if W == 1 else P
        # On one GPU the last slab is multiplied in four ranges of n, and each finished quarter of C
        # starts its way back to the host while the next one is computed.
        n_chunks = 4 if (W == 1 and n % 4 == 0) else 1
        slab_calls = []
        for s in range(n_slabs):
            lo, hi = starts[s], starts[s] + sizes[s]
            As_, Bs_ = sub(A, 3, lo, hi), sub(B, 1, lo, hi)
            beta = 0.0 if s == 0 else 1.0
            if s == n_slabs - 1 and n_chunks > 1:
                calls = []
                for q in range(n_chunks):
                    n0, n1 = q * n // n_chunks, (q + 1) * n // n_chunks
                    Bq, Cq = sub(Bs_, 3, n0, n1), sub(acc, 3, n0, n1)
                    tree = tb.ContractionTree.optimize(subs, [As_.dims(), Bq.dims()])
                    calls.append(tb.PreparedEinsum(tree, [As_, Bq], Cq, 1.0, beta))
                slab_calls.append(calls)
            else:
                tree = tb.ContractionTree.optimize(subs, [As_.dims(), Bs_.dims()])
                slab_calls.append([tb.PreparedEinsum(tree, [As_, Bs_], acc, 1.0, beta)])
        copy_ctx = env.copy_ctx
        c_bytes = c_keep.numel() * 4

        def e2e_step():
            events = []
            for s in range(n_slabs):
                # (one upload stream: with the A and B slabs on two streams the step took 267 ms instead of
                # 202 ms - under the contraction kernel the uploads reach 42 GB/s of the link's 55.6 either way)
                lo, off = starts[s], starts[s] - l_lo
                copy_ctx.h2d(a_t.data_ptr() + lo * i * j * k * 4, C.c_void_p(ha_ptr + off * i * j * k * 4),
                             i * j * k * sizes[s] * 4)
                copy_ctx.h2d_2d(b_t.data_ptr() + lo * k * 4, k * l * 4, C.c_void_p(hb_ptr + off * k * 4), k * l_r * 4,
                                k * sizes[s] * 4, m * n)
                events.append(copy_ctx.record_event())
            for s in range(n_slabs):
                ctx.wait_event(events[s])
                last = s == n_slabs - 1 and n_chunks > 1
                for q, call in enumerate(slab_calls[s]):
                    call.run()
                    if last:
                        # this quarter of C is final: it leaves on the copy stream (the uploads are over)
                        copy_ctx.wait_event(ctx.record_event())
                        copy_ctx.d2h(C.c_void_p(hc_ptr + q * c_bytes // n_chunks), c_keep.data_ptr() + q * c_bytes // n_chunks,
                                     c_bytes // n_chunks)
            if n_chunks == 1:
                if W > 1:
                    scatter()
                ctx.d2h(C.c_void_p(hc_ptr), c_keep.data_ptr(), c_bytes)
            ctx.synchronize()
            copy_ctx.synchronize()

        h2d, d2h = (a_bytes + b_bytes) * W, c_bytes * W
        e2e_note = (f"each rank uploads its 1/{W} of A and B along l in {n_slabs} slabs of {sizes} l-values "
                    f"(pitched copy for B) on a second stream, multiplies slab s while slab s+1 travels, "
                    + ("reduce-scatters the partial C and reads its part back" if W > 1 else
                       "and reads C back in four parts, each as soon as the last slab has been added to it"))
    # The probe runs once before the workload (cool GPU) and once after (under the power cap the
    # clock has dropped by then); the larger figure is the burst rate.
    tf32_cold = ctx.probe_tf32_tflops()
    primary = "k" if (args.shard == "k" and W > 1) else "i"
    pm = modes[primary]

    def read_result():
        ctx.synchronize()
        return pm["result"].flatten()[:4096].cpu().numpy()

    cfg = {"parallelism": pm["mode"],
           "l2": f"inputs larger than L2: A and B hold {(a_t.numel() + b_t.numel()) * 4 >> 20} MiB", "flop_total": flops}
    if e2e_note:
        cfg["e2e_path"] = e2e_note
    return {
        "step": pm["step"], "work": flops, "read_result": read_result, "e2e_step": e2e_step, "h2d": h2d, "d2h": d2h,
        "kernel": "contract_tf32x3",
        "kernel_label": "contract_tf32x3_pair_kernel (tcgen05 cta_group::2, 256x256 tiles per CTA pair, 32-deep stages)",
        "per_launch": flops / W, "bound": "tensor", "tf32_cold": tf32_cold, "tf32x3": True,
        "extra_kernels": ["repack_operand"], "keep": (a_t, b_t, c_t, part_t, out_t),
        "check": pm["check"], "modes": modes, "primary": primary, "traffic": None,
        "config": cfg,
    }


def wl_grouped(env: Env):
    """4096 ragged 'ij,jk->ik' products, f32, dims from {16,32,64,128}, U(-1,1); table sharded."""
    from tenferro_b200 import sharding

    args, tb, ctx, torch = env.args, env.tb, env.ctx, env.torch
    table = grouped_table(3000, args.problems)
    bytes_p = 4 * (table[:, 0] * table[:, 1] + table[:, 1] * table[:, 2] + table[:, 0] * table[:, 2])
    # contiguous ranges of the table with equal byte counts
    cuts = sharding.split_table_by_bytes(bytes_p, env.world)
    lo, hi = cuts[env.rank], cuts[env.rank + 1]
    mine = table[lo:hi]
    dev = torch.device("cuda", env.local_rank)
    gen = torch.Generator(device=dev)
    gen.manual_seed(3001 + env.rank)
    na = int((mine[:, 0] * mine[:, 1]).sum())
    nb = int((mine[:, 1] * mine[:, 2]).sum())
    nc = int((mine[:, 0] * mine[:, 2]).sum())
    a_t = torch.rand(na, generator=gen, device=dev) * 2 - 1
    b_t = torch.rand(nb, generator=gen, device=dev) * 2 - 1
    c_t = torch.zeros(nc, device=dev)
    probs, offs, oa, ob, oc = [], [], 0, 0, 0
    for (pi, pj, pk) in mine:
        pi, pj, pk = int(pi), int(pj), int(pk)
        probs.append((pi, pk, pj, a_t.data_ptr() + 4 * oa, 1, pi, b_t.data_ptr() + 4 * ob, 1, pj,
                      c_t.data_ptr() + 4 * oc, 1, pi))
        offs.append((oa, ob, oc))
        oa, ob, oc = oa + pi * pj, ob + pj * pk, oc + pi * pk
    flops_all = float((2.0 * table[:, 0] * table[:, 1] * table[:, 2]).sum())
    bytes_all = float(bytes_p.sum())

    from tenferro_b200.prims import PreparedGroupedGemm

    call = PreparedGroupedGemm(probs, np.float32, 1.0, 0.0, ctx)
    step = call.run

    def read_result():
        ctx.synchronize()
        return c_t[:4096].cpu().numpy()

    def check():
        # 32 problems of this rank's range against float64 on the host
        rng = np.random.default_rng(33 + env.rank)
        ctx.synchronize()
        worst = 0.0
        for q in rng.choice(len(mine), size=min(32, len(mine)), replace=False):
            pi, pj, pk = (int(x) for x in mine[q])
            oa_, ob_, oc_ = offs[q]
            a = a_t[oa_:oa_ + pi * pj].cpu().numpy().astype(np.float64).reshape(pi, pj, order="F")
            b = b_t[ob_:ob_ + pj * pk].cpu().numpy().astype(np.float64).reshape(pj, pk, order="F")
            c = c_t[oc_:oc_ + pi * pk].cpu().numpy().astype(np.float64).reshape(pi, pk, order="F")
            worst = max(worst, float(np.linalg.norm(c - a @ b) / np.linalg.norm(a @ b)))
        return worst

    e2e_step = None
    if not args.no_e2e:
        e2e_step, _, _ = staged_e2e(env, [(a_t.data_ptr(), na * 4), (b_t.data_ptr(), nb * 4)], step,
                                    [(c_t.data_ptr(), nc * 4)])
    hbm = (env.peaks or {}).get("hbm_gbs")
    return {
        "step": step, "work": flops_all, "read_result": read_result, "e2e_step": e2e_step,
        "h2d": float(4 * (table[:, 0] * table[:, 1] + table[:, 1] * table[:, 2]).sum()),
        "d2h": float(4 * (table[:, 0] * table[:, 2]).sum()),
        "kernel": "grouped_tf32x3", "kernels_any": ["grouped_tf32x3", "grouped_tcgen05", "grouped_simt"],
        "kernel_label": "grouped_f32_kernel (persistent CTAs, host-built stage table, double-buffered cp.async panels)",
        "per_launch": float(bytes_p[lo:hi].sum()), "bound": "hbm",
        "peak": (lambda: hbm) if hbm else ctx.probe_hbm_gbs,
        "peak_source": "MEASURED_PEAKS.json hbm_gbs" if hbm else "library copy probe (MEASURED_PEAKS.json absent)",
        "extra_kernels": [], "keep": (a_t, b_t, c_t), "check": check,
        # dram__bytes_read + dram__bytes_write of one launch over the whole table, from an ncu capture
        # of this workload (121.8 MB read + 25.5 MB written)
        "traffic": 147.3e6 if (args.problems == 4096 and env.world == 1) else None,
        "config": {"parallelism": f"problem table split {env.world} ways by bytes",
                   "l2": f"inputs larger than L2: {bytes_all / 2**20:.0f} MiB touched per step",
                   "bytes_total": bytes_all, "flop_total": flops_all},
    }


def wl_network4(env: Env):
    args, tb, ctx = env.args, env.tb, env.ctx
    dim = max(8, int(round(96 * args.scale)))
    notation = "ijk,jlm,kmn,lnp->ip"
    arrays = [seeded_normal(4000 + t, (dim,) * 3, np.complex64) for t in range(4)]
    ops = [tb.Tensor.from_numpy(a, memory_space=env.space) for a in arrays]
    out = tb.Tensor.empty([dim, dim], np.complex64, env.space)
    tree = tb.ContractionTree.optimize(tb.Subscripts.parse(notation), [a.shape for a in arrays])
    call = tb.PreparedEinsum(tree, ops, out)
    flops = 8.0 * tree.macs
    tf32_cold = ctx.probe_tf32_tflops()

    def read_result():
        return out.to_numpy()

    def check():
        # 64 sampled entries of the output, each a float64 sum over the network's five inner labels
        # on the host (a chain of small matrix products per sampled (i, p))
        rng = np.random.default_rng(44 + env.rank)
        a0, a1, a2, a3 = (x.astype(np.complex128) for x in arrays)
        got_all = out.to_numpy()
        # T[k,l,m,n] = sum_j ... is large; contract per sampled i and p instead:
        #   out[i,p] = sum_{j,k,l,m,n} a0[i,j,k] a1[j,l,m] a2[k,m,n] a3[l,n,p]
        num, den = 0.0, 0.0
        for _ in range(64 if dim <= 48 else 8):
            ii, pp = int(rng.integers(dim)), int(rng.integers(dim))
            x = np.einsum("jk,jlm->klm", a0[ii], a1, optimize=True)      # [k,l,m]
            y = np.einsum("klm,kmn->ln", x, a2, optimize=True)           # [l,n]
            want = np.sum(y * a3[:, :, pp])
            num += abs(got_all[ii, pp] - want) ** 2
            den += abs(want) ** 2
        return float((num / den) ** 0.5)

    e2e_step, h2d, d2h = None, 0, 0
    if not args.no_e2e:
        e2e_step, h2d, d2h = staged_e2e(env, [(o._block.ptr, o._block.nbytes) for o in ops], call.run,
                                        [(out._block.ptr, out._block.nbytes)])
    return {
        "step": call.run, "work": flops * env.world, "read_result": read_result, "e2e_step": e2e_step,
        "h2d": h2d * env.world, "d2h": d2h * env.world, "kernel": "contract_tf32x3",
        "kernel_label": "contract_tf32x3 kernels (tcgen05; complex64 as one real product of doubled extents per tree node)",
        "per_launch": flops / 3.0, "bound": "tensor", "tf32_cold": tf32_cold, "tf32x3": True,
        "extra_kernels": ["pack_planes", "contract_tf32x3_finish"], "check": check,
        # ncu, per launch averaged over the three product launches of a call: the two large nodes moved
        # 667 MB and 703 MB; the third, whose operands (two 7 MB tensors) stay in L2, was not captured
        # and is counted as zero
        "traffic": (667.2e6 + 703.2e6) / 3.0 if dim == 96 else None,
        "config": {"tree": tree.pairs, "parallelism": f"{env.world} independent replica(s)",
                   "l2": f"intermediates of {dim ** 4 * 8 >> 20} MiB exceed L2" if dim >= 64 else "L2-resident (scaled down)",
                   "flop_total": flops},
    }


def wl_abc_bcd(env: Env):
    args, tb, ctx = env.args, env.tb, env.ctx
    notation = "abc,bcd->ad"
    a, b = seeded_normal(1000, (64, 64, 64), np.float64), seeded_normal(1001, (64, 64, 64), np.float64)
    A, B = tb.Tensor.from_numpy(a, memory_space=env.space), tb.Tensor.from_numpy(b, memory_space=env.space)
    out = tb.Tensor.empty([64, 64], np.float64, env.space)
    tree = tb.ContractionTree.optimize(tb.Subscripts.parse(notation), [a.shape, b.shape])
    call = tb.PreparedEinsum(tree, [A, B], out)
    flops = 2.0 * 64 ** 4

    def check():
        want = np.einsum("abc,bcd->ad", a, b)
        return float(np.linalg.norm(out.to_numpy() - want) / np.linalg.norm(want))

    e2e_step, h2d, d2h = None, 0, 0
    if not args.no_e2e:
        e2e_step, h2d, d2h = staged_e2e(env, [(A._block.ptr, a.nbytes), (B._block.ptr, b.nbytes)], call.run,
                                        [(out._block.ptr, 64 * 64 * 8)])
    return {
        "step": call.run, "work": flops * env.world, "read_result": out.to_numpy, "e2e_step": e2e_step,
        "h2d": h2d * env.world, "d2h": d2h * env.world,
        "kernel": "contract_dmma", "kernel_label": "contract_dmma_tma_kernel (f64, 32x32x16 tiles, K split over the CTAs)",
        "per_launch": flops, "bound": "tensor", "peak": ctx.probe_fp64_tflops, "check": check, "check_tol": 1e-12,
        "peak_source": "library DMMA probe", "extra_kernels": ["contract_dmma_fixup"], "graph_calls": 16,
        "config": {"parallelism": f"{env.world} replica(s)",
                   "l2": "L2-resident by construction (4 MiB of operands): a latency measurement",
                   "flop_total": flops},
    }


PERMUTE_CASES = {
    "transpose2d": (np.float32, (16384, 16384), (1, 0)),
    "rank4_reverse": (np.float32, (128, 128, 128, 128), (3, 2, 1, 0)),
    "rank4_pairswap": (np.float32, (128, 128, 128, 128), (1, 0, 3, 2)),
    "rank3_f64": (np.float64, (512, 512, 512), (2, 0, 1)),
    "mps_site_c128": (np.complex128, (512, 2, 512), (1, 2, 0)),
    "copy": (np.float32, (16384, 16384), (0, 1)),
}


def wl_permute(env: Env):
    args, tb, ctx, torch = env.args, env.tb, env.ctx, env.torch
    dtype, shape, perm = PERMUTE_CASES[args.case]
    shape = tuple(max(2, int(round(s * args.scale))) for s in shape)
    itemsize = np.dtype(dtype).itemsize
    n = int(np.prod(shape))
    dev = torch.device("cuda", env.local_rank)
    src_t = torch.randint(0, 255, (n * itemsize,), device=dev, dtype=torch.uint8)
    dst_t = torch.zeros(n * itemsize, device=dev, dtype=torch.uint8)
    src = tb.Tensor.from_device_pointer(src_t.data_ptr(), n * itemsize, shape, dtype, env.space, src_t)
    out_shape = [shape[p] for p in perm]
    dst = tb.Tensor.from_device_pointer(dst_t.data_ptr(), n * itemsize, out_shape, dtype, env.space, dst_t)
    modes = list(range(len(shape)))
    plan = tb.CudaBackend.plan(tb.PrimDescriptor.Permute(modes, [modes[p] for p in perm]), [shape, out_shape], dtype, ctx=ctx)

    def step():
        tb.CudaBackend.execute(plan, 1.0, [src], 0.0, dst)

    step()
    ctx.synchronize()
    hbm = (env.peaks or {}).get("hbm_gbs")
    bytes_step = 2.0 * n * itemsize

    def read_result():
        ctx.synchronize()
        return dst_t[:4096].cpu().numpy()

    def check():
        # bit-exact: the raw bytes of the whole output against numpy's transpose of the input
        ctx.synchronize()
        host = src_t.cpu().numpy().view(dtype).reshape(shape, order="F")
        want = np.asfortranarray(np.transpose(host, perm)).reshape(-1, order="F").view(np.uint8)
        return 0.0 if np.array_equal(dst_t.cpu().numpy(), want) else 1.0

    e2e_step, h2d, d2h = None, 0, 0
    if not args.no_e2e:
        e2e_step, h2d, d2h = staged_e2e(env, [(src_t.data_ptr(), n * itemsize)], step, [(dst_t.data_ptr(), n * itemsize)])
    return {
        "step": step, "work": bytes_step * env.world, "read_result": read_result, "e2e_step": e2e_step,
        "h2d": h2d * env.world, "d2h": d2h * env.world,
        "kernel": "permute_tiled", "kernel_label": "permute kernel (rows / tiled transpose / generic, whichever the layout selects)",
        "kernels_any": ["permute_rows", "permute_tiled", "permute_generic"],
        "per_launch": bytes_step, "bound": "hbm", "peak": (lambda: hbm) if hbm else ctx.probe_hbm_gbs,
        "peak_source": "MEASURED_PEAKS.json hbm_gbs" if hbm else "library copy probe (MEASURED_PEAKS.json absent)",
        "extra_kernels": [], "keep": (src_t, dst_t), "check": check, "check_tol": 0.0,
        # ncu capture of this case: 1.074 GB read + 1.031 GB written per launch
        "traffic": 2.105e9 if (args.case == "transpose2d" and args.scale == 1.0) else None,
        "config": {"parallelism": f"{env.world} replica(s)",
                   "l2": "inputs larger than L2" if n * itemsize > 200e6 else "fits L2 (small member of the set)",
                   "bytes_total": bytes_step},
    }


REDUCE_CASES = {
    "sum_axis0": (np.float32, (16384, 16384), [1], 0),
    "sum_axis1": (np.float32, (16384, 16384), [0], 0),
    "sum_mid_f64": (np.float64, (512, 512, 512), [0, 2], 0),
    "max_axis0": (np.float32, (16384, 16384), [1], 1),
}


def wl_reduce(env: Env):
    args, tb, ctx, torch = env.args, env.tb, env.ctx, env.torch
    dtype, shape, kept, op = REDUCE_CASES.get(args.case, REDUCE_CASES["sum_axis0"])
    itemsize = np.dtype(dtype).itemsize
    n = int(np.prod(shape))
    dev = torch.device("cuda", env.local_rank)
    tdt = torch.float32 if dtype == np.float32 else torch.float64
    src_t = torch.randn(n, device=dev, dtype=tdt)
    out_shape = [shape[kk] for kk in kept]
    dst_t = torch.zeros(int(np.prod(out_shape)), device=dev, dtype=tdt)
    src = tb.Tensor.from_device_pointer(src_t.data_ptr(), n * itemsize, shape, dtype, env.space, src_t)
    dst = tb.Tensor.from_device_pointer(dst_t.data_ptr(), dst_t.numel() * itemsize, out_shape, dtype, env.space, dst_t)
    modes = list(range(len(shape)))
    plan = tb.CudaBackend.plan(tb.PrimDescriptor.Reduce(modes, kept, tb.ReduceOp(op)), [shape, out_shape], dtype, ctx=ctx)

    def step():
        tb.CudaBackend.execute(plan, 1.0, [src], 0.0, dst)

    hbm = (env.peaks or {}).get("hbm_gbs")
    bytes_step = float(n * itemsize + dst_t.numel() * itemsize)

    def read_result():
        ctx.synchronize()
        return dst_t[:4096].cpu().numpy()

    def check():
        ctx.synchronize()
        host = src_t.cpu().numpy().reshape(shape, order="F").astype(np.float64)
        axes = tuple(ax for ax in range(len(shape)) if ax not in kept)
        want = (np.sum if op == 0 else np.max)(host, axis=axes).reshape(-1, order="F")
        got = dst_t.cpu().numpy().astype(np.float64)
        return float(np.linalg.norm(got - want) / np.linalg.norm(want))

    e2e_step, h2d, d2h = None, 0, 0
    if not args.no_e2e:
        e2e_step, h2d, d2h = staged_e2e(env, [(src_t.data_ptr(), n * itemsize)], step,
                                        [(dst_t.data_ptr(), dst_t.numel() * itemsize)])
    return {
        "step": step, "work": bytes_step * env.world, "read_result": read_result, "e2e_step": e2e_step,
        "h2d": h2d * env.world, "d2h": d2h * env.world,
        "kernel": "reduce", "kernel_label": "reduce_kernel", "per_launch": bytes_step, "bound": "hbm",
        "peak": (lambda: hbm) if hbm else ctx.probe_hbm_gbs,
        "peak_source": "MEASURED_PEAKS.json hbm_gbs" if hbm else "library copy probe (MEASURED_PEAKS.json absent)",
        "extra_kernels": ["reduce_finish"], "keep": (src_t, dst_t), "check": check,
        "check_tol": 1e-5 if dtype == np.float32 else 1e-12,
        # ncu capture of this case: 1.076 GB read + 19.4 MB written per launch
        "traffic": 1.095e9 if args.case == "sum_axis0" else None,
        "config": {"parallelism": f"{env.world} replica(s)", "l2": "inputs larger than L2", "bytes_total": bytes_step},
    }


WORKLOADS = {"dense": wl_dense, "chain": wl_chain, "grouped": wl_grouped, "network4": wl_network4,
             "abc_bcd": wl_abc_bcd, "permute": wl_permute, "reduce": wl_reduce}


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")

    import torch
    import tenferro_b200 as tb

    dist = None
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = tb.Context.get(local_rank)
    # One stream for the library's kernels and torch's collectives.
    stream = torch.cuda.Stream(device=local_rank)
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    env = Env(args, tb, ctx, rank, local_rank, world, dist, torch)
    metric, unit, dtype_name, scaling, workload_name = workload_identity(args)
    wl = WORKLOADS[args.workload](env)
    unit_scale = 1e9  # GFLOP/s and GB/s alike

    def barrier():
        ctx.synchronize()
        if dist is not None:
            dist.barrier()
        ctx.synchronize()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    warmup = max(args.warmup, 3)
    sampler = ClockSampler(visible_gpu_index(local_rank)) if rank == 0 else None
    if sampler:
        sampler.start()

    def timed(step, steps=args.steps, warm=warmup):
        """`warm` untimed steps, then exactly `steps` steps between barriers; device time, max over ranks."""
        for _ in range(warm):
            step()
        barrier()
        c0 = sampler.mark() if sampler else 0
        n0 = ctx.kernel_launch_count()
        e0 = ctx.record_event()
        for _ in range(steps):
            step()
        e1 = ctx.record_event()
        barrier()
        ms = max_over_ranks(e0.elapsed_ms(e1))
        if sampler:
            time.sleep(0.12)  # one more clock sample lands
        clocks = sampler.summary(c0, sampler.mark()) if sampler else None
        return ms, ctx.kernel_launch_count() - n0, clocks

    # ---- the timed region: K steps, inputs resident in HBM
    step = wl["step"]
    ms_total, launches, clocks = timed(step)
    value = wl["work"] * args.steps / (ms_total * 1e-3) / unit_scale
    if clocks and clocks.get("sm_mhz"):
        # time x clock: compares runs whose SM clocks differ (short runs escape the power limit)
        clocks["ms_per_step_x_sm_mhz"] = ms_total / args.steps * clocks["sm_mhz"]

    # ---- the kernels are run-to-run deterministic: one more step reproduces the result bit for bit
    first = wl["read_result"]()
    step()
    deterministic = bool(np.array_equal(first, wl["read_result"]()))

    # ---- result check on what this rank owns (after its last step); the worst rank is reported
    def run_check(fn, tol):
        if fn is None:
            return None
        err = fn()
        worst = max_over_ranks(float(err))
        return {"rel_frobenius": worst, "tol": tol, "ok": bool(worst <= tol), "ranks_checked": world}

    check = run_check(wl.get("check"), wl.get("check_tol", CHECK_TOL))
    if check and args.workload == "dense":
        check["sample"] = ("per rank: 8 random (i,j) rows x 2048 random (m,n) columns of what it owns, float64 sum "
                           "over all (k,l) on the host")

    # ---- dense, N > 1: the other sharding mode in the same process, nested in the line
    nested, nested_key = None, None
    modes = wl.get("modes") or {}
    if args.workload == "dense" and world > 1 and args.shard == "both":
        other = "k" if wl["primary"] == "i" else "i"
        mk = modes[other]
        ms_k, _, clocks_k = timed(mk["step"])
        nested_key = f"shard_{other}"
        nested = {"value": wl["work"] * args.steps / (ms_k * 1e-3) / unit_scale, "unit": unit,
                  "ms_per_step": ms_k / args.steps, "parallelism": mk["mode"]}
        if "compute" in mk:
            # where the time of a step goes: the product alone and the collective alone (each K steps,
            # device-timed, max over ranks).  One stream, so a step is their sum.
            ms_c, _, _ = timed(mk["compute"], warm=1)
            ms_r, _, _ = timed(mk["collective"], warm=1)
            full_c = 4.0 * modes["i"]["result"].numel()
            nested["compute_ms"] = ms_c / args.steps
            nested["reduce_scatter_ms"] = ms_r / args.steps
            nested["reduce_scatter_gbs_per_rank"] = full_c * (world - 1) / world / (ms_r / args.steps * 1e-3) / 1e9
            nested["limited_by"] = (f"the pair kernel on a rank's 1/{world} of K; NCCL's reduce-scatter of the "
                                    f"{full_c / 2**30:.2f} GiB partial C is {100.0 * ms_r / max(ms_c + ms_r, 1e-9):.0f} % "
                                    f"of a step")
        mk["step"]()
        nested["check"] = run_check(mk["check"], CHECK_TOL)
        if clocks_k:
            if clocks_k.get("sm_mhz"):
                clocks_k["ms_per_step_x_sm_mhz"] = ms_k / args.steps * clocks_k["sm_mhz"]
            nested["clocks"] = clocks_k

    # ---- launch-bound workloads: the same steps once more as a captured graph (tfb_ctx_capture_*),
    # which takes the host's per-call work out of the measurement; nested in `config.graph`
    graph_info = None
    if wl.get("graph_calls"):
        n_calls = int(wl["graph_calls"])
        ctx.synchronize()
        ctx.capture_begin()
        try:
            for _ in range(n_calls):
                step()
        finally:
            graph = ctx.capture_end()
        ms_g, _, _ = timed(graph.launch, warm=2)
        step_ms = ms_g / args.steps / n_calls
        graph_info = {"steps_per_graph": n_calls, "ms_per_step": step_ms,
                      "value": wl["work"] / (step_ms * 1e-3) / unit_scale, "unit": unit,
                      "check": run_check(wl.get("check"), wl.get("check_tol", CHECK_TOL)),
                      "note": "the timed steps replayed from one captured graph: device time without the host's enqueue work"}

    # ---- roofline of the dominant kernel: the same steps again with an event pair around every
    # launch (kept out of the timed region so that `value` carries no event overhead)
    ctx.profile_begin()
    for _ in range(args.steps):
        step()
    names = wl.get("kernels_any") or [wl["kernel"]]
    n_main, ms_main = 0, 0.0
    for nm in names:
        a, b = ctx.profile_read(nm)
        n_main, ms_main = n_main + a, ms_main + b
    extras = {nm: ctx.profile_read(nm) for nm in wl["extra_kernels"]}
    ctx.profile_end()
    scale = 1e12 if wl["bound"] == "tensor" else 1e9
    achieved = wl["per_launch"] / (ms_main / n_main * 1e-3) / scale if n_main else None
    roofline = {"bound": wl["bound"], "achieved": achieved, "unit": "TFLOP/s" if wl["bound"] == "tensor" else "GB/s"}
    if wl.get("tf32x3"):
        # f32 through 3xTF32: three MMAs per algorithmic MMA, so the relevant peak is a third of the
        # dense TF32 rate, measured here by the library's tcgen05 probe (MEASURED_PEAKS.json holds no
        # TF32 figure).  Two denominators: the burst rate of a cool GPU, and the rate the probe
        # sustains when launched back to back for seconds under the board's power limit - the one
        # that applies to a kernel timed inside a long step, as here.
        #
        # With the corrections as one bf16 MMA (the library's default, TFB_TC_BF16_CORRECTIONS) a k-step
        # costs the tensor pipe TWO MMAs' time - a bf16 MMA of K = 16 takes what a TF32 MMA of K = 8
        # takes - so the ceiling is HALF the TF32 rate and the fractions are quoted against that;
        # `frac_of_three_mma_form` is the same figure against the third, for comparison with numbers
        # taken before the bf16 form existed.
        mmas = 2.0 if int(os.environ.get("TFB_TC_BF16_CORRECTIONS", "1") or 0) != 0 else 3.0
        burst_tf32 = max(wl["tf32_cold"], ctx.probe_tf32_tflops())
        burst = burst_tf32 / mmas
        sustained_tf32 = None
        if args.sustained_seconds > 0 and rank == 0:
            sustained_tf32 = ctx.probe_tf32_tflops_sustained(args.sustained_seconds)
        sustained = sustained_tf32 / mmas if sustained_tf32 else None
        peak = sustained or burst
        share = "half" if mmas == 2.0 else "one third"
        roofline.update({
            "peak": peak, "frac": (achieved / peak) if achieved else None,
            "peak_burst": burst, "frac_burst": (achieved / burst) if achieved else None,
            "peak_sustained": sustained, "frac_sustained": (achieved / sustained) if (achieved and sustained) else None,
            "mma_per_k_step": int(mmas),
            "frac_of_three_mma_form": (achieved / ((sustained_tf32 or burst_tf32) / 3.0)) if achieved else None,
            "peak_source": (f"{share} of the dense TF32 rate of the library's tcgen05 probe on this GPU ({int(mmas)} MMAs' time per "
                            "k-step): `peak` is the "
                            f"sustained figure (probe launched back to back for {args.sustained_seconds:g} s, rate of "
                            "the last quarter), `peak_burst` the larger of a single probe before and one after the run")
            if sustained else
            (f"{share} of the dense TF32 rate of the library's tcgen05 probe on this GPU ({int(mmas)} MMAs' time per k-step; "
             "burst: the larger of a probe before and one after the run)")})
    else:
        peak = wl["peak"]()
        roofline.update({"peak": peak, "frac": (achieved / peak) if (achieved and peak) else None,
                         "peak_source": wl["peak_source"]})
    roofline.update({
        "traffic": wl.get("traffic"), "kernel": wl["kernel_label"], "launches": n_main,
        "avg_launch_us": ms_main / max(n_main, 1) * 1e3,
        "other_kernels": {k: {"launches": v[0], "avg_us": v[1] / max(v[0], 1) * 1e3} for k, v in extras.items()}})

    # ---- end to end through the public API from pinned host memory
    e2e = None
    if wl["e2e_step"] is not None:
        ms_e2e, _, _ = timed(wl["e2e_step"], warm=2)
        e2e = {"value": wl["work"] * args.steps / (ms_e2e * 1e-3) / unit_scale, "unit": unit,
               "h2d_bytes_per_step": wl["h2d"], "d2h_bytes_per_step": wl["d2h"], "ms_per_step": ms_e2e / args.steps,
               "h2d_gbs": wl["h2d"] / (ms_e2e / args.steps * 1e-3) / 1e9}
        if args.workload == "dense":
            e2e["check"] = run_check(modes["k" if world > 1 else "i"]["check"], CHECK_TOL)

    if sampler:
        sampler.stop()
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(args)

    failed = [c for c in (check, (nested or {}).get("check"), (e2e or {}).get("check"), (graph_info or {}).get("check"))
              if c and not c["ok"]]
    if rank == 0:
        config = {"workload": workload_name}
        config.update(wl["config"])
        config["deterministic_rerun"] = deterministic
        if nested:
            config[nested_key] = nested
        if graph_info:
            config["graph"] = graph_info
        print(json.dumps({
            "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": dtype_name, "data": "synthetic",
            "config": config, "check": check, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
            "roofline": roofline, "cpu_baseline": cpu,
        }))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if failed:
        raise SystemExit(f"result check failed: {failed}")


if __name__ == "__main__":
    main()
