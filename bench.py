#!/usr/bin/env python
"""Benchmark of the contraction hot path.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun)
    python bench.py --impl reference ...                     (the CPU path on the host cores)

Default workload `chain`: the MPS transfer-matrix chain - 32 sites, each tensor chi x d x chi
with chi = 512, d = 2, complex128, Re/Im ~ N(0, 1/chi); the left environment E (chi x chi) is
contracted with A and conj(A) site by site as 'ab,asc,bsd->cd' through the contraction tree.
One step = one pass over the 32-site chain (64 dependent contractions, 137.4 GFLOP).  It does
not shard (64 dependent steps on 512 x 512 outputs): N GPUs run N independent replicas.

Other workloads (`--workload`): `dense` ('ijkl,klmn->ijmn', f32 3xTF32, i=j=m=n=128, k=l=256;
`--shard i` splits a free index with no communication, `--shard k` splits the contracted pair
and reduce-scatters the partial outputs over NCCL), `grouped` (4096 ragged f32 products, table
sharded over the ranks), `network4` ('ijk,jlm,kmn,lnp->ip', complex64, dim 96), `abc_bcd`
('abc,bcd->ad', f64, dim 64), `permute` and `reduce` (bandwidth).

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


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="chain",
                    choices=["chain", "dense", "grouped", "network4", "abc_bcd", "permute", "reduce"])
    ap.add_argument("--sites", type=int, default=32)
    ap.add_argument("--chi", type=int, default=512)
    ap.add_argument("--phys", type=int, default=2)
    ap.add_argument("--shard", default="i", choices=["i", "k"], help="dense: free-index or contracted-index sharding")
    ap.add_argument("--scale", type=float, default=1.0, help="dense/network4/permute: scale the index extents")
    ap.add_argument("--problems", type=int, default=4096, help="grouped: number of problems")
    ap.add_argument("--case", default="transpose2d", help="permute/reduce: which member of the set")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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


# ------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi every 200 ms while the timed region runs."""

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
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        for line in self.lines:
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


def visible_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        parts = [p for p in vis.split(",") if p.strip()]
        if local_rank < len(parts) and parts[local_rank].strip().isdigit():
            return int(parts[local_rank])
    return local_rank


# ------------------------------------------------------------------------------------------
# CPU path (the oracle's TTGT restatement on OpenBLAS): baseline leg and --impl reference
# ------------------------------------------------------------------------------------------
def cpu_chain(env: np.ndarray, sites) -> np.ndarray:
    from oracle import oracle

    for a in sites:
        t = oracle.ttgt_contract([0, 1], env, [0, 2, 3], a, [1, 2, 3])          # ab,asc->bsc
        env = oracle.ttgt_contract([1, 2, 3], t, [1, 2, 4], np.conj(a), [3, 4])  # bsc,bsd->cd
    return env


def cpu_baseline_chain(chi: int, d: int, target_seconds: float):
    """Time the CPU path on a bounded sample of the chain: whole sites, repeated until about
    `target_seconds` of CPU work are done."""
    cores = os.cpu_count() or 1
    env = np.eye(chi, dtype=np.complex128)
    sites = [site_tensor(2000 + s, chi, d) for s in range(4)]
    cpu_chain(env, sites[:1])  # warm the BLAS threads
    t0 = time.perf_counter()
    cpu_chain(env, sites[:1])
    one = time.perf_counter() - t0
    n = int(max(4, min(4096, target_seconds / max(one, 1e-6))))
    t0 = time.perf_counter()
    done = 0
    while done < n:
        take = min(len(sites), n - done)
        env = cpu_chain(np.eye(chi, dtype=np.complex128), sites[:take])
        done += take
    dt = time.perf_counter() - t0
    return {"value": chain_flops(chi, d, n) / dt / 1e9, "unit": "GFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{n} site contractions of the chain (chi={chi}, d={d}; 4 distinct site tensors cycled) through "
                      f"numpy/OpenBLAS permute+GEMM, {dt:.1f} s"}


def cpu_baseline_einsum(notation, arrays, flops, target_seconds: float):
    from oracle import oracle

    cores = os.cpu_count() or 1
    ins, out = oracle.parse_notation(notation)
    run = lambda: np.einsum(*[x for pair in zip(arrays, ins) for x in pair], out, optimize=True)
    run()
    t0 = time.perf_counter()
    run()
    one = time.perf_counter() - t0
    n = int(max(1, min(200, target_seconds / max(one, 1e-6))))
    t0 = time.perf_counter()
    for _ in range(n):
        run()
    dt = time.perf_counter() - t0
    return {"value": flops * n / dt / 1e9, "unit": "GFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{n} x numpy.einsum('{notation}', optimize=True) on OpenBLAS, {dt:.1f} s"}


def run_reference(args, rank: int):
    """--impl reference: the reference's own CPU implementation cannot be built or run here (no
    Rust toolchain, bodies are todo!()), so this arm times the oracle's CPU port."""
    if rank != 0:
        return
    chi, d = args.chi, args.phys
    sample_sites = 2
    sites = [site_tensor(2000 + s, chi, d) for s in range(sample_sites)]
    env = np.eye(chi, dtype=np.complex128)
    for _ in range(args.warmup):
        cpu_chain(env, sites)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_chain(env, sites)
    dt = time.perf_counter() - t0
    flops = chain_flops(chi, d, sample_sites) * args.steps
    value = flops / dt / 1e9
    cores = os.cpu_count() or 1
    print(json.dumps({
        "impl": "reference", "metric": CHAIN_METRIC, "value": value, "unit": "GFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "c128 (f64 arithmetic)", "data": "synthetic",
        "config": {"workload": f"MPS transfer-matrix chain, chi={chi}, d={d}, complex128; each step is a bounded "
                               f"sample of {sample_sites} sites", "sites_per_step": sample_sites},
        "cpu_baseline": {"value": value, "unit": "GFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"{sample_sites} sites per step on numpy/OpenBLAS with {cores} threads"},
        "e2e": {"value": value, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------------------
# Workloads.  Each returns a dict:
#   step()            enqueue one step on the context's stream (inputs resident)
#   work              algorithmic flops (or bytes) of one step, summed over all ranks' shares
#   e2e_step()        one step from pinned host inputs to a host-visible result (or None)
#   h2d, d2h          bytes copied per e2e step
#   kernel, per_launch, bound, peak(), peak_source     roofline of the dominant kernel
# ------------------------------------------------------------------------------------------
class Env:
    def __init__(self, args, tb, ctx, rank, local_rank, world, dist, torch):
        self.args, self.tb, self.ctx = args, tb, ctx
        self.rank, self.local_rank, self.world, self.dist, self.torch = rank, local_rank, world, dist, torch
        self.space = tb.LogicalMemorySpace.GpuMemory(local_rank)
        self.peaks = load_peaks()


def pinned(ctx, nbytes, dtype):
    ptr = ctx.host_alloc(nbytes)
    arr = np.ctypeslib.as_array((C.c_char * nbytes).from_address(ptr)).view(dtype)
    return ptr, arr


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

    # End to end: the site tensors travel host -> device on a second stream, one event per site,
    # and each site's contraction waits only for its own tensor, so the copies of later sites
    # hide behind the contractions of earlier ones.
    copy_stream = env.torch.cuda.Stream(device=env.local_rank)
    compute_stream = env.torch.cuda.current_stream()

    def e2e_step():
        ctx.set_stream(copy_stream.cuda_stream)
        ctx.h2d(dev_env0._block.ptr, C.c_void_p(he_ptr), env_bytes)
        events = []
        for s in range(sites):
            ctx.h2d(dev_sites[s]._block.ptr, C.c_void_p(hs_ptr + s * site_bytes), site_bytes)
            events.append(ctx.record_event())
        ctx.set_stream(compute_stream.cuda_stream)
        for s in range(sites):
            ctx.wait_event(events[s])
            calls[s].run()
        ctx.d2h(C.c_void_p(ho_ptr), final_env._block.ptr, env_bytes)
        ctx.synchronize()

    return {
        "metric": CHAIN_METRIC, "unit": "GFLOP/s", "dtype": "c128 (f64 arithmetic)", "scaling": "weak",
        "step": step, "work": chain_flops(chi, d, sites) * env.world, "read_result": read_result,
        "e2e_step": e2e_step, "h2d": site_bytes * sites + env_bytes, "d2h": env_bytes,
        "kernel": "contract_dmma", "kernel_label": "contract_dmma_kernel (complex128, 64x64x16 tiles, m16n8k8 DMMA)",
        "per_launch": 8.0 * chi * chi * (d * chi), "bound": "tensor", "peak": ctx.probe_fp64_tflops,
        "peak_source": "measured on this GPU by the library's register-resident DMMA probe "
                       "(MEASURED_PEAKS.json holds no FP64 figure)",
        "extra_kernels": ["contract_dmma_fixup"],
        # dram__bytes_read + dram__bytes_write per launch from the ncu capture summarised in
        # profiles/contract_dmma_c128_mps_chain.md (12.6 and 16.8 MB on the two captured launches)
        "traffic": 14.74e6 if (chi, d) == (512, 2) else None,
        "config": {"workload": f"MPS transfer-matrix chain: {sites} sites, chi={chi}, d={d}, complex128, '{CHAIN}' "
                               f"per site via the contraction tree",
                   "parallelism": f"{env.world} independent replica(s)",
                   "l2": f"inputs larger than L2: each pass streams {sites * site_bytes >> 20} MiB of site tensors",
                   "tree_pairs": tree.pairs},
        "cpu": lambda: cpu_baseline_chain(chi, d, args.cpu_seconds),
    }


def wl_dense(env: Env):
    """'ijkl,klmn->ijmn', f32, N(0,1).  Strong scaling: the ranks split one contraction."""
    from tenferro_b200 import sharding

    args, tb, ctx, torch = env.args, env.tb, env.ctx, env.torch
    e = lambda x: max(4, int(round(x * args.scale / 4)) * 4)
    i = j = m = n = e(128)
    k = l = e(256)
    W, r = env.world, env.rank
    dev = torch.device("cuda", env.local_rank)
    gen = torch.Generator(device=dev)
    gen.manual_seed(5000)
    # Column-major tensors = torch tensors with reversed dims.  Every rank holds the full A and B
    # (same seed) and contracts a strided sub-view of them.
    a_t = torch.randn((l, k, j, i), generator=gen, device=dev, dtype=torch.float32)
    gen.manual_seed(5001)
    b_t = torch.randn((n, m, l, k), generator=gen, device=dev, dtype=torch.float32)
    wrap = lambda t, dims: tb.Tensor.from_device_pointer(t.data_ptr(), t.numel() * 4, dims, np.float32, env.space, t)
    A, B = wrap(a_t, [i, j, k, l]), wrap(b_t, [k, l, m, n])
    notation = "ijkl,klmn->ijmn"
    if args.shard == "i" or W == 1:
        if i % W:
            raise SystemExit("i must divide by the number of GPUs")
        c_t = torch.zeros((n, m, j, i), device=dev, dtype=torch.float32)
        Cfull = wrap(c_t, [i, j, m, n])
        view = lambda T, axis: tb.Tensor(T._block, *sharding.shard_view(T.dims(), T.strides(), 0, axis, W, r),
                                         np.float32, env.space)
        As, Cs = view(A, 0), view(Cfull, 0)
        tree = tb.ContractionTree.optimize(tb.Subscripts.parse(notation), [As.dims(), B.dims()])
        call = tb.PreparedEinsum(tree, [As, B], Cs)
        step = call.run
        mode = f"free index i split {W} ways, no communication"
        result_t, keep = c_t, (a_t, b_t, c_t)
    else:
        if l % W:
            raise SystemExit("l must divide by the number of GPUs")
        part_t = torch.zeros((n, m, j, i), device=dev, dtype=torch.float32)
        out_t = torch.zeros((n * m * j * i) // W, device=dev, dtype=torch.float32)
        P = wrap(part_t, [i, j, m, n])
        view = lambda T, axis: tb.Tensor(T._block, *sharding.shard_view(T.dims(), T.strides(), 0, axis, W, r),
                                         np.float32, env.space)
        As, Bs = view(A, 3), view(B, 1)
        tree = tb.ContractionTree.optimize(tb.Subscripts.parse(notation), [As.dims(), Bs.dims()])
        call = tb.PreparedEinsum(tree, [As, Bs], P)

        def step():
            call.run()
            env.dist.reduce_scatter_tensor(out_t, part_t.view(-1), op=env.dist.ReduceOp.SUM)

        mode = f"contracted pair (k,l) split {W} ways on l, partial outputs reduce-scattered over NCCL"
        result_t, keep = out_t, (a_t, b_t, part_t, out_t)
    flops = 2.0 * i * j * m * n * k * l
    # The probe runs once before the workload (cool GPU) and once after (under the power cap the
    # clock has dropped by then); the larger figure is the denominator.
    tf32_cold = ctx.probe_tf32_tflops()
    tf32 = lambda: max(tf32_cold, ctx.probe_tf32_tflops())

    def read_result():
        ctx.synchronize()
        return result_t.flatten()[:4096].cpu().numpy()

    return {
        "metric": "einsum GFLOP/s ('ijkl,klmn->ijmn', f32 via 3xTF32)", "unit": "GFLOP/s", "dtype": "f32 (3xTF32)",
        "scaling": "strong", "step": step, "work": flops, "read_result": read_result, "e2e_step": None, "h2d": 0, "d2h": 0,
        "kernel": "contract_tf32x3",
        "kernel_label": "contract_tf32x3_pair_kernel (tcgen05 cta_group::2, 256x256 tiles per CTA pair, 32-deep stages)",
        "per_launch": flops / W, "bound": "tensor", "peak": lambda: tf32() / 3.0,
        "peak_source": "one third of the dense TF32 rate measured on this GPU by the library's tcgen05 probe (three "
                       "MMAs per algorithmic MMA), the larger of a probe before and one after the run; MEASURED_PEAKS.json "
                       "holds no TF32 figure",
        "extra_kernels": [], "keep": keep,
        "config": {"workload": f"'{notation}' f32, i=j=m=n={i}, k=l={k}, N(0,1)", "parallelism": mode,
                   "l2": f"inputs larger than L2: A and B hold {(a_t.numel() + b_t.numel()) * 4 >> 20} MiB",
                   "flop_total": flops},
        "cpu": None,
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
    probs, oa, ob, oc = [], 0, 0, 0
    for (pi, pj, pk) in mine:
        pi, pj, pk = int(pi), int(pj), int(pk)
        probs.append((pi, pk, pj, a_t.data_ptr() + 4 * oa, 1, pi, b_t.data_ptr() + 4 * ob, 1, pj,
                      c_t.data_ptr() + 4 * oc, 1, pi))
        oa, ob, oc = oa + pi * pj, ob + pj * pk, oc + pi * pk
    flops_all = float((2.0 * table[:, 0] * table[:, 1] * table[:, 2]).sum())
    bytes_all = float(bytes_p.sum())

    from tenferro_b200.prims import PreparedGroupedGemm

    call = PreparedGroupedGemm(probs, np.float32, 1.0, 0.0, ctx)
    step = call.run

    def read_result():
        ctx.synchronize()
        return c_t[:4096].cpu().numpy()

    hbm = (env.peaks or {}).get("hbm_gbs")
    return {
        "metric": "einsum GFLOP/s (grouped 'bij,bjk->bik', f32, ragged)", "unit": "GFLOP/s", "dtype": "f32",
        "scaling": "strong", "step": step, "work": flops_all, "read_result": read_result, "e2e_step": None, "h2d": 0,
        "d2h": 0, "kernel": "grouped_tf32x3", "kernels_any": ["grouped_fma", "grouped_tf32x3", "grouped_simt"],
        "kernel_label": "grouped_f32_kernel (persistent CTAs, host-built stage table, double-buffered cp.async panels)",
        "per_launch": float(bytes_p[lo:hi].sum()), "bound": "hbm",
        "peak": (lambda: hbm) if hbm else ctx.probe_hbm_gbs,
        "peak_source": "MEASURED_PEAKS.json hbm_gbs" if hbm else "library copy probe (MEASURED_PEAKS.json absent)",
        "extra_kernels": [], "keep": (a_t, b_t, c_t),
        # profiles/grouped_tf32x3_ragged_4096.md: 121.8 MB read + 25.5 MB written
        "traffic": 147.3e6 if (args.problems == 4096 and env.world == 1) else None,
        "config": {"workload": f"{args.problems} problems 'ij,jk->ik', dims drawn from {{16,32,64,128}} (seed 3000), "
                               f"U(-1,1), f32", "parallelism": f"problem table split {env.world} ways by bytes",
                   "l2": f"inputs larger than L2: {bytes_all / 2**20:.0f} MiB touched per step",
                   "bytes_total": bytes_all, "flop_total": flops_all},
        "cpu": None,
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

    return {
        "metric": "einsum GFLOP/s ('ijk,jlm,kmn,lnp->ip', complex64)", "unit": "GFLOP/s", "dtype": "c64 (f32 arithmetic)",
        "scaling": "weak", "step": call.run, "work": flops * env.world, "read_result": read_result, "e2e_step": None,
        "h2d": 0, "d2h": 0, "kernel": "contract_tf32x3",
        "kernel_label": "contract_tf32x3 kernels (tcgen05; complex64 as one real product of doubled extents per tree node)",
        "per_launch": flops / 3.0, "bound": "tensor", "peak": lambda: max(tf32_cold, ctx.probe_tf32_tflops()) / 3.0,
        "peak_source": "one third of the library's dense TF32 probe: a complex multiply-add (8 flop) costs four real "
                       "ones, each three TF32 MMAs (24 TF32 flop)",
        "extra_kernels": ["pack_planes", "contract_tf32x3_finish"],
        # ncu, per launch averaged over the three product launches of a call: the two large nodes moved
        # 667 MB and 703 MB (profiles/contract_tf32x3_shortk_network4_c64.md); the third, whose operands
        # (two 7 MB tensors) stay in L2, was not captured and is counted as zero
        "traffic": (667.2e6 + 703.2e6) / 3.0 if dim == 96 else None,
        "config": {"workload": f"'{notation}' complex64, every index {dim}, N(0,1) parts; tree {tree.pairs}",
                   "parallelism": f"{env.world} independent replica(s)",
                   "l2": f"intermediates of {dim ** 4 * 8 >> 20} MiB exceed L2" if dim >= 64 else "L2-resident (scaled down)",
                   "flop_total": flops},
        "cpu": (lambda: cpu_baseline_einsum(notation, arrays, flops, args.cpu_seconds)) if dim <= 48 else None,
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
    return {
        "metric": "einsum GFLOP/s ('abc,bcd->ad', f64, dims 64)", "unit": "GFLOP/s", "dtype": "f64", "scaling": "weak",
        "step": call.run, "work": flops * env.world, "read_result": out.to_numpy, "e2e_step": None, "h2d": 0, "d2h": 0,
        "kernel": "contract_dmma", "kernel_label": "contract_dmma_kernel (f64, 64x64x16 tiles, split over K)",
        "per_launch": flops, "bound": "tensor", "peak": ctx.probe_fp64_tflops,
        "peak_source": "library DMMA probe", "extra_kernels": ["contract_dmma_fixup"],
        "config": {"workload": f"'{notation}' f64, a=b=c=d=64, N(0,1)", "parallelism": f"{env.world} replica(s)",
                   "l2": "L2-resident by construction (4 MiB of operands): a latency measurement",
                   "flop_total": flops},
        "cpu": lambda: cpu_baseline_einsum(notation, [a, b], flops, min(args.cpu_seconds, 5.0)),
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
    kernel = {"permute": "permute_tiled"}.get(plan.kernel_name, "permute_tiled")
    # which of the three permute kernels ran is not reported by the plan; time all of them
    hbm = (env.peaks or {}).get("hbm_gbs")
    bytes_step = 2.0 * n * itemsize

    def read_result():
        ctx.synchronize()
        return dst_t[:4096].cpu().numpy()

    return {
        "metric": f"permute GB/s ({args.case})", "unit": "GB/s", "dtype": np.dtype(dtype).name, "scaling": "weak",
        "step": step, "work": bytes_step * env.world, "read_result": read_result, "e2e_step": None, "h2d": 0, "d2h": 0,
        "kernel": kernel, "kernel_label": "permute kernel (rows / tiled transpose / generic, whichever the layout selects)",
        "kernels_any": ["permute_rows", "permute_tiled", "permute_generic"],
        "per_launch": bytes_step, "bound": "hbm", "peak": (lambda: hbm) if hbm else ctx.probe_hbm_gbs,
        "peak_source": "MEASURED_PEAKS.json hbm_gbs" if hbm else "library copy probe (MEASURED_PEAKS.json absent)",
        "extra_kernels": [], "keep": (src_t, dst_t),
        # profiles/permute_tiled_vec_transpose2d_f32.md: 1.074 GB read + 1.031 GB written
        "traffic": 2.105e9 if (args.case == "transpose2d" and args.scale == 1.0) else None,
        "config": {"workload": f"permute {list(shape)} {np.dtype(dtype).name} by {list(perm)}",
                   "parallelism": f"{env.world} replica(s)",
                   "l2": "inputs larger than L2" if n * itemsize > 200e6 else "fits L2 (small member of the set)",
                   "bytes_total": bytes_step},
        "cpu": None,
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

    return {
        "metric": f"reduce GB/s ({args.case})", "unit": "GB/s", "dtype": np.dtype(dtype).name, "scaling": "weak",
        "step": step, "work": bytes_step * env.world, "read_result": read_result, "e2e_step": None, "h2d": 0, "d2h": 0,
        "kernel": "reduce", "kernel_label": "reduce_kernel", "per_launch": bytes_step, "bound": "hbm",
        "peak": (lambda: hbm) if hbm else ctx.probe_hbm_gbs,
        "peak_source": "MEASURED_PEAKS.json hbm_gbs" if hbm else "library copy probe (MEASURED_PEAKS.json absent)",
        "extra_kernels": ["reduce_finish"], "keep": (src_t, dst_t),
        # profiles/reduce_sum_axis0_f32.md: 1.076 GB read + 19.4 MB written
        "traffic": 1.095e9 if args.case == "sum_axis0" else None,
        "config": {"workload": f"reduce {list(shape)} {np.dtype(dtype).name} keeping modes {kept}, op {op}",
                   "parallelism": f"{env.world} replica(s)", "l2": "inputs larger than L2", "bytes_total": bytes_step},
        "cpu": None,
    }


WORKLOADS = {"chain": wl_chain, "dense": wl_dense, "grouped": wl_grouped, "network4": wl_network4,
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
    wl = WORKLOADS[args.workload](env)
    step = wl["step"]
    unit_scale = 1e9  # GFLOP/s and GB/s alike

    def barrier():
        ctx.synchronize()
        if dist is not None:
            dist.barrier()
        ctx.synchronize()

    def max_over_ranks(ms: float) -> float:
        if dist is None:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- warm-up, then the timed region: K steps, inputs resident in HBM
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    barrier()
    sampler = ClockSampler(visible_gpu_index(local_rank)) if rank == 0 else None
    if sampler:
        sampler.start()
    launches0 = ctx.kernel_launch_count()
    barrier()
    e0 = ctx.record_event()
    for _ in range(args.steps):
        step()
    e1 = ctx.record_event()
    barrier()
    ms_total = max_over_ranks(e0.elapsed_ms(e1))
    launches = ctx.kernel_launch_count() - launches0
    clocks = sampler.stop() if sampler else None
    value = wl["work"] * args.steps / (ms_total * 1e-3) / unit_scale

    # ---- the kernels are run-to-run deterministic: one more step reproduces the result bit for bit
    first = wl["read_result"]()
    step()
    deterministic = bool(np.array_equal(first, wl["read_result"]()))

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
    peak = wl["peak"]()
    scale = 1e12 if wl["bound"] == "tensor" else 1e9
    achieved = wl["per_launch"] / (ms_main / n_main * 1e-3) / scale if n_main else None
    roofline = {
        "bound": wl["bound"], "achieved": achieved, "peak": peak, "unit": "TFLOP/s" if wl["bound"] == "tensor" else "GB/s",
        "frac": (achieved / peak) if (achieved and peak) else None, "traffic": wl.get("traffic"),
        "kernel": wl["kernel_label"], "peak_source": wl["peak_source"], "launches": n_main,
        "avg_launch_us": ms_main / max(n_main, 1) * 1e3,
        "other_kernels": {k: {"launches": v[0], "avg_us": v[1] / max(v[0], 1) * 1e3} for k, v in extras.items()},
    }

    # ---- end to end through the public API from pinned host memory
    e2e = None
    if wl["e2e_step"] is not None:
        for _ in range(2):
            wl["e2e_step"]()
        barrier()
        t0 = ctx.record_event()
        for _ in range(args.steps):
            wl["e2e_step"]()
        t1 = ctx.record_event()
        barrier()
        ms_e2e = max_over_ranks(t0.elapsed_ms(t1))
        e2e = {"value": wl["work"] * args.steps / (ms_e2e * 1e-3) / unit_scale, "unit": wl["unit"],
               "h2d_bytes_per_step": wl["h2d"], "d2h_bytes_per_step": wl["d2h"], "ms_per_step": ms_e2e / args.steps}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and wl["cpu"] is not None:
        cpu = wl["cpu"]()

    if rank == 0:
        config = dict(wl["config"])
        config["deterministic_rerun"] = deterministic
        print(json.dumps({
            "metric": wl["metric"], "value": value, "unit": wl["unit"], "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": wl["scaling"], "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
            "config": config, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline,
            "cpu_baseline": cpu,
        }))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
