#!/usr/bin/env python
"""Benchmark of the contraction hot path.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun)
    python bench.py --impl reference ...                     (the CPU path on the host cores)

Default workload: the MPS transfer-matrix chain - 32 sites, each tensor chi x d x chi with
chi = 512, d = 2, complex128, Re/Im ~ N(0, 1/chi); the left environment E (chi x chi) is
contracted with A and conj(A) site by site as 'ab,asc,bsd->cd' through the contraction tree.
One step = one pass over the 32-site chain (64 dependent contractions, 137.4 GFLOP).

The metric is einsum GFLOP/s (algorithmic: 8 flop per complex multiply-add).  `value` is
measured with inputs resident in HBM; `e2e` through the public API from pinned host buffers
with the host<->device copies inside the timed region.  The chain does not shard (64
dependent steps on 512 x 512 outputs), so N GPUs run N independent replicas.
"""
from __future__ import annotations

import argparse
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
METRIC = "einsum GFLOP/s (MPS transfer-matrix chain, complex128)"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--sites", type=int, default=32)
    ap.add_argument("--chi", type=int, default=512)
    ap.add_argument("--phys", type=int, default=2)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="target length of the CPU-baseline sample")
    return ap.parse_args()


def chain_flops(chi: int, d: int, sites: int) -> float:
    # per site two contractions of chi * chi * (d chi) complex multiply-adds, 8 flop each
    return sites * 2 * 8.0 * chi * chi * (d * chi)


def site_tensor(seed: int, chi: int, d: int) -> np.ndarray:
    from oracle import oracle

    return oracle.normal(seed, (chi, d, chi), np.complex128, scale=(1.0 / chi) ** 0.5)


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
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(smax)), "power_w_max": float(max(power)),
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


def cpu_baseline(chi: int, d: int, target_seconds: float):
    """Time the CPU path on a bounded sample of the chain (whole sites, >= 1)."""
    cores = os.cpu_count() or 1
    env = np.eye(chi, dtype=np.complex128)
    a0 = site_tensor(2000, chi, d)
    cpu_chain(env, [a0])  # warm the BLAS threads
    t0 = time.perf_counter()
    cpu_chain(env, [a0])
    one = time.perf_counter() - t0
    n = int(max(1, min(32, target_seconds / max(one, 1e-6))))
    sites = [site_tensor(2000 + s, chi, d) for s in range(min(n, 4))]
    t0 = time.perf_counter()
    done = 0
    while done < n:
        env = cpu_chain(env, sites[: min(len(sites), n - done)])
        done += min(len(sites), n - done)
    dt = time.perf_counter() - t0
    return {"value": chain_flops(chi, d, n) / dt / 1e9, "unit": "GFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{n} of the chain's sites (chi={chi}, d={d}) through numpy/OpenBLAS permute+GEMM, "
                      f"{dt:.1f} s"}


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
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "c128 (f64 arithmetic)", "data": "synthetic",
        "config": {"workload": f"MPS transfer-matrix chain, chi={chi}, d={d}, complex128; each step is a bounded "
                               f"sample of {sample_sites} sites", "sites_per_step": sample_sites},
        "cpu_baseline": {"value": value, "unit": "GFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"{sample_sites} sites per step on numpy/OpenBLAS with {cores} threads"},
        "e2e": {"value": value, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


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
        if args.gpus != 1 or world != 1:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")

    import ctypes as C

    import torch
    import tenferro_b200 as tb

    dist = None
    if world > 1:
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    chi, d, sites = args.chi, args.phys, args.sites
    space = tb.LogicalMemorySpace.GpuMemory(local_rank)
    ctx = tb.Context.get(local_rank)
    flops_step = chain_flops(chi, d, sites)
    site_bytes = chi * d * chi * 16
    env_bytes = chi * chi * 16

    # Inputs: pinned host copies (for the end-to-end leg) and resident device tensors.  Each rank
    # (replica) draws its own chain: seed = 2000 + 100 * rank + site.
    host_sites_ptr = ctx.host_alloc(site_bytes * sites)
    host_env_ptr = ctx.host_alloc(env_bytes)
    host_out_ptr = ctx.host_alloc(env_bytes)
    host_sites = np.ctypeslib.as_array((C.c_char * (site_bytes * sites)).from_address(host_sites_ptr)).view(
        np.complex128).reshape(sites, chi * d * chi)
    host_env = np.ctypeslib.as_array((C.c_char * env_bytes).from_address(host_env_ptr)).view(np.complex128)
    host_out = np.ctypeslib.as_array((C.c_char * env_bytes).from_address(host_out_ptr)).view(np.complex128)
    for s in range(sites):
        host_sites[s] = site_tensor(2000 + 100 * rank + s, chi, d).reshape(-1, order="F")
    host_env[:] = np.eye(chi, dtype=np.complex128).reshape(-1, order="F")

    dev_sites = [tb.Tensor.empty([chi, d, chi], np.complex128, space) for _ in range(sites)]
    dev_env0 = tb.Tensor.empty([chi, chi], np.complex128, space)
    envs = [tb.Tensor.empty([chi, chi], np.complex128, space) for _ in range(2)]

    def upload():
        for s in range(sites):
            ctx.h2d(dev_sites[s]._block.ptr, C.c_void_p(host_sites_ptr + s * site_bytes), site_bytes)
        ctx.h2d(dev_env0._block.ptr, C.c_void_p(host_env_ptr), env_bytes)

    upload()
    ctx.synchronize()

    tree = tb.ContractionTree.optimize(tb.Subscripts.parse(CHAIN), [[chi, chi], [chi, d, chi], [chi, d, chi]])
    # One prepared call per site: E_{s+1} = einsum(E_s, A_s, conj(A_s)); conj is a view flag
    # folded into the operand loads, nothing is materialised.
    calls = []
    for s in range(sites):
        src = dev_env0 if s == 0 else envs[(s - 1) % 2]
        dst = envs[s % 2]
        calls.append(tb.PreparedEinsum(tree, [src, dev_sites[s], dev_sites[s].into_conj()], dst))
    final_env = envs[(sites - 1) % 2]

    def chain_step():
        for c in calls:
            c.run()

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
    for _ in range(max(args.warmup, 3)):
        chain_step()
    barrier()
    sampler = ClockSampler(visible_gpu_index(local_rank)) if rank == 0 else None
    if sampler:
        sampler.start()
    launches0 = ctx.kernel_launch_count()
    barrier()
    e0 = ctx.record_event()
    for _ in range(args.steps):
        chain_step()
    e1 = ctx.record_event()
    barrier()
    ms_total = max_over_ranks(e0.elapsed_ms(e1))
    launches = ctx.kernel_launch_count() - launches0
    clocks = sampler.stop() if sampler else None
    value = flops_step * args.steps * world / (ms_total * 1e-3) / 1e9

    # ---- parity guard on the timed configuration: the environment the timed steps produced is
    # reproduced bit for bit by one more pass (the kernels are run-to-run deterministic)
    ctx.d2h(C.c_void_p(host_out_ptr), final_env._block.ptr + 0, env_bytes)
    ctx.synchronize()
    first = host_out.copy()
    chain_step()
    ctx.d2h(C.c_void_p(host_out_ptr), final_env._block.ptr + 0, env_bytes)
    ctx.synchronize()
    deterministic = bool(np.array_equal(first, host_out))

    # ---- roofline of the dominant kernel: the same steps again with an event pair around every
    # launch (kept out of the timed region so that `value` carries no event overhead)
    ctx.profile_begin()
    for _ in range(args.steps):
        chain_step()
    n_main, ms_main = ctx.profile_read("contract_dmma")
    n_fix, ms_fix = ctx.profile_read("contract_dmma_fixup")
    ctx.profile_end()
    flops_launch = 8.0 * chi * chi * (d * chi)
    achieved = flops_launch / (ms_main / max(n_main, 1) * 1e-3) / 1e12 if n_main else None
    peak = ctx.probe_fp64_tflops()
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
        "frac": (achieved / peak) if (achieved and peak) else None, "traffic": None,
        "kernel": "contract_dmma_kernel (complex128, 64x64x8 tiles)",
        "peak_source": "measured on this GPU by the library's register-resident DMMA probe "
                       "(MEASURED_PEAKS.json holds no FP64 figure)",
        "launches": n_main, "avg_launch_us": ms_main / max(n_main, 1) * 1e3,
        "fixup_launches": n_fix, "fixup_avg_us": ms_fix / max(n_fix, 1) * 1e3,
    }

    # ---- end to end: every step copies its inputs from pinned host memory, runs the chain
    # through the public API and reads the final environment back
    def e2e_step():
        upload()
        chain_step()
        ctx.d2h(C.c_void_p(host_out_ptr), final_env._block.ptr + 0, env_bytes)
        ctx.synchronize()

    for _ in range(2):
        e2e_step()
    barrier()
    t0 = ctx.record_event()
    for _ in range(args.steps):
        e2e_step()
    t1 = ctx.record_event()
    barrier()
    ms_e2e = max_over_ranks(t0.elapsed_ms(t1))
    e2e = {"value": flops_step * args.steps * world / (ms_e2e * 1e-3) / 1e9, "unit": "GFLOP/s",
           "h2d_bytes_per_step": site_bytes * sites + env_bytes, "d2h_bytes_per_step": env_bytes,
           "ms_per_step": ms_e2e / args.steps}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(chi, d, args.cpu_seconds)

    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "c128 (f64 arithmetic)", "data": "synthetic",
            "config": {"workload": f"MPS transfer-matrix chain: {sites} sites, chi={chi}, d={d}, complex128, "
                                   f"'{CHAIN}' per site via the contraction tree",
                       "flop_per_step": flops_step, "parallelism": f"{world} independent replica(s)",
                       "l2": f"inputs larger than L2: each pass streams {sites * site_bytes >> 20} MiB of site tensors",
                       "tree_pairs": tree.pairs, "deterministic_rerun": deterministic},
            "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
        }))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
