#!/usr/bin/env python
"""Benchmark of the Hyrax commitment hot path: MSM points/s on one LLaMA-2-7B-shaped layer, and the
proof time per layer of the same model shape.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

One step commits the seven weight matrices of one decoder layer (4 x 4096x4096, 2 x 11008x4096,
1 x 4096x11008, int16-range entries held as int32, flattened into rows of 4096 scalars over 4096
generators): 49 408 row commitments, 202 375 168 (scalar, generator) pairs.  With N > 1 the rows of
that ONE layer are dealt to the ranks in contiguous blocks, every rank commits its block and one NCCL
all-gather hands every rank all the commitments (strong scaling; the time includes the gather).  The
line also carries `layer_proof`: every rank proves its own batch of four decoder layers (seq 2048), the
second half of the headline metric.  Rank 0 prints one JSON line.

--impl reference times the reference's own commit kernels (its unmodified sources built into
oracle/_ref) on the same workload; it never loads this repository's library.
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
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WD = 4096                      # scalars (= generators) per commitment row
SEED = 0xC4
LAYER_PAIRS = 4 * 4096 * 4096 + 3 * 4096 * 11008   # elements of the seven weight matrices of one layer
MUL_INSTR_PER_FIELD_MUL = 264  # 8-limb Montgomery product: 128 lo/hi multiply-add pairs + 8 single multiplies
MUL_INSTR_PER_FIELD_SQR = 208  # dedicated squaring: 100 pairs + 8
FIELD_MUL_PER_ADD = 10         # mixed XYZZ += affine addition: 8 products + 2 squarings
ADDS_PER_PAIR_INT16 = 2        # byte windows of a 16-bit magnitude (the reference's cost model)
ALGO_MUL_INSTR_PER_PAIR = MUL_INSTR_PER_FIELD_MUL * FIELD_MUL_PER_ADD * ADDS_PER_PAIR_INT16  # 5280
EXEC_MUL_INSTR_PER_ADD = 8 * MUL_INSTR_PER_FIELD_MUL + 2 * MUL_INSTR_PER_FIELD_SQR              # 2528
NCU_DRAM_BYTES_PER_PAIR = 69.8  # measured with ncu on a reduced case: 585 MB read+write for 8.4 M pairs
METRIC = "hyrax_msm_points_per_s"
UNIT = "points/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="grape_b200", choices=["grape_b200", "reference"])
    ap.add_argument("--window-bits", type=int, default=16, choices=[8, 16])
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="target length of the CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--proof-layers", type=int, default=4,
                    help="layers per batch of the proof timing carried in `layer_proof` (seq 2048); 0 = skip it")
    ap.add_argument("--proof-window-bits", type=int, default=13)
    ap.add_argument("--proof-scope", default="layer", choices=["layer", "ffn"])
    ap.add_argument("--workload", default="commit", choices=["commit", "matmul", "lookup", "lookup-bucket", "commit-bls12-381", "matmul-sharded", "layer-proof", "fold"],
                    help="commit = C4 (the headline); matmul = C2 prove_matmul; lookup = C3 range lookup")
    ap.add_argument("--shrink", type=int, default=1, help="divide the matmul / lookup sizes (profiling cases)")
    ap.add_argument("--rows", type=int, default=0, help="commit only this many rows (reduced case for profiling)")
    ap.add_argument("--affine", default="", help="B,chunks: commit with the affine-accumulator kernel, B slots per lane "
                                                 "(0,0 = chosen by its planner), or 'auto': where its planner "
                                                 "expects a gain; profiling cases")
    ap.add_argument("--gens", type=int, default=WD, help="generators = scalars per row (reduced case for profiling)")
    return ap.parse_args()


def workload_config():
    """The same dictionary in both arms (the window width of this library's table is a top-level key)."""
    return {"workload": "C4: Hyrax commit of one LLaMA-2-7B-shaped layer (4x4096x4096 + 3x4096x11008 int16-range "
                        "weights, 4096 generators)", "pairs_per_step": LAYER_PAIRS, "rows_per_step": LAYER_PAIRS // WD,
            "row_len": WD, "curve": "BN254 G1 (the curve the reference compiles)",
            "l2_policy": "inputs (809 MB) exceed L2"}


def quantised_normal_np(rng, n, std=0.02, scale=1 << 16, lo=-(1 << 15), hi=(1 << 15) - 1):
    """clip(round(N(0, std) * scale), lo, hi) as int32 (numpy only: the reference arm imports nothing of the package)."""
    out = np.empty(n, dtype=np.int32)
    step = 1 << 24
    for a in range(0, n, step):
        b = min(n, a + step)
        x = rng.standard_normal(b - a, dtype=np.float32) * np.float32(std * scale)
        out[a:b] = np.clip(np.rint(x), lo, hi).astype(np.int32)
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML while the timed region runs (the same
    counters `nvidia-smi --query-gpu=clocks.sm,clocks_event_reasons.*` prints)."""
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, device_index: int):
        self.idx = device_index
        self.sm: list[int] = []
        self.power: list[float] = []
        self.mask = 0
        self.max_sm = None
        self.stop_flag = threading.Event()
        self.thread = None
        self.error = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            # NVML enumerates physical devices; honour CUDA_VISIBLE_DEVICES when it lists indices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            phys = self.idx
            if vis and all(t.strip().isdigit() for t in vis.split(",")):
                phys = int(vis.split(",")[self.idx])
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # noqa: BLE001
            self.error = f"NVML unavailable: {e}"
            return
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def _loop(self):
        nv = self.nv
        while not self.stop_flag.is_set():
            try:
                self.sm.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                self.mask |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0)
            except Exception as e:  # noqa: BLE001
                self.error = str(e)
                return
            time.sleep(0.02)

    def stop(self):
        self.stop_flag.set()
        if self.thread:
            self.thread.join(timeout=2)
        reasons = sorted(k for k, bit in self.REASONS.items() if self.mask & bit)
        out = {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_sm,
               "samples": len(self.sm), "reasons": reasons,
               "power_w_max": max(self.power) if self.power else None}
        if self.error:
            out["note"] = self.error
        return out


def cpu_baseline(gens: np.ndarray, scalars: np.ndarray, target_seconds: float, check_rows=None):
    """Times the C restatement of the reference's byte-window commit on all host cores over a row
    sample sized for about `target_seconds`; returns (dict, rows_used, records)."""
    from oracle import cport
    cport.build()
    cores = cport.threads()
    table = cport.table_build(gens)  # setup, not timed (the reference precomputes it offline)
    probe_rows = max(2 * cores, 8)
    t = time.perf_counter()
    cport.commit_i32(scalars, WD, table, 0, probe_rows)
    dt = time.perf_counter() - t
    rows = int(max(probe_rows, min(scalars.size // WD, target_seconds / (dt / probe_rows))))
    rows = max(cores, rows // cores * cores)
    t = time.perf_counter()
    rec = cport.commit_i32(scalars, WD, table, 0, rows)
    dt = time.perf_counter() - t
    value = rows * WD / dt
    return ({"value": value, "unit": UNIT, "cores": cores, "kind": "port",
             "sample": f"first {rows} of {scalars.size // WD} rows of the same layer ({rows * WD} pairs, {dt:.1f} s), "
                       "fixed-base 8-bit-window table as in the reference"}, rows, rec)


REF_HARNESS = ROOT / "oracle" / "_ref" / "ref_harness"


def _run_harness(argv, timeout):
    if not REF_HARNESS.exists():
        return None
    env = dict(os.environ, OMP_NUM_THREADS="1")
    try:
        res = subprocess.run([str(REF_HARNESS), *map(str, argv)], capture_output=True, text=True, env=env, timeout=timeout)
    except (OSError, subprocess.TimeoutExpired) as e:
        return {"unavailable": str(e)}
    for ln in reversed(res.stdout.strip().splitlines()):
        if ln.startswith("{"):
            return json.loads(ln)
    return {"unavailable": (res.stderr or res.stdout)[-300:]}


def reference_cuda(rows: int, steps: int, warmup: int = 1):
    """The reference's own commit kernels (its unmodified src/*.cu built into oracle/_ref by
    `make -C oracle ref`), timed on this GPU by oracle/ref_harness.cu.  None when that build is absent."""
    d = _run_harness(["commit-bench", rows, steps, warmup], 900)
    if d is not None and "unavailable" not in d:
        d["what"] = ("reference CUDA (fixed-base 8-bit windows, one warp per row), unmodified sources, "
                     "libff replaced by a stand-in; same rows x 4096 int16-range workload")
    return d


def reference_cuda_secondary(mode: str, a: int, steps: int, what: str, extra=()):
    """`ref_harness matmul-bench|lookup-bench`: the reference's own prove_matmul / tLookupRange::prove on
    this GPU at the same sizes.  None when that build is absent."""
    d = _run_harness([mode, a, steps, *extra], 900)
    if d is not None and "unavailable" not in d:
        d["what"] = what
    return d


def run_reference(args):
    """The reference arm: the reference's own CUDA commit kernels on GPU 0 (the reference has no CPU
    implementation of this path); the C restatement on the host cores only when that build is absent.
    Nothing of the grape_b200 package is imported here."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = workload_config()
    sampler = ClockSampler(0)   # over the whole child process: its table build and warm-up are inside
    sampler.start()
    ref = reference_cuda(cfg["rows_per_step"], max(args.steps, 1), max(args.warmup, 1))
    clocks = sampler.stop()
    clocks["note"] = (clocks.get("note", "") + " sampled while the reference's process ran (set-up, warm-up and timed steps)").strip()
    if ref and "points_per_s" in ref and ref.get("cuda_status") == "no error":
        line = {"impl": "reference", "metric": METRIC, "value": ref["points_per_s"], "unit": UNIT, "n_gpus": args.gpus,
                "gpus_used": 1, "steps": args.steps, "warmup": ref.get("warmup", 1), "ms_per_step": ref["ms_per_step"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "u32 limbs (254-bit fields)", "data": "synthetic", "config": cfg,
                "cpu_baseline": {"value": ref["points_per_s"], "unit": UNIT, "cores": 1, "kind": "reference",
                                 "sample": "whole layer (49 408 rows); the reference's implementation of this path is "
                                           "CUDA, so its own kernels run on GPU 0 driven by one host thread"},
                "e2e": {"value": ref["e2e_points_per_s"], "unit": UNIT, "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0, "ms_per_step": ref["e2e_ms_per_step"],
                        "note": "the reference's own data movement (cudaMemcpy from pageable memory) is inside"},
                "gpu_launches": 0, "clocks": clocks, "reference_build": ref["what"],
                "multi_gpu_note": "the reference has no multi-GPU path: at any N its kernels run on one GPU"}
        print(json.dumps(line))
        return
    from oracle import bn254, cport   # the one other place bench.py may execute oracle/
    cport.build()
    rng = np.random.default_rng(SEED)
    rows_avail = 4096
    scalars = quantised_normal_np(rng, rows_avail * WD)
    # generators [rho_i](1,2): computed with the oracle's own table code from one base point
    base = np.frombuffer(bn254.jacobian_to_bytes(bn254.G1_GEN), dtype=np.uint32).reshape(1, 24)
    base_table = cport.table_build(base)
    rho = np.frombuffer(b"".join(bn254.fr_to_bytes(v) for v in bn254.SplitMix64(SEED).fr_vec(WD)),
                        dtype=np.uint32).reshape(-1, 8)
    gens = cport.commit_fr(rho, 1, base_table)
    table = cport.table_build(gens)
    cores = cport.threads()
    t = time.perf_counter()
    cport.commit_i32(scalars, WD, table, 0, 2 * cores)
    per_row = (time.perf_counter() - t) / (2 * cores)
    total_steps = args.steps + args.warmup
    rows = int(min(rows_avail, max(cores, (90.0 / max(total_steps, 1)) / per_row)))
    rows = max(cores, rows // cores * cores)
    for _ in range(args.warmup):
        cport.commit_i32(scalars, WD, table, 0, rows)
    t = time.perf_counter()
    for _ in range(args.steps):
        cport.commit_i32(scalars, WD, table, 0, rows)
    dt = time.perf_counter() - t
    value = rows * WD * args.steps / dt
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u32 limbs (254-bit fields)",
            "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                             "sample": f"each step = first {rows} rows ({rows * WD} pairs) of the layer"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def layer_proof(ctx, layers: int, window_bits: int, scope: str, seed: int = 0xC5, pieces: bool = False):
    """Proof of `layers` LLaMA-2-7B-shaped decoder layers in one batch (seq 2048, dim 4096, ffn 11008) in
    the call order of the reference's end-to-end driver test/llm.cu:73-611.  scope "layer": everything
    (11 matmul sumchecks, 3 Hadamard sumchecks, 14 range and 2 mapping lookups, 3 claim batchings and the
    openings); scope "ffn": the feed-forward half only (test/llm.cu:73-239).  The timed region is what the
    reference's own timer brackets (test/llm.cu:69-75, 613-614: total_prove_time over the batch)."""
    import grape_b200 as g
    from grape_b200 import host, layer, layer_full, workloads as wl
    t_syn = time.perf_counter()
    if scope == "ffn":
        shape = layer.FFNShape(layer_num=layers, tokens=2048, dim=4096, ffn=11008)
        t = layer.synthesize_ffn(shape, seed=seed, x_range=1 << 13, matmul=wl.exact_matmul_cuda)
    else:
        shape = layer_full.LayerShape(layer_num=layers, tokens=2048, dim=4096, ffn=11008)
        t = layer_full.synthesize_layer(shape, seed=seed, x_range=1 << 13, matmul=wl.exact_matmul_cuda)
    # the loader's buffers: page-locked, so that the uploads inside the timed region run at PCIe speed
    for k, v in list(t.items()):
        if isinstance(v, np.ndarray) and v.nbytes >= (1 << 20):
            p = ctx.pinned_array(v.shape, v.dtype)
            p[...] = v
            t[k] = p
    synth_s = time.perf_counter() - t_syn
    gens = wl.make_generators(ctx, shape.ffn_pad * 16, 0xC5)
    t0 = time.perf_counter()
    table = g.GeneratorTable(ctx, gens, window_bits, 1)
    ctx.sync()
    table_s = time.perf_counter() - t0
    ctx.seed(1)
    if scope == "ffn":
        prover = layer.FFNProver(ctx, shape, table, gens[0], t["swiglu_table"])
        run = prover.prove
    else:
        prover = layer_full.LayerProver(ctx, shape, table, gens[0], t["swiglu_table"], t["exp_table"])
        run = prover.prove_layer
    prover.prefetch_inputs = True   # the inputs are page-locked: upload them behind the first proof steps
    run(t)  # warm-up (allocations)
    ctx.sync()
    t0 = time.perf_counter()
    run(t)
    ctx.sync()
    dt = time.perf_counter() - t0
    prover.timing = True
    trace = run(t)
    out = {"scope": scope, "layers": layers, "seconds": dt, "seconds_per_layer": dt / layers,
           "by_step_with_syncs": trace.seconds,
           "lookup_ms_in_walk_order": [round(dt * 1e3, 1) for kind, dt in trace.steps if kind == "lookup"],
           "window_bits": window_bits, "table_gib": table.nbytes / 2**30,
           "table_build_s": table_s, "synthesis_s": synth_s, "opens": trace.opens, "lookups": trace.lookups,
           "matmul_sumchecks": trace.matmuls,
           "upload_s": getattr(prover, "upload_seconds", None),
           "note": "host int32 tensors (page-locked) are uploaded inside the timed region, as the reference's driver loads them"}
    prover.release_pool()
    if pieces:
        # one piece of the walk alone, at the shape the reference build is timed on beside it: the range
        # lookup of a 4 x 2048 x 4096 remainder tensor (2^25 queries, 2^16 table, rows of 65 536 generators)
        D = 1 << 25
        rng = np.random.default_rng(7)
        q = rng.integers(-(1 << 15), 1 << 15, size=D).astype(np.int32)
        dq, dS, dA = ctx.upload(q), ctx.alloc(D * 32), ctx.alloc(D * 32)
        lk = host.Lookup(ctx, -(1 << 15), 1 << 16)
        vv = host.decode_field(ctx.random_fr(25))
        ms = []
        for it in range(3):
            ctx.fr_from_i32(dq, D, dS)
            ctx.timer_begin()
            lk.prove(dS, D, dA, vv, table=table, msm_size=4096)
            ms.append(ctx.timer_end())
        out["piece_range_lookup_2p25_ms"] = float(np.mean(ms[1:]))
        for b in (dq, dS, dA):
            b.free()
    table.close()
    return out


def set_affine(ctx, spec: str):
    """--affine B,chunks forces the affine-accumulator kernel; --affine auto leaves the choice to its planner."""
    if spec == "auto":
        ctx.set_affine_commit(1)
    else:
        ctx.set_affine_commit(2, *(int(v) for v in spec.split(",")))


def run_own(args):
    import grape_b200 as g
    from grape_b200 import parallel, workloads as wl

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    headline = args.gens == WD and not args.rows
    # The reference's own kernels are timed first, while this process holds nothing on the GPU
    # (timed after this library's runs, with its context and tables alive, the other process
    # measured up to three times slower).
    ref_cuda = ref_pieces = None
    if world == 1 and headline:
        ref_cuda = reference_cuda(LAYER_PAIRS // WD, 3, 3)   # three warm-up steps: an idle GPU takes a while to clock up
        if args.proof_layers:
            ref_pieces = {
                "range_lookup_2p25": reference_cuda_secondary(
                    "lookup-bench", 25, 1, "reference CUDA tLookupRange::prove: 2^25 queries (a 4 x 2048 x 4096 remainder "
                    "tensor), 2^16 table, commitments over rows of 65 536 generators; host wall clock around the call",
                    extra=(65536,)),
                "matmul_c2": reference_cuda_secondary(
                    "matmul-bench", 1, 2, "reference CUDA prove_matmul, A 2048x4096 . B 4096x4096, Fr tensors resident")}
    ctx = g.Context(local_rank)
    if args.affine:
        set_affine(ctx, args.affine)

    wd = args.gens
    n = LAYER_PAIRS if not args.rows else args.rows * wd
    rows = n // wd
    if rows % world:
        raise SystemExit(f"{rows} rows do not divide over {world} ranks")
    gens = wl.make_generators(ctx, wd, SEED)                  # same generators on every rank
    bits = 16
    n_windows = 1 if args.window_bits == 16 else 2
    adds_per_pair = 1 if args.window_bits == 16 else 2
    table = g.GeneratorTable(ctx, gens, args.window_bits, n_windows)
    ctx.sync()

    # the layer is the same on every rank; rank r owns the contiguous row block [r0, r1)
    rng = np.random.default_rng(SEED)
    h_scalars = ctx.pinned_array((n,), np.int32)
    wl.quantised_normal(rng, n, out=h_scalars)
    r0, r1 = parallel.row_block(rows, rank, world)
    block = r1 - r0
    h_out = ctx.pinned_array((rows, 24), np.uint32)
    d_scalars = ctx.upload(h_scalars)                         # whole layer resident (the block is a slice of it)
    d_out = ctx.alloc(rows * 96)                              # all commitments, rank order = row order
    d_local = ctx.alloc(block * 96) if world > 1 else d_out
    h_scalars_dev = ctx.host_device_pointer(h_scalars) if world > 1 else None
    lib = ctx.lib

    def step_device():
        parallel.commit_rows_sharded_device(ctx, table, d_scalars.at(r0 * wd * 4), block, wd, d_local, d_out, dist,
                                            max_bits=bits)

    def step_host():
        if world == 1:
            g.commit_i32_host(ctx, table, h_scalars, wd, max_bits=bits, out=h_out)
            return
        # this rank's block is read by the kernel where it lies in page-locked host memory (as the
        # library's host-buffer entry point does at N = 1), then the gather, then all commitments back to
        # every rank's host
        g.commit_i32(ctx, table, h_scalars_dev + r0 * wd * 4, block * wd, wd, d_local, max_bits=bits)
        parallel.gather_rows_device(ctx, d_local, block, d_out, dist)
        ctx._check(lib.grape_d2h(ctx.handle, h_out.ctypes.data, d_out.ptr, rows * 96))

    def barrier():
        ctx.sync()
        if dist is not None:
            import torch
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if dist is None:
            return ms
        import torch
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing -------------------------------------------------------------
    for _ in range(args.warmup):
        step_device()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = ctx.launches
    ctx.prof_enable(True)
    ctx.timer_begin()
    for _ in range(args.steps):
        step_device()
    ms = ctx.timer_end()
    barrier()
    kernel_ms, kernel_launches = ctx.prof_read()
    ctx.prof_enable(False)
    launches = ctx.launches - launches0
    clocks = sampler.stop() if rank == 0 else None
    ms = max_over_ranks(ms)
    status = ctx.status()
    value = n * args.steps / (ms * 1e-3)        # the ONE layer's pairs over the slowest rank's time, gather included
    dev_records = ctx.download(d_out, rows * 96).reshape(rows, 24)

    # ---- end to end through host buffers -----------------------------------------------------
    for _ in range(max(1, min(args.warmup, 2))):
        step_host()
    barrier()
    ctx.timer_begin()
    for _ in range(args.steps):
        step_host()
    e2e_ms = max_over_ranks(ctx.timer_end())
    barrier()
    e2e_value = n * args.steps / (e2e_ms * 1e-3)
    host_path_matches = bool(np.array_equal(dev_records, h_out))

    # ---- the same commitment by the affine-accumulator kernel (off by default), N = 1 -----------------
    affine = None
    if world == 1 and headline and not args.affine:
        d_alt = ctx.alloc(rows * 96)
        ctx.set_affine_commit(2)
        for _ in range(3):   # the first calls grow the scratch arena
            g.commit_i32(ctx, table, d_scalars, n, wd, d_alt, max_bits=bits)
        ctx.prof_enable(True)
        ctx.timer_begin()
        for _ in range(args.steps):
            g.commit_i32(ctx, table, d_scalars, n, wd, d_alt, max_bits=bits)
        alt_ms = ctx.timer_end() / args.steps
        alt_kernel_ms, alt_launches = ctx.prof_read()
        ctx.prof_enable(False)
        ctx.set_affine_commit(-1)
        affine = {"what": "commit_accumulate_affine_kernel: affine accumulators in device memory, one inversion shared "
                          "by the additions of a batch of rows (5 multiplications + 1 squaring per addition); selectable "
                          "with grape_commit_set_affine, not the default",
                  "ms_per_step": alt_ms, "kernel_ms": alt_kernel_ms / max(alt_launches, 1), "value": n / (alt_ms * 1e-3),
                  "unit": UNIT,
                  "identical_output": bool(np.array_equal(ctx.download(d_alt, rows * 96).reshape(rows, 24), dev_records))}
        d_alt.free()

    # ---- N > 1: every rank commits the whole layer alone (the check of the sharded result, and the
    # weak-scaling figure: N layers on N GPUs, no collective) --------------------------------------
    multi = None
    if world > 1:
        d_full = ctx.alloc(rows * 96)
        g.commit_i32(ctx, table, d_scalars, n, wd, d_full, max_bits=bits)
        barrier()
        ctx.timer_begin()
        for _ in range(3):
            g.commit_i32(ctx, table, d_scalars, n, wd, d_full, max_bits=bits)
        weak_ms = max_over_ranks(ctx.timer_end()) / 3
        full = ctx.download(d_full, rows * 96).reshape(rows, 24)
        same = bool(np.array_equal(full, dev_records))
        import torch
        flag = torch.tensor([1 if same else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        multi = {"sharding": f"rows dealt to {world} ranks in contiguous blocks of {block}; one NCCL all-gather of "
                             f"{block * 96} B per rank on the library's stream inside every step",
                 "gathered_equals_unsharded_on_every_rank": bool(flag.item()),
                 "weak_scaling": {"value": world * n / (weak_ms * 1e-3), "unit": UNIT, "ms_per_step": weak_ms,
                                  "what": "every rank commits a whole layer, no collective"},
                 "single_gpu_ms_per_layer": weak_ms}
        d_full.free()

    # ---- roofline of the dominant kernel (commit_accumulate), rank 0's launches -------------------
    roofline = None
    if rank == 0:
        peak_instr = ctx.measure_int_peak(2)        # lo/hi multiply-add instructions per second, measured now
        peak_fmul = ctx.measure_int_peak(3)
        peak_fsqr = ctx.measure_int_peak(5)
        peak_madd = ctx.measure_madd_peak()         # mixed additions/s on register-resident operands
        k_ms = kernel_ms / max(kernel_launches, 1)
        pairs_per_launch = block * wd
        adds_per_launch = pairs_per_launch * adds_per_pair
        achieved = adds_per_launch * EXEC_MUL_INSTR_PER_ADD / (k_ms * 1e-3)
        cost_model = pairs_per_launch * ALGO_MUL_INSTR_PER_PAIR / (k_ms * 1e-3)
        peaks_file = ROOT / "MEASURED_PEAKS.json"
        hbm_peak = json.loads(peaks_file.read_text())["hbm_gbs"] if peaks_file.exists() else 6650.0
        algo_bytes = pairs_per_launch * 4 + adds_per_launch * 64 + block * 128   # scalars + gathered table points + partial sums
        roofline = {"bound": "int32-multiply pipe (not hbm, not tensor: no dense contraction on this path)",
                    "kernel": "commit_accumulate_kernel", "achieved": achieved / 1e12, "peak": peak_instr / 1e12,
                    "unit": "T multiply-instr/s", "frac": achieved / peak_instr,
                    "frac_of": "measured peak (this run: dependent-free mad.lo.cc/madc.hi loop at full occupancy)",
                    "executed_instr_per_add": EXEC_MUL_INSTR_PER_ADD, "adds_per_pair": adds_per_pair,
                    "cost_model_frac": cost_model / peak_instr,
                    "cost_model_note": "the reference's algorithm as the unit: 2 byte-window additions x 10 field "
                                       "multiplications x 264 multiply instructions = 5280 per int16 pair; this kernel "
                                       "executes one addition per pair, so this figure can exceed 1",
                    "kernel_ms": k_ms, "pairs_per_launch": pairs_per_launch,
                    "field_mul_peak_per_s": peak_fmul, "field_sqr_peak_per_s": peak_fsqr,
                    "adds_per_s": adds_per_launch / (k_ms * 1e-3), "register_resident_add_peak_per_s": peak_madd,
                    "frac_of_add_peak": adds_per_launch / (k_ms * 1e-3) / peak_madd,
                    "traffic": int(pairs_per_launch * NCU_DRAM_BYTES_PER_PAIR),
                    "traffic_source": "ncu dram bytes of a reduced case (8.4 M pairs: 585 MB read+write = 69.8 B/pair) "
                                      "scaled by pairs; algorithmic 68 B/pair",
                    "hbm": {"achieved_gbs": algo_bytes / (k_ms * 1e-3) / 1e9, "peak_gbs": hbm_peak,
                            "frac": algo_bytes / (k_ms * 1e-3) / 1e9 / hbm_peak,
                            "peak_source": "MEASURED_PEAKS.json" if peaks_file.exists() else "fallback"}}

    # ---- the other half of the metric: proof seconds per layer (every rank proves its own batch) -----
    proof = None
    if args.proof_layers and headline:
        table.close()
        for b in (d_scalars, d_out, d_local if world > 1 else None):
            if b is not None:
                b.free()
        barrier()
        res = layer_proof(ctx, args.proof_layers, args.proof_window_bits, args.proof_scope, seed=0xC5 + rank,
                          pieces=(world == 1))
        slowest = max_over_ranks(res["seconds"] * 1e3) / 1e3
        proof = {"metric": "proof_seconds_per_layer", "seconds_per_layer": slowest / (args.proof_layers * world),
                 "unit": "s/layer", "layers_per_rank": args.proof_layers, "layers_total": args.proof_layers * world,
                 "slowest_batch_s": slowest, "scaling": "weak (one batch of layers per GPU, no data-path collective)",
                 "timing": "host wall clock around the batch on each rank, synchronised on both sides, max over ranks",
                 "rank0": res}
        if ref_pieces is not None:
            proof["reference_pieces"] = ref_pieces
            proof["reference_note"] = ("the reference's whole-layer driver needs the model's tensor dumps and cannot run "
                                       "here; these are its provers on pieces of the same shapes, same GPU, timed before "
                                       "this library created its context")

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    assert roofline["frac"] <= 1.0 or args.rows, "executed-work fraction above the measured peak: check the instruction count"
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "u32 limbs (254-bit fields)", "data": "synthetic",
            "config": workload_config() if headline else
            {"workload": f"reduced case for profiling: {rows} rows x {wd} generators"},
            "window_bits": args.window_bits, "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(n * 4),
                    "d2h_bytes_per_step": int(world * rows * 96), "ms_per_step": e2e_ms / args.steps,
                    "matches_device_path": host_path_matches},
            "gpu_launches": int(launches), "roofline": roofline, "device_status": status,
            "table_bytes": int(2 ** (args.window_bits - 1) * n_windows * wd * 64)}
    if multi is not None:
        line["multi_gpu"] = multi
    if affine is not None:
        line["affine_commit"] = affine
    if ref_cuda is not None:
        line["reference_cuda"] = ref_cuda
    if proof is not None:
        line["layer_proof"] = proof
    if not args.no_cpu_baseline and headline and world == 1:   # host-core baseline: N = 1 only
        base, rows_used, rec = cpu_baseline(gens, np.asarray(h_scalars), args.cpu_seconds)
        base["matches_gpu_rows"] = bool(np.array_equal(rec, dev_records[:rows_used]))
        line["cpu_baseline"] = base
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def run_secondary(args):
    """C2 (matmul sumcheck) and C3 (range lookup) as stand-alone timings with the roofline of their
    dominant kernel; single GPU."""
    import grape_b200 as g
    from grape_b200 import host, workloads as wl
    ctx = g.Context(int(os.environ.get("LOCAL_RANK", "0")))
    if args.affine:
        set_affine(ctx, args.affine)
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    hbm_peak = json.loads(peaks_file.read_text())["hbm_gbs"] if peaks_file.exists() else 6650.0
    rng = np.random.default_rng(0xC2)
    times = []
    if args.workload == "matmul":
        L, N, M, K = 1, 2048 // args.shrink, 4096 // args.shrink, 4096
        A = wl.quantised_normal(rng, N * K, lo=-2**31, hi=2**31 - 1)
        B = wl.quantised_normal(rng, M * K, lo=-2**31, hi=2**31 - 1)
        dAi, dBi = ctx.upload(A), ctx.upload(B)
        dA, dB = ctx.alloc(N * K * 32), ctx.alloc(M * K * 32)
        ctx.seed(0xC2)
        lM, lN, lK = (M - 1).bit_length(), (N - 1).bit_length(), (K - 1).bit_length()
        u = host.decode_field(ctx.random_fr(lM + lN))
        v = host.decode_field(ctx.random_fr(lK))
        du = ctx.fr_upload(u)
        a_, b_, one = ctx.alloc(K * 32), ctx.alloc(K * 32), ctx.alloc(32)
        ctx.fr_from_i32(dAi, N * K, dA)
        ctx.fr_from_i32(dBi, M * K, dB)
        ctx.fr_fold(dA, N * K, du.at(lM * 32), N, K, a_)
        ctx.fr_fold(dB, M * K, du, M, K, b_)
        ctx.fr_binary("mul", a_, b_, a_, K)
        ctx.fr_sum(a_, K, one)
        claim = ctx.fr_download(one, 1)[0]
        launches = 0
        for it in range(args.warmup + args.steps):
            ctx.fr_from_i32(dAi, N * K, dA)
            ctx.fr_from_i32(dBi, M * K, dB)
            if it == args.warmup:
                ctx.prof_enable(True)
            l0 = ctx.launches
            ctx.timer_begin()
            host.prove_matmul(ctx, dA, dB, L, N, M, K, u, v, claim)
            ms = ctx.timer_end()
            if it >= args.warmup:
                times.append(ms)
                launches += ctx.launches - l0
        k_ms, k_n = ctx.prof_read()
        ctx.prof_enable(False)
        # the same proof straight from the int32 tensors (no conversion, folds read 4 B per element)
        times_i32 = []
        for it in range(args.warmup + args.steps):
            ctx.timer_begin()
            r_i32 = host.prove_matmul_i32(ctx, dAi, dBi, L, N, M, K, u, v, claim)
            ms = ctx.timer_end()
            if it >= args.warmup:
                times_i32.append(ms)
        algo_bytes = 32.0 * (N * K + M * K)   # the two axis folds read every element once
        per_launch = k_ms / max(k_n, 1)
        achieved = algo_bytes / 2 / (per_launch * 1e-3) / 1e9 if k_n else 0.0  # two launches (A and B) per proof
        line = {"metric": "prove_matmul_ms", "value": float(np.mean(times)), "unit": "ms", "higher_is_better": False,
                "config": {"workload": f"C2: prove_matmul A {N}x{K} . B {M}x{K}^T, Fr tensors resident in HBM"},
                "roofline": {"bound": "hbm", "kernel": "k_fold_axis", "achieved": achieved, "peak": hbm_peak,
                             "unit": "GB/s", "frac": achieved / hbm_peak, "traffic": None,
                             "note": "mean over the A-fold and B-fold launches; 32 B read and one field "
                                     "multiplication per element, so the integer pipe caps it near 2.2 TB/s"},
                "gpu_launches": int(launches),
                "from_int32_ms": float(np.mean(times_i32)),
                "from_int32_note": "grape_prove_matmul_i32 on the int32 tensors the Fr tensors are built from: same "
                                   "claims and transcript, no conversion pass, folds at 4 B per element"}
        # host-core baseline and full-size parity: the C restatement of the reference's prove_matmul on all
        # host cores, same tensors, same challenges; its claims and round polynomials must equal the GPU's
        if not args.no_cpu_baseline:
            from oracle import cport
            cport.build()
            enc = lambda xs: host.encode_field(xs)
            t0 = time.perf_counter()
            rc, ca, cb, cfinal, ctr = cport.prove_matmul_l1(A, B, N, M, K, enc(u), enc(v), enc([claim]))
            cpu_s = time.perf_counter() - t0
            same = (rc == 0 and host.decode_field(ca.reshape(1, 8))[0] == r_i32[0]
                    and host.decode_field(cb.reshape(1, 8))[0] == r_i32[1]
                    and host.decode_field(cfinal.reshape(1, 8))[0] == r_i32[2]
                    and [host.decode_field(ctr[i]) for i in range(ctr.shape[0])] == [p[:3] for p in r_i32[3]])
            line["cpu_baseline"] = {"value": cpu_s * 1e3, "unit": "ms", "cores": cport.threads(), "kind": "port",
                                    "sample": "the full C2 proof once (int32 -> Fr, two folds, 12 rounds)",
                                    "matches_gpu_claims_and_transcript": bool(same)}
        ctx.sync()
        line["reference_cuda"] = reference_cuda_secondary(
            "matmul-bench", args.shrink, 3, "reference CUDA prove_matmul (unmodified sources, libff stand-in), same shape, "
            "Fr tensors resident, host wall clock around the call")
    elif args.workload == "fold":
        # Axis fold (FrTensor::partial_eval, src/fr-tensor.cu:53-72,168-188) of an [8192][16384] tensor over its
        # first axis, from int32 data (4 B per element) and from Fr data (32 B per element).
        c, gap = 8192 // args.shrink, 16384
        n = c * gap
        t_i = ctx.upload(wl.quantised_normal(rng, n, lo=-2**31, hi=2**31 - 1))
        ctx.seed(0xF0)
        du = ctx.upload(ctx.random_fr((c - 1).bit_length()))
        out = ctx.alloc(gap * 32)
        res = {}
        launches = 0
        for label in ("int32", "fr"):
            if label == "fr":
                t_f = ctx.alloc(n * 32)
                ctx.fr_from_i32(t_i, n, t_f)
            ctx.prof_read()
            for it in range(args.warmup + args.steps):
                if it == args.warmup:
                    ctx.prof_enable(True)
                l0 = ctx.launches
                if label == "int32":
                    ctx.fold_i32(t_i, n, du, c, gap, out)
                else:
                    ctx.fr_fold(t_f, n, du, c, gap, out)
                if it >= args.warmup:
                    launches += ctx.launches - l0
            ctx.sync()
            k_ms, k_n = ctx.prof_read()
            ctx.prof_enable(False)
            per = k_ms / max(k_n, 1)
            nbytes = n * (4 if label == "int32" else 32)
            res[label] = {"kernel_ms": per, "bytes": nbytes, "gbs": nbytes / (per * 1e-3) / 1e9 if per else 0.0}
        line = {"metric": "fold_axis_gbs", "value": res["int32"]["gbs"], "unit": "GB/s", "higher_is_better": True,
                "config": {"workload": f"axis fold of a {c} x {gap} tensor over its first axis; inputs ({n * 4 >> 20} MiB int32, "
                                       f"{n * 32 >> 20} MiB Fr) exceed L2"},
                "roofline": {"bound": "hbm", "kernel": "k_fold_axis<int32 source>", "achieved": res["int32"]["gbs"],
                             "peak": hbm_peak, "unit": "GB/s", "frac": res["int32"]["gbs"] / hbm_peak, "traffic": None,
                             "note": "algorithmic bytes = 4 per element (the tensor is read once); eight multiply-adds per element"},
                "fr_source": {"kernel": "k_fold_axis<Fr source>", "achieved_gbs": res["fr"]["gbs"],
                              "frac_of_hbm": res["fr"]["gbs"] / hbm_peak, "kernel_ms": res["fr"]["kernel_ms"],
                              "note": "32 B and one full field multiplication per element: bound by the multiply pipe"},
                "kernel_ms": res["int32"]["kernel_ms"], "gpu_launches": int(launches)}
    elif args.workload == "lookup-bucket":
        # One range lookup whose rows (2^18 elements) are four times longer than its table (2^16 entries), proved
        # with the commitment of A by the direct kernel and by the bucket method: same commitments, two timings.
        D, Nt, msm = (1 << 24) // args.shrink, 1 << 16, 16384
        gens = wl.make_generators(ctx, msm * 16, 3)
        table = g.GeneratorTable(ctx, gens, 13, 1)
        ctx.seed(1)
        lk = host.Lookup(ctx, -(1 << 15), Nt)
        q = rng.integers(-(1 << 15), 1 << 15, size=D).astype(np.int32)
        dq, dS, dA, com = ctx.upload(q), ctx.alloc(D * 32), ctx.alloc(D * 32), ctx.alloc(D // (msm * 16) * 96)
        vv = host.decode_field(ctx.random_fr((D - 1).bit_length()))
        res, coms, launches = {}, {}, 0
        for label, mode in (("direct", 0), ("bucket", 2)):
            ctx.set_bucket_commit(mode)
            ts = []
            for it in range(args.warmup + args.steps):
                ctx.fr_from_i32(dq, D, dS)
                l0 = ctx.launches
                ctx.timer_begin()
                lk.prove(dS, D, dA, vv, table=table, msm_size=msm, d_com_A=com)
                ms = ctx.timer_end()
                if it >= args.warmup:
                    ts.append(ms)
                    launches += ctx.launches - l0
            res[label] = float(np.mean(ts))
            coms[label] = ctx.download(com, D // (msm * 16) * 96).tobytes()
        ctx.set_bucket_commit(1)
        line = {"metric": "lookup_prove_ms (A committed by the bucket method)", "value": res["bucket"], "unit": "ms",
                "higher_is_better": False, "direct_kernel_ms": res["direct"],
                "commitments_identical": coms["direct"] == coms["bucket"], "gpu_launches": int(launches),
                "config": {"workload": f"range lookup, {D} queries, 2^16 table, commitment rows of {msm * 16} elements "
                                       f"({D // (msm * 16)} rows), 13-bit windows"}}
    elif args.workload == "commit-bls12-381":
        # The C4 shape over BLS12-381 G1 (the reference compiles BN254 only; reported separately).
        wd = args.gens
        n = LAYER_PAIRS // args.shrink if not args.rows else args.rows * wd
        n -= n % wd
        rows = n // wd
        gens = wl.make_generators_bls12_381(ctx, wd, SEED)
        table = g.GeneratorTable(ctx, gens, args.window_bits, 1 if args.window_bits == 16 else 2, curve="bls12_381")
        h_scalars = wl.quantised_normal(rng, n)
        d_scalars, d_out = ctx.upload(h_scalars), ctx.alloc(rows * 144)
        launches = 0
        for it in range(args.warmup + args.steps):
            if it == args.warmup:
                ctx.prof_enable(True)
            l0 = ctx.launches
            ctx.timer_begin()
            g.commit_i32(ctx, table, d_scalars, n, wd, d_out, max_bits=16)
            ms = ctx.timer_end()
            if it >= args.warmup:
                times.append(ms)
                launches += ctx.launches - l0
        k_ms, k_n = ctx.prof_read()
        per_launch = k_ms / max(k_n, 1)
        mul_peak = ctx.measure_bls12_381_mul_peak()
        adds = n * (1 if args.window_bits == 16 else 2)
        muls_per_s = adds * 10 / (per_launch * 1e-3)
        line = {"metric": "Hyrax MSM points/s over BLS12-381 G1", "value": n / (float(np.mean(times)) * 1e-3),
                "unit": "points/s", "higher_is_better": True, "ms_per_step": float(np.mean(times)),
                "config": {"workload": f"C4 shape over BLS12-381: {rows} rows x {wd} generators, int16 scalars, "
                                       f"{args.window_bits}-bit signed windows; inputs resident in HBM"},
                "roofline": {"bound": "int32-multiply pipe", "kernel": "commit_accumulate_kernel<Bls12381>",
                             "achieved": muls_per_s / 1e9, "peak": mul_peak / 1e9, "unit": "G 12-limb field mul/s",
                             "frac": muls_per_s / mul_peak, "kernel_ms": per_launch, "traffic": None,
                             "note": "10 field multiplications per mixed addition (8 products + 2 squarings); peak = "
                                     "the same multiplication looped on registers, measured in this run"},
                "gpu_launches": int(launches), "table_bytes": table.nbytes, "device_status": ctx.status()}
    else:
        D, Nt = (1 << 22) // args.shrink, 1 << 16
        gens = wl.make_generators(ctx, 4096, 0xC3)
        table = g.GeneratorTable(ctx, gens, args.window_bits if args.window_bits != 16 else 13, 1)
        ctx.seed(0xC3)
        lk = host.Lookup(ctx, -(1 << 15), Nt)
        q = rng.integers(-(1 << 15), 1 << 15, size=D).astype(np.int32)
        dqi, dS, dAq = ctx.upload(q), ctx.alloc(D * 32), ctx.alloc(D * 32)
        vv = host.decode_field(ctx.random_fr((D - 1).bit_length()))
        launches = 0
        res = {}
        for label, tab in (("without_commitments", None), ("with_commitments", table)):
            ts = []
            for it in range(args.warmup + args.steps):
                ctx.fr_from_i32(dqi, D, dS)
                if it == args.warmup and tab is not None:
                    ctx.prof_enable(True)
                l0 = ctx.launches
                ctx.timer_begin()
                lk.prove(dS, D, dAq, vv, table=tab, msm_size=256 if tab else 0)
                ms = ctx.timer_end()
                if it >= args.warmup:
                    ts.append(ms)
                    launches += ctx.launches - l0
            res[label] = float(np.mean(ts))
        k_ms, k_n = ctx.prof_read()
        ctx.prof_enable(False)
        wbits = args.window_bits if args.window_bits != 16 else 13
        adds = D * ((254 + wbits - 1) // wbits)
        acc_ms = k_ms / max(args.steps, 1)          # commit_accumulate launches (A and m) per proof
        peak_madd = ctx.measure_madd_peak()
        line = {"metric": "lookup_prove_ms", "value": res["with_commitments"], "unit": "ms", "higher_is_better": False,
                "config": {"workload": f"C3: range lookup, {D} queries into a 2^16 table, commitments of A and m over 4096 generators"},
                "without_commitments_ms": res["without_commitments"], "gpu_launches": int(launches),
                "roofline": {"bound": "int32-multiply pipe", "kernel": "commit_accumulate_kernel<Bn254, Fr scalars>",
                             "achieved": adds / (acc_ms * 1e-3) / 1e9 if acc_ms else 0.0, "peak": peak_madd / 1e9,
                             "unit": "G mixed additions/s", "frac": adds / (acc_ms * 1e-3) / peak_madd if acc_ms else 0.0,
                             "kernel_ms_per_proof": acc_ms, "traffic": None,
                             "note": f"{(254 + wbits - 1) // wbits} additions per query ({wbits}-bit signed windows over "
                                     "254-bit scalars); peak = the same addition looped on registers, measured in this run"}}
        # host-core baseline and full-size parity: the C restatement of tLookupRange::prove on all host cores
        # with the same queries, alpha, u and v; multiplicities, claims and round polynomials must equal the GPU's
        if not args.no_cpu_baseline:
            from oracle import cport
            cport.build()
            lD = (D - 1).bit_length()
            ctx.seed(0xC33)
            u_enc = ctx.random_fr(lD)              # what the prover will draw inside the next call
            ctx.seed(0xC33)
            ctx.fr_from_i32(dqi, D, dS)
            g_claim, g_tr = lk.prove(dS, D, dAq, vv)
            g_m = lk.table("m")
            t0 = time.perf_counter()
            rc, c_m, c_claim, c_final, c_tr = cport.lookup_range(q, -(1 << 15), Nt, host.encode_field([lk.alpha])[0],
                                                                 u_enc, host.encode_field(vv))
            cpu_s = time.perf_counter() - t0
            same = (rc == 0 and [int(x) for x in c_m] == g_m and host.decode_field(c_claim.reshape(1, 8))[0] == g_claim
                    and [host.decode_field(c_tr[i]) for i in range(c_tr.shape[0])] == g_tr)
            line["cpu_baseline"] = {"value": cpu_s * 1e3, "unit": "ms", "cores": cport.threads(), "kind": "port",
                                    "sample": "the full C3 lookup proof once, without the two commitments",
                                    "matches_gpu_multiplicities_claim_and_transcript": bool(same)}
        if args.shrink == 1:
            ctx.sync()
            line["reference_cuda"] = reference_cuda_secondary(
                "lookup-bench", 22, 3, "reference CUDA tLookupRange::prove (unmodified sources, libff stand-in): 2^22 "
                "queries, 2^16 table, its commitments of A and m over 4096 generators; host wall clock around the call")
    line.update({"n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "data": "synthetic",
                 "dtype": "u32 limbs (381-bit base field)" if args.workload == "commit-bls12-381"
                 else "u32 limbs (254-bit fields)", "vs_baseline": None})
    print(json.dumps(line))


def run_matmul_sharded(args):
    """C2 with the inner dimension dealt to the ranks by residue class (one rank per GPU under
    torchrun): per-rank folds and local rounds, one NCCL all-gather of the partial sums, finish on
    every rank.  Tensors are born sharded (each rank synthesises its own columns)."""
    import torch
    import grape_b200 as g
    from grape_b200 import host, parallel, workloads as wl
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = g.Context(local_rank)
    L, N, M, K = 1, 2048 // args.shrink, 4096 // args.shrink, 4096
    kl = K // world
    rng = np.random.default_rng(0xC2 + rank)
    A = wl.quantised_normal(rng, N * kl, lo=-2**31, hi=2**31 - 1)
    B = wl.quantised_normal(rng, M * kl, lo=-2**31, hi=2**31 - 1)
    dAi, dBi = ctx.upload(A), ctx.upload(B)
    dA, dB = ctx.alloc(N * kl * 32), ctx.alloc(M * kl * 32)
    ctx.seed(0xC2)
    lM, lN, lK = (M - 1).bit_length(), (N - 1).bit_length(), (K - 1).bit_length()
    u = host.decode_field(ctx.random_fr(lM + lN))
    v = host.decode_field(ctx.random_fr(lK))
    # the claim: sum over ranks of <fold(A_r), fold(B_r)>, all-reduced as integers on the host side
    du = ctx.fr_upload(u)
    a_, b_, one = ctx.alloc(kl * 32), ctx.alloc(kl * 32), ctx.alloc(32)
    ctx.fr_from_i32(dAi, N * kl, dA)
    ctx.fr_from_i32(dBi, M * kl, dB)
    ctx.fr_fold(dA, N * kl, du.at(lM * 32), N, kl, a_)
    ctx.fr_fold(dB, M * kl, du, M, kl, b_)
    ctx.fr_binary("mul", a_, b_, a_, kl)
    ctx.fr_sum(a_, kl, one)
    mine = ctx.fr_download(one, 1)[0]
    if dist is not None:
        words = torch.tensor([(mine >> (32 * i)) & 0xFFFFFFFF for i in range(8)], dtype=torch.int64, device="cuda")
        allw = [torch.empty_like(words) for _ in range(world)]
        dist.all_gather(allw, words)
        claim = sum(sum(int(x) << (32 * i) for i, x in enumerate(w.tolist())) for w in allw) % host.FR_MODULUS
    else:
        claim = mine

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    times, launches, result = [], 0, None
    for it in range(args.warmup + args.steps):
        ctx.fr_from_i32(dAi, N * kl, dA)
        ctx.fr_from_i32(dBi, M * kl, dB)
        barrier()
        l0 = ctx.launches
        t0 = time.perf_counter()
        result = parallel.prove_matmul_sharded(ctx, dA, dB, L, N, M, K, u, v, claim, dist)
        ctx.sync()
        ms = (time.perf_counter() - t0) * 1e3      # the call synchronises with the host on both sides
        if it >= args.warmup:
            times.append(ms)
            launches += ctx.launches - l0
    ms = float(np.mean(times))
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        print(json.dumps({"metric": "prove_matmul_ms (inner dimension sharded over the GPUs)", "value": ms, "unit": "ms",
                          "higher_is_better": False, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                          "scaling": "strong", "data": "synthetic", "dtype": "u32 limbs (254-bit fields)",
                          "vs_baseline": None, "gpu_launches": int(launches),
                          "config": {"workload": f"C2: prove_matmul A {N}x{K} . B {M}x{K}^T, each rank holds K/{world} "
                                                 f"columns as Fr tensors in HBM; one all-gather of "
                                                 f"{host.matmul_partial_elems(L, kl) * 32} B per rank",
                                     "timing": "host wall clock around the call (it synchronises), max over ranks"},
                          "rounds": len(result[3])}))
    if dist is not None:
        dist.destroy_process_group()


def run_layer_proof(args):
    """C5: every rank proves its own batch of `--proof-layers` (default 4) decoder layers; the batches
    of a 32-layer model are independent, so there is no data-path collective (weak scaling).  The
    reported time per layer is the slowest rank's batch time divided by all the layers proven."""
    import torch
    import grape_b200 as g
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = g.Context(local_rank)
    if args.affine:
        set_affine(ctx, args.affine)
    layers = args.proof_layers or 4
    if dist is not None:
        dist.barrier()
    res = layer_proof(ctx, layers, args.proof_window_bits, args.proof_scope, seed=0xC5 + rank)
    t = torch.tensor([res["seconds"]], device="cuda", dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    slowest = float(t.item())
    if rank == 0:
        print(json.dumps({"metric": "proof_seconds_per_layer", "value": slowest / (layers * world), "unit": "s/layer",
                          "higher_is_better": False, "n_gpus": world, "steps": 1, "warmup": 1, "scaling": "weak",
                          "data": "synthetic", "dtype": "u32 limbs (254-bit fields)", "vs_baseline": None,
                          "config": {"workload": f"C5: {world} batch(es) of {layers} LLaMA-2-7B-shaped decoder layers "
                                                 f"(seq 2048, dim 4096, ffn 11008), one batch per GPU, scope {args.proof_scope}"},
                          "slowest_batch_s": slowest, "rank0": res}))
    if dist is not None:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "layer-proof":
        run_layer_proof(args)
    elif args.workload == "matmul-sharded":
        run_matmul_sharded(args)
    elif args.workload != "commit":
        run_secondary(args)
    else:
        run_own(args)


if __name__ == "__main__":
    main()
