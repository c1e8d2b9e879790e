#!/usr/bin/env python
"""Benchmark of the B200 quantized GEMM suite.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One JSON line on stdout (rank 0).  A *step* is one pass of the hot path over one batch of
synthetic input: one GEMM of the workload's shape (plus, on N > 1 GPUs, the all-gather of C).

Workloads
  bf16_8192   bf16 GEMM M=N=K=8192, N(0,1) inputs, fp32 accumulate, bf16 out   (default)
  int8_8192   int8 GEMM M=N=K=8192, uniform [-127,127], int32 out
  fp16_8192   fp16 GEMM M=N=K=8192
  int8_4096   int8 GEMM M=N=K=4096
  w8a8        int8 W8A8 linear M=8192, N=28672, K=8192, per-row/per-column scales, bf16 out

On N > 1 GPUs (launched by torchrun, one rank per GPU) the rows of A are split across the ranks,
B is replicated and every rank ends the step with the complete [M, N] C; total work is fixed
("strong").  By default the GEMM's epilogue stores each finished tile of the rank's slab into
every rank's copy of C over NVLink (peer memory) and a one-warp marker kernel tells the ranks
when all slabs have landed; `--gather nccl` runs the plain GEMM followed by an in-place NCCL
all-gather instead.  Both variants' pieces are timed separately as well (`gemm_phase`,
`all_gather`, `fused_kernel_ms`).

`value` is whole-job throughput with inputs resident in HBM; `e2e` is the same metric through
the host-buffer C entry point (pinned host memory, copies inside the timed region).
`--impl reference` times the reference's own CPU loop (matrixMulCPU, compiled unmodified into
oracle/_ref/) on the host cores instead; see reference_arm() for how the sample is bounded.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (kind, M, N, K, in_bytes, out_bytes, unit)
    "bf16_8192": ("bf16", 8192, 8192, 8192, 2, 2, "TFLOP/s"),
    "fp16_8192": ("f16", 8192, 8192, 8192, 2, 2, "TFLOP/s"),
    "int8_8192": ("i8", 8192, 8192, 8192, 1, 4, "TOP/s"),
    "int8_4096": ("i8", 4096, 4096, 4096, 1, 4, "TOP/s"),
    "w8a8": ("w8a8", 8192, 28672, 8192, 1, 2, "TOP/s"),
}
NOMINAL_PEAK = {"bf16": 2250.0, "f16": 2250.0, "i8": 4500.0, "w8a8": 4500.0}  # dense, per GPU
METRIC = "int8 TOPS & bf16/fp16 TFLOPS per GPU at 8192^3; % of dense tensor peak"

# DRAM bytes per launch of the dominant kernel measured by ncu (dram__bytes_read.sum +
# dram__bytes_write.sum); None until a capture of that workload is summarised under profiles/.
NCU_TRAFFIC_BYTES = {
    "bf16_8192": 704302000 + 139248000,   # profiles/gemm_umma_bf16_8192x8192x8192.md
    "int8_8192": 317102848 + 231789312,   # profiles/gemm_umma_int8_8192x8192x8192.md
    "w8a8": 841799424 + 458604544,        # profiles/gemm_umma_w8a8_8192x28672x8192.md
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "burst": d["bf16_tflops"], "sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "burst": 1590.0, "sustained": 1400.0, "source": "fallback"}


# ----------------------------------------------------------------------------- clock sampling

class ClockSampler:
    """SM clock and clock-event reasons of one GPU, polled by a separate `nvidia-smi` process
    (every 100 ms) from before the warm-up until after the timed region.

    The poller is a process of its own on purpose: NVML queries issued from inside a rank (a
    sampling thread) take a lock that the rank's own kernel launches need, which slowed an
    8-rank step by 40 to 130 %.  Only rank 0 polls, and only its own GPU.  Because a timed
    region can be shorter than one polling period, the caller keeps the same load running,
    untimed, until the poller has had `min_seconds` of it."""

    FIELDS = ["clocks.sm", "clocks.max.sm", "clocks_event_reasons.hw_slowdown",
              "clocks_event_reasons.hw_thermal_slowdown", "clocks_event_reasons.sw_thermal_slowdown",
              "clocks_event_reasons.sw_power_cap"]

    def __init__(self, torch_device_index: int, enabled: bool = True, min_seconds: float = 0.8):
        self.proc, self.error, self.t_start, self.min_seconds = None, None, None, min_seconds
        self.out = ""
        if not enabled:
            self.error = "clocks are sampled on rank 0 only"
            return
        try:
            import subprocess

            import torch

            uuid = str(torch.cuda.get_device_properties(torch_device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", uuid, "--query-gpu=" + ",".join(self.FIELDS), "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t_start = time.perf_counter()
        except Exception as e:
            self.error = repr(e)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.out, _ = self.proc.communicate(timeout=5)
            except Exception:
                self.proc.kill()
            self.proc = None

    def summary(self):
        if self.error:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "error": self.error}
        clocks, max_mhz, reasons = [], None, set()
        for line in self.out.splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) != len(self.FIELDS):
                continue
            try:
                clocks.append(int(parts[0]))
                max_mhz = int(parts[1])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:]):
                if val == "Active":
                    reasons.add(name)
        loaded = sorted(clocks[1:] if len(clocks) > 2 else clocks)  # the first sample may predate the load
        med = loaded[len(loaded) // 2] if loaded else None
        return {"sm_mhz": med, "sm_max_mhz": max_mhz, "reasons": sorted(reasons), "samples": len(clocks),
                "how": "nvidia-smi -lms 100 in a separate process, from warm-up to the end of an untimed "
                       "continuation of the same load"}


# ----------------------------------------------------------------------------- workload set-up

def make_inputs(kind, M_local, N, K, device, seed, only_a=False):
    """Seeded synthetic inputs of the workload's distributions, resident on the device.  A (this
    rank's rows) depends on `seed`; B is the same on every rank.  only_a: B is not generated
    (returned as None)."""
    import torch

    g = torch.Generator(device=device).manual_seed(seed)
    gb = torch.Generator(device=device).manual_seed(999)
    extra, b = {}, None
    if kind in ("bf16", "f16"):
        dt = torch.bfloat16 if kind == "bf16" else torch.float16
        a = torch.randn((M_local, K), device=device, generator=g).to(dt)
        if not only_a:
            b = torch.randn((K, N), device=device, generator=gb).to(dt)
    elif kind == "i8":
        a = torch.randint(-127, 128, (M_local, K), dtype=torch.int8, device=device, generator=g)
        if not only_a:
            b = torch.randint(-127, 128, (K, N), dtype=torch.int8, device=device, generator=gb)
    else:  # w8a8: quantise N(0,1) fp32 sources with the library's own quantiser
        import cudaintro_b200 as cb

        x = torch.randn((M_local, K), device=device, generator=g)
        a, rs = cb.quantize_absmax(x, 0)
        del x
        extra = {"row_scale": rs}
        if not only_a:
            w = torch.randn((K, N), device=device, generator=gb)
            b, cs = cb.quantize_absmax(w, 1)
            del w
            extra["col_scale"] = cs
    return a, b, extra


def out_dtype(kind):
    import torch

    return {"bf16": torch.bfloat16, "f16": torch.float16, "i8": torch.int32, "w8a8": torch.bfloat16}[kind]


def launch(kind, a, b, c_slab, extra):
    import cudaintro_b200 as cb

    if kind == "bf16":
        cb.gemm_bf16(a, b, out=c_slab)
    elif kind == "f16":
        cb.gemm_f16(a, b, out=c_slab)
    elif kind == "i8":
        cb.gemm_i8_i32(a, b, out=c_slab)
    else:
        cb.gemm_w8a8_bf16(a, b, extra["row_scale"], extra["col_scale"], out=c_slab)


# ----------------------------------------------------------------------------- parity of the sharded result

def sharded_rows_parity(kind, c_full, b, extra, M, N, K, world, device):
    """Rank 0, outside any timed region: rows of the assembled C from EVERY rank's slab (first, last
    and one inner row of each) against the CPU oracle.  The other ranks' rows of A are regenerated
    here from their seeds (make_inputs is deterministic per seed and shape).  Bit-exact for the
    integer kinds; relative Frobenius error within the stated tolerance for bf16 / fp16.  Returns
    (ok, text): a short description, or which rows differed."""
    import numpy as np
    import torch

    import oracle as O

    slot = -(-M // world)
    checked = 0
    for r in range(world):
        row0 = min(M, r * slot)
        rows_r = max(0, min(M, (r + 1) * slot) - row0)
        if rows_r == 0:
            continue
        a_r, _, extra_r = make_inputs(kind, rows_r, N, K, device, seed=1234 + r, only_a=True)
        # first, last and an inner row of every slab; with one or two slabs also rows next to the 128- and
        # 256-row tile edges and more inner rows (about 16 rows in all)
        picks = {0, rows_r - 1, rows_r // 2}
        if world <= 2:
            picks |= {127, 128, 255, 256} | {(i * rows_r) // 6 for i in range(6)}
        elif world == 4:
            picks |= {255, 256}
        local = sorted(i for i in picks if 0 <= i < rows_r)
        got = c_full[[row0 + i for i in local]].cpu()
        a_np = a_r[local].cpu()
        if kind == "i8":
            want = O.gemm_i8_i32(a_np.numpy(), b.cpu().numpy(), len(local), N, K)
            ok = np.array_equal(got.numpy(), want)
        elif kind == "w8a8":
            want = O.gemm_w8a8_bf16(a_np.numpy(), b.cpu().numpy(), extra_r["row_scale"][local].cpu().numpy(),
                                    extra["col_scale"].cpu().numpy(), len(local), N, K)
            ok = np.array_equal(got.view(torch.int16).numpy().view(np.uint16), want)
        else:
            _, o32 = O.gemm_h16(a_np.view(torch.int16).numpy().view(np.uint16),
                                b.cpu().view(torch.int16).numpy().view(np.uint16), len(local), N, K, kind == "bf16")
            err = float(np.linalg.norm(got.float().numpy().astype(np.float64) - o32) / np.linalg.norm(o32))
            ok = err <= (1e-2 if kind == "bf16" else 2e-3)
        if not ok:
            return False, f"sharded {kind} GEMM: rows {local} of rank {r}'s slab differ from the CPU oracle"
        checked += len(local)
        del a_r, extra_r
    return True, f"oracle rows ok ({checked} rows from {world} slab(s), every rank's among them)"


# ----------------------------------------------------------------------------- CPU legs

def cpu_baseline_port(kind, M, N, K, target_seconds=10.0):
    """The oracle (OpenMP restatement of the reference loop) on a bounded row sample of the workload."""
    import numpy as np

    import oracle as O

    rng = np.random.default_rng(0)
    threads = O.num_threads()

    def run(rows):
        idx = np.arange(rows, dtype=np.int64)
        if kind in ("bf16", "f16"):
            a = rng.standard_normal((rows, K)).astype(np.float32)
            b = rng.standard_normal((K, N)).astype(np.float32)
            if kind == "bf16":
                ab, bb = O.f32_to_bf16_bits(a), O.f32_to_bf16_bits(b)
            else:
                ab, bb = a.astype(np.float16).view(np.uint16), b.astype(np.float16).view(np.uint16)
            t0 = time.perf_counter()
            O.gemm_h16(ab, bb, rows, N, K, kind == "bf16", O.ROW_MAJOR, idx)
            return time.perf_counter() - t0
        a = rng.integers(-127, 128, (rows, K)).astype(np.int8)
        b = rng.integers(-127, 128, (K, N)).astype(np.int8)
        if kind == "i8":
            t0 = time.perf_counter()
            O.gemm_i8_i32(a, b, rows, N, K, O.ROW_MAJOR, idx)
            return time.perf_counter() - t0
        rs = np.full(rows, 0.01, dtype=np.float32)
        cs = np.full(N, 0.01, dtype=np.float32)
        t0 = time.perf_counter()
        O.gemm_w8a8_bf16(a, b, rs, cs, rows, N, K, idx)
        return time.perf_counter() - t0

    probe_rows = max(threads, 8)
    t = run(probe_rows)
    rows = int(min(M, max(probe_rows, probe_rows * target_seconds / max(t, 1e-3))))
    rows = max(threads, rows // threads * threads)
    t = run(rows)
    ops = 2.0 * rows * N * K
    return {"value": ops / t / 1e12, "unit": WORKLOADS_UNIT[kind], "cores": threads, "kind": "port",
            "sample": f"{rows} of {M} rows of C (all N, all K) in {t:.2f} s; OpenMP restatement of the reference loop, "
                      f"linear in rows: full problem would take {t * M / rows:.0f} s"}


WORKLOADS_UNIT = {"bf16": "TFLOP/s", "f16": "TFLOP/s", "i8": "TOP/s", "w8a8": "TOP/s"}


def reference_arm(args, wl_name):
    """The reference's own CPU GEMM (matrixMulCPU, TileProgramming/tensor_utils.cu:35-45, built
    unmodified into oracle/_ref/) on the host cores.  The function is square, fp32 and single
    threaded, so a step runs T concurrent calls (one per host thread) on T distinct w x w x w
    sub-blocks of the workload, with the workload's values widened to fp32."""
    import numpy as np

    import oracle as O

    kind, M, N, K, _, _, unit = WORKLOADS[wl_name]
    threads = os.cpu_count() or 1
    have_ref = O.load_ref() is not None
    w = 384
    rng = np.random.default_rng(1)
    blocks = []
    for _ in range(threads):
        if kind in ("bf16", "f16"):
            a = rng.standard_normal((w, w)).astype(np.float32)
            b = rng.standard_normal((w, w)).astype(np.float32)
            if kind == "bf16":
                a, b = O.bf16_bits_to_f32(O.f32_to_bf16_bits(a)), O.bf16_bits_to_f32(O.f32_to_bf16_bits(b))
            else:
                a, b = a.astype(np.float16).astype(np.float32), b.astype(np.float16).astype(np.float32)
        else:
            a = rng.integers(-127, 128, (w, w)).astype(np.float32)
            b = rng.integers(-127, 128, (w, w)).astype(np.float32)
        blocks.append((a, b))

    def one(i):
        a, b = blocks[i]
        if have_ref:
            O.ref_matrix_mul_cpu(a, b, w)
        else:
            O.gemm_f32(a, b, w, w, w)

    def step():
        if have_ref:
            ts = [threading.Thread(target=one, args=(i,)) for i in range(threads)]
            for t in ts:
                t.start()
            for t in ts:
                t.join()
        else:  # the port is already parallel inside
            for i in range(threads):
                one(i)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    ops = 2.0 * w ** 3 * threads * args.steps
    value = ops / dt / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": {"bf16": "bf16", "f16": "f16", "i8": "int8", "w8a8": "int8"}[kind], "data": "synthetic",
        "config": {"workload": wl_name, "M": M, "N": N, "K": K},
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads,
                         "kind": "reference" if have_ref else "port",
                         "sample": f"each step = {threads} concurrent matrixMulCPU calls on distinct {w}^3 sub-blocks "
                                   f"of the {M}x{N}x{K} problem (values widened to fp32)"},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- failing together

_CLEANUPS = []  # callables that release peer-mapped / multicast-bound memory, newest last


def agree(ok, message, world, device):
    """Every rank calls this with its own verdict.  If any rank's check failed, ALL ranks release their
    peer-mapped and multicast-bound buffers in the same order, leave the process group and exit 1
    together: no rank is killed from outside while its memory is still bound to an NVLink multicast
    object or mapped by a peer."""
    import torch
    import torch.distributed as dist

    t = torch.tensor([1 if ok else 0], device=device, dtype=torch.int32)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if int(t.item()) == 1:
        return
    if not ok:
        print(message, file=sys.stderr, flush=True)
    torch.cuda.synchronize()
    for fn in reversed(_CLEANUPS):
        try:
            fn()
        except Exception as e:  # keep releasing the rest
            print(f"cleanup: {e!r}", file=sys.stderr, flush=True)
    _CLEANUPS.clear()
    if world > 1:
        dist.destroy_process_group()
    sys.exit(1)


# ----------------------------------------------------------------------------- the sharded W8A8 configuration

def timed_ms(fn, steps, barrier, warmup=3):
    """Average milliseconds per call of `fn` over `steps` back-to-back calls (CUDA events on the
    current stream), after `warmup` untimed calls and a barrier."""
    import torch

    for _ in range(warmup):
        fn()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def w8a8_sharded_record(world, rank, device, steps, barrier, max_over_ranks, multicast=False):
    """The row-sharded W8A8 linear (M=8192, N=28672, K=8192, bf16 out, C complete on every rank) on
    the GPUs of this run, whatever the main workload is: fused step, GEMM phase alone, NCCL
    all-gather alone, and the one-GPU time of the whole product measured on rank 0 in the same run,
    from which eff_compute = T1 / (G * T_gemm) and eff_e2e = T1 / (G * T_step) follow.  The
    assembled C is checked against the CPU oracle (rank 0, untimed) before anything is timed."""
    import torch

    import cudaintro_b200 as cb
    from cudaintro_b200 import capi
    from cudaintro_b200.sharded import FusedShardedGemm, ShardedGemm

    kind, M, N, K, in_b, out_b, unit = WORKLOADS["w8a8"]
    sharded = ShardedGemm(M, N, torch.bfloat16, device)
    M_local = sharded.part.rows
    a, b, extra = make_inputs(kind, M_local, N, K, device, seed=1234 + rank)
    ops = 2.0 * M * N * K
    rec = {"workload": "w8a8", "M": M, "N": N, "K": K, "n_gpus": world, "steps": steps, "unit": unit}

    def gemm_only():
        launch(kind, a, b, sharded.c_slab, extra)

    if world == 1:
        gemm_only()
        cb.check_device()
        ok, rec["parity"] = sharded_rows_parity(kind, sharded.result(), b, extra, M, N, K, 1, device)
        agree(ok, rec["parity"], 1, device)
        t1 = timed_ms(gemm_only, steps, barrier)
        cb.check_device()
        rec.update({"one_gpu_ms": t1, "step_ms": t1, "gemm_phase_ms": t1, "value": ops / (t1 * 1e-3) / 1e12,
                    "eff_compute": 1.0, "eff_e2e": 1.0})
        return rec

    fused = FusedShardedGemm(M, N, torch.bfloat16, device, multicast=multicast)
    _CLEANUPS.append(fused.close)
    rec["gather"] = "nvls (multimem.st to a multicast mapping)" if multicast else "fused (one TMA store per rank)"

    def fused_step():
        fused.step(capi.W8A8, a, b, extra["row_scale"], extra["col_scale"])

    sharded.step(lambda slab: launch(kind, a, b, slab, extra))
    fused_step()
    cb.check_device()
    barrier()
    agree(torch.equal(fused.result().view(torch.int16), sharded.result().view(torch.int16)),
          f"rank {rank}: W8A8 fused GEMM + all-gather differs from GEMM + NCCL all-gather", world, device)
    ok = True
    if rank == 0:
        ok, rec["parity"] = sharded_rows_parity(kind, fused.result(), b, extra, M, N, K, world, device)
    agree(ok, rec.get("parity", ""), world, device)
    step_ms = timed_ms(fused_step, steps, barrier)
    cb.check_device()
    barrier()
    gemm_ms = timed_ms(gemm_only, steps, barrier)
    barrier()
    gather_ms = timed_ms(sharded.gather, steps, barrier)
    barrier()
    step_ms, gemm_ms, gather_ms = max_over_ranks([step_ms, gemm_ms, gather_ms])
    # the whole product on one GPU (rank 0; the other ranks wait at the barrier)
    t1 = 0.0
    if rank == 0:
        a_full = torch.cat([make_inputs(kind, sharded.part.slot_rows, N, K, device, seed=1234 + r, only_a=True)[0]
                            for r in range(world)])[:M]
        rs_full = torch.ones(M, device=device)
        c_one = sharded.c_full[:M]
        one = {"row_scale": rs_full, "col_scale": extra["col_scale"]}
        t1 = timed_ms(lambda: launch(kind, a_full, b, c_one, one), steps, lambda: torch.cuda.synchronize())
        del a_full
    barrier()
    (t1,) = max_over_ranks([t1])
    c_bytes = M * N * out_b
    rec.update({
        "one_gpu_ms": t1, "step_ms": step_ms, "gemm_phase_ms": gemm_ms, "nccl_all_gather_ms": gather_ms,
        "gemm_plus_nccl_all_gather_ms": gemm_ms + gather_ms, "value": ops / (step_ms * 1e-3) / 1e12,
        "eff_compute": t1 / (world * gemm_ms), "eff_e2e": t1 / (world * step_ms),
        "ingress_gbs": c_bytes * (world - 1) / world / (step_ms * 1e-3) / 1e9,
        "nccl_bus_gbs": c_bytes * (world - 1) / world / (gather_ms * 1e-3) / 1e9,
        "note": "step = multi-destination GEMM (every tile stored into every rank's C over NVLink) + completion "
                "marker; every GPU receives (G-1)/G of C; eff_* against the one-GPU time of the same run"})
    fused.close()
    _CLEANUPS.remove(fused.close)
    return rec


# ----------------------------------------------------------------------------- main

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="bf16_8192", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-suite", action="store_true", help="skip the per-type side measurements")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-w8a8-record", action="store_true", help="skip the sharded W8A8 side record")
    ap.add_argument("--gather", default="auto", choices=["auto", "fused", "nvls", "nccl"],
                    help="N>1: auto = nvls for bf16 / fp16 outputs where the machine has NVLink multicast, else fused; fused = the GEMM epilogue stores each tile into every rank's C over NVLink (one TMA "
                         "store per rank); nvls = it writes each tile once with multimem.st to a multicast mapping "
                         "of C (replicated in the NVSwitch); nccl = GEMM, then NCCL all-gather")
    ap.add_argument("--clock-sampling", default="rank0", choices=["rank0", "off"],
                    help="rank0: a separate nvidia-smi process polls rank 0's GPU; off: no clock record")
    ap.add_argument("--multi-tile", default="", metavar="CG,BN",
                    help="force the tiling of every GEMM of the run (CTA grouping, tile width), e.g. 1,128; "
                         "for measurements of the multi-destination epilogue")
    ap.add_argument("--register-stores", action="store_true",
                    help="write C straight from registers instead of staged TMA stores (for comparison)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            reference_arm(args, args.workload)
        return 0

    import torch
    import torch.distributed as dist

    import cudaintro_b200 as cb
    from cudaintro_b200 import capi

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the GEMM suite has no CPU path")
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    kind, M, N, K, in_b, out_b, unit = WORKLOADS[args.workload]
    if args.register_stores:
        capi.set_store_policy(True)
    if args.multi_tile:
        cg_, bn_ = (int(x) for x in args.multi_tile.split(","))
        cb.set_tile_policy(cg_, bn_, 0)
    from cudaintro_b200.sharded import ShardedGemm

    sharded = ShardedGemm(M, N, out_dtype(kind), device)
    M_local = sharded.part.rows
    a, b, extra = make_inputs(kind, M_local, N, K, device, seed=1234 + rank)
    c_slab = sharded.c_slab

    def nccl_step():
        sharded.step(lambda slab: launch(kind, a, b, slab, extra))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # How C is completed on every rank.  auto: for 16-bit outputs of 16-bit products the epilogue writes each
    # tile once to a multicast mapping (fewer bytes leave the GPU; measured faster at 2, 4 and 8 GPUs), where the
    # machine offers one; store-heavy products (int32 or W8A8 outputs) are bound by what every GPU must take
    # in, which the multicast's loop-back copy only adds to, so they store once per rank with TMA.
    gather = args.gather
    if gather == "auto":
        gather = "nvls" if (world > 1 and kind in ("bf16", "f16")) else "fused"
    fused = None
    step = nccl_step
    if world > 1 and gather in ("fused", "nvls"):
        from cudaintro_b200.sharded import FusedShardedGemm

        if gather == "nvls":
            try:
                fused = FusedShardedGemm(M, N, out_dtype(kind), device, multicast=True)
            except RuntimeError as e:  # no multicast on this machine: the same on every rank
                if args.gather == "nvls":
                    raise
                if rank == 0:
                    print(f"multicast gather not available ({e}); using per-rank TMA stores", file=sys.stderr)
                gather = "fused"
        if fused is None:
            fused = FusedShardedGemm(M, N, out_dtype(kind), device)
        _CLEANUPS.append(fused.close)
        what = {"bf16": capi.BF16, "f16": capi.F16, "i8": capi.I8, "w8a8": capi.W8A8}[kind]

        def step():
            fused.step(what, a, b, extra.get("row_scale"), extra.get("col_scale"))

        # untimed check: the fused path must assemble what GEMM + NCCL all-gather assembles: bit for bit for
        # the integer kinds; to rounding for the 16-bit types, whose K order depends on the tiling, and the
        # single-destination GEMM of the NCCL path may run on other tiles than the multi-destination one
        nccl_step()
        step()
        barrier()
        if kind in ("i8", "w8a8"):
            same = torch.equal(fused.result().view(torch.uint8), sharded.result().view(torch.uint8))
        else:
            want = sharded.result().float()
            same = bool((fused.result().float() - want).norm() <= 1e-2 * want.norm())
            del want
        agree(same, f"rank {rank}: fused GEMM + all-gather differs from GEMM + NCCL all-gather", world, device)

    # untimed check of the assembled C against the CPU oracle: rows from every rank's slab
    if fused is None:
        nccl_step()
        barrier()
    ok, parity = True, None
    if rank == 0:
        ok, parity = sharded_rows_parity(kind, (fused or sharded).result(), b, extra, M, N, K, world, device)
    agree(ok, parity or "", world, device)

    clocks = ClockSampler(local_rank, enabled=(rank == 0 and args.clock_sampling != "off"))
    for _ in range(max(args.warmup, 3)):
        step()
    cb.check_device()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gemm_ms = 0.0
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    cb.check_device()
    # same load, untimed, until the clock poller has covered enough of it (all ranks take part:
    # a step involves every rank)
    extra_rounds = torch.zeros(1, dtype=torch.int32, device=device)
    if rank == 0 and clocks.proc is not None:
        per_round = max(ms / args.steps * 8 * 1e-3, 1e-4)
        extra_rounds[0] = int(max(0.0, clocks.min_seconds - (time.perf_counter() - clocks.t_start)) / per_round) + 1
    if world > 1:
        dist.broadcast(extra_rounds, src=0)
    for _ in range(int(extra_rounds.item()) * 8):
        step()
    barrier()
    clocks.stop()

    # Average duration of the GEMM kernel alone.  On one GPU a step is exactly one launch, so it
    # is the timed region itself; with a collective in the step it is measured right after.
    if world == 1:
        gemm_ms = ms / args.steps
    else:
        barrier()
        g0.record()
        for _ in range(args.steps):
            launch(kind, a, b, c_slab, extra)
        g1.record()
        torch.cuda.synchronize()
        gemm_ms = g0.elapsed_time(g1) / args.steps

    gather_ms = 0.0
    if world > 1:  # the all-gather alone, same buffers
        barrier()
        g0.record()
        for _ in range(args.steps):
            sharded.gather()
        g1.record()
        torch.cuda.synchronize()
        gather_ms = g0.elapsed_time(g1) / args.steps

    fused_kernel_ms = 0.0
    if fused is not None:  # the fused kernel without the completion marker that ends a step
        barrier()
        g0.record()
        for _ in range(args.steps):
            fused.launch(what, a, b, extra.get("row_scale"), extra.get("col_scale"))
        g1.record()
        torch.cuda.synchronize()
        fused_kernel_ms = g0.elapsed_time(g1) / args.steps

    t = torch.tensor([ms, gemm_ms, gather_ms, fused_kernel_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, gemm_ms, gather_ms, fused_kernel_ms = float(t[0]), float(t[1]), float(t[2]), float(t[3])
    fused_in_step = fused is not None

    ops_step = 2.0 * M * N * K
    value = ops_step * args.steps / (ms * 1e-3) / 1e12

    def max_over_ranks(values):
        tt = torch.tensor(values, device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return [float(x) for x in tt]

    # ---- end to end through the host-buffer C entry points (pinned memory, copies timed).
    # B (the operand every row of C needs; the weights of a linear layer) is uploaded once with
    # b200_host_weights_upload, outside the timed region; a step then moves this rank's rows of A up
    # and its rows of C down through b200_gemm_host_weights.
    e2e = None
    if kind != "w8a8" and not args.no_e2e:
        code = {"bf16": capi.BF16, "f16": capi.F16, "i8": capi.I8}[kind]
        ha = torch.empty((M_local, K), dtype=a.dtype).pin_memory()
        hb = torch.empty((K, N), dtype=b.dtype).pin_memory()
        hc = torch.empty((M_local, N), dtype=out_dtype(kind)).pin_memory()
        ha.copy_(a)
        hb.copy_(b)
        e2e_steps = min(args.steps, 20)
        weights = capi.HostWeights(code, hb, K, N)

        def host_call():
            weights.matmul(ha, hc, M_local)

        for _ in range(3):
            host_call()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            host_call()
        (dt,) = max_over_ranks([time.perf_counter() - t0])
        # rows of the result against the device-side product of the same operands
        # (bit for bit for int8; to rounding for the 16-bit types, whose K order depends on the tiling)
        dev_rows = sharded.c_slab[:8].cpu()
        same = torch.equal(hc[:8], dev_rows) if kind == "i8" else bool(
            (hc[:8].float() - dev_rows.float()).norm() <= 1e-2 * dev_rows.float().norm())
        agree(same, f"rank {rank}: host-buffer result differs from the device-buffer result", world, device)
        e2e = {"value": ops_step * e2e_steps / dt / 1e12, "unit": unit,
               "h2d_bytes_per_step": world * M_local * K * in_b, "d2h_bytes_per_step": M * N * out_b,
               "steps": e2e_steps, "ms_per_step": dt / e2e_steps * 1e3,
               "api": "b200_gemm_host_weights (pinned host buffers; B uploaded once by b200_host_weights_upload "
                      "before the timed region, every step moves each rank's rows of A up and its rows of C down)"}
        if world == 1:  # the call that moves both operands every time, for comparison
            def cold_call():
                st = capi.lib.b200_gemm_host(code, ha.data_ptr(), hb.data_ptr(), hc.data_ptr(), M_local, N, K,
                                             cb.ROW_MAJOR)
                if st:
                    raise cb.B200Error(st, capi.lib.b200_last_error().decode())

            cold_call()
            t0 = time.perf_counter()
            for _ in range(5):
                cold_call()
            dt = (time.perf_counter() - t0) / 5
            e2e["both_operands_every_step"] = {"value": ops_step / dt / 1e12, "ms_per_step": dt * 1e3,
                                               "h2d_bytes_per_step": (M * K + K * N) * in_b, "api": "b200_gemm_host"}
        weights.close()
        capi.lib.b200_host_release()
        del ha, hb, hc

    w8a8_rec = None
    if not args.no_w8a8_record:
        if fused is not None:
            fused.close()
            _CLEANUPS.remove(fused.close)
            fused = None
        if args.workload == "w8a8" and world == 1:
            w8a8_rec = None  # the main line already is that measurement
        else:
            torch.cuda.empty_cache()
            w8a8_rec = w8a8_sharded_record(world, rank, device, min(args.steps, 20), barrier, max_over_ranks,
                                           multicast=(args.gather == "nvls"))  # auto: per-rank TMA stores

    if rank != 0:
        if world > 1:
            if fused is not None:
                fused.close()
            dist.barrier()
            dist.destroy_process_group()
        return 0

    peaks = measured_peaks()
    timed_seconds = ms * 1e-3
    peak_kind = "sustained" if timed_seconds > 2.0 else "burst"
    scale = {"bf16": 1.0, "f16": 1.0, "i8": 2.0, "w8a8": 2.0}[kind]  # int8 runs at twice the bf16 rate
    peak = peaks[peak_kind] * scale
    gemm_ops = 2.0 * M_local * N * K
    achieved = gemm_ops / (gemm_ms * 1e-3) / 1e12
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
        "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
        "kernel": "gemm_umma_kernel", "avg_launch_ms": gemm_ms,
        "peak_source": f"{peaks['source']} cuBLAS bf16 {peak_kind}" + (" x2 for int8" if scale == 2.0 else ""),
        "frac_of_nominal": achieved / NOMINAL_PEAK[kind],
        "algorithmic_bytes_per_launch": (M_local * K + K * N) * in_b + M_local * N * out_b,
    }

    line = {
        "metric": METRIC, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None,
        "dtype": {"bf16": "bf16", "f16": "f16", "i8": "int8", "w8a8": "int8"}[kind], "data": "synthetic",
        "config": {"workload": args.workload, "M": M, "N": N, "K": K, "layout": "row-major",
                   "parallelism": f"rows of A over {world} GPU(s), B replicated" + (
                       "" if world == 1 else ((", tiles written once by the GEMM epilogue to a multicast mapping of C "
                                               "(multimem.st, replicated in the NVSwitch)") if gather == "nvls" else
                                              ", tiles stored into every rank's C by the GEMM epilogue (peer stores over NVLink)"
                                              if fused_in_step else ", NCCL all-gather of C")),
                   "l2": "inputs larger than L2 (no flush needed)" if (M_local * K + K * N) * in_b > 126e6
                         else "inputs fit L2: back-to-back launches re-use it"},
        "roofline": roofline,
        "clocks": clocks.summary(),
        # kernels of this library launched inside the timed region, all ranks together: one GEMM per
        # rank and step, plus the completion-marker kernel when the epilogue does the gather
        "gpu_launches": args.steps * world * (2 if fused_in_step else 1),
        "frac_of_nominal_peak": value / world / NOMINAL_PEAK[kind],
    }
    if e2e is not None:
        line["e2e"] = e2e
    if parity is not None:
        line["parity"] = parity
    if w8a8_rec is not None:
        line["w8a8_sharded"] = w8a8_rec
    if world > 1:
        line["gather"] = {"nvls": "multimem.st from the GEMM epilogue to a multicast mapping of C",
                          "fused": "one TMA store per rank from the GEMM epilogue (peer memory)",
                          "nccl": "GEMM, then NCCL all-gather"}[gather]
        line["gemm_phase"] = {"ms": gemm_ms, "value": ops_step / (gemm_ms * 1e-3) / 1e12, "unit": unit,
                              "note": "all ranks' GEMMs without the all-gather"}
        if fused_in_step:
            line["gemm_plus_nccl_all_gather_ms"] = gemm_ms + gather_ms
            line["fused_kernel_ms"] = fused_kernel_ms
            line["fused_ingress_gbs"] = M * N * out_b * (world - 1) / world / (ms / args.steps * 1e-3) / 1e9
        c_bytes = M * N * out_b
        line["all_gather"] = {"ms": gather_ms, "bytes_received_per_gpu": c_bytes * (world - 1) // world,
                              "bus_gbs": c_bytes * (world - 1) / world / (gather_ms * 1e-3) / 1e9,
                              "note": "NCCL all-gather of C alone; every GPU receives (G-1)/G of C over NVLink"}

    if world == 1 and not args.no_suite:
        line["suite"] = side_measurements(device, args.workload)
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline_port(kind, M, N, K)

    print(json.dumps(line), flush=True)
    if world > 1:
        if fused is not None:
            fused.close()
        dist.barrier()
        dist.destroy_process_group()
    return 0


def side_measurements(device, main_workload):
    """The other types of the metric at 8192^3 (and the W8A8 linear), each timed alone: best of 10
    single launches.  Also the vendor library's GEMM on the same shapes as a yardstick, its launches
    alternating with this library's."""
    import torch

    from cudaintro_b200 import capi

    out = {}
    for name in ("int8_8192", "bf16_8192", "fp16_8192", "w8a8"):
        kind, M, N, K, _, _, unit = WORKLOADS[name]
        a, b, extra = make_inputs(kind, M, N, K, device, seed=77)
        c = torch.empty((M, N), dtype=out_dtype(kind), device=device)
        what = {"bf16": capi.BF16, "f16": capi.F16, "i8": capi.I8, "w8a8": capi.W8A8}[kind]
        if kind in ("bf16", "f16"):
            vendor = lambda: torch.matmul(a, b)  # noqa: E731
        elif kind == "i8":
            vendor = lambda: torch._int_mm(a, b)  # noqa: E731
        else:
            vendor = None

        def vendor_ms():
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            vendor()
            e.record()
            torch.cuda.synchronize()
            return s.elapsed_time(e)

        def own_ms():
            return capi.time_gemm(what, a, b, c, M, N, K, iters=1, row_scale=extra.get("row_scale"),
                                  col_scale=extra.get("col_scale"))

        # Both implementations are warmed, then timed in turn (own, vendor, own, vendor, ...), so that
        # neither gets the cooler or the hotter half of the measurement.
        vendor_error = None
        try:
            for _ in range(3):
                own_ms()
                if vendor is not None:
                    vendor()
        except Exception as ex:  # the vendor call failing must not cost the own measurement
            vendor_error, vendor = repr(ex)[:120], None
        own, theirs = [], []
        for _ in range(10):
            own.append(own_ms())
            if vendor is not None:
                try:
                    theirs.append(vendor_ms())
                except Exception as ex:
                    vendor_error, vendor = repr(ex)[:120], None
        best = min(own)
        val = 2.0 * M * N * K / (best * 1e-3) / 1e12
        entry = {"value": val, "unit": unit, "ms": best, "frac_of_nominal_peak": val / NOMINAL_PEAK[kind]}
        if vendor_error is not None:
            entry["vendor_library"] = {"error": vendor_error}
        elif theirs:
            entry["vendor_library"] = {"value": 2.0 * M * N * K / (min(theirs) * 1e-3) / 1e12, "ms": min(theirs)}
        out[name] = entry
        del a, b, c, extra
        torch.cuda.empty_cache()
    # the remaining BASELINE shapes, one kernel each (see cudaintro_b200/measure.py)
    from cudaintro_b200 import measure

    keep = ("bound", "ms_best", "achieved", "unit", "peak", "frac")
    for name, res in measure.run_cases(
            ["int8_4096_colmajor", "linear_m16", "linear_m128", "linear_m1024", "linear_m4096", "fp32_1024_ffma",
             "fp32_1024_3xtf32", "quantize_rows_8192x8192", "quantize_cols_8192x28672"], reps=5, device=device).items():
        out[name] = {k: res[k] for k in keep if k in res}
    return out


if __name__ == "__main__":
    sys.exit(main())
