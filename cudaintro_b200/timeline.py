"""Per-k-block timeline of the skinny (at most 128 rows) tensor-core kernel.

    python -m cudaintro_b200.build --stamps      # once: the measurement build of the library
    python -m cudaintro_b200.timeline            # one JSON line per case
    python -m cudaintro_b200.timeline --umma     # wait accounting of the large tensor-core kernel instead

The measurement build (``libb200gemm_stamps.so``, compiled with ``-DB200_SKINNY_STAMPS``) makes every CTA of
``gemm_skinny_kernel`` record ``%globaltimer`` (32 ns resolution) for its first 64 k-blocks at four points:
the load-issuing lane after its wait for a free stage and after issuing the stage's TMA loads, the
MMA-issuing lane after its wait for the full stage and after issuing the stage's MMAs and commit; and once
per CTA the phases of the tail (accumulator complete, moved to the exchange slots, barrier, sums stored).  This script
runs the fp16 linear layer [4096 -> 11008] of the decode sweep through that build (weights rotated through
five copies so that they come from HBM), back to back, and reduces the stamps of the last launch to
percentiles and a histogram of the time between consecutive "stage full" events of a CTA.  The stamps
themselves cost two timer reads and two global stores per k-block and lane (about 30 ns per k-block).
"""
from __future__ import annotations

import ctypes as C
import json
import os
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(PKG, "libb200gemm_stamps.so")
CASES = ((16, 0), (64, 0), (128, 192), (128, 128))  # (rows M, forced tile width of the skinny kernel; 0 = its own choice)


def main() -> int:
    import numpy as np
    import torch

    if not os.path.exists(LIB):
        raise SystemExit("build the measurement library first: python -m cudaintro_b200.build --stamps")
    lib = C.CDLL(LIB)
    lib.b200_last_error.restype = C.c_char_p
    i64, p = C.c_int64, C.c_void_p
    lib.b200_gemm_f16.argtypes = [p, p, p, i64, i64, i64, i64, i64, i64, C.c_int, p]
    lib.b200_set_tile_policy.argtypes = [C.c_int, C.c_int, C.c_int]
    lib.b200_debug_set_skinny_stamps.argtypes = [p]
    lib.b200_check_device.argtypes = [p]
    dev = "cuda"
    K, N = 4096, 11008
    for M, bn in CASES:
        g = torch.Generator(device=dev).manual_seed(M)
        x = torch.randn((M, K), device=dev, generator=g).half()
        ws = [(torch.randn((K, N), device=dev, generator=g) * 0.02).half() for _ in range(5)]
        y = torch.empty((M, N), device=dev, dtype=torch.float16)
        if lib.b200_set_tile_policy(3, bn, 0) != 0:
            raise SystemExit(lib.b200_last_error().decode())
        stamps = torch.zeros((148 * 2, 6, 64), dtype=torch.int64, device=dev)
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)

        def run(w):
            if lib.b200_gemm_f16(x.data_ptr(), w.data_ptr(), y.data_ptr(), M, N, K, 0, 0, 0, 0, st) != 0:
                raise SystemExit(lib.b200_last_error().decode())

        for i in range(6):
            run(ws[i % 5])
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for i in range(50):
            run(ws[i % 5])
        e.record()
        torch.cuda.synchronize()
        per = s.elapsed_time(e) / 50 * 1e3
        lib.b200_debug_set_skinny_stamps(stamps.data_ptr())
        for i in range(3):  # back to back: the last launch's stamps survive
            run(ws[i % 5])
        torch.cuda.synchronize()
        lib.b200_debug_set_skinny_stamps(None)
        if lib.b200_check_device(st) != 0:
            raise SystemExit(lib.b200_last_error().decode())
        t = stamps.cpu().numpy()
        t = t[[c for c in range(t.shape[0]) if t[c, 4, 0] != 0]]
        nkb = int((t[0, 0] != 0).sum())

        def q(a):
            return [round(float(v), 3) for v in np.percentile(a, [10, 50, 90, 99])]

        full_to_full = np.diff(t[:, 2, :nkb], axis=1) / 1e3
        hist, edges = np.histogram(full_to_full, bins=[0, .3, .4, .5, .6, .8, 1.0, 1.5, 100])
        rec = {
            "M": M, "forced_tile_width": bn, "ctas": int(t.shape[0]), "kblocks_per_cta": nkb,
            "us_per_launch_back_to_back_in_this_build": round(per, 2),
            "percentiles": "p10, p50, p90, p99 in us",
            "dependency_wait_to_first_stage_full": q((t[:, 2, 0] - t[:, 4, 0]) / 1e3),
            "stage_full_to_next_stage_full": q(full_to_full),
            "loads_issued_to_stage_full": q((t[:, 2, :nkb] - t[:, 1, :nkb]) / 1e3),
            "load_lane_free_stage_to_loads_issued": q((t[:, 1, :nkb] - t[:, 0, :nkb]) / 1e3),
            "load_lane_loads_issued_to_next_free_stage": q((t[:, 0, 1:nkb] - t[:, 1, :nkb - 1]) / 1e3),
            "mma_lane_stage_full_to_mmas_issued": q((t[:, 3, :nkb] - t[:, 2, :nkb]) / 1e3),
            "first_full_to_last_mma_issued_median_us": round(float(np.median(t[:, 3, nkb - 1] - t[:, 2, 0]) / 1e3), 2),
            "tail_last_mma_issued_to_accumulator_complete": q((t[:, 5, 0] - t[:, 3, nkb - 1]) / 1e3),
            "tail_tensor_memory_to_exchange_slots": q((t[:, 5, 1] - t[:, 5, 0]) / 1e3),
            "tail_barrier": q((t[:, 5, 2] - t[:, 5, 1]) / 1e3),
            "tail_sum_convert_store": q((t[:, 5, 3] - t[:, 5, 2]) / 1e3),
            "launch_span_first_cta_start_to_last_cta_end_us": round(float((t[:, 5, 3].max() - t[:, 4, 0].min()) / 1e3), 2),
            "histogram_stage_full_to_next_stage_full": {f"{edges[i]:.1f}-{edges[i + 1]:.1f} us": int(h)
                                                        for i, h in enumerate(hist)},
        }
        print(json.dumps(rec), flush=True)
    lib.b200_set_tile_policy(0, 0, 0)
    return 0


def umma_waits() -> int:
    """Wait accounting of the large tensor-core kernel (``python -m cudaintro_b200.timeline --umma``).

    In the measurement build every CTA of ``gemm_umma_kernel`` adds up SM cycles per role: the MMA lane
    waiting for full stages and for free accumulators and its whole loop, the producer lane waiting for
    free stages, the epilogue from "accumulator complete" to "accumulator handed back".  One JSON line
    per (type, shape, tiling): bf16 and int8 at 8192^3 and 4096^3 on 256-row and on 512-row CTA-pair tiles."""
    import torch

    if not os.path.exists(LIB):
        raise SystemExit("build the measurement library first: python -m cudaintro_b200.build --stamps")
    lib = C.CDLL(LIB)
    lib.b200_last_error.restype = C.c_char_p
    i64, p = C.c_int64, C.c_void_p
    for name in ("b200_gemm_bf16", "b200_gemm_i8_i32"):
        getattr(lib, name).argtypes = [p, p, p, i64, i64, i64, i64, i64, i64, C.c_int, p]
    lib.b200_set_tile_policy.argtypes = [C.c_int, C.c_int, C.c_int]
    lib.b200_debug_set_umma_waits.argtypes = [p]
    dev = "cuda"
    for kind in ("bf16", "int8"):
        for n in (8192, 4096):
            if kind == "bf16":
                a = torch.randn((n, n), device=dev).bfloat16()
                b = torch.randn((n, n), device=dev).bfloat16()
                c = torch.empty((n, n), device=dev, dtype=torch.bfloat16)
                fn = lib.b200_gemm_bf16
            else:
                a = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=dev)
                b = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=dev)
                c = torch.empty((n, n), device=dev, dtype=torch.int32)
                fn = lib.b200_gemm_i8_i32
            for cta_group, rows in ((2, 256), (4, 512)):
                if lib.b200_set_tile_policy(cta_group, 256, 0) != 0:
                    raise SystemExit(lib.b200_last_error().decode())
                waits = torch.zeros((148, 16), dtype=torch.int64, device=dev)
                for _ in range(3):
                    if fn(a.data_ptr(), b.data_ptr(), c.data_ptr(), n, n, n, 0, 0, 0, 0, None) != 0:
                        raise SystemExit(lib.b200_last_error().decode())
                torch.cuda.synchronize()
                lib.b200_debug_set_umma_waits(waits.data_ptr())
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                for _ in range(5):  # back to back: the last launch's record survives
                    fn(a.data_ptr(), b.data_ptr(), c.data_ptr(), n, n, n, 0, 0, 0, 0, None)
                stop.record()
                torch.cuda.synchronize()
                lib.b200_debug_set_umma_waits(None)
                t = waits.cpu().double()
                lead = t[0::2]  # the even CTA of a pair issues the MMAs
                loop = lead[:, 2].mean().item()
                print(json.dumps({
                    "type": kind, "shape": [n, n, n], "tile_rows": rows,
                    "us_per_launch": round(start.elapsed_time(stop) / 5 * 1e3, 1),
                    "mma_loop_cycles": round(loop),
                    "mma_waiting_full_pct": round(lead[:, 0].mean().item() / loop * 100, 1),
                    "k_blocks_not_yet_full_when_asked": round(lead[:, 7].mean().item()),
                    "mma_waiting_accumulator_pct": round(lead[:, 1].mean().item() / loop * 100, 1),
                    "producer_waiting_free_stage_pct": round(t[:, 3].mean().item() / max(t[:, 4].mean().item(), 1) * 100, 1),
                    "epilogue_complete_to_handed_back_cycles": round(t[:, 8].mean().item()),
                }), flush=True)
    lib.b200_set_tile_policy(0, 0, 0)
    return 0


if __name__ == "__main__":
    sys.exit(umma_waits() if "--umma" in sys.argv else main())
