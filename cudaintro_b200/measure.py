"""Per-kernel measurements of the GEMM suite on one GPU.

    python -m cudaintro_b200.measure                 # every case, one JSON line each
    python -m cudaintro_b200.measure linear_m16 ...  # selected cases
    python -m cudaintro_b200.measure --list

Each case runs one entry point of the library on synthetic inputs of a BASELINE shape, timed
with CUDA events on the launching stream (3 warm-ups, then the median and best of `--reps`
single launches), and reports throughput against the bound that applies: tensor peak for the
large products, HBM bandwidth for the small-M linear layers and the quantiser, the FP32 pipe for
the FFMA kernel.  Cases whose operands would fit in L2 rotate through enough copies of the large
operand to exceed it, so that HBM and not L2 is measured.  The same commands are what the ncu
summaries under profiles/ were captured from (`--reps 1 --warmup 1` keeps a capture short).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

L2_BYTES = 126e6
NOMINAL = {"bf16": 2250.0, "f16": 2250.0, "i8": 4500.0, "w8a8": 4500.0, "tf32x3": 1125.0 / 3}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def _time(fn, reps, warmup):
    """(median, best) milliseconds per call.  Calls are timed in back-to-back batches long enough
    (about half a millisecond) that the gap between the host recording the first event and the
    first kernel reaching the GPU does not count as kernel time."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()

    def batch(n):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(n):
            fn()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / n

    if reps <= 1:
        return (batch(1),) * 2
    per_call = batch(4)
    inner = max(1, min(64, int(0.5 / max(per_call, 1e-3))))
    ts = sorted(batch(inner) for _ in range(reps))
    return ts[len(ts) // 2], ts[0]


def _randn(shape, dtype, device, seed, scale=1.0):
    import torch

    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(shape, device=device, generator=g) * scale).to(dtype)


def _randint8(shape, device, seed):
    import torch

    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randint(-127, 128, shape, dtype=torch.int8, device=device, generator=g)


def case_gemm(kind, M, N, K, layout_name="ROW_MAJOR"):
    """Large tensor-core products: bf16 / f16 / i8 (int32 out)."""
    def run(args, device):
        import torch

        import cudaintro_b200 as cb

        layout = getattr(cb, layout_name)
        sa, sb = ((M, K), (K, N)) if layout == cb.ROW_MAJOR else ((K, M), (N, K))
        if kind == "i8":
            a, b = _randint8(sa, device, 1), _randint8(sb, device, 2)
            fn = lambda: cb.gemm_i8_i32(a, b, layout, out=c)  # noqa: E731
            c = torch.empty((M, N) if layout == cb.ROW_MAJOR else (N, M), dtype=torch.int32, device=device)
        else:
            dt = torch.bfloat16 if kind == "bf16" else torch.float16
            a, b = _randn(sa, dt, device, 1), _randn(sb, dt, device, 2)
            c = torch.empty((M, N) if layout == cb.ROW_MAJOR else (N, M), dtype=dt, device=device)
            fn = (lambda: cb.gemm_bf16(a, b, layout, out=c)) if kind == "bf16" else (lambda: cb.gemm_f16(a, b, layout, out=c))
        med, best = _time(fn, args.reps, args.warmup)
        cb.check_device()
        ops = 2.0 * M * N * K
        _, tpeak, src = _peaks()
        peak = tpeak * (2.0 if kind == "i8" else 1.0)
        return {"bound": "tensor", "ms_median": med, "ms_best": best, "achieved": ops / (best * 1e-3) / 1e12,
                "unit": "TOP/s" if kind == "i8" else "TFLOP/s", "peak": peak,
                "peak_source": f"{src} cuBLAS bf16 burst" + (" x2" if kind == "i8" else ""),
                "frac": ops / (best * 1e-3) / 1e12 / peak, "frac_of_nominal": ops / (best * 1e-3) / 1e12 / NOMINAL[kind],
                "algorithmic_bytes": (M * K + K * N) * a.element_size() + M * N * c.element_size()}
    return run


def case_linear(M, K=4096, N=11008):
    """fp16 activations [M,K] ~ N(0,1) times weights [K,N] ~ N(0,0.02): the decode-to-prefill sweep."""
    def run(args, device):
        import torch

        import cudaintro_b200 as cb

        x = _randn((M, K), torch.float16, device, 1)
        copies = max(1, int(L2_BYTES * 3 // (K * N * 2)) + 1) if M <= 1024 else 1
        ws = [_randn((K, N), torch.float16, device, 10 + i, 0.02) for i in range(copies)]
        out = torch.empty((M, N), dtype=torch.float16, device=device)
        state = {"i": 0}

        def fn():
            cb.gemm_f16(x, ws[state["i"] % copies], out=out)
            state["i"] += 1

        med, best = _time(fn, max(args.reps, copies), max(args.warmup, copies))
        cb.check_device()
        byts = (M * K + K * N + M * N) * 2
        ops = 2.0 * M * N * K
        hbm, tpeak, src = _peaks()
        hbm_bound = byts / (hbm * 1e9) > ops / (tpeak * 1e12)
        res = {"bound": "hbm" if hbm_bound else "tensor", "ms_median": med, "ms_best": best,
               "algorithmic_bytes": byts, "weight_copies_rotated": copies,
               "gbs": byts / (med * 1e-3) / 1e9, "tflops": ops / (med * 1e-3) / 1e12}
        if hbm_bound:
            res.update(achieved=res["gbs"], unit="GB/s", peak=hbm, peak_source=f"{src} HBM copy", frac=res["gbs"] / hbm)
        else:
            res.update(achieved=res["tflops"], unit="TFLOP/s", peak=tpeak, peak_source=f"{src} cuBLAS bf16 burst",
                       frac=res["tflops"] / tpeak)
        return res
    return run


def case_w8a8(M=8192, N=28672, K=8192):
    def run(args, device):
        import torch

        import cudaintro_b200 as cb

        a, b = _randint8((M, K), device, 1), _randint8((K, N), device, 2)
        rs = torch.rand(M, device=device) * 0.01 + 0.001
        cs = torch.rand(N, device=device) * 0.01 + 0.001
        c = torch.empty((M, N), dtype=torch.bfloat16, device=device)
        med, best = _time(lambda: cb.gemm_w8a8_bf16(a, b, rs, cs, out=c), args.reps, args.warmup)
        cb.check_device()
        ops = 2.0 * M * N * K
        _, tpeak, src = _peaks()
        return {"bound": "tensor", "ms_median": med, "ms_best": best, "achieved": ops / (best * 1e-3) / 1e12,
                "unit": "TOP/s", "peak": 2 * tpeak, "peak_source": f"{src} cuBLAS bf16 burst x2",
                "frac": ops / (best * 1e-3) / 1e12 / (2 * tpeak), "frac_of_nominal": ops / (best * 1e-3) / 1e12 / 4500.0,
                "algorithmic_bytes": M * K + K * N + 2 * M * N + 4 * (M + N)}
    return run


def case_w8a8_decode(M, K=4096, N=11008):
    """int8 activations [M,K] times int8 weights [K,N] with per-row x per-column scales, bf16 out: the
    quantised form of the decode-shape linear layer.  Weight copies are rotated so that they come from DRAM."""
    def run(args, device):
        import torch

        import cudaintro_b200 as cb

        x = _randint8((M, K), device, 1)
        copies = int(L2_BYTES * 3 // (K * N)) + 1
        ws = [_randint8((K, N), device, 10 + i) for i in range(copies)]
        rs = torch.rand(M, device=device) * 0.01 + 0.001
        cs = torch.rand(N, device=device) * 0.01 + 0.001
        out = torch.empty((M, N), dtype=torch.bfloat16, device=device)
        state = {"i": 0}

        def fn():
            cb.gemm_w8a8_bf16(x, ws[state["i"] % copies], rs, cs, out=out)
            state["i"] += 1

        med, best = _time(fn, max(args.reps, copies), max(args.warmup, copies))
        cb.check_device()
        byts = M * K + K * N + 2 * M * N + 4 * (M + N)
        hbm, _, src = _peaks()
        return {"bound": "hbm", "ms_median": med, "ms_best": best, "algorithmic_bytes": byts,
                "weight_copies_rotated": copies, "achieved": byts / (med * 1e-3) / 1e9, "unit": "GB/s", "peak": hbm,
                "peak_source": f"{src} HBM copy", "frac": byts / (med * 1e-3) / 1e9 / hbm}
    return run


def case_f32(n, mode_name):
    def run(args, device):
        import torch

        import cudaintro_b200 as cb

        a = cb.fill(torch.empty((n, n), dtype=torch.float32, device=device), 0x3234)
        b = cb.fill(torch.empty((n, n), dtype=torch.float32, device=device), 0x7776)
        c = torch.empty((n, n), dtype=torch.float32, device=device)
        mode = getattr(cb, mode_name)
        med, best = _time(lambda: cb.gemm_f32(a, b, mode=mode, out=c), args.reps, args.warmup)
        cb.check_device()
        ops = 2.0 * n ** 3
        sms = cb.lib.b200_sm_count()
        ffma_peak = sms * 128 * 2 * 1.965e9 / 1e12  # FP32 lanes x 2 flop x max SM clock
        if mode_name == "F32_FFMA":
            peak, src = ffma_peak, f"{sms} SMs x 128 FP32 lanes x 2 x 1.965 GHz"
        elif mode_name == "F32_TF32":
            peak, src = 1125.0, "nominal dense tf32"
        else:
            peak, src = NOMINAL["tf32x3"], "nominal dense tf32 / 3 products per term"
        return {"bound": "fp32 pipe" if mode_name == "F32_FFMA" else "tensor", "ms_median": med, "ms_best": best,
                "achieved": ops / (best * 1e-3) / 1e12, "unit": "TFLOP/s", "peak": peak, "peak_source": src,
                "frac": ops / (best * 1e-3) / 1e12 / peak, "algorithmic_bytes": 3 * n * n * 4}
    return run


def case_fc(batch, in_f, out_f, mode_name):
    """The hidden layer of the reference's two-layer network (784 -> 512 on a batch of 20000, weights
    [in, out], bias, ReLU) as one fused launch; `torch_ms` is the same layer as three torch calls."""
    def run(args, device):
        import torch

        import cudaintro_b200 as cb

        x = _randn((batch, in_f), torch.float32, device, 1)
        w = _randn((in_f, out_f), torch.float32, device, 2, 0.05)
        b = _randn((out_f,), torch.float32, device, 3, 0.1)
        y = torch.empty((batch, out_f), dtype=torch.float32, device=device)
        mode = getattr(cb, mode_name)
        med, best = _time(lambda: cb.linear(x, w, b, cb.ROW_MAJOR, relu=True, bias_first=True, mode=mode, out=y),
                          args.reps, args.warmup)
        cb.check_device()
        torch.backends.cuda.matmul.allow_tf32 = mode_name != "F32_FFMA"
        tmed, _ = _time(lambda: torch.relu(torch.addmm(b, x, w)), args.reps, args.warmup)
        torch.backends.cuda.matmul.allow_tf32 = False
        ops = 2.0 * batch * in_f * out_f
        sms = cb.lib.b200_sm_count()
        if mode_name == "F32_FFMA":
            peak, src, bound = sms * 128 * 2 * 1.965e9 / 1e12, f"{sms} SMs x 128 FP32 lanes x 2 x 1.965 GHz", "fp32 pipe"
        else:
            peak, src, bound = 1125.0, "nominal dense tf32", "tensor"
        return {"bound": bound, "ms_median": med, "ms_best": best, "achieved": ops / (best * 1e-3) / 1e12,
                "unit": "TFLOP/s", "peak": peak, "peak_source": src, "frac": ops / (best * 1e-3) / 1e12 / peak,
                "algorithmic_bytes": 4 * (batch * in_f + in_f * out_f + out_f + batch * out_f), "torch_ms_median": tmed}
    return run


def case_quantize(R, C, along):
    def run(args, device):
        import cudaintro_b200 as cb
        import torch

        x = _randn((R, C), torch.float32, device, 3)
        med, best = _time(lambda: cb.quantize_absmax(x, along), args.reps, args.warmup)
        # Per-row scales: a row is read once (it stays in registers between the two passes) and
        # written once: 5 B per element.  Per-column scales of a matrix far larger than L2 need the
        # maxima of all rows before the first element can be quantised: two reads and one write, 9 B.
        per_elem = 5 if along == 0 else 9
        byts = R * C * per_elem + 4 * (R if along == 0 else C)
        hbm, _, src = _peaks()
        return {"bound": "hbm", "ms_median": med, "ms_best": best, "achieved": byts / (med * 1e-3) / 1e9, "unit": "GB/s",
                "peak": hbm, "peak_source": f"{src} HBM copy", "frac": byts / (med * 1e-3) / 1e9 / hbm,
                "algorithmic_bytes": byts, "bytes_per_element": per_elem}
    return run


CASES = {
    "bf16_8192": case_gemm("bf16", 8192, 8192, 8192),
    "fp16_8192": case_gemm("f16", 8192, 8192, 8192),
    "int8_8192": case_gemm("i8", 8192, 8192, 8192),
    "int8_4096": case_gemm("i8", 4096, 4096, 4096),
    "int8_4096_colmajor": case_gemm("i8", 4096, 4096, 4096, "COL_MAJOR_NN"),
    "bf16_4096_colmajor": case_gemm("bf16", 4096, 4096, 4096, "COL_MAJOR_NN"),
    "fp16_4096_colmajor": case_gemm("f16", 4096, 4096, 4096, "COL_MAJOR_NN"),
    "w8a8": case_w8a8(),
    "w8a8_decode_m16": case_w8a8_decode(16),
    "w8a8_decode_m128": case_w8a8_decode(128),
    "linear_m16": case_linear(16),
    "linear_m128": case_linear(128),
    "linear_m1024": case_linear(1024),
    "linear_m4096": case_linear(4096),
    "fp32_1024_ffma": case_f32(1024, "F32_FFMA"),
    "fp32_4096_ffma": case_f32(4096, "F32_FFMA"),
    "fp32_1024_3xtf32": case_f32(1024, "F32_3XTF32"),
    "fp32_4096_3xtf32": case_f32(4096, "F32_3XTF32"),
    "fp32_1024_tf32": case_f32(1024, "F32_TF32"),
    "fp32_4096_tf32": case_f32(4096, "F32_TF32"),
    "fc_20000x784x512_ffma": case_fc(20000, 784, 512, "F32_FFMA"),
    "fc_20000x784x512_tf32": case_fc(20000, 784, 512, "F32_TF32"),
    "quantize_rows_8192x8192": case_quantize(8192, 8192, 0),
    "quantize_cols_8192x28672": case_quantize(8192, 28672, 1),
}


def run_cases(names, reps=10, warmup=3, device=None):
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("measure needs a CUDA device: the GEMM suite has no CPU path")
    device = device or torch.device("cuda", torch.cuda.current_device())
    ns = argparse.Namespace(reps=reps, warmup=warmup)
    out = {}
    for name in names:
        res = CASES[name](ns, device)
        res["case"] = name
        out[name] = res
        torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("cases", nargs="*")
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--policy", default="", help="tile policy for every case: cta_group,tile_n (e.g. 1,128 forces the "
                    "general kernel with 128-wide tiles, 3,0 the skinny K-split kernel); default: automatic")
    args = ap.parse_args()
    if args.list:
        print("\n".join(CASES))
        return 0
    names = args.cases or list(CASES)
    for n in names:
        if n not in CASES:
            raise SystemExit(f"unknown case {n!r}; try --list")
    if args.policy:
        import cudaintro_b200 as cb

        cg, bn = (int(v) for v in args.policy.split(","))
        cb.set_tile_policy(cg, bn, 0)
    for name in names:
        res = run_cases([name], args.reps, args.warmup)[name]
        if args.policy:
            res["tile_policy"] = args.policy
        print(json.dumps(res), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
