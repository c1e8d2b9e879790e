"""Generates the golden fixtures of this directory from the REFERENCE's own code.

Run where the reference tree is mounted (it is not needed to *use* the fixtures):

    make -C oracle ref REF=<reference tree>
    python tests/golden/make_golden.py

For every case the inputs come from a seeded numpy generator and the expected output from the
reference's unmodified ``matrixMulCPU`` (TileProgramming/tensor_utils.cu:35-45, compiled into
``oracle/_ref/libref_matmulcpu.so``).  The 8-bit and 16-bit cases feed it the widened values:

* int8 values are exact in fp32 and, for K <= 1024, every partial sum stays below 2**24, so the
  fp32 loop returns the exact integers an int32 accumulator holds;
* the product of two bf16 (or two fp16) numbers is exact in fp32, so the fp32 loop over widened
  inputs is exactly "fp32 accumulate in ascending k" before the final rounding to 16 bits.

Each fixture is one ``.npz`` with the raw inputs, the reference output and the seed.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle as O  # noqa: E402


def main():
    if O.load_ref() is None:
        raise SystemExit("build the reference loop first: make -C oracle ref REF=<reference tree>")
    rng = np.random.default_rng(20240607)

    for w in (32, 96):
        a = rng.uniform(-1, 1, (w, w)).astype(np.float32)
        b = rng.uniform(-1, 1, (w, w)).astype(np.float32)
        np.savez_compressed(os.path.join(HERE, f"ref_f32_{w}.npz"), a=a, b=b, c=O.ref_matrix_mul_cpu(a, b, w))

    # the reference driver's own distribution: rand()/RAND_MAX in [0, 1] (TileProgramming/tensor_utils.h:60)
    w = 64
    a = rng.uniform(0, 1, (w, w)).astype(np.float32)
    b = rng.uniform(0, 1, (w, w)).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "ref_f32_unit_64.npz"), a=a, b=b, c=O.ref_matrix_mul_cpu(a, b, w))

    w = 128
    a = rng.integers(-127, 128, (w, w)).astype(np.int8)
    b = rng.integers(-127, 128, (w, w)).astype(np.int8)
    c = O.ref_matrix_mul_cpu(a.astype(np.float32), b.astype(np.float32), w)
    assert np.all(c == np.rint(c))
    np.savez_compressed(os.path.join(HERE, "ref_i8_128.npz"), a=a, b=b, c=c.astype(np.int32))

    # the suite's own int8 generator (quantization/GEMM_int8.cu:8-19, seeds :44-45), 64 x 64
    w = 64
    a = O.fill_int8(w * w, 0x4234).reshape(w, w)
    b = O.fill_int8(w * w, 0x6676).reshape(w, w)
    c = O.ref_matrix_mul_cpu(a.astype(np.float32), b.astype(np.float32), w)
    np.savez_compressed(os.path.join(HERE, "ref_i8_suitefill_64.npz"), a=a, b=b, c=c.astype(np.int32))

    w = 96
    for name, to_bits, widen in (
        ("bf16", O.f32_to_bf16_bits, O.bf16_bits_to_f32),
        ("f16", lambda x: x.astype(np.float16).view(np.uint16), O.f16_bits_to_f32),
    ):
        a = to_bits(rng.standard_normal((w, w)).astype(np.float32))
        b = to_bits(rng.standard_normal((w, w)).astype(np.float32))
        c32 = O.ref_matrix_mul_cpu(widen(a), widen(b), w)
        np.savez_compressed(os.path.join(HERE, f"ref_{name}_{w}.npz"), a=a, b=b, c32=c32)
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    main()
