"""GPU tests of the two epilogue store paths (staged TMA stores / register stores) and of the
multi-destination GEMM that the sharded path uses to place its tiles in every rank's C.
On one GPU the destinations are several local buffers; the 2-GPU test maps real peer memory."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def to_dev(x, device, dtype=None):
    import torch

    t = torch.from_numpy(np.ascontiguousarray(x)).to(device)
    return t.view(dtype) if dtype is not None else t


@pytest.fixture
def policies(cb):
    from cudaintro_b200 import capi

    yield cb.set_tile_policy, capi.set_store_policy
    cb.set_tile_policy(0, 0, 0)
    capi.set_store_policy(False)


@pytest.mark.parametrize("register_stores", [False, True])
@pytest.mark.parametrize("cg,bn", [(1, 256), (1, 128), (1, 64), (2, 256)])
@pytest.mark.parametrize("shape", [(200, 328, 256), (520, 1040, 1024), (128, 32, 64), (257, 8, 128)])
def test_store_paths_bit_exact_int8_and_w8a8(cb, oracle, device, policies, shape, cg, bn, register_stores):
    import torch

    set_tiles, set_stores = policies
    M, N, K = shape
    rng = np.random.default_rng(M * 7 + N * 3 + K + cg + bn)
    a = rng.integers(-127, 128, (M, K)).astype(np.int8)
    b_t = rng.integers(-127, 128, (N, K)).astype(np.int8)  # [N, K]: any N works for the int8 tile widths
    set_tiles(cg, bn, 0)
    set_stores(register_stores)
    c = cb.gemm_i8_i32(to_dev(a, device), to_dev(b_t, device), cb.ROW_MAJOR_BT)
    cb.check_device()
    want = oracle.gemm_i8_i32(a, np.ascontiguousarray(b_t.T), M, N, K)
    assert np.array_equal(c.cpu().numpy(), want)
    if N % 16 == 0 and bn >= 128:
        b = np.ascontiguousarray(b_t.T)
        sx = rng.uniform(0.001, 0.02, M).astype(np.float32)
        sw = rng.uniform(0.001, 0.02, N).astype(np.float32)
        cw = cb.gemm_w8a8_bf16(to_dev(a, device), to_dev(b, device), to_dev(sx, device), to_dev(sw, device))
        cb.check_device()
        assert np.array_equal(cw.view(torch.int16).cpu().numpy().view(np.uint16),
                              oracle.gemm_w8a8_bf16(a, b, sx, sw, M, N, K))


@pytest.mark.parametrize("register_stores", [False, True])
def test_store_paths_leave_padding_alone(cb, device, policies, register_stores):
    """Canary around C with ldc > N and rows past M, for both store paths and both CTA groupings."""
    import torch
    from cudaintro_b200 import capi

    set_tiles, set_stores = policies
    set_stores(register_stores)
    M, N, K, ldc = 300, 264, 512, 288
    g = torch.Generator(device=device).manual_seed(11)
    a = torch.randn((M, K), device=device, generator=g).to(torch.bfloat16)
    b = torch.randn((N, K), device=device, generator=g).to(torch.bfloat16)
    for cg in (1, 2, 4):
        set_tiles(cg, 256, 0)
        out = torch.full((M + 4, ldc), 7.0, dtype=torch.bfloat16, device=device)
        st = capi.lib.b200_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, K, K, ldc, cb.ROW_MAJOR_BT, None)
        assert st == 0, capi.lib.b200_last_error()
        torch.cuda.synchronize()
        ref = (a.float() @ b.float().t())
        assert float((out[:M, :N].float() - ref).norm() / ref.norm()) < 1e-2
        assert bool((out[:M, N:] == 7.0).all()) and bool((out[M:] == 7.0).all())


@pytest.mark.parametrize("tiles", [(0, 0), (1, 256), (1, 128), (2, 256), (4, 256)])
def test_multi_destination_under_every_tiling(cb, oracle, device, policies, tiles):
    """b200_gemm_multi under every tiling it can take: all destinations (peers first, destination 0
    last) bit-exact against the oracle, twice in a row."""
    import torch
    from cudaintro_b200 import capi

    set_tiles, _ = policies
    M, N, K = 520, 784, 640
    rng = np.random.default_rng(17)
    a = rng.integers(-127, 128, (M, K)).astype(np.int8)
    b = rng.integers(-127, 128, (K, N)).astype(np.int8)
    want = oracle.gemm_i8_i32(a, b, M, N, K)
    ad, bd = to_dev(a, device), to_dev(b, device)
    set_tiles(tiles[0], tiles[1], 0)
    for _ in range(2):
        outs = [torch.full((M, N), -1, dtype=torch.int32, device=device) for _ in range(5)]
        capi.gemm_multi(capi.I8, ad, bd, [o.data_ptr() for o in outs], M, N, K)
        cb.check_device()
        for o in outs:
            assert np.array_equal(o.cpu().numpy(), want)


@pytest.mark.parametrize("register_stores", [False, True])
def test_multi_destination_gemm_on_one_gpu(cb, oracle, device, policies, register_stores):
    import torch
    from cudaintro_b200 import capi

    _, set_stores = policies
    set_stores(register_stores)
    M, N, K = 392, 528, 1024
    rng = np.random.default_rng(3)
    a = rng.integers(-127, 128, (M, K)).astype(np.int8)
    b = rng.integers(-127, 128, (K, N)).astype(np.int8)
    sx = rng.uniform(0.001, 0.02, M).astype(np.float32)
    sw = rng.uniform(0.001, 0.02, N).astype(np.float32)
    ad, bd, sxd, swd = to_dev(a, device), to_dev(b, device), to_dev(sx, device), to_dev(sw, device)
    # destinations: the same slab position (row 16) inside three separate "full C" buffers
    fulls = [torch.zeros((M + 32, N), dtype=torch.int32, device=device) for _ in range(3)]
    capi.gemm_multi(capi.I8, ad, bd, [f[16:].data_ptr() for f in fulls], M, N, K)
    cb.check_device()
    want = oracle.gemm_i8_i32(a, b, M, N, K)
    for f in fulls:
        assert np.array_equal(f[16:16 + M].cpu().numpy(), want)
        assert int(f[:16].abs().sum()) == 0 and int(f[16 + M:].abs().sum()) == 0
    outs = [torch.zeros((M, N), dtype=torch.bfloat16, device=device) for _ in range(8)]
    capi.gemm_multi(capi.W8A8, ad, bd, [o.data_ptr() for o in outs], M, N, K, sxd, swd)
    cb.check_device()
    want16 = oracle.gemm_w8a8_bf16(a, b, sx, sw, M, N, K)
    for o in outs:
        assert np.array_equal(o.view(torch.int16).cpu().numpy().view(np.uint16), want16)


@pytest.mark.parametrize("cg", [0, 1])
@pytest.mark.parametrize("shape", [(4096, 4096, 1024), (4000, 4704, 1152), (2304, 6400, 2048)])
def test_partly_filled_last_wave_int8_and_w8a8_bit_exact(cb, device, policies, shape, cg):
    """Shapes whose tiles leave the last wave of the persistent grid less than half full (CTA pairs
    with cg = 0, single CTAs with cg = 1), checked in full against the one-thread-per-element
    kernel, twice (the second launch starts from the state the first one left)."""
    import torch

    set_tiles, _ = policies
    M, N, K = shape
    g = torch.Generator(device=device).manual_seed(M + N + K + cg)
    a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=device, generator=g)
    b = torch.randint(-127, 128, (K, N), dtype=torch.int8, device=device, generator=g)
    rs = torch.rand(M, device=device, generator=g) * 0.01 + 0.001
    cs = torch.rand(N, device=device, generator=g) * 0.01 + 0.001
    want = cb.gemm_naive(a, b)
    want_w = ((want.float() * rs[:, None]) * cs[None, :]).to(torch.bfloat16)
    set_tiles(cg, 256 if cg else 0, 0)
    for _ in range(2):
        c = cb.gemm_i8_i32(a, b)
        cb.check_device()
        assert torch.equal(c, want)
    cw = cb.gemm_w8a8_bf16(a, b, rs, cs)
    cb.check_device()
    assert torch.equal(cw.view(torch.int16), want_w.view(torch.int16))


def test_completion_marker_passes_when_all_flags_arrive_and_gives_up_when_one_never_does(cb, oracle, device):
    """Failure detection without a fault: the marker's wait is bounded.  Here "rank 1" is just a
    second flag array on the same GPU that nobody ever writes for us, so rank 0's wait for it runs
    out after its two-second limit; the kernel returns, the status says so, and the context keeps
    working (a GEMM right after is still bit-exact)."""
    import ctypes as C
    import time

    import torch
    from cudaintro_b200 import capi

    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # world of one: the only flag it waits for is the one it writes itself
    solo = torch.zeros(8, dtype=torch.int32, device=device)
    arr1 = (C.c_void_p * 1)(C.c_void_p(solo.data_ptr()))
    assert capi.lib.b200_peer_marker(arr1, 1, 0, 1, stream) == 0
    cb.check_device()
    assert int(solo[0]) == 1

    mine = torch.zeros(8, dtype=torch.int32, device=device)
    other = torch.zeros(8, dtype=torch.int32, device=device)
    arr2 = (C.c_void_p * 2)(C.c_void_p(mine.data_ptr()), C.c_void_p(other.data_ptr()))
    t0 = time.perf_counter()
    assert capi.lib.b200_peer_marker(arr2, 2, 0, 1, stream) == 0
    with pytest.raises(cb.B200Error) as e:
        cb.check_device()
    waited = time.perf_counter() - t0
    assert e.value.status == 4            # B200_ERR_DEVICE_WAIT
    assert 1.5 < waited < 10.0            # it waited for its bound, not for ever
    assert int(mine[0]) == 1 and int(other[0]) == 1 and int(mine[1]) == 0
    cb.check_device()                     # the record was cleared by the failed check

    # a peer that does arrive (its slot in our array already holds the step number): no wait
    mine[1] = 2
    assert capi.lib.b200_peer_marker(arr2, 2, 0, 2, stream) == 0
    cb.check_device()

    rng = np.random.default_rng(1)
    a = rng.integers(-127, 128, (128, 256)).astype(np.int8)
    b = rng.integers(-127, 128, (256, 128)).astype(np.int8)
    c = cb.gemm_i8_i32(to_dev(a, device), to_dev(b, device))
    cb.check_device()
    assert np.array_equal(c.cpu().numpy(), oracle.gemm_i8_i32(a, b, 128, 128, 256))


def test_multi_destination_argument_checks(cb, device):
    import ctypes as C

    import torch
    from cudaintro_b200 import capi

    t = torch.zeros(1024, dtype=torch.int8, device=device)
    arr = (C.c_void_p * 9)(*[C.c_void_p(t.data_ptr())] * 9)
    assert capi.lib.b200_gemm_multi(capi.I8, t.data_ptr(), t.data_ptr(), arr, 9, None, None, 16, 16, 16, 0, 0, 0, None) == 1
    assert capi.lib.b200_gemm_multi(capi.I8, t.data_ptr(), t.data_ptr(), arr, 0, None, None, 16, 16, 16, 0, 0, 0, None) == 1
    assert capi.lib.b200_gemm_multi(capi.F32, t.data_ptr(), t.data_ptr(), arr, 1, None, None, 16, 16, 16, 0, 0, 0, None) == 1
    assert capi.lib.b200_gemm_multi(capi.W8A8, t.data_ptr(), t.data_ptr(), arr, 1, None, None, 16, 16, 16, 0, 0, 0, None) == 1


_TWO_GPU_SCRIPT = r"""
import os, sys
sys.path.insert(0, os.environ["B200_ROOT"])
import numpy as np, torch, torch.distributed as dist
import cudaintro_b200 as cb
from cudaintro_b200 import capi
from cudaintro_b200.sharded import FusedShardedGemm, ShardedGemm
import oracle as O
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank); dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
M, N, K = 1000, 784, 2048      # 500 rows per rank: slab edges inside a tile
rng = np.random.default_rng(9)
a = rng.integers(-127, 128, (M, K)).astype(np.int8); b = rng.integers(-127, 128, (K, N)).astype(np.int8)
sx = rng.uniform(0.001, 0.02, M).astype(np.float32); sw = rng.uniform(0.001, 0.02, N).astype(np.float32)
fs = FusedShardedGemm(M, N, torch.bfloat16, dev)
p = fs.part
a_loc = torch.from_numpy(a[p.row0:p.row0 + p.rows]).to(dev); b_d = torch.from_numpy(b).to(dev)
sx_loc = torch.from_numpy(sx[p.row0:p.row0 + p.rows]).to(dev); sw_d = torch.from_numpy(sw).to(dev)
for _ in range(2):
    fs.step(capi.W8A8, a_loc, b_d, sx_loc, sw_d)
torch.cuda.synchronize(); cb.check_device()
want = O.gemm_w8a8_bf16(a, b, sx, sw, M, N, K)
got = fs.result().view(torch.int16).cpu().numpy().view(np.uint16)
assert np.array_equal(got, want), f"rank {rank}: fused result differs from the oracle"
sg = ShardedGemm(M, N, torch.bfloat16, dev)
sg.step(lambda slab: cb.gemm_w8a8_bf16(a_loc, b_d, sx_loc, sw_d, out=slab))
torch.cuda.synchronize()
assert torch.equal(sg.result().view(torch.int16), fs.result().view(torch.int16))
fs.close()
dist.barrier(); dist.destroy_process_group()
print(f"rank {rank} ok")
"""


def test_fused_gather_on_two_gpus(cb, device, tmp_path):
    """Real peer memory: two ranks, each GPU's epilogue stores its tiles into both copies of C."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "two_gpu.py"
    script.write_text(_TWO_GPU_SCRIPT)
    env = dict(os.environ, B200_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                         capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "rank 0 ok" in res.stdout and "rank 1 ok" in res.stdout


_TWO_GPU_MULTICAST_SCRIPT = _TWO_GPU_SCRIPT.replace(
    "fs = FusedShardedGemm(M, N, torch.bfloat16, dev)",
    "fs = FusedShardedGemm(M, N, torch.bfloat16, dev, multicast=True)\nassert fs.multicast and fs.mc_slab_ptr")


def test_multicast_gather_on_two_gpus(cb, device, tmp_path):
    """b200_gemm_multicast on real hardware: two ranks, C in symmetric memory with an NVLink multicast
    mapping, every tile written once with multimem.st and delivered to both copies by the switch.
    Bit-exact against the oracle on both ranks and equal to GEMM + NCCL all-gather.  No rank leaves
    in this test (a process that dies while bound to a multicast object disturbs the other GPUs)."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "two_gpu_mc.py"
    script.write_text(_TWO_GPU_MULTICAST_SCRIPT)
    env = dict(os.environ, B200_ROOT=ROOT)
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29534", str(script)],
                         capture_output=True, text=True, env=env, timeout=600)
    if "no NVLink multicast mapping" in res.stderr:
        pytest.skip("this machine offers no NVLink multicast")
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "rank 0 ok" in res.stdout and "rank 1 ok" in res.stdout
