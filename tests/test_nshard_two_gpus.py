"""The N-sharded product on two GPUs (one process each): the NCCL all-gather form and the form whose epilogue
stores straight into the peer's result buffer give the same full product as one GPU.  Needs two devices; the
single-GPU run skips it."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist
    import __graft_entry__ as ge

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    pkg = ge.load_package()
    from fluidaudio_web_b200 import sharding

    ctx = pkg.CudaContext(rank)
    try:
        rng = np.random.default_rng(2)
        M, K, N = 1024, 512, 768
        a = rng.standard_normal((M, K)).astype(np.float32)
        w = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float16).astype(np.float32)
        A = ctx.upload(a, M, K)
        ws = sharding.column_shard(w, world, rank)
        Ws = ctx.uploadF16(ws, K, ws.shape[1])
        gathered = ctx.download(sharding.matmul_n_sharded(ctx, A, Ws)).reshape(M, N)
        res = sharding.ScatterResult(ctx, M, N)
        sharding.matmul_n_sharded_scatter(ctx, A, Ws, res)
        sharding.stream_barrier(ctx)
        fused = ctx.download(res.local).reshape(M, N)
        whole = ctx.download(ctx.matmul(A, ctx.uploadF16(w, K, N))).reshape(M, N)
        res.close()
        np.save(os.path.join(out_dir, f"r{rank}.npy"), np.stack([gathered, fused, whole]))
    finally:
        ctx.destroy()
        dist.destroy_process_group()


def test_two_gpu_forms_agree(tmp_path):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    port = 29700 + os.getpid() % 200
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "r0.npy"), np.load(tmp_path / "r1.npy")
    for r in (r0, r1):
        gathered, fused, whole = r
        # the same f16 operands and f32 accumulation everywhere; a thin column block may split K over a cluster, which
        # changes the order of the f32 sums, so the forms agree to f32 rounding, not bit for bit
        tol = 2e-6 * float(np.abs(whole).max()) * np.sqrt(512)
        assert np.abs(gathered - whole).max() <= tol
        assert np.abs(fused - whole).max() <= tol
    assert np.array_equal(r0, r1)  # both ranks end with the same full product
