"""N > 1 host path on CPU: two gloo ranks shard the windows, encode their blocks on the CPU oracle
backend (the engine is backend-agnostic), gather on rank 0, and the result equals the one-process run.
Also ragged and empty shards."""
import os
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, n_windows, out_path):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import __graft_entry__ as ge

    ge.load_package()
    from fluidaudio_web_b200 import sharding
    from fluidaudio_web_b200.engines import fastconformer, synth
    from oracle.wasm_oracle import WasmOracle

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        ora = WasmOracle()
        w = synth.encoder_weights(synth.TINY, seed=3)
        mels = [synth.log_mel(a, 32).reshape(-1) for a in synth.synth_audio(n_windows, samples=16000, seed=3)]
        got, Tsub = sharding.encode_windows_sharded(ora, fastconformer.load_encoder(ora, w), mels, world, rank, batch=2)
        if rank == 0:
            np.save(out_path, got)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_windows", [5, 1])
def test_two_rank_gloo_matches_single_process(pkg, tmp_path, n_windows):
    from fluidaudio_web_b200 import sharding
    from fluidaudio_web_b200.engines import fastconformer, synth
    from oracle.wasm_oracle import WasmOracle

    out = str(tmp_path / "g.npy")
    port = 29600 + os.getpid() % 200 + n_windows
    mp.spawn(_worker, args=(2, port, n_windows, out), nprocs=2, join=True)
    got = np.load(out)
    ora = WasmOracle()
    w = synth.encoder_weights(synth.TINY, seed=3)
    mels = [synth.log_mel(a, 32).reshape(-1) for a in synth.synth_audio(n_windows, samples=16000, seed=3)]
    ref, _ = sharding.encode_windows_sharded(ora, fastconformer.load_encoder(ora, w), mels, 1, 0, batch=2)
    assert got.shape == ref.shape
    # batches group windows differently per rank; windows are independent, so frames agree to rounding
    assert np.abs(got - ref).max() < 1e-4


def test_shard_ranges_cover_and_order(pkg):
    from fluidaudio_web_b200 import sharding

    for n in (0, 1, 7, 8, 256):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(4, 2, 2)


def _nshard_worker(rank, world, port, out_path):
    """N-sharded product on two gloo ranks: each multiplies by its column block on the CPU oracle backend,
    the blocks are all-gathered along rows and unsharded into the row-major product."""
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import __graft_entry__ as ge

    ge.load_package()
    from fluidaudio_web_b200 import sharding
    from oracle.wasm_oracle import WasmOracle

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(2)
        a = rng.standard_normal((6, 40)).astype(np.float32)
        w = rng.standard_normal((40, 24)).astype(np.float32)
        ora = WasmOracle()
        ws = sharding.column_shard(w, world, rank)
        local = ora.matmul(ora.upload(a, 6, 40), ora.upload(ws, 40, ws.shape[1])).array()
        gathered = torch.empty((world * 6, ws.shape[1]), dtype=torch.float32)
        dist.all_gather_into_tensor(gathered, torch.from_numpy(np.ascontiguousarray(local)))
        full = sharding.unshard_cols_host(gathered.numpy(), world)
        np.save(out_path + f".{rank}.npy", full)
    finally:
        dist.destroy_process_group()


def test_n_sharded_product_two_gloo_ranks(pkg, tmp_path):
    from oracle.wasm_oracle import WasmOracle

    out = str(tmp_path / "ns")
    port = 29850 + os.getpid() % 100
    mp.spawn(_nshard_worker, args=(2, port, out), nprocs=2, join=True)
    rng = np.random.default_rng(2)
    a = rng.standard_normal((6, 40)).astype(np.float32)
    w = rng.standard_normal((40, 24)).astype(np.float32)
    ora = WasmOracle()
    ref = ora.matmul(ora.upload(a, 6, 40), ora.upload(w, 40, 24)).array()
    for r in range(2):  # every rank ends with the whole product, bit for bit (same per-column arithmetic)
        assert np.array_equal(np.load(out + f".{r}.npy"), ref)


def test_column_shard_rejects_uneven(pkg):
    from fluidaudio_web_b200 import sharding

    with pytest.raises(ValueError):
        sharding.column_shard(np.zeros((4, 10), np.float32), 4, 0)
    parts = [sharding.column_shard(np.arange(24, dtype=np.float32).reshape(2, 12), 3, r) for r in range(3)]
    assert np.array_equal(np.concatenate(parts, axis=1), np.arange(24, dtype=np.float32).reshape(2, 12))
