"""The N > 1 path on CPU: two gloo ranks, each holding its output-feature shard, one all-gather of the slices.

The per-shard products here come from the CPU oracle (the test exercises the slicing, the collective and the
re-assembly, not the CUDA kernels); the same index rules are used by b200q_weight_upload on the device."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rocmforge_b200 import shard, synth


def _rank_main(rank, world, port, qt, n, k, m, tmpdir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import cpu_oracle as orc
    rng = synth.rng_for(42)
    data = synth.gen_packed(qt, synth.GGUF, n * k, rng)          # every rank draws the same tensor
    x = synth.gen_activations(m, k, rng)
    mine = shard.shard_bytes(data, qt, synth.GGUF, n, k, rank, world)
    row0, rows = shard.shard_rows(n, rank, world)
    w = orc.dequantize(qt, synth.GGUF, mine, rows * k).reshape(rows, k)
    y_slice = torch.from_numpy(orc.matmul_f32(x, w, nk=True))
    y_all = torch.empty((world, m, rows), dtype=torch.float32)
    dist.all_gather_into_tensor(y_all.view(world * m, rows), y_slice)     # [G*m, n/G]: slices stacked along dim 0
    y = shard.gathered_to_matrix(y_all).numpy()
    if rank == 0:
        wf = orc.dequantize(qt, synth.GGUF, data, n * k).reshape(n, k)
        ref = orc.matmul_f32(x, wf, nk=True)
        np.save(os.path.join(tmpdir, "ok.npy"), np.array([np.array_equal(y.view(np.uint32), ref.view(np.uint32))]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("qt,n,k", [(synth.Q4_K, 256, 512), (synth.MXFP4, 128, 1024), (synth.Q6_K, 64, 896)])
def test_two_ranks_gather_to_the_unsharded_result(tmp_path, qt, n, k):
    port = 29500 + (os.getpid() % 1000) + qt
    mp.spawn(_rank_main, args=(2, port, qt, n, k, 3, str(tmp_path)), nprocs=2, join=True)
    assert np.load(tmp_path / "ok.npy")[0]


def test_shard_index_rules():
    assert shard.shard_rows(28672, 3, 8) == (3 * 3584, 3584)
    with pytest.raises(ValueError):
        shard.shard_rows(10, 0, 3)
    with pytest.raises(ValueError):
        shard.shard_rows(8, 2, 2)
    data = np.arange(8 * 144, dtype=np.uint8)                     # 8 Q4_K super-blocks = 4 rows x 512
    assert shard.shard_bytes(data, synth.Q4_K, synth.GGUF, 4, 512, 1, 2).tolist() == data[4 * 144:].tolist()
    with pytest.raises(ValueError):
        shard.shard_bytes(data, synth.Q4_K, synth.GGUF, 16, 128, 0, 16)   # one row of 128 is half a super-block
    y_all = torch.arange(2 * 3 * 4, dtype=torch.float32).reshape(2, 3, 4)
    y = shard.gathered_to_matrix(y_all)
    assert y.shape == (3, 8) and y[1, 4:].tolist() == y_all[1, 1].tolist()
