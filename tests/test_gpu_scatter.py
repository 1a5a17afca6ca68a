"""b200q_matmul_scatter: the gather of a sharded product fused into the kernels' epilogues. On one GPU the
"peers" are further buffers of the same device (the stores are the same instructions); with two or more GPUs
a second test runs two processes that write into each other's outputs through IPC-mapped pointers."""
import os
import subprocess
import sys

import numpy as np
import pytest

from rocmforge_b200 import _lib, synth
from rocmforge_b200._lib import B200QError
from rocmforge_b200.backend import QuantizedWeight

from gpu_util import backend, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("qt,m,tol", [(synth.Q4_K, 1, 1e-4), (synth.Q6_K, 3, 1e-4), (synth.MXFP4, 8, 1e-4),
                                       (synth.Q4_K, 200, 2e-3), (synth.Q8_0, 64, 2e-3), (synth.Q4_K, 600, 2e-3), (synth.Q6_K, 1030, 2e-3)],
                         ids=["decode-q4k", "decode-q6k", "decode-mxfp4", "prefill-q4k-streamk", "prefill-q8_0",
                              "prefill-q4k-three-token-tiles", "prefill-q6k-five-token-tiles"])
def test_every_shard_lands_in_every_output(oracle, qt, m, tol):
    be = backend()
    rng = synth.rng_for(6100 + qt + m)
    n, k, shards, copies = 512, 1024, 4, 3
    data = synth.gen_packed(qt, synth.GGUF, n * k, rng)
    x = synth.gen_activations(m, k, rng)
    xb = be.allocate_buffer(x.nbytes)
    xb.copy_from_host(x)
    outs = [be.allocate_buffer(m * n * 4) for _ in range(copies)]
    for o in outs:
        o.fill(0xFF)
    ws = [QuantizedWeight(be, data, qt, synth.GGUF, n, k, shard_rank=r, shard_count=shards) for r in range(shards)]
    for w in ws:
        w.matmul_scatter(xb, outs, m, n)
    be.synchronize()
    wf = oracle.dequantize(qt, synth.GGUF, data, n * k).reshape(n, k)
    ref = oracle.matmul_f32(x, wf, nk=True, threads=8)
    got = [o.to_numpy(np.float32, m * n).reshape(m, n) for o in outs]
    assert rel_err(got[0], ref) <= tol
    for g in got[1:]:
        assert np.array_equal(g, got[0])            # every copy holds the same bits
    for w in ws:
        w.free()


def _bf16_bits(a):
    """fp32 -> bf16 with round-to-nearest-even, as 16-bit patterns (finite inputs)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


@pytest.mark.parametrize("m", [200, 520])
@pytest.mark.parametrize("qt", [synth.Q4_K, synth.MXFP4, synth.Q8_0, synth.MXFP6_E2M3], ids=["q4k", "mxfp4", "q8_0", "mxfp6"])
def test_bf16_outputs_are_the_fp32_ones_rounded_once(qt, m):
    """B200Q_MM_SCATTER_BF16: the same accumulators, rounded to bf16 in the epilogue, in every copy (m = 520: three
    token tiles, the last one ragged)."""
    be = backend()
    rng = synth.rng_for(6300 + qt)
    n, k, shards, copies = 512, 1024, 2, 3
    data = synth.gen_packed(qt, synth.GGUF, n * k, rng)
    x = synth.gen_activations(m, k, rng)
    xb = be.allocate_buffer(x.nbytes)
    xb.copy_from_host(x)
    o32 = [be.allocate_buffer(m * n * 4) for _ in range(copies)]
    o16 = [be.allocate_buffer(m * n * 2) for _ in range(copies)]
    for o in o32 + o16:
        o.fill(0xFF)
    ws = [QuantizedWeight(be, data, qt, synth.GGUF, n, k, shard_rank=r, shard_count=shards) for r in range(shards)]
    for w in ws:
        w.matmul_scatter(xb, o32, m, n)
        w.matmul_scatter(xb, o16, m, n, flags=_lib.MM_SCATTER_BF16)
    be.synchronize()
    want = _bf16_bits(o32[0].to_numpy(np.float32, m * n))
    for o in o16:
        assert np.array_equal(o.to_numpy(np.uint16, m * n), want)
    with pytest.raises(B200QError) as e:
        ws[0].matmul_scatter(xb, o16, 4, n, flags=_lib.MM_SCATTER_BF16)     # the decode kernel writes fp32
    assert e.value.status == _lib.ERR_UNSUPPORTED
    for w in ws:
        w.free()


def test_scatter_argument_errors():
    be = backend()
    rng = synth.rng_for(6200)
    n, k = 256, 512
    data = synth.gen_packed(synth.MXFP6_E3M2, synth.GGUF, n * k, rng)
    w = QuantizedWeight(be, data, synth.MXFP6_E3M2, synth.GGUF, n, k, shard_rank=1, shard_count=2)
    x = be.allocate_buffer(k * 4)
    y = be.allocate_buffer(n * 4)
    with pytest.raises(B200QError) as e:
        w.matmul_scatter(x, [y, y], 1, n)            # MXFP6 E3M2 has no tensor-core decode kernel
    assert e.value.status == _lib.ERR_UNSUPPORTED
    with pytest.raises(B200QError) as e:
        w.matmul_scatter(x, [y], 1, n // 2)          # ldy ends before this shard's columns
    assert e.value.status == _lib.ERR_INVALID
    with pytest.raises(B200QError) as e:
        w.matmul_scatter(x, [y] * 9, 1, n)
    assert e.value.status == _lib.ERR_INVALID
    w.free()


_CHILD = r"""
import os, sys
import numpy as np
import torch, torch.distributed as dist
sys.path.insert(0, os.environ["B200Q_REPO"]); sys.path.insert(0, os.path.join(os.environ["B200Q_REPO"], "tests"))
from rocmforge_b200 import synth
from rocmforge_b200.backend import B200Backend, QuantizedWeight
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
be = B200Backend(rank, stream=torch.cuda.current_stream().cuda_stream)
n, k = 1024, 1024
ok = True
for qt, m in ((synth.Q4_K, 1), (synth.Q4_K, 256)):
    rng = synth.rng_for(6300 + m)
    data = synth.gen_packed(qt, synth.GGUF, n * k, rng)
    x = synth.gen_activations(m, k, rng)
    xt = torch.from_numpy(x).cuda()
    y_full = be.allocate_buffer(m * n * 4); y_full.fill(0xFF)
    flags = be.allocate_buffer(64); flags.fill(0)
    handles = [None] * world
    dist.all_gather_object(handles, (be.ipc_handle(y_full), be.ipc_handle(flags)))
    peers = [y_full.as_ptr() if r == rank else be.ipc_open(handles[r][0]) for r in range(world)]
    peer_flags = [flags.as_ptr() if r == rank else be.ipc_open(handles[r][1]) for r in range(world)]
    w = QuantizedWeight(be, data, qt, synth.GGUF, n, k, shard_rank=rank, shard_count=world)
    full = QuantizedWeight(be, data, qt, synth.GGUF, n, k)
    dist.barrier()                                   # every rank has mapped the others' buffers
    for epoch in (1, 2):                             # no collective between the product and the read: flags only
        if epoch == 1:
            w.matmul_scatter(xt.data_ptr(), peers, m, n)
            be.peer_signal(peer_flags, rank, epoch)
        else:
            w.matmul_scatter_signal(xt.data_ptr(), peers, m, n, peer_flags, rank, epoch)
        be.peer_wait(flags, world, rank, epoch)
    be.synchronize()
    yb = torch.empty((m, n), dtype=torch.float32, device="cuda")
    full.matmul(xt.data_ptr(), yb.data_ptr(), m)
    be.synchronize()
    got = y_full.to_numpy(np.float32, m * n).reshape(m, n)
    ref = yb.cpu().numpy()
    scale = np.abs(ref).max()
    ok = ok and bool(np.abs(got - ref).max() <= 2e-3 * scale)
    dist.barrier()
    for r in range(world):
        if r != rank:
            be.ipc_close(peers[r])
            be.ipc_close(peer_flags[r])
    dist.barrier()
t = torch.tensor([1.0 if ok else 0.0], device="cuda")
dist.all_reduce(t, op=dist.ReduceOp.MIN)
dist.destroy_process_group()
sys.exit(0 if t.item() == 1.0 else 3)
"""


def test_peer_wait_gives_up_when_no_peer_signals():
    """A rank that never hears from a peer (it died between steps) must not hang its GPU: the wait is bounded, the
    next synchronise reports a recoverable time-out, and the context goes on working. The failure is made on the
    host: nothing ever writes the flag."""
    be = backend()
    flags = be.allocate_buffer(64)
    flags.fill(0)
    be.peer_wait(flags, 2, 0, 7)                     # slot 1 never becomes 7
    with pytest.raises(B200QError) as e:
        be.synchronize()
    assert e.value.status == _lib.ERR_TIMEOUT and e.value.recoverable
    be.synchronize()                                 # the status was consumed; the context is usable
    import numpy as np
    one = np.array([0, 7] + [0] * 14, dtype=np.int32)
    flags.copy_from_host(one)
    be.peer_wait(flags, 2, 0, 7)                     # the flag is there: returns at once
    be.synchronize()
    with pytest.raises(B200QError):
        be.peer_wait(flags, 9, 0, 1)
    flags.free()


def test_two_processes_write_into_each_others_outputs(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, B200Q_REPO=repo, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                       env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
