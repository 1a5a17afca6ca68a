"""B200Q_MM_MX_NATIVE: GGUF MXFP4 codes and their E8M0 block scales straight into the block-scaled tensor-core MMA
(tcgen05.mma.kind::mxf8f6f4.block_scale), activations quantised to MXFP8 on the way in.

Two kinds of check against the CPU oracle. (1) Activations that MXFP8 represents exactly (integers of at most four
significant bits times a power of two per block of 32): every product is then exact and only the fp32 summation
order differs from the oracle's, so the tolerance is 2e-5 — this pins the operand layouts, the element order of a
block, both scale planes and the accumulation. (2) Random activations: the result carries the rounding of E4M3's
3-bit mantissa; tolerance 5e-2 of the largest output, stated here because it is far from the 2e-3 of the default
path, which is why the mode is opt-in.
"""
import numpy as np
import pytest

from rocmforge_b200 import _lib, synth
from rocmforge_b200._lib import B200QError

from gpu_util import QuantizedWeight, backend, gpu_matmul, rel_err

pytestmark = pytest.mark.gpu


def exact_activations(m, k, rng):
    ints = rng.integers(-15, 16, size=(m, k)).astype(np.float32)
    ints[:, ::32] = 15.0                                   # every block reaches the largest magnitude: the scale is fixed by it
    scale = np.exp2(rng.integers(-6, 7, size=(m, k // 32))).astype(np.float32)
    return (ints.reshape(m, k // 32, 32) * scale[:, :, None]).reshape(m, k)


def reference(oracle, data, n, k, x, qt=synth.MXFP4):
    w = oracle.dequantize(qt, synth.GGUF, data, n * k, threads=8).reshape(n, k)
    return oracle.matmul_f64(x, w, nk=True)


@pytest.mark.parametrize("qt", [synth.MXFP6_E2M3, synth.MXFP6_E3M2], ids=["e2m3", "e3m2"])
@pytest.mark.parametrize("n,k,m", [(128, 128, 16), (300, 1024, 100), (256, 2048, 300), (512, 8192, 520)],
                         ids=["one-stage", "ragged", "two-token-tiles", "k8192-ragged-m"])
def test_mxfp6_codes_go_in_as_they_are(oracle, qt, n, k, m):
    """The 6-bit code plane by TMA as 16 x U6 -> 16-byte containers; E3M2 has no other tensor-core path that keeps
    its codes exact (its values are not 8-bit integers times a power of two)."""
    be = backend()
    rng = synth.rng_for(9150 + qt + n + k + m)
    data = synth.gen_packed(qt, synth.GGUF, n * k, rng).copy()
    blocks = data.reshape(-1, 25)
    blocks[:, 1:] = rng.integers(0, 256, size=(blocks.shape[0], 24)).astype(np.uint8)     # every code in every position
    x = exact_activations(m, k, rng)
    w = QuantizedWeight(be, data, qt, synth.GGUF, n, k)
    y = gpu_matmul(be, w, x, m, flags=_lib.MM_MX_NATIVE)
    assert rel_err(y, reference(oracle, data, n, k, x, qt)) <= 2e-5
    w.free()


@pytest.mark.parametrize("n,k,m", [(128, 128, 16), (128, 512, 64), (300, 1024, 100), (256, 1024, 300), (1024, 2048, 512), (384, 8192, 520)],
                         ids=["one-stage", "four-stages", "ragged", "two-token-tiles", "m512", "k8192-ragged-m"])
def test_exactly_representable_activations_give_the_fp32_result(oracle, n, k, m):
    be = backend()
    rng = synth.rng_for(9100 + n + k + m)
    data = synth.gen_packed(synth.MXFP4, synth.GGUF, n * k, rng)
    x = exact_activations(m, k, rng)
    w = QuantizedWeight(be, data, synth.MXFP4, synth.GGUF, n, k)
    y = gpu_matmul(be, w, x, m, flags=_lib.MM_MX_NATIVE)
    assert rel_err(y, reference(oracle, data, n, k, x)) <= 2e-5
    y2 = gpu_matmul(be, w, x, m, flags=_lib.MM_MX_NATIVE)      # second call: the weight's scale plane comes from its cache
    assert np.array_equal(y, y2)
    w.free()


def test_every_block_exponent_and_code(oracle):
    """All 16 codes in every position of a block, block exponents from 2^-40 to 2^40 (the scales stay E8M0 end to end,
    nothing passes through f16)."""
    be = backend()
    n, k, m = 128, 1024, 32
    rng = synth.rng_for(9200)
    data = synth.gen_packed(synth.MXFP4, synth.GGUF, n * k, rng).copy()
    blocks = data.reshape(-1, 17)
    blocks[:, 0] = rng.integers(87, 168, size=blocks.shape[0]).astype(np.uint8)
    blocks[:, 1:] = rng.integers(0, 256, size=(blocks.shape[0], 16)).astype(np.uint8)
    x = exact_activations(m, k, rng)
    w = QuantizedWeight(be, data, synth.MXFP4, synth.GGUF, n, k)
    y = gpu_matmul(be, w, x, m, flags=_lib.MM_MX_NATIVE)
    ref = reference(oracle, data, n, k, x)
    assert np.all(np.isfinite(y))
    # rows differ by many orders of magnitude: compare row by row
    err = np.abs(y - ref).max(axis=0) / np.maximum(np.abs(ref).max(axis=0), 1e-30)
    assert float(err.max()) <= 2e-5
    w.free()


@pytest.mark.parametrize("m", [64, 512])
def test_random_activations_within_the_mxfp8_tolerance(oracle, m):
    be = backend()
    n, k = 512, 4096
    rng = synth.rng_for(9300 + m)
    data = synth.gen_packed(synth.MXFP4, synth.GGUF, n * k, rng)
    x = synth.gen_activations(m, k, rng)
    w = QuantizedWeight(be, data, synth.MXFP4, synth.GGUF, n, k)
    y = gpu_matmul(be, w, x, m, flags=_lib.MM_MX_NATIVE)
    ref = reference(oracle, data, n, k, x)
    e = rel_err(y, ref)
    assert e <= 5e-2, e
    assert e > 1e-4          # it IS the lower-precision path (the default one meets 2e-3 on the same input)
    assert rel_err(gpu_matmul(be, w, x, m), ref) <= 2e-3
    w.free()


def test_other_formats_and_small_m(oracle):
    be = backend()
    n, k = 128, 256
    rng = synth.rng_for(9400)
    data = synth.gen_packed(synth.Q4_K, synth.GGUF, n * k, rng)
    w = QuantizedWeight(be, data, synth.Q4_K, synth.GGUF, n, k)
    x = synth.gen_activations(16, k, rng)
    with pytest.raises(B200QError) as e:
        gpu_matmul(be, w, x, 16, flags=_lib.MM_MX_NATIVE)
    assert e.value.status == _lib.ERR_UNSUPPORTED
    w.free()
    data = synth.gen_packed(synth.MXFP4, synth.GGUF, n * k, rng)
    w = QuantizedWeight(be, data, synth.MXFP4, synth.GGUF, n, k)
    x = synth.gen_activations(4, k, rng)
    y = gpu_matmul(be, w, x, 4, flags=_lib.MM_MX_NATIVE)        # m <= 8: the flag is ignored, the decode kernel runs
    wf = oracle.dequantize(synth.MXFP4, synth.GGUF, data, n * k).reshape(n, k)
    assert rel_err(y, oracle.matmul_f32(x, wf, nk=True)) <= 1e-4
    w.free()


def test_bf16_activations_a_row_pitch_and_bf16_outputs(oracle):
    """The exactly representable activations are bf16 values too, so the bf16 entry gives the same fp32 result; a
    row pitch larger than k and a bf16 output go through the same kernel."""
    import torch
    be = backend()
    n, k, m, ldx = 256, 1024, 72, 1024 + 64
    rng = synth.rng_for(9500)
    data = synth.gen_packed(synth.MXFP4, synth.GGUF, n * k, rng)
    x = exact_activations(m, k, rng)
    w = QuantizedWeight(be, data, synth.MXFP4, synth.GGUF, n, k)
    ref = reference(oracle, data, n, k, x)
    xp = np.zeros((m, ldx), dtype=np.float32)
    xp[:, :k] = x
    xp[:, k:] = 1e30                                            # never read
    xb = be.allocate_buffer(xp.nbytes); xb.copy_from_host(xp)
    yb = be.allocate_buffer(m * n * 4)
    w.matmul(xb, yb, m, flags=_lib.MM_MX_NATIVE, ldx=ldx)
    be.synchronize()
    assert rel_err(yb.to_numpy(np.float32, m * n).reshape(m, n), ref) <= 2e-5
    x16 = torch.from_numpy(x).to(torch.bfloat16)
    assert np.array_equal(x16.float().numpy(), x)               # nothing is lost on the way in
    xb16 = be.allocate_buffer(m * k * 2); xb16.copy_from_host(x16.view(torch.int16).numpy())
    w.matmul(xb16, yb, m, x_dtype=_lib.BF16, flags=_lib.MM_MX_NATIVE)
    be.synchronize()
    y = yb.to_numpy(np.float32, m * n).reshape(m, n)
    assert rel_err(y, ref) <= 2e-5
    y16 = be.allocate_buffer(m * n * 2)
    w.matmul(xb16, y16, m, x_dtype=_lib.BF16, y_dtype=_lib.BF16, flags=_lib.MM_MX_NATIVE)
    be.synchronize()
    got = torch.from_numpy(y16.to_numpy(np.int16, m * n)).view(torch.bfloat16).float().numpy().reshape(m, n)
    assert np.array_equal(got, torch.from_numpy(y).to(torch.bfloat16).float().numpy())
    for b in (xb, xb16, yb, y16):
        b.free()
    w.free()


@pytest.mark.parametrize("row_tiles,m", [(94, 512), (75, 512), (84, 500), (75, 300)],
                         ids=["40-of-188-tiles", "2-of-150-tiles", "20-of-168-tiles-ragged-m", "2-of-150-tiles-ragged-m"])
def test_last_wave_cut_into_pieces(oracle, row_tiles, m):
    """More tiles than SMs with a small remainder: the tiles of the last wave are cut along the activation rows into
    two pieces of 128 (188 tiles on 148 SMs -> 40 tiles in 80 pieces). Checked on sampled weight rows: the first and
    last tiles and the cut ones."""
    be = backend()
    n, k = 128 * row_tiles, 512
    rng = synth.rng_for(9600 + row_tiles + m)
    data = synth.gen_packed(synth.MXFP4, synth.GGUF, n * k, rng)
    x = exact_activations(m, k, rng)
    w = QuantizedWeight(be, data, synth.MXFP4, synth.GGUF, n, k)
    y = gpu_matmul(be, w, x, m, flags=_lib.MM_MX_NATIVE)
    rows = np.unique(np.concatenate([np.arange(0, 256), np.arange(n - 6 * 128, n), rng.integers(0, n, size=256)]))
    blocks = np.frombuffer(bytes(data), dtype=np.uint8).reshape(-1, 17)
    sel = np.concatenate([blocks[r * k // 32:(r + 1) * k // 32] for r in rows]).reshape(-1)
    wsel = oracle.dequantize(synth.MXFP4, synth.GGUF, sel, rows.size * k, threads=8).reshape(rows.size, k)
    ref = oracle.matmul_f64(x, wsel, nk=True)
    assert np.all(np.isfinite(y))
    assert float(np.max(np.abs(y[:, rows] - ref))) / float(np.max(np.abs(ref))) <= 2e-5
    w.free()


@pytest.mark.parametrize("qt", [synth.MXFP4, synth.MXFP6_E2M3], ids=["mxfp4", "mxfp6"])
@pytest.mark.parametrize("n,k", [(28672, 8192), (8192, 28672)], ids=["28672x8192", "8192x28672"])
def test_config5_full_size(oracle, qt, n, k):
    """BASELINE config 5's shapes at full size, M = 512: 448 (128) tiles on 148 SMs, the last wave cut in two.
    Sampled weight rows against the oracle on exactly representable activations."""
    be = backend()
    m = 512
    rng = synth.rng_for(9700 + qt + n)
    data = synth.gen_packed(qt, synth.GGUF, n * k, rng)
    x = exact_activations(m, k, rng)
    w = QuantizedWeight(be, data, qt, synth.GGUF, n, k)
    y = gpu_matmul(be, w, x, m, flags=_lib.MM_MX_NATIVE)
    rows = np.unique(np.concatenate([rng.integers(0, n, size=96), np.arange(n - 130, n), [0, 127, 128]]))
    bb = synth.block_bytes(qt, synth.GGUF)
    blocks = np.frombuffer(bytes(data), dtype=np.uint8).reshape(-1, bb)
    sel = np.concatenate([blocks[r * k // 32:(r + 1) * k // 32] for r in rows]).reshape(-1)
    wsel = oracle.dequantize(qt, synth.GGUF, sel, rows.size * k, threads=8).reshape(rows.size, k)
    ref = oracle.matmul_f64(x, wsel, nk=True)
    assert np.all(np.isfinite(y))
    assert float(np.max(np.abs(y[:, rows] - ref))) / float(np.max(np.abs(ref))) <= 2e-5
    w.free()


@pytest.mark.parametrize("qt", [synth.MXFP4, synth.MXFP6_E3M2], ids=["mxfp4", "e3m2"])
@pytest.mark.parametrize("n,k,m", [(1024, 2048, 512), (384, 1024, 256), (128 * 151, 512, 512)],
                         ids=["four-pair-tiles", "odd-row-tiles", "more-items-than-pairs"])
def test_cta_pairs(oracle, qt, n, k, m, monkeypatch):
    """B200Q_MX_PAIR=1: two CTAs of a cluster share a 256 x 256 tile (tcgen05 cta_group::2), each holding 128 weight
    rows and half of the activation tile. Same exact result; an odd number of row tiles leaves the last pair's second
    CTA on rows past the end."""
    monkeypatch.setenv("B200Q_MX_PAIR", "1")
    be = backend()
    rng = synth.rng_for(9800 + qt + n + m)
    data = synth.gen_packed(qt, synth.GGUF, n * k, rng)
    x = exact_activations(m, k, rng)
    w = QuantizedWeight(be, data, qt, synth.GGUF, n, k)
    y = gpu_matmul(be, w, x, m, flags=_lib.MM_MX_NATIVE)
    rows = np.unique(np.concatenate([np.arange(0, min(n, 300)), np.arange(max(0, n - 300), n), rng.integers(0, n, size=128)]))
    bb = synth.block_bytes(qt, synth.GGUF)
    blocks = np.frombuffer(bytes(data), dtype=np.uint8).reshape(-1, bb)
    sel = np.concatenate([blocks[r * k // 32:(r + 1) * k // 32] for r in rows]).reshape(-1)
    wsel = oracle.dequantize(qt, synth.GGUF, sel, rows.size * k, threads=8).reshape(rows.size, k)
    ref = oracle.matmul_f64(x, wsel, nk=True)
    assert np.all(np.isfinite(y))
    assert float(np.max(np.abs(y[:, rows] - ref))) / float(np.max(np.abs(ref))) <= 2e-5
    w.free()
