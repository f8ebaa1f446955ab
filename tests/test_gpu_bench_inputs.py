"""bench.py generates its synthetic expert weights on the GPU with torch; those quantisers
must be the reference converters' rules bit for bit. tests/golden/quant_vectors.npz holds the
outputs of c/tools/convert_fp8_to_int4.py:79-109 (quant_int4_grouped) and
c/tools/make_deepseek_v4_tiny.py:97-121 (quantize_fp4) on seeded weights."""
import os

import numpy as np
import pytest

import bench

pytestmark = pytest.mark.gpu
QV = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quant_vectors.npz"))


@pytest.mark.parametrize("nm", ["a", "c"])
def test_torch_int4_g32_generator_matches_reference_converter(nm):
    import torch
    w = torch.from_numpy(QV[f"w.{nm}"]).cuda()
    pk, sc = bench.quant_int4_g32_torch(torch, w, fp16_scales=False)
    assert np.array_equal(sc.cpu().numpy().reshape(-1).view(np.uint32), QV[f"i4g32.{nm}.s"].view(np.uint32))
    assert np.array_equal(pk.cpu().numpy(), QV[f"i4g32.{nm}.q"])
    # the benchmark's variant rounds the scale to fp16 first and derives the codes from it
    from colibri_b200.quant import quant_int4_grouped
    pk16, sc16 = bench.quant_int4_g32_torch(torch, w, fp16_scales=True)
    q_np, s_np = quant_int4_grouped(QV[f"w.{nm}"], 32, np.float16)
    assert np.array_equal(sc16.cpu().numpy().reshape(-1).view(np.uint32), s_np.view(np.uint32))
    assert np.array_equal(pk16.cpu().numpy(), q_np)


@pytest.mark.parametrize("nm", ["a", "c"])
def test_torch_mxfp4_generator_matches_reference_converter(nm):
    import torch
    w = torch.from_numpy(QV[f"w.{nm}"]).cuda()
    pk, e = bench.quant_mxfp4_torch(torch, w)
    assert np.array_equal(e.cpu().numpy(), QV[f"fp4.{nm}.e"])
    assert np.array_equal(pk.cpu().numpy(), QV[f"fp4.{nm}.q"])
