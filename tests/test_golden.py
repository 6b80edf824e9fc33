"""Committed golden vectors (tests/golden/golden.npz, made by tests/golden/make_golden.py from the reference's own
in-code generators): the CPU oracle must still reproduce them, and the CUDA path must match them."""
import os

import numpy as np
import pytest

from oracle import oracle as orc
from tests import helpers as H

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden.npz"))
TYPES = {"q4_0": 2, "q8_0": 8, "q4_k": 12, "iq4_nl": 20}
ROWS, COLS = 24, 512


@pytest.mark.parametrize("name", sorted(TYPES))
def test_oracle_reproduces_golden_vectors(name):
    t, packed, x = TYPES[name], G[f"{name}_bytes"], G["x"]
    assert np.array_equal(orc.dequantize(t, packed, ROWS * COLS).view(np.uint32), G[f"{name}_dequant"].view(np.uint32))
    # fixed summation order, no contraction: the dot products are reproducible bit for bit
    assert np.array_equal(orc.matvec(t, packed, ROWS, COLS, x[0]).view(np.uint32), G[f"{name}_matvec"].view(np.uint32))
    assert np.array_equal(orc.matmul(t, packed, ROWS, COLS, x).view(np.uint32), G[f"{name}_matmul"].view(np.uint32))
    half = len(packed) // 2
    # expf comes from libm: allow its last-bit differences between C libraries
    np.testing.assert_allclose(orc.gated_silu_matvec(t, packed[:half], packed[half:], ROWS // 2, COLS, x[0]), G[f"{name}_gated"], rtol=2e-6, atol=1e-7)


def test_oracle_reproduces_golden_encoder_and_router():
    assert np.array_equal(orc.encode_q4_k(G["q4_k_encode_in"]), G["q4_k_encode_bytes"])
    ids, w = orc.route_softmax_logits(G["route_logits"], 4, 1.5, True)
    assert np.array_equal(ids, G["route_ids"])
    np.testing.assert_allclose(w, G["route_weights"], rtol=2e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(TYPES))
def test_cuda_path_matches_golden_vectors(name):
    from tests.gpu_util import ctx, dev, host

    t, packed, x = TYPES[name], G[f"{name}_bytes"], G["x"]
    w = ctx().prepare_weight(t, packed, ROWS, COLS)
    assert np.array_equal(host(ctx().dequantize(w)).reshape(-1).view(np.uint32), G[f"{name}_dequant"].view(np.uint32))
    assert H.max_rel_error(host(ctx().linear(dev(x[:1]), w))[0], G[f"{name}_matvec"]) <= 2e-3
    assert H.max_rel_error(host(ctx().linear(dev(x), w)), G[f"{name}_matmul"]) <= 2e-3
    half = len(packed) // 2
    wg, wu = ctx().prepare_weight(t, packed[:half], ROWS // 2, COLS), ctx().prepare_weight(t, packed[half:], ROWS // 2, COLS)
    assert H.max_rel_error(host(ctx().gated_linear(dev(x[:1]), wg, wu))[0], G[f"{name}_gated"]) <= 2e-3


@pytest.mark.gpu
def test_cuda_q4_k_encoder_matches_golden_bytes():
    import torch
    from tests.gpu_util import ctx

    values = torch.from_numpy(G["q4_k_encode_in"].reshape(4, 256)).cuda()
    got = ctx().quantize(12, values)
    got = got.cpu().numpy().reshape(-1) if hasattr(got, "cpu") else np.asarray(got).reshape(-1)
    assert np.array_equal(got, G["q4_k_encode_bytes"])
