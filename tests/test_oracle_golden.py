"""The oracle against the fixtures the real reference produced (CPU only)."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import dlrnet_oracle as O
from oracle import build_oracle

from conftest import GOLDEN, load_golden

SMALL = ["toy_d64_r8", "toy_d256_r32", "toy_d256_r32_stress", "toy_d512_r64_stress"]
FULL = ["cfg1_d1024_r32", "cfg1_d1024_r32_stress", "cfg2_d2048_r64", "cfg3_d4096_r128", "cfg4_d5120_r256"]


def _case(name):
    g = load_golden(name)
    m = g["meta"]
    p, x = O.seeded_case(m["d"], m["r"], m["L"], m["M"], m["seed"], m["alpha"], m["gain_jitter"])
    return g, m, p, x


@pytest.mark.parametrize("name", SMALL + FULL)
def test_oracle_reproduces_reference_outputs(name):
    g, m, p, x = _case(name)
    # the seeded generator reproduces the reference constructor's draws
    assert torch.equal(x, g["x"])
    # bf16 forward: same op order on the same torch build -> bit-equal on this image;
    # the tolerance only allows for a different CPU matmul blocking on another host.
    y1 = O.forward_eager(x, p)
    assert O.rel_l2(y1, g["y_bf16"]) <= 2e-3
    y2 = O.forward_fp32(x, p)
    assert O.rel_l2(y2, g["y_fp32"]) <= 1e-5


def test_parameter_checksums_match_reference():
    g, m, _, _ = _case("toy_d256_r32")
    p = O.seeded_params(m["d"], m["r"], m["L"], m["seed"], m["alpha"], m["gain_jitter"])
    assert abs(float(p.V.double().sum()) - m["v_sum"]) < 1e-6
    assert abs(float(p.U.double().sum()) - m["u_sum"]) < 1e-6


def test_depth_table_and_param_count():
    # examples/smoke_test.py:90-95 pins these four depths
    for (d, d_ff, r), L in {(1024, 3072, 32): 141, (2048, 6144, 64): 142,
                            (4096, 12288, 128): 143, (5120, 25600, 256): 149}.items():
        assert O.depth_for_budget(d, d_ff, r) == L
        assert O.param_count(d, r, L) <= 3 * d * d_ff
    with open(os.path.join(GOLDEN, "depth_table.json")) as f:
        table = json.load(f)
    for key, (L, n) in table.items():
        d, d_ff, r = map(int, key.split(","))
        assert O.depth_for_budget(d, d_ff, r) == L
        assert O.param_count(d, r, L) == n


def test_identity_at_alpha_zero_is_bit_exact():
    # examples/smoke_test.py:73-75
    p = O.seeded_params(64, 8, 12, seed=3, alpha=0.0)
    x = torch.randn(4, 7, 64)
    assert torch.equal(O.forward_eager(x, p), x)


@pytest.mark.parametrize("name", ["toy_d64_r8", "toy_d256_r32", "toy_d256_r32_stress"])
def test_fold_matches_reference_packer(name):
    g, m, p, _ = _case(name)
    Vf, Uf = O.fold_weights(p)
    # the reference packer stores V'^T as (L,D,R) and U'^T as (L,R,D)
    assert torch.equal(Vf.transpose(1, 2), g["packed_Vs"])
    assert torch.equal(Uf.transpose(1, 2), g["packed_Us"])


@pytest.mark.parametrize("name", ["toy_d64_r8", "toy_d256_r32_stress"])
def test_folded_algebra_equals_module_algebra(name):
    g, m, p, x = _case(name)
    Vf, Uf = O.fold_weights(p)
    y = O.forward_folded_fp32(x, Vf, Uf)
    assert O.rel_l2(y, g["y_fp32"]) <= 3e-3
    assert O.rel_l2_update(y, g["y_fp32"], x) <= 2e-2


@pytest.mark.parametrize("name", ["toy_d64_r8", "toy_d256_r32", "toy_d256_r32_stress"])
def test_c_oracle_agrees(name):
    g, m, p, x = _case(name)
    p32 = p.to(torch.float32)
    y = build_oracle.forward_f32(x.float().numpy(), p32.V.numpy(), p32.U.numpy(), p32.w.numpy(),
                                 p32.alpha.numpy(), O.EPS)
    assert O.rel_l2(torch.from_numpy(y), g["y_fp32"]) <= 1e-5


def test_update_metric_flags_an_identity_kernel():
    g, m, p, x = _case("cfg1_d1024_r32")
    assert O.rel_l2(x, g["y_bf16"]) < 1e-2          # the plain gate would pass...
    assert O.rel_l2_update(x, g["y_fp32"], x) > 0.99  # ...the update gate does not
