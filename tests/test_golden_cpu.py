"""Pins the CPU oracle against outputs of the reference's own CUDA code.

tests/golden/reference_vectors.npz was produced by tests/golden/make_golden.py on a GPU from the reference's sources
(compiled where they lie by oracle/build_ref.py); the inputs are rebuilt here from the same seeds.  Integer work is
compared exactly, floating point within the parity bars (the oracle uses IEEE libm where the GPU uses its fast
approximations, so a few rays per thousand may gain or lose a sample at a voxel boundary)."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

from helpers import ABS_RGB, REL_MLP, half_bits, half_vals, rel_err  # noqa: E402
from oracle_pipeline import OracleField  # noqa: E402

PATH = os.path.join(HERE, "golden", "reference_vectors.npz")
AUX_PATH = os.path.join(HERE, "golden", "device_level_scales.npz")   # not reference output: see make_golden.py


@pytest.fixture(scope="module")
def golden():
    if not os.path.exists(PATH):
        pytest.skip("tests/golden/reference_vectors.npz has not been generated yet (needs a GPU run of make_golden.py)")
    return np.load(PATH)


@pytest.fixture(scope="module")
def inputs():
    import make_golden
    return make_golden.golden_inputs(), make_golden.FIELD, make_golden.MARCH


@pytest.mark.parametrize("tag,b", [("b1447", 1.447), ("b13819", 1.3819)])
def test_field_step_against_reference_outputs(orc, golden, inputs, tag, b):
    inp, f, _ = inputs
    fi = inp["field"]
    aux = np.load(AUX_PATH)
    scales, sscales = aux["%s_scales" % tag], aux["%s_scatter_scales" % tag]
    dls = int(aux["%s_dense_level_start" % tag][0])
    assert dls == orc.dense_level_start(f["T"], f["base"], b, f["L"])
    assert np.allclose(orc.level_scales(f["base"], b, f["L"]), scales, rtol=2e-6)
    field = OracleField(f["L"], f["T"], f["base"], b, scales, dls, f["density"], f["color"], fi["table"], fi["dens"][0], fi["dens"][1],
                        fi["col"][0], fi["col"][1], sscales)
    tgt8 = np.zeros((f["n"], 8), np.float32); tgt8[:, :3] = fi["tgt3"]
    r = field.forward_backward(fi["pos"], fi["dirs"], half_bits(tgt8), f["loss_scale"], f["density_bias"])
    assert rel_err(r["d_out"], golden["field_%s_density_out" % tag]) <= REL_MLP
    assert np.max(np.abs(r["c_out"][:, :3] - golden["field_%s_color_out" % tag])) <= 1e-2
    g_cin = golden["field_%s_color_in" % tag]
    assert np.array_equal(r["c_in"][:, 16:], g_cin[:, 16:])                       # SH: same formula, same rounding
    assert rel_err(half_vals(r["c_in"][:, :16]), half_vals(g_cin[:, :16])) <= REL_MLP
    g_hash = np.zeros(f["L"] * f["T"] * 2, np.float32)
    g_hash[golden["field_%s_hash_grad_idx" % tag]] = golden["field_%s_hash_grad_val" % tag]
    assert rel_err(r["g_table"], g_hash) <= 3 * REL_MLP
    assert np.mean((r["g_table"] != 0) != (g_hash != 0)) < 1e-3                   # same touched entries
    for net, (gw, gb, dims) in enumerate(((r["g_dW"], r["g_db"], f["density"]), (r["g_cW"], r["g_cb"], f["color"]))):
        i, h, o, nl = dims
        wo = bo = 0
        for l in range(nl):
            ki, ko = (i if l == 0 else h), (o if l == nl - 1 else h)
            assert rel_err(gw[wo:wo + ki * ko], golden["field_%s_dW_%d_%d" % (tag, net, l)]) <= 3 * REL_MLP, (net, l)
            assert rel_err(gb[bo:bo + ko], golden["field_%s_db_%d_%d" % (tag, net, l)]) <= 3 * REL_MLP, (net, l)
            wo += ki * ko; bo += ko


@pytest.mark.parametrize("tag,cascades,spv", [("c1", 1, 1), ("c2", 2, 1), ("k2", 1, 2)])
def test_march_against_reference_outputs(orc, golden, inputs, tag, cascades, spv):
    from test_oracle_nerf_cpu import speckled_bitfield
    inp, _, m = inputs
    o, d = inp["rays_o"], inp["rays_d"]
    amin, amax = [-m["aabb"]] * 3, [m["aabb"]] * 3
    G = lambda k: golden["march_%s_%s" % (tag, k)]
    d_inv, near, far = orc.ray_aabb(o, d, amin, amax, cascades)
    assert np.allclose(d_inv, G("dinv"), rtol=2e-6) and np.allclose(near, G("near"), rtol=1e-5, atol=1e-6) and np.allclose(far, G("far"), rtol=1e-5)
    bits = speckled_bitfield(orc, m["res"], m["levels"], cascades)
    # walk with the reference's own reciprocal directions and entry / exit distances
    cnt = orc.march_count(o, d, G("dinv"), G("near"), G("far"), bits, m["res"], amin, amax, cascades, m["levels"], spv)
    ref_cnt = G("steps")
    assert np.mean(cnt != ref_cnt) <= 1e-2 and np.max(np.abs(cnt.astype(np.int64) - ref_cnt.astype(np.int64))) <= 2 * spv
    assert ref_cnt.sum() > 2000
    # integer pipeline on the reference's counts: exact
    assert np.array_equal(orc.exclusive_sum(ref_cnt), G("offs"))
    assert np.array_equal(G("ray"), np.repeat(np.arange(len(ref_cnt), dtype=np.uint32), ref_cnt))
    offs = orc.exclusive_sum(cnt)
    t, ray, pos = orc.march_emit(o, d, G("dinv"), G("near"), G("far"), bits, m["res"], amin, amax, cascades, m["levels"], spv, offs, 0, int(cnt.sum()))
    good = np.nonzero(cnt == ref_cnt)[0]
    mine = np.concatenate([np.arange(offs[r], offs[r] + cnt[r]) for r in good])
    theirs = np.concatenate([np.arange(G("offs")[r], G("offs")[r] + ref_cnt[r]) for r in good])
    assert np.allclose(t[mine], G("t")[theirs], rtol=2e-5, atol=2e-6)
    assert np.allclose(pos[mine][:, :3], G("pos")[theirs], atol=2e-6)


def test_compositing_and_loss_gradients_against_reference_outputs(orc, golden, inputs):
    c = inputs[0]["comp"]
    R = c["R"]
    sigma = np.exp(np.minimum(c["dens"][:, 0] - np.float32(c["bias"]), 8)).astype(np.float32)
    rgb, depth, phi, dw, ws = orc.render_rays_distortion(R, c["off"], c["counts"], c["t"], sigma, c["col"], c["target"], c["lam"], 0.0, c["bg"])
    assert np.max(np.abs(rgb - golden["comp_rgb"])) <= ABS_RGB and np.max(np.abs(phi - golden["comp_phi"])) <= 2 * ABS_RGB
    assert np.allclose(depth, golden["comp_depth"], rtol=1e-4, atol=1e-4)
    assert rel_err(dw, golden["comp_dw"]) <= REL_MLP and rel_err(ws, golden["comp_ws"]) <= REL_MLP
    col8 = np.zeros((len(c["t"]), 8), np.float32); col8[:, :3] = c["col"]
    grad, dsig = orc.color_grad(R, c["counts"], c["off"], c["t"], c["dens"], col8, golden["comp_phi"], golden["comp_rgb"], golden["comp_dw"],
                                golden["comp_ws"], c["scale"], c["bias"], R, 8)
    assert rel_err(half_vals(grad)[:, :3], half_vals(golden["comp_grad"])) <= REL_MLP
    assert rel_err(dsig, golden["comp_dsig"]) <= REL_MLP
    i_rgb, _, _ = orc.render_rays(R, 0, 0, c["off"], c["counts"], c["t"], sigma, c["col"], None, c["bg"])
    assert np.max(np.abs(i_rgb - golden["comp_infer_rgb"])) <= ABS_RGB


def test_occupancy_sample_jitter_against_reference_outputs(orc, golden, inputs):
    """cuRAND Philox4x32-10 as the reference seeds it (one subsequence per thread): restated in the oracle."""
    _, _, m = inputs
    s = orc.sample_aabb([-m["aabb"]] * 3, [m["aabb"]] * 3, (16, 16, 16), 16 ** 3, 16 ** 3, 0, 5)
    ref = golden["occ_samples"]
    assert np.array_equal(s[:, 3], ref[:, 3])                                      # cell ids
    assert np.allclose(s[:, :3], ref[:, :3], atol=2e-6)
