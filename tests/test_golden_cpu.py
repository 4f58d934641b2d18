"""CPU: the oracle must reproduce what the reference's own kernels produced on a B200
(tests/golden/ref_mgpu_*.npz, written by tests/golden/make_golden.py mgpu)."""
import os
import zlib

import numpy as np
import pytest

from common import REF_CONFIGS, ROOT, load_oracle, make_case

GOLD = os.path.join(ROOT, "tests", "golden")
STEPS, SEED, LR = 4, 0x00C0FFEE, 0.5


@pytest.mark.parametrize("tag", ["tiny", "small", "muon_tiny", "tok_tiny", "tok_small", "ntt1_tiny", "ntt2_tiny", "ntt3_small"])
def test_oracle_reproduces_reference_kernel_outputs(tag):
    path = os.path.join(GOLD, "ref_mgpu_%s.npz" % tag)
    g = np.load(path)
    O = load_oracle()
    kw = REF_CONFIGS[tag]
    cfg, ocfg, model0, data = make_case(kw, data_len=50000)
    pop, S = kw["population_size"], kw["seq_len"]
    model, opt = model0.copy(), np.zeros(O.opt_bytes(ocfg), np.uint8)
    muon = kw.get("use_muon", 0)
    for step in range(STEPS):
        losses = O.eval_losses(ocfg, model, data, step * S, SEED + step, 0, pop)
        if muon and step > 0:
            break       # later Muon generations start from weights that may differ by tolerance-level flips: see the Muon test below
        assert (losses == g["losses"][step]).all(), "losses of generation %d" % step
        fit = O.fitness(losses)
        assert (fit == g["fitness"][step]).all()
        n = O.update(ocfg, model, opt, fit, SEED + step, LR)
        if not muon:
            assert n == int(g["updates"][step])
    if not muon:
        changed = np.nonzero(model != model0)[0]
        assert len(changed) == int(g["changed_count"])
        assert (changed[:2048] == g["changed_idx"]).all() and (model[changed[:2048]] == g["changed_val"]).all()
        assert zlib.crc32(model.tobytes()) == int(g["model_crc"])
        assert zlib.crc32(opt.tobytes()) == int(g["opt_crc"]), "fp32 optimiser state is not bit-identical to the reference kernels"
        assert len(changed) > 0


@pytest.mark.parametrize("tag", ["tiny", "small"])
def test_oracle_reproduces_deggs_worker_kernels_with_overlays(tag):
    """Six generations of the d-eggs worker's own kernels on a B200 (tests/golden/ref_deggs_*.npz, written by
    make_golden.py deggs): losses, update counts, adaptive-noise overlays, weights and fp32 state, with the
    worker's seed chain."""
    from common import DEGGS_CONFIGS, deggs_initial_scales
    g = np.load(os.path.join(GOLD, "ref_deggs_%s.npz" % tag))
    O = load_oracle()
    kw = DEGGS_CONFIGS[tag]
    cfg, ocfg, model0, data = make_case(kw, data_len=50000)
    pop, S = kw["population_size"], kw["seq_len"]
    model, opt = model0.copy(), np.zeros(O.opt_bytes(ocfg), np.uint8)
    scales = deggs_initial_scales(O.scales_bytes(ocfg))
    seed, step = 42, 0
    gens = len(g["losses"]) if tag == "tiny" else 3          # the later generations of the larger case only cost time
    for gen in range(gens):
        losses = O.eval_losses(ocfg, model, data, step * S, seed, 0, pop, scales=scales)
        assert (losses == g["losses"][gen]).all(), "losses of generation %d" % gen
        n = O.update_scaled(ocfg, model, opt, O.fitness(losses), seed, 0.5, scales)
        assert n == int(g["updates"][gen])
        assert zlib.crc32(scales.tobytes()) == int(g["scales_crc"][gen]), "overlays after generation %d" % gen
        step += 1
        seed = O.hash_rng(seed, step)
    if gens == len(g["losses"]):
        assert (scales == g["scales_final"]).all()
        changed = np.nonzero(model != model0)[0]
        assert len(changed) == int(g["changed_count"]) and len(changed) > 0
        assert (changed[:2048] == g["changed_idx"]).all() and (model[changed[:2048]] == g["changed_val"]).all()
        assert zlib.crc32(model.tobytes()) == int(g["model_crc"])
        assert zlib.crc32(opt.tobytes()) == int(g["opt_crc"])


@pytest.mark.parametrize("tag", ["muon_tiny", "muon_small"])
def test_oracle_muon_step_within_tolerance_of_reference_muon(tag):
    """One Muon generation of the reference's own kernels (momentum, cuBLAS Newton-Schulz, quantised apply;
    muon_internal.cuh:15-342) from zero state, recorded on a B200 (tests/golden/ref_muon_step_*.npz, make_golden.py
    muon): the oracle's double-accumulating Newton-Schulz must reproduce a seeded sample of 8192 fp32 state values
    within 1e-5 relative; int8 weights that flip differently are counted (a flip happens when an accumulator
    crosses 1, so tolerance-level differences can move single flips)."""
    g = np.load(os.path.join(GOLD, "ref_muon_step_%s.npz" % tag))
    O = load_oracle()
    kw = REF_CONFIGS[tag]
    cfg, ocfg, model0, data = make_case(kw, data_len=50000)
    pop = kw["population_size"]
    model, opt = model0.copy(), np.zeros(O.opt_bytes(ocfg), np.uint8)
    losses = O.eval_losses(ocfg, model, data, 0, SEED, 0, pop)
    assert (losses == g["losses"][0]).all()
    fit = O.fitness(losses)
    assert (fit == g["fitness"][0]).all()
    O.update(ocfg, model, opt, fit, SEED, LR)
    got = opt.view(np.float32)[g["sample_idx"]].astype(np.float64)
    want = g["sample_val"][0].astype(np.float64)
    err = np.abs(got - want)
    tol = 1e-5 * np.maximum(np.abs(got), np.abs(want)) + 2e-6
    assert (err <= tol).all(), "%d of %d sampled state values beyond 1e-5 relative (max abs err %g)" % ((err > tol).sum(), len(err), err.max())
    ref_changed = {int(i): int(v) for i, v in zip(g["changed_idx"][0], g["changed_val"][0]) if i >= 0}
    mine = np.nonzero(model != model0)[0]
    if int(g["changed_count"][0]) <= 4096:
        differing = sum(1 for i in mine if ref_changed.get(int(i)) != int(model[i])) + sum(1 for i in ref_changed if model[i] == model0[i])
        assert differing <= max(4, model.size // 20000), "%d weights flip differently from the reference" % differing
