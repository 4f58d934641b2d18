"""CPU: the oracle must reproduce what the reference's own kernels produced on a B200
(tests/golden/ref_mgpu_*.npz, written by tests/golden/make_golden.py mgpu)."""
import os
import zlib

import numpy as np
import pytest

from common import REF_CONFIGS, ROOT, load_oracle, make_case

GOLD = os.path.join(ROOT, "tests", "golden")
STEPS, SEED, LR = 4, 0x00C0FFEE, 0.5


@pytest.mark.parametrize("tag", ["tiny", "small", "muon_tiny"])
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
            break       # Muon's fp32 Newton–Schulz is compared at tolerance (cuBLAS order unpinned): weights may drift
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
