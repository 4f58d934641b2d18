"""GPU parity of sampling (egg_generate ≙ generate_sequence_kernel): the sampled bytes must equal the
reference kernel's (golden vectors from a B200 run, and the kernel run live where oracle/_ref holds it) and the
CPU oracle's, including the thread-major order of the reference's weighted draw when hidden_dim < vocab."""
import json
import os

import numpy as np
import pytest

from common import DEGGS_CONFIGS, ROOT, deggs_binary, load_oracle, load_pkg, make_case, run_ref_generate

pytestmark = pytest.mark.gpu
GOLD = os.path.join(ROOT, "tests", "golden", "ref_generate.json")


def _ctx(pkg, cfg, model):
    ctx = pkg.Context(cfg, 0, 2)
    ctx.upload_model(model)
    return ctx


def test_generate_matches_golden_reference_kernel():
    pkg = load_pkg()
    cases = json.load(open(GOLD))
    assert len(cases) >= 6
    for c in cases:
        cfg, ocfg, model, data = make_case(DEGGS_CONFIGS[c["tag"]], data_len=50000, model_kind=c["model_kind"], model_seed=5)
        ctx = _ctx(pkg, cfg, model)
        got = ctx.generate(data[100:100 + c["seed_len"]], c["gen_len"], c["seed"], c["temp"], c["min_p"], c["penalty"])
        assert got.tolist() == c["tokens"], (c["tag"], c["model_kind"], c["seed"])
        ctx.close()


@pytest.mark.parametrize("kw,sl,gl", [(dict(hidden_dim=512, n_layers=2, seq_len=64, population_size=8), 16, 40),
                                      (dict(hidden_dim=384, n_layers=1, seq_len=32, population_size=8, device_mask=3), 3, 29),
                                      (dict(hidden_dim=1024, n_layers=1, seq_len=32, population_size=8), 8, 8)])
def test_generate_matches_oracle_other_widths(kw, sl, gl):
    pkg, O = load_pkg(), load_oracle()
    cfg, ocfg, model, data = make_case(kw, data_len=20000, model_kind="random_all", model_seed=11)
    ctx = _ctx(pkg, cfg, model)
    for seed, temp, mp, pen in ((5, 0.6, 0.08, 0.2), (6, 1.0, 0.0, 0.0)):
        want = O.generate(ocfg, model, data[:sl], gl, seed, temp, mp, pen)
        got = ctx.generate(data[:sl], gl, seed, temp, mp, pen)
        assert (got == want).all(), (seed, got[sl:sl + 8], want[sl:sl + 8])
    with pytest.raises(pkg.EggError):
        ctx.generate(data[:sl], kw["seq_len"], 1)          # longer than the RoPE table
    ctx.close()


def test_generate_matches_reference_kernel_run_here():
    if not deggs_binary("small"):
        pytest.skip("oracle/_ref/ref_deggs_small not built")
    pkg = load_pkg()
    cfg, ocfg, model, data = make_case(DEGGS_CONFIGS["small"], data_len=30000, data_seed=9, model_kind="random_all", model_seed=21)
    ctx = _ctx(pkg, cfg, model)
    want = run_ref_generate("small", model, data[5:15], 22, 31337, 0.7, 0.05, 0.5)
    got = ctx.generate(data[5:15], 22, 31337, 0.7, 0.05, 0.5)
    assert (got == want).all()
    ctx.close()
