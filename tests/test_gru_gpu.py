"""GPU parity of the recurrent model (full_trained_egg.c) through the C ABI: per-member losses, pair
fitness, carried recurrent states and post-update int8 weights, bit-exact against the CPU oracle and
against the reference's own CPU trainer functions (oracle/_ref/ref_cpu_gru) where they were built."""
import numpy as np
import pytest

from common import load_oracle, load_pkg, ref_gru_binary, run_ref_gru

pytestmark = pytest.mark.gpu
SEED = 0x00C0FFEE


def _run_generations(pkg, O, kw, tokens, gens, model0, data, seeds_starts, check_oracle=True):
    gcfg, ocfg = pkg.default_gru_config(**kw), O.make_gru_config(**kw)
    assert pkg.gru_model_bytes(gcfg) == O.gru_model_bytes(ocfg) and pkg.gru_state_bytes(gcfg) == O.gru_state_bytes(ocfg)
    ctx = pkg.GruContext(gcfg, 0)
    ctx.upload_model(model0)
    ctx.set_dataset(data)
    model, states = model0.copy(), np.zeros(O.gru_state_bytes(ocfg), np.int8)
    out = []
    for g in range(gens):
        seed, start = seeds_starts[g]
        losses, fit = ctx.generation(seed, start, tokens, True)
        out.append((losses, fit))
        if check_oracle:
            wl, wf = O.gru_generation(ocfg, model, states, data, seed, start, tokens, True)
            assert (losses == wl).all(), "losses of generation %d: %s vs %s" % (g, losses[:6], wl[:6])
            assert (fit == wf).all()
            assert (ctx.download_states() == states).all(), "recurrent states after generation %d" % g
            assert (ctx.download_model() == model).all(), "weights after generation %d" % g
    res = dict(gens=out, model=ctx.download_model(), states=ctx.download_states(), launches=ctx.launch_count())
    ctx.close()
    return res


def test_gru_small_config_three_generations_against_oracle():
    """H 128, 2 layers, population 64; 40 tokens = two replays of the 16-token graph + 8 single steps."""
    pkg, O = load_pkg(), load_oracle()
    from egg_c_b200 import synth
    kw = dict(hidden_dim=128, n_layers=2, seq_len=64, population_size=64)
    ocfg = O.make_gru_config(**kw)
    model0 = O.gru_init_model(ocfg, 42)
    data = synth.zipf_bytes(1, 20000)
    r = _run_generations(pkg, O, kw, 40, 3, model0, data, [(SEED, 0), (SEED ^ 0x9e3779b9, 64), (77, 12345)])
    assert (r["model"] != model0).any()
    assert r["launches"] >= 3 * 40 * (6 * 2 + 4)


def test_gru_reference_sizes_against_oracle_uniform_weights():
    """The reference's compiled-in sizes (H 512, 4 layers, population 128), weights uniform in [-127, 127]."""
    pkg, O = load_pkg(), load_oracle()
    from egg_c_b200 import synth
    ocfg = O.make_gru_config()
    model0 = synth.uniform_int8(0, O.gru_model_bytes(ocfg))
    data = synth.zipf_bytes(1, 300000)
    _run_generations(pkg, O, {}, 6, 2, model0, data, [(SEED, 0), (SEED ^ 0x9e3779b9, 4096)])


def test_gru_against_reference_cpu_trainer_run_here():
    if not ref_gru_binary():
        pytest.skip("oracle/_ref/ref_cpu_gru not built")
    pkg, O = load_pkg(), load_oracle()
    from egg_c_b200 import synth
    ocfg = O.make_gru_config()
    model0 = O.gru_init_model(ocfg, 42)
    data = synth.zipf_bytes(3, 300000)
    tokens = 20
    ref = run_ref_gru(model0, data, 4242, tokens, steps=2)
    seeds = [(4242, 0), (4242 ^ 0x9e3779b9, 4096)]
    r = _run_generations(pkg, O, {}, tokens, 2, model0, data, seeds, check_oracle=False)
    for g in range(2):
        assert (r["gens"][g][0] == ref["losses"][g]).all(), "losses of generation %d" % g
        assert (r["gens"][g][1] == ref["fitness"][g]).all()
    assert (r["states"] == ref["states"]).all()
    assert (r["model"] == ref["model"]).all()
    assert (r["model"] != model0).any()


def test_gru_full_generation_matches_reference_golden():
    """One whole generation of full_trained_egg.c at its compiled-in size -- 128 members x 4096 tokens, fitness, the
    25 threshold-vote matrix updates (full_trained_egg.c:527-577) -- against what the reference's own code produced
    on the CPU (tests/golden/ref_cpu_gru_full.npz, written by tests/golden/make_golden.py gru; minutes of CPU time,
    hence a committed fixture)."""
    import os
    import zlib
    from common import ROOT
    pkg, O = load_pkg(), load_oracle()
    from egg_c_b200 import synth
    g = np.load(os.path.join(ROOT, "tests", "golden", "ref_cpu_gru_full.npz"))
    ocfg = O.make_gru_config()
    model0 = synth.uniform_int8(0, O.gru_model_bytes(ocfg))
    data = synth.zipf_bytes(1, 1 << 20)
    r = _run_generations(pkg, O, {}, ocfg.seq_len, 1, model0, data, [(SEED, 0)], check_oracle=False)
    losses, fit = r["gens"][0]
    assert (losses == g["losses"]).all(), "%d of 128 losses differ" % (losses != g["losses"]).sum()
    assert (fit == g["fitness"]).all()
    changed = np.nonzero(r["model"] != model0)[0]
    assert len(changed) == int(g["changed_count"]) and len(changed) > 0
    assert (changed[:4096] == g["changed_idx"]).all() and (r["model"][changed[:4096]] == g["changed_val"]).all()
    assert zlib.crc32(r["model"].tobytes()) == int(g["model_crc"])
    assert (r["states"][:2048] == g["states_head"]).all()
    assert zlib.crc32(r["states"].tobytes()) == int(g["states_crc"])
