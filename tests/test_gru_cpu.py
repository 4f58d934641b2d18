"""CPU: the oracle's restatement of full_trained_egg.c (the recurrent GRU + MLP trainer) against the
reference itself — its lines 1-476 compiled unmodified into oracle/_ref/ref_cpu_gru — on the same seeded
case at the reference's compiled-in sizes (H 512, 4 layers, population 128): losses, fitness, recurrent
states and post-update weights, bit for bit, over two generations (so that carried states and updated
weights feed the second one)."""
import numpy as np
import pytest

from common import load_oracle, load_pkg, ref_gru_binary, run_ref_gru

SEED = 0x00C0FFEE


def _case(O, gcfg, kind):
    load_pkg()
    from egg_c_b200 import synth
    if kind == "init":
        model = O.gru_init_model(gcfg, 42)                         # the reference's own initial weights
    else:
        model = synth.uniform_int8(0, O.gru_model_bytes(gcfg))     # every byte uniform in [-127, 127]
    return model, synth.zipf_bytes(1, 300000)


@pytest.mark.parametrize("kind,tokens", [("init", 24), ("uniform", 12)])
def test_gru_oracle_matches_reference_cpu_trainer(kind, tokens):
    if not ref_gru_binary():
        pytest.skip("oracle/_ref/ref_cpu_gru not built (reference tree absent)")
    O = load_oracle()
    gcfg = O.make_gru_config()
    model0, data = _case(O, gcfg, kind)
    ref = run_ref_gru(model0, data, SEED, tokens, steps=2)
    assert ref["sizes"]["model_bytes"] == O.gru_model_bytes(gcfg)
    model, states = model0.copy(), np.zeros(O.gru_state_bytes(gcfg), np.int8)
    for step in range(2):
        seed = SEED ^ ((step * 0x9e3779b9) & 0xFFFFFFFF)
        losses, fit = O.gru_generation(gcfg, model, states, data, seed, step * gcfg.seq_len, tokens, True)
        assert (losses == ref["losses"][step]).all(), "losses of generation %d" % step
        assert (fit == ref["fitness"][step]).all()
    assert (states == ref["states"]).all()
    assert (model == ref["model"]).all()
    assert (model != model0).any(), "the update changed nothing: the case does not exercise update_matrix"
