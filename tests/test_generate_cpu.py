"""CPU: the oracle's sampling restatement against the continuations the d-eggs generate_sequence_kernel produced
on a B200 (tests/golden/ref_generate.json, written by tests/golden/make_golden.py generate)."""
import json
import os

from common import DEGGS_CONFIGS, ROOT, load_oracle, make_case


def test_oracle_generate_reproduces_reference_kernel():
    O = load_oracle()
    cases = json.load(open(os.path.join(ROOT, "tests", "golden", "ref_generate.json")))
    for c in cases:
        cfg, ocfg, model, data = make_case(DEGGS_CONFIGS[c["tag"]], data_len=50000, model_kind=c["model_kind"], model_seed=5)
        got = O.generate(ocfg, model, data[100:100 + c["seed_len"]], c["gen_len"], c["seed"], c["temp"], c["min_p"], c["penalty"])
        assert got.tolist() == c["tokens"], (c["tag"], c["model_kind"], c["seed"])
