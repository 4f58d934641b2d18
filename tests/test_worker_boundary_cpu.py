"""CPU: the d-eggs worker boundary of the library (wire messages, trit codec, chunk fitness, seed chain)
against the reference's own protocol.h / ternary_pack.h outputs and against the oracle."""
import json
import os
import sys

import numpy as np
import pytest

from common import ROOT, load_oracle, load_pkg

KAT = json.load(open(os.path.join(ROOT, "tests", "golden", "rng_kat_mask15.json")))


def test_wire_messages_match_reference_serialisers():
    pkg = load_pkg()
    for case in KAT["wire"]:
        m = pkg.WireMsg(opcode=case["opcode"], payload_size=case["payload_size"], seed=case["seed"], last_step=case["last_step"],
                        data_position=case["data_position"], updates_count=case["updates_count"], sum_loss=case["sum_loss"])
        enc = pkg.wire_encode(m)
        assert enc.hex() == case["hex"]
        back, total = pkg.wire_decode(enc)
        assert total == len(enc) - 10 + case["payload_size"]
        for f in ("opcode", "seed", "last_step", "data_position"):
            assert getattr(back, f) == case[f]
        if case["opcode"] != 0:
            assert back.payload_size == case["payload_size"]
        if case["opcode"] == 1:
            assert back.updates_count == case["updates_count"] and back.sum_loss == case["sum_loss"]


def test_wire_rejects_bad_magic_and_version():
    pkg = load_pkg()
    good = bytearray(pkg.wire_encode(pkg.WireMsg(opcode=0, seed=1)))
    bad = bytes([0]) + bytes(good[1:])
    with pytest.raises(pkg.EggError) as e1:
        pkg.wire_decode(bad)
    assert e1.value.code == -1
    good[4] = 9
    with pytest.raises(pkg.EggError) as e2:
        pkg.wire_decode(bytes(good))
    assert e2.value.code == -2


def test_ternary_codec_matches_reference_and_oracle():
    pkg, O = load_pkg(), load_oracle()
    for case in KAT["ternary"]:
        vals = np.array(case["values"], np.int32)
        assert pkg.ternary_pack(vals).tolist() == case["packed"]
        assert pkg.ternary_unpack(np.array(case["packed"], np.uint8), len(vals)).tolist() == case["values"]
    rng = np.random.default_rng(3)
    for n in (0, 1, 4, 5, 6, 1023, 20480, 131072):        # ragged tails and the fitness sizes of the benchmark configurations
        v = rng.integers(-1, 2, n).astype(np.int32)
        p = pkg.ternary_pack(v)
        assert len(p) == (n + 4) // 5 and (p == O.ternary_pack(v)).all()
        assert (pkg.ternary_unpack(p, n) == v).all()


@pytest.mark.parametrize("mean_filter,adaptive", [(1, 1), (0, 1), (1, 0), (0, 0)])
def test_chunk_fitness_matches_oracle(mean_filter, adaptive):
    pkg, O = load_pkg(), load_oracle()
    rng = np.random.default_rng(7)
    for n, bias in ((64, 0), (4096, 37), (4096, -5), (2, 0)):
        losses = (rng.integers(10000, 20000, n) + bias * (np.arange(n) % 2)).astype(np.int32)
        got, gs = pkg.deggs_chunk_fitness(losses, mean_filter, 1.2, adaptive, 0.1)
        want, ws = O.deggs_chunk_fitness(losses, mean_filter, 1.2, adaptive, 0.1)
        assert (got == want).all() and gs == ws == int(losses.astype(np.int64).sum())
        assert set(np.unique(got)) <= {-1, 0, 1}
    # all-equal losses: with the MAD threshold the reference's comparison "|diff| < 0" is false and a zero
    # difference falls through to -1 (worker.cu:672-676); the plain pairwise rule gives 0
    got, _ = pkg.deggs_chunk_fitness(np.full(16, 5, np.int32), 1, 1.2, 1, 0.1)
    assert (got == -1).all()
    got, _ = pkg.deggs_chunk_fitness(np.full(16, 5, np.int32), 1, 1.2, 0, 0.1)
    assert (got == 0).all()


def test_seed_chain_is_the_reference_hash():
    pkg, O = load_pkg(), load_oracle()
    for s, i, h in KAT["hash_rng"]:
        assert pkg.next_seed(s, i) == h
    assert pkg.next_seed(42, 1) == O.hash_rng(42, 1)


def test_chunk_fitness_matches_reference_worker_lines():
    """The library and the oracle against d-eggs/src/worker.cu:635-687 itself: those lines, cut by line range and
    compiled unmodified into oracle/_ref/ref_worker_fitness, produced tests/golden/ref_worker_fitness.json
    (tests/golden/make_golden.py worker); where the binary is present it is also run live on fresh vectors."""
    import json
    import subprocess
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import make_golden
    pkg, O = load_pkg(), load_oracle()
    gold = json.load(open(os.path.join(ROOT, "tests", "golden", "ref_worker_fitness.json")))
    vectors = make_golden.worker_vectors()
    assert len(gold["cases"]) == 4 * len(vectors)
    for case in gold["cases"]:
        losses = vectors[case["vector"]]
        bits = np.unpackbits(np.array(case["fitness_packed"], np.uint8))[:2 * case["pairs"]].reshape(-1, 2)
        want = (bits[:, 0] * 2 + bits[:, 1]).astype(np.int32) - 1
        for impl in (pkg, O):
            got, sl = impl.deggs_chunk_fitness(losses, case["mean_filter"], 1.2, case["adaptive"], 0.1)
            assert sl == case["sum_loss"]
            assert (got == want).all(), (case["vector"], case["mean_filter"], case["adaptive"])
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_worker_fitness")
    if os.path.exists(exe):
        rng = np.random.default_rng(123)
        for n in (2, 6, 1000, 4096):
            losses = rng.integers(-50000, 50000, n).astype(np.int32)
            for mf in (0, 1):
                for ad in (0, 1):
                    r = subprocess.run([exe, str(mf), str(ad)], input=" ".join(str(int(x)) for x in losses), capture_output=True, text=True, check=True)
                    o = json.loads(r.stdout)
                    got, sl = pkg.deggs_chunk_fitness(losses, mf, 1.2, ad, 0.1)
                    assert sl == o["sum_loss"] and got.tolist() == o["fitness"]
