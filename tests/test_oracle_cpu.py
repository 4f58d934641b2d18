"""CPU tests: the oracle against the reference's known answers, host logic, ABI surface."""
import ctypes as C
import json
import os
import re

import numpy as np
import pytest

from common import ROOT, load_oracle, load_pkg, cfg_pair

GOLD = os.path.join(ROOT, "tests", "golden")


def _kat(mask):
    return json.load(open(os.path.join(GOLD, "rng_kat_mask%d.json" % mask)))


@pytest.mark.parametrize("mask", [15, 3])
def test_hash_and_noise_match_reference_known_answers(mask):
    O = load_oracle()
    k = _kat(mask)
    cfg = O.make_config(device_mask=mask)
    for s, i, h in k["hash_rng"]:
        assert O.hash_rng(s, i) == h
    for ent in k["noise"]:
        got = [O.noise(cfg, ent["seed"], i) for i in range(len(ent["values"]))]
        assert got == ent["values"]
    st = C.c_uint32(k["gen_noise_host"]["state"])
    got = [O.lib().oracle_gen_noise_host(C.byref(cfg), C.byref(st)) for _ in k["gen_noise_host"]["values"]]
    assert got == k["gen_noise_host"]["values"]


def test_ternary_codec_matches_reference_cases():
    O = load_oracle()
    for case in _kat(15)["ternary"]:
        vals = np.array(case["values"], np.int32)
        packed = O.ternary_pack(vals)
        assert packed.tolist() == case["packed"]
        assert O.ternary_unpack(packed, len(vals)).tolist() == case["values"]
    # size law of ternary_pack_estimate_size: 5 trits per byte
    assert [O.lib().oracle_ternary_packed_size(n) for n in (0, 1, 5, 6, 10, 11)] == [0, 1, 1, 2, 2, 3]


def test_struct_sizes_match_reference_sizeof():
    # sizeof(TransformerModel) / sizeof(AdamModel) printed by the reference TUs at the benchmark configurations
    O = load_oracle()
    c2 = O.make_config(hidden_dim=512, n_layers=4, seq_len=256, population_size=40960)
    assert (O.model_bytes(c2), O.opt_bytes(c2)) == (14834688, 178016256)
    c5 = O.make_config(hidden_dim=1024, n_layers=12, seq_len=512, population_size=262144)
    assert (O.model_bytes(c5), O.opt_bytes(c5), O.scales_bytes(c5)) == (159766528, 1917198336, 353536)


def test_library_sizes_agree_with_oracle():
    pkg, O = load_pkg(), load_oracle()
    for kw in (dict(hidden_dim=128, n_layers=1), dict(hidden_dim=512, n_layers=4), dict(hidden_dim=1024, n_layers=12),
               dict(hidden_dim=256, n_layers=2, use_muon=1)):
        cfg, ocfg = cfg_pair(**kw)
        assert pkg.model_bytes(cfg) == O.model_bytes(ocfg)
        assert pkg.opt_state_bytes(cfg) == O.opt_bytes(ocfg)


def test_library_exports_every_declared_symbol():
    pkg = load_pkg()
    hdr = open(os.path.join(ROOT, "include", "egg_b200.h")).read()
    declared = set(re.findall(r"\b(egg_[a-z0-9_]+)\s*\(", hdr))
    declared -= {"egg_config", "egg_ctx"}
    L = pkg.lib()
    for name in sorted(declared):
        assert hasattr(L, name), name
    assert declared == set(pkg.EXPORTS)


def test_header_is_plain_c():
    """The boundary is a C ABI: the header must compile as C99 on its own (no C++ in the signatures)."""
    import shutil
    import subprocess
    if not shutil.which("gcc"):
        pytest.skip("no gcc")
    r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-fsyntax-only", "-x", "c", os.path.join(ROOT, "include", "egg_b200.h")],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_config_validation_messages():
    pkg = load_pkg()
    L = pkg.lib()
    for kw in (dict(hidden_dim=100), dict(seq_len=8), dict(seq_len=2048), dict(vocab_size=300), dict(vocab_size=128), dict(vocab_size=131072), dict(population_size=7), dict(head_dim=32)):
        cfg = pkg.default_config(**kw)
        why = C.c_char_p()
        assert L.egg_config_validate(C.byref(cfg), C.byref(why)) == pkg.EGG_E_INVALID
        assert why.value
    cfg = pkg.default_config()
    assert L.egg_config_validate(C.byref(cfg), None) == 0
    for vocab in (512, 8192, 65536):          # the tokenizer build: any multiple of 256 that 16 bits can index
        cfg = pkg.default_config(vocab_size=vocab)
        assert L.egg_config_validate(C.byref(cfg), None) == 0


def test_oracle_tokenizer_variant_reads_32_bit_tokens():
    """vocab_size != 256 switches the token stream to uint32 (TokenType, mgpu.cu:58-66): the embedding table grows with
    the vocabulary, a byte stream is refused, and stream positions count tokens rather than bytes."""
    O = load_oracle()
    kw = dict(hidden_dim=128, n_layers=1, seq_len=16, population_size=8, device_mask=15)
    o256, o512 = O.make_config(**kw), O.make_config(vocab_size=512, **kw)
    assert O.model_bytes(o512) - O.model_bytes(o256) == 256 * 128
    m512 = O.init_model(o512, 42)
    data = (np.arange(4000, dtype=np.uint32) * 2654435761 >> 7) % 512
    a = O.eval_losses(o512, m512, data.astype(np.uint32), 0, 11, 0, 8)
    b = O.eval_losses(o512, m512, data.astype(np.uint32), 0, 11, 0, 8)
    assert (a == b).all() and (a > 0).all()
    with pytest.raises(AssertionError):
        O.eval_losses(o512, m512, data.astype(np.uint8), 0, 11, 0, 8)
    # positions count tokens, not bytes: shifting the start by one token shifts by four bytes of the stream
    c = O.eval_losses(o512, m512, data[1:].astype(np.uint32), 0, 11, 0, 8)
    d = O.eval_losses(dict_same_data(O, o512), m512, data.astype(np.uint32), 1, 11, 0, 8)
    e = O.eval_losses(dict_same_data(O, o512), m512, data[1:].astype(np.uint32), 0, 11, 0, 8)
    assert (d == e).all() and c.shape == d.shape


def dict_same_data(O, cfg):
    """A copy of the oracle configuration with USE_SAME_DATA = 1 (every pair reads the same window)."""
    import copy
    c2 = copy.copy(cfg)
    c2.use_same_data = 1
    return c2


def test_no_gpu_fails_loudly():
    """Without a device the context must refuse; nothing computes on the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    pkg = load_pkg()
    with pytest.raises(pkg.EggError):
        pkg.Context(pkg.default_config())


def test_tables_shape_and_known_values():
    O = load_oracle()
    exp, act, rope = O.init_tables(O.make_config(seq_len=16))
    assert exp[0] == 1 << 18 and exp[75] == 0 and exp[74] > 0      # exp(-i/6)*2^18 drops below 1 at i=75
    assert act[0] == 0 and act[127] == 127 and act[(-128) & 0xFF] == 0
    assert rope[0] == 1 << 20 and rope[1] == 0                      # t=0: cos=1, sin=0


def test_eval_is_deterministic_and_antithetic_pairs_share_data():
    O = load_oracle()
    cfg = O.make_config(hidden_dim=128, n_layers=1, seq_len=16, population_size=8)
    model = O.init_model(cfg, 42)
    rng = np.random.default_rng(5)
    data = rng.integers(0, 256, 5000).astype(np.uint8)
    a = O.eval_losses(cfg, model, data, 0, 1234, 0, 8)
    b = O.eval_losses(cfg, model, data, 0, 1234, 0, 8)
    assert (a == b).all()
    # chunked evaluation equals whole evaluation
    c = np.concatenate([O.eval_losses(cfg, model, data, 0, 1234, off, 2) for off in range(0, 8, 2)])
    assert (a == c).all()
    # with no noise magnitude both members of a pair see the same model: equal losses, zero fitness
    cfg0 = O.make_config(hidden_dim=128, n_layers=1, seq_len=16, population_size=8, device_mask=0)
    l0 = O.eval_losses(cfg0, model, data, 0, 1234, 0, 8)
    assert (l0[0::2] == l0[1::2]).all() and (O.fitness(l0) == 0).all()


def test_vote_matrix_linearity_and_update_count():
    O = load_oracle()
    cfg = O.make_config(hidden_dim=128, n_layers=1, seq_len=16, population_size=64)
    rng = np.random.default_rng(0)
    f1 = rng.integers(-1, 2, 32).astype(np.int32)
    f2 = rng.integers(-1, 2, 32).astype(np.int32)
    v1 = O.vote_matrix(cfg, f1, 128, 128, 200, 201, 0, 77)
    v2 = O.vote_matrix(cfg, f2, 128, 128, 200, 201, 0, 77)
    v12 = O.vote_matrix(cfg, f1 + f2, 128, 128, 200, 201, 0, 77)
    assert (v1 + v2 == v12).all()
    model = O.init_model(cfg, 42)
    before = model.copy()
    opt = np.zeros(O.opt_bytes(cfg), np.uint8)
    # one AdamW step from zero state moves acc by ~0.45*lr: weights flip only after a few steps
    assert O.update(cfg, model, opt, f1, 77, 0.5) == 0 and (model == before).all()
    n = sum(O.update(cfg, model, opt, f1, 77, 0.5) for _ in range(5))
    assert n > 0 and n >= int((model != before).sum())
    assert np.abs(model.astype(int) - before.astype(int)).max() <= 5


def test_newton_schulz_orthogonalises():
    O = load_oracle()
    rng = np.random.default_rng(1)
    for shape in ((64, 64), (32, 128), (128, 32)):
        x = rng.standard_normal(shape).astype(np.float32)
        y = O.newton_schulz(x).astype(np.float64)
        g = y @ y.T if shape[0] <= shape[1] else y.T @ y
        # 5 cubic iterations from Frobenius normalisation move singular values toward 1 (not all the way)
        s = np.linalg.svd(y, compute_uv=False)
        assert s.max() < 1.3 and np.isfinite(g).all()


def test_index_math_selftest_runs_on_the_host():
    """FastDiv (the multiply-shift division of the per-tile index arithmetic) against C division, through the C ABI."""
    pkg = load_pkg()
    pkg.selftest_index_math()


def test_oracle_window_transforms_against_their_definitions():
    """ntt_mode 1 is the Walsh-Hadamard transform in natural order; modes 2 and 3 at their full lengths (256, 65536)
    are number-theoretic transforms with root 3: X[k] = sum_n x[n] 3^(n k) mod p.  At shorter lengths the reference
    keeps the full-length root in its twiddles (egg_ntt.cuh:349-362), so only the first stages agree with a true
    transform; those lengths are pinned by the reference-kernel goldens instead."""
    O = load_oracle()
    rng = np.random.default_rng(3)
    x = rng.integers(0, 256, 64).astype(np.int32)
    h = np.array([[1]])
    while h.shape[0] < 64:
        h = np.block([[h, h], [h, -h]])
    assert (O.window_transform(O.make_config(ntt_mode=1), x) == h @ x).all()
    x = rng.integers(0, 256, 256).astype(np.int32)
    n = np.arange(256)
    pw = np.array([pow(3, int(e), 257) for e in range(256)], np.int64)
    want = np.array([(x.astype(np.int64) * pw[(n * k) % 256]).sum() % 257 for k in range(256)])
    assert (O.window_transform(O.make_config(ntt_mode=2), x) == want).all()
    # mode 3 at a short length: every output stays below the prime and the transform is linear mod p
    a, b = rng.integers(0, 65537, 32).astype(np.int32), rng.integers(0, 65537, 32).astype(np.int32)
    c3 = O.make_config(ntt_mode=3)
    ta, tb, tab = O.window_transform(c3, a), O.window_transform(c3, b), O.window_transform(c3, ((a.astype(np.int64) + b) % 65537).astype(np.int32))
    assert ta.max() < 65537 and ta.min() >= 0
    assert (((ta.astype(np.int64) + tb) % 65537) == tab).all()


def test_ntt_mode_layout_and_validation():
    pkg, O = load_pkg(), load_oracle()
    kw = dict(hidden_dim=128, n_layers=1, seq_len=16)
    for mode in (1, 2, 3):
        cfg, ocfg = cfg_pair(ntt_mode=mode, **kw)
        assert pkg.model_bytes(cfg) == O.model_bytes(ocfg) == O.model_bytes(O.make_config(**kw)) + 3 * 256 * 128
        assert pkg.opt_state_bytes(cfg) == O.opt_bytes(ocfg) == O.opt_bytes(O.make_config(**kw)) + 3 * 256 * 128 * 12
    L = pkg.lib()
    for bad in (dict(ntt_mode=4), dict(ntt_mode=1, seq_len=48), dict(ntt_mode=1, seq_len=256, hidden_dim=128),
                dict(ntt_mode=2, seq_len=512, hidden_dim=512)):
        cfg = pkg.default_config(**bad)
        assert L.egg_config_validate(C.byref(cfg), None) == pkg.EGG_E_INVALID, bad
