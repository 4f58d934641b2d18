"""GPU: the reference's tokenizer build (VOCAB_SIZE != 256: uint32 tokens, embedding rows and head columns over a
wider vocabulary, the strided two-pass cross-entropy of mgpu.cu:969-1023) against the oracle and, where the harness
binaries exist, the reference's own kernels."""
import numpy as np
import pytest

from common import REF_CONFIGS, load_oracle, load_pkg, make_case, ref_binary, run_ref_mgpu

pytestmark = pytest.mark.gpu
SEED = 0x5EED1234


def _ctx(cfg, wave=0):
    return load_pkg().Context(cfg, 0, wave)


@pytest.mark.parametrize("tag", ["tok_tiny", "tok_small"])
def test_generations_match_oracle_and_reference_kernels(tag):
    """Four chained generations (evaluate, fitness, AdamW on every parameter, the V-wide embedding included)."""
    O = load_oracle()
    kw = REF_CONFIGS[tag]
    cfg, ocfg, model, data = make_case(kw, data_len=50000)
    assert data.dtype == np.uint32 and int(data.max()) >= 256
    pop, S = kw["population_size"], kw["seq_len"]
    ctx = _ctx(cfg)
    ctx.upload_model(model)
    ctx.set_dataset(data)
    omodel, oopt = model.copy(), np.zeros(O.opt_bytes(ocfg), np.uint8)
    rmodel, ropt = model.copy(), None
    for step in range(4):
        seed = SEED + step
        ctx.eval_chunk(seed, step * S, 0, pop)
        ctx.compute_fitness_pairs(0, pop // 2)
        losses, fit = ctx.read_losses(0, pop), ctx.read_fitness(0, pop // 2)
        want = O.eval_losses(ocfg, omodel, data, step * S, seed, 0, pop)
        assert (losses == want).all(), "generation %d: %s vs %s" % (step, losses[:6], want[:6])
        assert (fit == O.fitness(want)).all()
        n_gpu = ctx.apply_update(seed, 0.5)
        n_orc = O.update(ocfg, omodel, oopt, fit, seed, 0.5)
        got = ctx.download_model()
        assert (got == omodel).all(), "generation %d: %d weights differ" % (step, (got != omodel).sum())
        assert n_gpu == n_orc
        assert (ctx.download_opt_state() == oopt).all()
        if ref_binary(tag):
            ref = run_ref_mgpu(tag, rmodel, data, seed, step * S, 0, pop, lr=0.5, do_update=True, opt_state=ropt)
            assert (ref["losses"] == want).all(), "oracle differs from the reference kernels"
            assert (ref["model"] == omodel).all() and ref["updates"] == n_orc
            rmodel, ropt = ref["model"], ref["opt"]
            assert (ropt == oopt).all()
    assert (omodel != model).any()
    ctx.close()


@pytest.mark.parametrize("hidden,layers,seq,vocab,pop,wave", [(512, 2, 64, 2048, 16, 0), (256, 1, 48, 768, 12, 4), (1024, 1, 32, 512, 8, 0)])
def test_evaluation_at_wider_shapes_matches_oracle(hidden, layers, seq, vocab, pop, wave):
    """Row-owning projections (hidden 512, 1024), the two-kernel path (seq 48), several head tiles per row, short waves."""
    O = load_oracle()
    kw = dict(hidden_dim=hidden, n_layers=layers, seq_len=seq, population_size=pop, device_mask=3, vocab_size=vocab)
    cfg, ocfg, model, data = make_case(kw, data_len=40000, model_kind="random")
    ctx = _ctx(cfg, wave)
    ctx.upload_model(model)
    ctx.set_dataset(data)
    ctx.eval_chunk(SEED, 7, 0, pop)
    got = ctx.read_losses(0, pop)
    want = O.eval_losses(ocfg, model, data, 7, SEED, 0, pop)
    assert (got == want).all(), (got, want)
    ctx.close()


def test_generation_through_host_buffers_and_same_data_mode():
    O = load_oracle()
    kw = dict(hidden_dim=128, n_layers=1, seq_len=32, population_size=16, device_mask=15, vocab_size=1024, use_same_data=1)
    cfg, ocfg, model, data = make_case(kw, data_len=20000)
    ctx = _ctx(cfg)
    ctx.upload_model(model)
    losses = np.zeros(16, np.int32)
    n = ctx.generation_host(data, 0, SEED, 0.5, losses)
    want = O.eval_losses(ocfg, model, data, 0, SEED, 0, 16)
    assert (losses == want).all()
    omodel, oopt = model.copy(), np.zeros(O.opt_bytes(ocfg), np.uint8)
    assert n == O.update(ocfg, omodel, oopt, O.fitness(want), SEED, 0.5)
    assert (ctx.download_model() == omodel).all()
    ctx.close()


def test_token_width_and_range_are_checked():
    pkg = load_pkg()
    kw = dict(hidden_dim=128, n_layers=1, seq_len=16, population_size=8, device_mask=15)
    wide, narrow = _ctx(pkg.default_config(vocab_size=512, **kw)), _ctx(pkg.default_config(**kw))
    L = pkg.lib()
    toks32 = np.arange(1000, dtype=np.uint32) % 512
    toks8 = (np.arange(1000) % 256).astype(np.uint8)
    assert L.egg_set_dataset(wide._h, toks8.ctypes.data, 1000) == pkg.EGG_E_INVALID
    assert L.egg_set_dataset_tokens(narrow._h, toks32.ctypes.data, 1000) == pkg.EGG_E_INVALID
    bad = toks32.copy(); bad[777] = 512
    assert L.egg_set_dataset_tokens(wide._h, bad.ctypes.data, 1000) == pkg.EGG_E_INVALID
    assert b"777" in L.egg_last_error()
    assert L.egg_set_dataset_tokens(wide._h, toks32.ctypes.data, 1000) == 0
    wide.upload_model(np.zeros(pkg.model_bytes(wide.cfg), np.int8))
    with pytest.raises(pkg.EggError):
        wide.generate(np.array([1, 2, 3], np.uint8), 4, 1)
    wide.close(); narrow.close()
