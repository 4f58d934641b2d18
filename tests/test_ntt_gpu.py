"""GPU: the reference's transformed-window variants (NTT_MODE 1 Walsh-Hadamard, 2 Fermat-257, 3 Fermat-65537,
egg_ntt.cuh; three more embedding tables indexed by the coefficient bytes, mgpu.cu:877-887, 916-929, updated at half
the learning rate, mgpu.cu:1645-1668) against the oracle and, where the harness binaries exist, the reference's own
kernels."""
import numpy as np
import pytest

from common import REF_CONFIGS, load_oracle, load_pkg, make_case, ref_binary, run_ref_mgpu

pytestmark = pytest.mark.gpu
SEED = 0x0177C0DE


def _ctx(cfg, wave=0):
    return load_pkg().Context(cfg, 0, wave)


@pytest.mark.parametrize("tag", ["ntt1_tiny", "ntt2_tiny", "ntt3_small"])
def test_generations_match_oracle_and_reference_kernels(tag):
    O = load_oracle()
    kw = REF_CONFIGS[tag]
    cfg, ocfg, model, data = make_case(kw, data_len=50000)
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


@pytest.mark.parametrize("mode,hidden,seq,vocab", [(1, 512, 256, 256), (2, 256, 256, 256), (3, 512, 512, 256), (3, 256, 64, 1024), (1, 1024, 128, 256)])
def test_evaluation_at_wider_shapes_matches_oracle(mode, hidden, seq, vocab):
    """Full-length Fermat-257 (seq 256), windows of 512 tokens, negative Walsh-Hadamard coefficients (their sign byte
    picks rows of the third table), uint32 tokens reduced mod 65537, several waves."""
    O = load_oracle()
    kw = dict(hidden_dim=hidden, n_layers=1, seq_len=seq, population_size=12, device_mask=3, vocab_size=vocab, ntt_mode=mode)
    cfg, ocfg, model, data = make_case(kw, data_len=40000, model_kind="random")
    ctx = _ctx(cfg, 4)
    ctx.upload_model(model)
    ctx.set_dataset(data)
    ctx.eval_chunk(SEED, 11, 0, 12)
    got = ctx.read_losses(0, 12)
    want = O.eval_losses(ocfg, model, data, 11, SEED, 0, 12)
    assert (got == want).all(), (got, want)
    ctx.close()


def test_overlays_and_sampling_are_refused():
    pkg = load_pkg()
    cfg = pkg.default_config(hidden_dim=128, n_layers=1, seq_len=16, population_size=8, ntt_mode=1)
    ctx = _ctx(cfg)
    ctx.upload_model(np.zeros(pkg.model_bytes(cfg), np.int8))
    with pytest.raises(pkg.EggError):
        ctx.upload_scales(np.zeros(pkg.scales_bytes(cfg), np.int8))
    with pytest.raises(pkg.EggError):
        ctx.generate(np.array([1, 2, 3], np.uint8), 4, 1)
    ctx.close()
