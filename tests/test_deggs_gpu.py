"""GPU parity of the d-eggs worker path: evaluation under adaptive-noise overlays (AdaptiveScales),
chunk-relative losses, the update followed by the overlay steps, and the worker's seed chain — against
the golden vectors taken from the d-eggs worker's own kernels, against those kernels run on the same
GPU (where oracle/_ref holds them) and against the CPU oracle.  Everything here is bit-exact."""
import os
import zlib

import numpy as np
import pytest

from common import (DEGGS_CHUNK, DEGGS_CONFIGS, ROOT, deggs_binary, deggs_initial_scales, load_oracle, load_pkg, make_case,
                    run_ref_deggs)

pytestmark = pytest.mark.gpu
GOLD = os.path.join(ROOT, "tests", "golden")


def _worker_generations(ctx, pkg, O, kw, chunk, gens, seed, lr, data_S):
    """The worker's loop (d-eggs/src/worker.cu:390-717) over the library: per chunk eval_chunk + read_losses
    (chunk-relative), sign fitness, write_fitness, apply_update (+ overlay steps), seed = next_seed(seed, step+1)."""
    pop = kw["population_size"]
    step, out = 0, dict(losses=[], updates=[], scales=[])
    for _ in range(gens):
        losses = np.zeros(pop, np.int32)
        for off in range(0, pop, chunk):
            ctx.eval_chunk(seed, step * data_S, off, chunk)
            losses[off:off + chunk] = ctx.read_losses(0 if kw.get("chunk_relative_loss") else off, chunk)
        ctx.write_fitness(O.fitness(losses), 0)
        out["losses"].append(losses)
        out["updates"].append(ctx.apply_update(seed, lr))
        out["scales"].append(ctx.download_scales())
        step += 1
        seed = pkg.next_seed(seed, step)
    return out


@pytest.mark.parametrize("tag", ["tiny", "small"])
def test_worker_generations_match_golden_reference_kernels(tag):
    pkg, O = load_pkg(), load_oracle()
    g = np.load(os.path.join(GOLD, "ref_deggs_%s.npz" % tag))
    kw = DEGGS_CONFIGS[tag]
    cfg, ocfg, model0, data = make_case(kw, data_len=50000)
    scales0 = deggs_initial_scales(pkg.scales_bytes(cfg))
    assert pkg.scales_bytes(cfg) == O.scales_bytes(ocfg)
    ctx = pkg.Context(cfg, 0, 0 if tag == "tiny" else 24)       # the larger case also splits chunks into waves
    ctx.upload_model(model0)
    ctx.upload_scales(scales0)
    ctx.set_dataset(data)
    gens = len(g["losses"])
    r = _worker_generations(ctx, pkg, O, kw, DEGGS_CHUNK[tag], gens, 42, 0.5, kw["seq_len"])
    for gen in range(gens):
        assert (r["losses"][gen] == g["losses"][gen]).all(), "losses of generation %d" % gen
        assert r["updates"][gen] == int(g["updates"][gen]), "update count of generation %d" % gen
        assert zlib.crc32(r["scales"][gen].tobytes()) == int(g["scales_crc"][gen]), "overlays after generation %d" % gen
    assert (r["scales"][-1] == g["scales_final"]).all()
    model, opt = ctx.download_model(), ctx.download_opt_state()
    changed = np.nonzero(model != model0)[0]
    assert len(changed) == int(g["changed_count"]) and len(changed) > 0
    assert zlib.crc32(model.tobytes()) == int(g["model_crc"])
    assert zlib.crc32(opt.tobytes()) == int(g["opt_crc"]), "fp32 optimiser state is not bit-identical to the worker's kernels"
    ctx.close()


@pytest.mark.parametrize("tag", ["tiny", "small"])
def test_worker_generations_match_reference_kernels_run_here(tag):
    """Another seed, a random model and another overlay draw, against the worker's kernels on this GPU."""
    if not deggs_binary(tag):
        pytest.skip("oracle/_ref/ref_deggs_%s not built" % tag)
    pkg, O = load_pkg(), load_oracle()
    kw = DEGGS_CONFIGS[tag]
    cfg, ocfg, model0, data = make_case(kw, data_len=40000, data_seed=5, model_kind="random_all", model_seed=3)
    scales0 = deggs_initial_scales(pkg.scales_bytes(cfg), seed=11)
    opt0 = np.zeros(pkg.opt_state_bytes(cfg), np.uint8)
    gens, seed, lr = 4, 0xBEEF, 0.25
    ref = run_ref_deggs(tag, model0, opt0, scales0, data, seed, 0, gens, lr)
    ctx = pkg.Context(cfg, 0, 0)
    ctx.upload_model(model0)
    ctx.upload_scales(scales0)
    ctx.set_dataset(data)
    r = _worker_generations(ctx, pkg, O, kw, DEGGS_CHUNK[tag], gens, seed, lr, kw["seq_len"])
    for gen in range(gens):
        assert (r["losses"][gen] == ref["losses"][gen]).all(), "losses of generation %d" % gen
        assert r["updates"][gen] == ref["updates"][gen]
        assert (r["scales"][gen] == ref["scales"][gen]).all(), "overlays after generation %d" % gen
    assert (ctx.download_model() == ref["model"]).all()
    assert (ctx.download_opt_state() == ref["opt"]).all()
    ctx.close()


def test_overlays_against_oracle_other_width_and_switching_off():
    """hidden_dim 384 (three 128-wide chunks per row), global loss indexing, Gaussian noise; then the
    overlays are switched off again and the unscaled losses come back."""
    pkg, O = load_pkg(), load_oracle()
    kw = dict(hidden_dim=384, n_layers=2, seq_len=16, population_size=48, device_mask=7, device_gaussian=1)
    cfg, ocfg, model0, data = make_case(kw, data_len=30000, model_kind="random_all", model_seed=9)
    scales = deggs_initial_scales(pkg.scales_bytes(cfg), seed=3)
    model, opt = model0.copy(), np.zeros(O.opt_bytes(ocfg), np.uint8)
    oscales = scales.copy()
    ctx = pkg.Context(cfg, 0, 10)
    ctx.upload_model(model0)
    ctx.upload_scales(scales)
    ctx.set_dataset(data)
    seed = 1234
    for gen in range(3):
        want = O.eval_losses(ocfg, model, data, 16 * gen, seed, 0, 48, scales=oscales)
        ctx.eval_chunk(seed, 16 * gen, 0, 48)
        got = ctx.read_losses(0, 48)
        assert (got == want).all(), "losses of generation %d" % gen
        fit = O.fitness(want)
        n_want = O.update_scaled(ocfg, model, opt, fit, seed, 0.5, oscales)
        ctx.write_fitness(fit, 0)
        assert ctx.apply_update(seed, 0.5) == n_want
        assert (ctx.download_scales() == oscales).all()
        assert (ctx.download_model() == model).all()
        seed = pkg.next_seed(seed, gen + 1)
    ctx.upload_scales(None)
    want = O.eval_losses(ocfg, model, data, 0, 77, 0, 48)
    ctx.eval_chunk(77, 0, 0, 48)
    assert (ctx.read_losses(0, 48) == want).all()
    with pytest.raises(pkg.EggError):
        ctx.download_scales()
    ctx.close()


@pytest.mark.parametrize("hidden,level", [(256, 2), (256, 1), (1024, 2)])
def test_overlays_with_row_owning_projections_against_oracle(hidden, level):
    """seq_len 128, so the row-owning projections (and at level 2 the norm inside MLP-down; at hidden_dim 1024 the pairs of
    thread blocks) run under adaptive-noise overlays: scaled A vectors and bias deltas come from the noise table, the row
    dots are recomputed with per-term truncation after the fused norm.  Two generations with updates against the oracle."""
    pkg, O = load_pkg(), load_oracle()
    kw = dict(hidden_dim=hidden, n_layers=2 if hidden < 1024 else 1, seq_len=128, population_size=8, device_mask=7)
    cfg, ocfg, model0, data = make_case(kw, data_len=30000, model_kind="random_all", model_seed=5)
    scales = deggs_initial_scales(pkg.scales_bytes(cfg), seed=7)
    model, opt = model0.copy(), np.zeros(O.opt_bytes(ocfg), np.uint8)
    oscales = scales.copy()
    ctx = pkg.Context(cfg, 0, 0)
    ctx.set_fused_epilogues(level)
    assert ctx.fused_epilogues_active() == level
    ctx.upload_model(model0)
    ctx.upload_scales(scales)
    ctx.set_dataset(data)
    seed = 4321
    for gen in range(2):
        want = O.eval_losses(ocfg, model, data, 128 * gen, seed, 0, 8, scales=oscales)
        ctx.eval_chunk(seed, 128 * gen, 0, 8)
        got = ctx.read_losses(0, 8)
        assert (got == want).all(), "losses of generation %d: %s vs %s" % (gen, got, want)
        fit = O.fitness(want)
        n_want = O.update_scaled(ocfg, model, opt, fit, seed, 0.5, oscales)
        ctx.write_fitness(fit, 0)
        assert ctx.apply_update(seed, 0.5) == n_want
        assert (ctx.download_scales() == oscales).all()
        assert (ctx.download_model() == model).all()
        seed = pkg.next_seed(seed, gen + 1)
    ctx.close()
