"""GPU parity tests: the CUDA library (through the C ABI) against the CPU oracle and,
where oracle/_ref holds them, against the reference's own kernels run on the same GPU.
Integer results must be bit-exact; fp32 optimiser state within 1e-5 relative."""
import numpy as np
import pytest

from common import REF_CONFIGS, assert_losses_match_racy_reference, cfg_pair, load_oracle, load_pkg, make_case, ref_binary, run_ref_mgpu

pytestmark = pytest.mark.gpu

SEED = 0x00C0FFEE


def _ctx(cfg, wave=0):
    pkg = load_pkg()
    return pkg.Context(cfg, 0, wave)


@pytest.mark.parametrize("rows,K,N,rpm,mask", [(512, 256, 256, 64, 3), (256, 128, 384, 16, 15), (1024, 512, 128, 32, 3),
                                                 (384, 256, 512, 64, 3)])
def test_perturbed_projection_matches_oracle(rows, K, N, rpm, mask):
    pkg, O = load_pkg(), load_oracle()
    from egg_c_b200 import synth
    cfg, ocfg = cfg_pair(device_mask=mask)
    x = synth.normal_int8(3, rows * K)
    w = synth.uniform_int8(0, K * N)
    want = O.projection(ocfg, x, w, K, N, rpm, 7, 200, 201, 7, 8)
    y = np.zeros((rows, N), np.int8)
    ctx = _ctx(cfg, 2)
    ctx.perturbed_projection(x, w, y, rows, K, N, rpm, 7, 200, 201, 7, 8)
    assert (y == want).all(), "mismatches: %d of %d" % ((y != want).sum(), y.size)
    ctx.close()


@pytest.mark.parametrize("tag", ["tiny", "small"])
def test_eval_losses_match_oracle_and_reference(tag):
    O = load_oracle()
    kw = REF_CONFIGS[tag]
    cfg, ocfg, model, data = make_case(kw, data_len=50000)
    pop = kw["population_size"]
    want = O.eval_losses(ocfg, model, data, 0, SEED, 0, pop)
    ctx = _ctx(cfg)
    ctx.upload_model(model)
    ctx.set_dataset(data)
    ctx.eval_chunk(SEED, 0, 0, pop)
    got = ctx.read_losses(0, pop)
    assert (got == want).all(), (got[:8], want[:8])
    if ref_binary(tag):
        ref = run_ref_mgpu(tag, model, data, SEED, 0, 0, pop)
        assert (ref["losses"] == want).all(), "oracle differs from the reference kernels"
    ctx.close()


def test_eval_longest_sequence():
    """seq_len 1024, the longest the configuration check admits: a head's K and V fill 150 KB of shared memory, the
    limb sums leave the 23-bit range of the short-sequence division path, the causal loop runs 32 key blocks."""
    O = load_oracle()
    kw = dict(hidden_dim=128, n_layers=1, seq_len=1024, population_size=4, device_mask=15)
    cfg, ocfg, model, data = make_case(kw, data_len=30000, model_kind="random")
    want = O.eval_losses(ocfg, model, data, 5, SEED + 9, 0, 4)
    for fused in (2, 0):
        ctx = _ctx(cfg)
        ctx.set_fused_epilogues(fused)
        ctx.upload_model(model)
        ctx.set_dataset(data)
        ctx.eval_chunk(SEED + 9, 5, 0, 4)
        got = ctx.read_losses(0, 4)
        assert (got == want).all(), (fused, got, want)
        ctx.close()


def test_eval_waves_and_chunks_are_consistent():
    """Small waves, an odd number of waves, chunked calls and a later start index give the same losses."""
    O = load_oracle()
    kw = dict(hidden_dim=128, n_layers=2, seq_len=32, population_size=48, device_mask=15)
    cfg, ocfg, model, data = make_case(kw, data_len=30000, model_kind="random")
    want = O.eval_losses(ocfg, model, data, 96, SEED + 5, 0, 48)
    ctx = _ctx(cfg, wave=10)       # 5 waves of 10 members, the last one short
    ctx.upload_model(model)
    ctx.set_dataset(data)
    ctx.eval_chunk(SEED + 5, 96, 0, 48)
    assert (ctx.read_losses(0, 48) == want).all()
    ctx.eval_chunk(SEED + 5, 96, 16, 8)
    assert (ctx.read_losses(16, 8) == want[16:24]).all()
    ctx.close()


@pytest.mark.parametrize("hidden", [256, 384])
def test_eval_partial_tiles_with_256_wide_projections(hidden):
    """Waves whose row count is not a multiple of the 128-row tile, on a model wide enough for the 256-column tiles
    (residual boxes fetched by the copy engine, output boxes clipped at the last row, row-per-lane head); hidden 384
    takes the 128-column tiles for the residual and QKV projections."""
    O = load_oracle()
    kw = dict(hidden_dim=hidden, n_layers=2, seq_len=32, population_size=44, device_mask=3)
    cfg, ocfg, model, data = make_case(kw, data_len=30000, model_kind="random")
    want = O.eval_losses(ocfg, model, data, 64, SEED + 9, 0, 44)
    ctx = _ctx(cfg, wave=10)       # 320 rows per wave = 2.5 tiles; the last wave has 4 members = 1 tile
    ctx.upload_model(model)
    ctx.set_dataset(data)
    ctx.eval_chunk(SEED + 9, 64, 0, 44)
    assert (ctx.read_losses(0, 44) == want).all()
    ctx.close()


def test_eval_gaussian_noise_and_random_norm_weights():
    O = load_oracle()
    kw = dict(hidden_dim=256, n_layers=1, seq_len=16, population_size=16, device_mask=7, device_gaussian=1)
    cfg, ocfg, model, data = make_case(kw, data_len=20000, model_kind="random_all")
    want = O.eval_losses(ocfg, model, data, 0, 99, 0, 16)
    ctx = _ctx(cfg)
    ctx.upload_model(model)
    ctx.set_dataset(data)
    ctx.eval_chunk(99, 0, 0, 16)
    assert (ctx.read_losses(0, 16) == want).all()
    ctx.close()


def _opt_close(a_bytes, b_bytes, rtol=1e-5):
    a, b = a_bytes.view(np.float32).astype(np.float64), b_bytes.view(np.float32).astype(np.float64)
    err = np.abs(a - b)
    tol = rtol * np.maximum(np.abs(a), np.abs(b)) + 1e-7
    return int((err > tol).sum()), float(err.max())


@pytest.mark.parametrize("tag", ["tiny", "small"])
def test_update_matches_oracle_and_reference(tag):
    O = load_oracle()
    kw = REF_CONFIGS[tag]
    cfg, ocfg, model, data = make_case(kw, data_len=50000)
    pop = kw["population_size"]
    ctx = _ctx(cfg)
    ctx.upload_model(model)
    ctx.set_dataset(data)
    omodel, oopt = model.copy(), np.zeros(O.opt_bytes(ocfg), np.uint8)
    rmodel, ropt = model.copy(), None
    lr = 0.5
    for step in range(4):       # several generations so that weights actually flip
        seed = SEED + step
        ctx.eval_chunk(seed, step * kw["seq_len"], 0, pop)
        ctx.compute_fitness_pairs(0, pop // 2)
        fit = ctx.read_fitness(0, pop // 2)
        losses = ctx.read_losses(0, pop)
        want_l = O.eval_losses(ocfg, omodel, data, step * kw["seq_len"], seed, 0, pop)
        assert (losses == want_l).all(), "step %d losses" % step
        assert (fit == O.fitness(want_l)).all()
        n_gpu = ctx.apply_update(seed, lr)
        n_orc = O.update(ocfg, omodel, oopt, fit, seed, lr)
        got_model = ctx.download_model()
        assert (got_model == omodel).all(), "step %d: %d weights differ" % (step, (got_model != omodel).sum())
        assert n_gpu == n_orc
        gopt = ctx.download_opt_state()
        bad, mx = _opt_close(gopt, oopt)
        assert bad == 0, "optimiser state: %d elements off, max err %g" % (bad, mx)
        assert (gopt == oopt).all(), "optimiser state is within tolerance but not bit-identical to the oracle"
        if ref_binary(tag):
            ref = run_ref_mgpu(tag, rmodel, data, seed, step * kw["seq_len"], 0, pop, lr=lr, do_update=True, opt_state=ropt)
            assert (ref["losses"] == want_l).all()
            assert (ref["model"] == omodel).all(), "reference kernels: %d weights differ" % (ref["model"] != omodel).sum()
            assert ref["updates"] == n_orc
            rmodel, ropt = ref["model"], ref["opt"]
            assert (ropt == ctx.download_opt_state()).all(), "optimiser state not bit-identical to the reference kernels"
    assert (omodel != model).any()
    ctx.close()


@pytest.mark.parametrize("tag", ["muon_tiny"])
def test_muon_update_within_tolerance(tag):
    O = load_oracle()
    kw = REF_CONFIGS[tag]
    cfg, ocfg, model, data = make_case(kw, data_len=50000)
    pop = kw["population_size"]
    ctx = _ctx(cfg)
    ctx.upload_model(model)
    ctx.set_dataset(data)
    omodel, oopt = model.copy(), np.zeros(O.opt_bytes(ocfg), np.uint8)
    for step in range(3):
        seed = SEED + step
        ctx.eval_chunk(seed, 0, 0, pop)
        ctx.compute_fitness_pairs(0, pop // 2)
        fit = ctx.read_fitness(0, pop // 2)
        ctx.apply_update(seed, 0.5)
        O.update(ocfg, omodel, oopt, fit, seed, 0.5)
        ctx.upload_model(omodel)     # keep both sides on the same weights: tolerance-level fp32 differences may flip a weight
        bad, mx = _opt_close(ctx.download_opt_state(), oopt, rtol=1e-4)
        assert bad == 0, "step %d: %d state elements off (max %g)" % (step, bad, mx)
        ctx.upload_opt_state(oopt)
    ctx.close()


@pytest.mark.parametrize("ternary", [True, False])
def test_update_reconstruct_matches_oracle(ternary):
    pkg, O = load_pkg(), load_oracle()
    cfg, ocfg = cfg_pair(device_mask=3, population_size=2 * 300)
    rng = np.random.default_rng(4)
    fit = (rng.integers(-1, 2, 300) if ternary else rng.integers(-127, 128, 300)).astype(np.int32)
    want = O.vote_matrix(ocfg, fit, 256, 128, 402, 403, 1000, 2)
    vote = np.zeros(256 * 128, np.int32)
    ctx = _ctx(cfg, 2)
    ctx.update_reconstruct(fit, 300, 256, 128, 402, 403, 1000, 2, vote)
    assert (vote == want).all()
    ctx.close()


def test_benchmark_config_sample_matches_reference_kernels():
    """Full benchmark configuration (H=512, L=4, S=256, POP=40960): two 64-member slices of the
    population against the reference's own kernels, and the whole-population loss checksum is stable
    across wave sizes."""
    if not ref_binary("c2"):
        pytest.skip("oracle/_ref/ref_mgpu_c2 not built")
    pkg = load_pkg()
    from egg_c_b200 import synth
    kw = REF_CONFIGS["c2"]
    cfg, ocfg = cfg_pair(**kw)
    model = synth.random_model(cfg, 0, "uniform")
    data = synth.zipf_bytes(1, 8 << 20)
    ctx = _ctx(cfg, wave=64)
    ctx.upload_model(model)
    ctx.set_dataset(data)
    for off in (0, 40960 - 64):
        ctx.eval_chunk(SEED, 256, off, 64)
        got = ctx.read_losses(off, 64)
        ref = run_ref_mgpu("c2", model, data, SEED, 256, off, 64)
        assert_losses_match_racy_reference("c2", model, data, SEED, 256, off, got, ref["losses"])
    ctx.close()
    ctx2 = _ctx(cfg, wave=48)      # a wave size that leaves a ragged last wave
    ctx2.upload_model(model)
    ctx2.set_dataset(data)
    ctx2.eval_chunk(SEED, 256, 40960 - 64, 64)
    assert (ctx2.read_losses(40960 - 64, 64) == got).all()
    ctx2.close()


def test_deggs_scale_config_sample_matches_reference_kernels():
    """d-eggs-scale shapes (H=1024, 16 heads, L=12, S=512, POP=262144, ternary weight values in the
    reference int8 layout): a 16-member slice against the reference's own kernels."""
    if not ref_binary("c5"):
        pytest.skip("oracle/_ref/ref_mgpu_c5 not built")
    pkg = load_pkg()
    from egg_c_b200 import synth
    kw = REF_CONFIGS["c5"]
    cfg, ocfg = cfg_pair(**kw)
    model = synth.random_model(cfg, 0, "ternary")
    data = synth.zipf_bytes(1, 8 << 20)
    ctx = _ctx(cfg, wave=16)
    ctx.upload_model(model)
    ctx.set_dataset(data)
    off = 262144 - 16
    ctx.eval_chunk(SEED, 512, off, 16)
    got = ctx.read_losses(off, 16)
    ref = run_ref_mgpu("c5", model, data, SEED, 512, off, 16)
    assert_losses_match_racy_reference("c5", model, data, SEED, 512, off, got, ref["losses"])
    ctx.close()
