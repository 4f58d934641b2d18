"""GPU parity at the sizes the benchmark configurations name.

* one whole generation of the Int8NativeFormer configuration (40 960 members, H 512, 4 layers, 256 tokens) beside the
  reference's own kernels: every loss, every fitness value, the update count, the weights and the fp32 AdamW state;
* the Muon step against the reference's own Muon (cuBLAS Newton-Schulz) at 1e-5 relative;
* the isolated projection at 262 144 x 4096 x 4096 and the isolated vote reconstruction at 4096 x 4096 with 32 768
  pairs of int8 fitness, on seeded samples of rows that the CPU oracle can afford.
"""
import numpy as np
import pytest

from common import REF_CONFIGS, assert_losses_match_racy_reference, cfg_pair, load_oracle, load_pkg, make_case, ref_binary, run_ref_mgpu

pytestmark = pytest.mark.gpu

SEED = 0x00C0FFEE


def test_whole_benchmark_generation_matches_reference_kernels():
    """full_cuda_train_transformer_adam_mgpu.cu:1506-1688 at POPULATION_SIZE 40960: evaluation of every member, host
    fitness, the whole LAUNCH_ADAM_* list.

    The reference's train_sequence_kernel is not deterministic at this size: two runs of it on identical inputs differ
    in a handful of the 40 960 losses (its three back-to-back adaptive_qkv_normalize calls share one scratch array with
    no barrier between one call's reads and the next call's writes, egg_adaptive_normalize.h:29-41 called at
    mgpu.cu:782-784).  So: every loss must equal the reference's, except that a member whose loss differs must equal
    the reference re-run on that pair alone (where its race does not show) -- and there may only be a few of them.
    The update is then compared on the reference's own fitness vector, so that its raced losses cannot leak into the
    comparison: update count, weights and fp32 AdamW state bit-identical."""
    if not ref_binary("c2"):
        pytest.skip("oracle/_ref/ref_mgpu_c2 not built")
    pkg = load_pkg()
    from egg_c_b200 import synth
    kw = REF_CONFIGS["c2"]
    cfg, ocfg = cfg_pair(**kw)
    pop = kw["population_size"]
    model = synth.random_model(cfg, 0, "uniform")
    data = synth.zipf_bytes(1, 8 << 20)
    lr = 2.5        # from zero state |m / sqrt(v)| = 0.1 / sqrt(0.05) = 0.447: a rate above 2.24 makes weights flip in the first step
    ctx = pkg.Context(cfg, 0, 0)
    ctx.upload_model(model)
    ctx.set_dataset(data)
    ctx.eval_chunk(SEED, 256, 0, pop)
    losses = ctx.read_losses(0, pop)
    ctx.compute_fitness_pairs(0, pop // 2)
    fit = ctx.read_fitness(0, pop // 2)
    ref = run_ref_mgpu("c2", model, data, SEED, 256, 0, pop, lr=lr, do_update=True)
    bad = assert_losses_match_racy_reference("c2", model, data, SEED, 256, 0, losses, ref["losses"], max_bad=64)
    bad_pairs = sorted(set(int(m) // 2 for m in bad))
    print("members where the reference's full-population run differs from its own single-pair run:", bad)
    same = np.ones(pop // 2, bool)
    same[bad_pairs] = False
    assert (fit[same] == ref["fitness"][same]).all()
    ctx.write_fitness(ref["fitness"], 0)
    n_gpu = ctx.apply_update(SEED, lr)
    got_model, got_opt = ctx.download_model(), ctx.download_opt_state()
    ctx.close()
    assert n_gpu == ref["updates"] and n_gpu > 0
    assert (got_model == ref["model"]).all(), "%d weights differ" % (got_model != ref["model"]).sum()
    assert (got_opt == ref["opt"]).all(), "fp32 AdamW state is not bit-identical to the reference kernels"
    assert (got_model != model).any()


def _state_diff(a_bytes, b_bytes, rtol=1e-5, atol=2e-6):
    a, b = a_bytes.view(np.float32).astype(np.float64), b_bytes.view(np.float32).astype(np.float64)
    err = np.abs(a - b)
    tol = rtol * np.maximum(np.abs(a), np.abs(b)) + atol
    return int((err > tol).sum()), float((err / (np.maximum(np.abs(a), np.abs(b)) + 1e-30)).max()), float(err.max())


@pytest.mark.parametrize("tag", ["muon_tiny", "muon_small"])
def test_muon_step_matches_reference_muon(tag):
    """muon_internal.cuh:182-342 called from mgpu.cu:1587-1595 (cuBLAS SGEMM Newton-Schulz) beside the library's own
    Newton-Schulz: three generations, each from inputs identical on both sides (the reference's previous outputs).
    fp32 state within 1e-5 relative; int8 weights that differ are counted and reported (a weight flips when `acc`
    crosses 1, so a tolerance-level difference in fp32 can move a flip by one generation)."""
    if not ref_binary(tag):
        pytest.skip("oracle/_ref/ref_mgpu_%s not built" % tag)
    pkg = load_pkg()
    kw = REF_CONFIGS[tag]
    cfg, ocfg, model, data = make_case(kw, data_len=50000)
    pop, S = kw["population_size"], kw["seq_len"]
    ctx = pkg.Context(cfg, 0, 0)
    ctx.set_dataset(data)
    opt = None
    flips_total = 0
    for step in range(3):
        ctx.upload_model(model)
        if opt is not None:
            ctx.upload_opt_state(opt)
        losses = np.zeros(pop, np.int32)
        ctx.generation_host(None, step, SEED + step, 0.5, losses)
        ref = run_ref_mgpu(tag, model, data, SEED + step, step * S, 0, pop, lr=0.5, do_update=True, opt_state=opt)
        assert (losses == ref["losses"]).all()
        got_model, got_opt = ctx.download_model(), ctx.download_opt_state()
        bad, max_rel, max_abs = _state_diff(got_opt, ref["opt"])
        flips = int((got_model != ref["model"]).sum())
        flips_total += flips
        print("%s step %d: state max rel err %.3g, max abs err %.3g, %d of %d int8 weights differ from the reference's"
              % (tag, step, max_rel, max_abs, flips, got_model.size))
        assert bad == 0, "step %d: %d optimiser-state elements beyond 1e-5 relative (max rel %g, max abs %g)" % (step, bad, max_rel, max_abs)
        assert flips <= max(4, got_model.size // 20000), "step %d: %d weights differ" % (step, flips)
        model, opt = ref["model"], ref["opt"]
    ctx.close()


def test_isolated_projection_at_benchmark_size_sample():
    """W 4096 x 4096, 4096 members x 64 tokens = 262 144 rows, noise magnitudes in [-3, 3]: `>> 8` and clip
    (full_cuda_train_egg_transformer.cu:249 on compute_linear_projection, mgpu.cu:553-572).  Activations are drawn on
    the device (clamp(round(N(0, 32)))); 16 population pairs = 2048 rows are checked against the oracle."""
    import torch
    pkg, O = load_pkg(), load_oracle()
    from egg_c_b200 import synth
    cfg, ocfg = cfg_pair(device_mask=3)
    K = N = 4096
    rpm, members = 64, 4096
    rows = rpm * members
    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    x = torch.empty((rows, K), dtype=torch.int8, device="cuda")
    step = 16384
    for r0 in range(0, rows, step):
        x[r0:r0 + step] = torch.clamp(torch.round(torch.randn((step, K), generator=g, device="cuda") * 32.0), -127, 127).to(torch.int8)
    w = synth.uniform_int8(0, K * N)
    d_w = torch.from_numpy(w).cuda()
    y = torch.zeros((rows, N), dtype=torch.int8, device="cuda")
    ctx = pkg.Context(cfg, 0, 2)
    torch.cuda.synchronize()
    ctx.perturbed_projection(x.data_ptr(), d_w.data_ptr(), y.data_ptr(), rows, K, N, rpm, 7, 200, 201, 7, 8, on_device=True)
    rng = np.random.default_rng(5)
    pairs = sorted(set([0, members // 2 - 1] + rng.integers(0, members // 2, 14).tolist()))
    for j in pairs:
        r0 = j * 2 * rpm
        xs = x[r0:r0 + 2 * rpm].cpu().numpy()
        want = O.projection(ocfg, xs, w, K, N, rpm, 7 + j, 200, 201, 7, 8)
        got = y[r0:r0 + 2 * rpm].cpu().numpy()
        assert (got == want).all(), "pair %d: %d of %d outputs differ" % (j, (got != want).sum(), got.size)
    assert int(y.min()) >= -127             # the reference clips to [-127, 127], never -128
    ctx.close()


def test_isolated_vote_reconstruction_at_benchmark_size_sample():
    """4096 x 4096 weight, 65 536 members = 32 768 pairs, int8 rank-normalised fitness, noise magnitudes in [-3, 3]
    (update_matrix_adam_kernel's vote, mgpu.cu:1085-1098): 64 output columns x 4096 inputs against the oracle, and
    linearity over disjoint pair ranges (votes(all pairs) == votes(first half) + votes(second half))."""
    import torch
    pkg, O = load_pkg(), load_oracle()
    cfg, ocfg = cfg_pair(device_mask=3, population_size=65536)
    R = Cn = 4096
    pairs = 32768
    rng = np.random.RandomState(2)
    rank = np.argsort(np.argsort(rng.randn(pairs)))
    fit = np.clip(np.round(rank / (pairs - 1) * 254.0 - 127.0), -127, 127).astype(np.int32)
    ctx = pkg.Context(cfg, 0, 2)
    d_fit = torch.from_numpy(fit).cuda()
    votes = torch.zeros(R * Cn, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    ctx.update_reconstruct(d_fit.data_ptr(), pairs, R, Cn, 402, 403, 1000, 2, votes.data_ptr(), on_device=True)
    v = votes.cpu().numpy().reshape(R // 4, Cn, 4)                   # packed index order [k/4][n][4]
    n_list = np.unique(np.concatenate([[0, Cn - 1], np.random.default_rng(6).integers(0, Cn, 62)])).astype(np.int32)
    want = O.vote_columns(ocfg, fit, R, 402, 403, 1000, 2, n_list)
    for i, n in enumerate(n_list):
        got = v[:, n, :].reshape(-1)
        assert (got == want[i]).all(), "output column %d: %d of %d votes differ" % (n, (got != want[i]).sum(), R)
    # linearity over the pair index
    lo, hi = fit.copy(), fit.copy()
    lo[pairs // 2:] = 0
    hi[:pairs // 2] = 0
    parts = []
    for f in (lo, hi):
        d_f = torch.from_numpy(f).cuda()
        out = torch.zeros(R * Cn, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        ctx.update_reconstruct(d_f.data_ptr(), pairs, R, Cn, 402, 403, 1000, 2, out.data_ptr(), on_device=True)
        parts.append(out)
    assert torch.equal(parts[0] + parts[1], votes)
    ctx.close()


def _packed_index(k, n, cols_n):
    return ((k >> 2) * cols_n + n) * 4 + (k & 3)


@pytest.mark.parametrize("int8fit", [False, True])
def test_isolated_matrix_update_adamw_matches_oracle(int8fit):
    """egg_update_matrix (one launch of update_matrix_adam_kernel, mgpu.cu:1067-1111): two chained ES-AdamW steps of a
    256 x 384 matrix from 1000 pairs, ternary and int8 fitness; weights, fp32 state and the change count bit-exact."""
    import torch
    pkg, O = load_pkg(), load_oracle()
    cfg, ocfg = cfg_pair(device_mask=3, population_size=2000)
    R, Cn, pairs = 256, 384, 1000
    rng = np.random.default_rng(21)
    w = rng.integers(-127, 128, R * Cn).astype(np.int8)
    st = np.zeros((R * Cn, 3), np.float32)
    d_w, d_st = torch.from_numpy(w.copy()).cuda(), torch.zeros(R * Cn * 3, dtype=torch.float32, device="cuda")
    ctx = pkg.Context(cfg, 0, 2)
    for step in range(2):
        fit = (rng.integers(-127, 128, pairs) if int8fit else rng.integers(-1, 2, pairs)).astype(np.int32)
        d_fit = torch.from_numpy(fit).cuda()
        torch.cuda.synchronize()
        n_gpu = ctx.update_matrix(d_w.data_ptr(), d_st.data_ptr(), R, Cn, 402, 403, 1000, d_fit.data_ptr(), pairs, 5 + step, 0.7,
                                  optimizer=0, split=int8fit)
        votes = O.vote_matrix(ocfg, fit, R, Cn, 402, 403, 1000, 5 + step)
        n_orc = O.adam_from_votes(ocfg, w, st, votes, 0.7)
        assert n_gpu == n_orc
        assert (d_w.cpu().numpy() == w).all(), "step %d: %d weights differ" % (step, (d_w.cpu().numpy() != w).sum())
        assert (d_st.cpu().numpy().view(np.uint32) == st.reshape(-1).view(np.uint32)).all(), "fp32 AdamW state not bit-identical"
    ctx.close()


def test_isolated_matrix_update_muon_matches_oracle():
    """egg_update_matrix with the Muon sequence (muon_internal.cuh:15-342) on a 512 x 1024 matrix from 300 pairs: momentum
    exact, accumulator within 1e-5 relative of the oracle's double-accumulating Newton-Schulz."""
    import torch
    pkg, O = load_pkg(), load_oracle()
    cfg, ocfg = cfg_pair(device_mask=3, population_size=600, use_muon=1)
    R, Cn, pairs = 512, 1024, 300
    rng = np.random.default_rng(22)
    w = rng.integers(-127, 128, R * Cn).astype(np.int8)
    fit = rng.integers(-1, 2, pairs).astype(np.int32)
    d_w, d_st = torch.from_numpy(w.copy()).cuda(), torch.zeros(R * Cn * 2, dtype=torch.float32, device="cuda")
    d_fit = torch.from_numpy(fit).cuda()
    ctx = pkg.Context(cfg, 0, 2)
    torch.cuda.synchronize()
    lr = 0.5
    ctx.update_matrix(d_w.data_ptr(), d_st.data_ptr(), R, Cn, 400, 401, 2000, d_fit.data_ptr(), pairs, 9, lr, optimizer=1)
    st = d_st.cpu().numpy().reshape(-1, 2)
    votes = O.vote_matrix(ocfg, fit, R, Cn, 400, 401, 2000, 9).astype(np.float32)          # from zero state: m = votes
    assert (st[:, 0] == votes).all()
    idx = np.arange(R * Cn)
    n_of, k_of = (idx >> 2) % Cn, ((idx >> 2) // Cn) * 4 + (idx & 3)
    m_rowmajor = np.zeros((R, Cn), np.float32)
    m_rowmajor[k_of, n_of] = votes
    u = O.newton_schulz(m_rowmajor)[k_of, n_of].astype(np.float64)
    acc_want = -lr * (u + 0.01 * w.astype(np.float64))
    wrapped = np.abs(acc_want) >= 1.0                                                      # the quantised step subtracts 1 there
    err = np.abs(st[:, 1].astype(np.float64) - acc_want)[~wrapped]
    tol = 1e-5 * np.abs(acc_want[~wrapped]) + 2e-6
    assert (err <= tol).all(), "max err %g over %d elements" % (err.max(), (~wrapped).sum())
    ctx.close()


def test_isolated_matrix_update_at_benchmark_size_sample():
    """4096 x 4096 weight, 32 768 pairs of int8 rank-normalised fitness, one ES-AdamW step from zero state: the weights and
    fp32 state of 64 sampled output columns against the oracle (votes of those columns, then the element step)."""
    import torch
    pkg, O = load_pkg(), load_oracle()
    from egg_c_b200 import synth
    cfg, ocfg = cfg_pair(device_mask=3, population_size=65536)
    R = Cn = 4096
    pairs = 32768
    rng = np.random.RandomState(2)
    rank = np.argsort(np.argsort(rng.randn(pairs)))
    fit = np.clip(np.round(rank / (pairs - 1) * 254.0 - 127.0), -127, 127).astype(np.int32)
    w0 = synth.uniform_int8(0, R * Cn)
    d_w = torch.from_numpy(w0.copy()).cuda()
    d_st = torch.zeros(R * Cn * 3, dtype=torch.float32, device="cuda")
    d_fit = torch.from_numpy(fit).cuda()
    ctx = pkg.Context(cfg, 0, 2)
    torch.cuda.synchronize()
    lr = 2.5           # |m/sqrt(v)| = 0.1/sqrt(0.05) ~ 0.447 after the first step: lr above 2.24 makes weights flip at once
    n_gpu = ctx.update_matrix(d_w.data_ptr(), d_st.data_ptr(), R, Cn, 402, 403, 1000, d_fit.data_ptr(), pairs, 2, lr, optimizer=0, split=True)
    assert n_gpu > 0
    w1 = d_w.cpu().numpy()
    st1 = d_st.cpu().numpy().reshape(-1, 3)
    assert int((w1 != w0).sum()) == n_gpu
    n_list = np.unique(np.concatenate([[0, Cn - 1], np.random.default_rng(8).integers(0, Cn, 62)])).astype(np.int32)
    votes = O.vote_columns(ocfg, fit, R, 402, 403, 1000, 2, n_list)
    k = np.arange(R)
    for i, n in enumerate(n_list):
        idx = _packed_index(k, int(n), Cn)
        w = w0[idx].copy()
        st = np.zeros((R, 3), np.float32)
        O.adam_from_votes(ocfg, w, st, votes[i], lr)
        assert (w1[idx] == w).all(), "output column %d: %d weights differ" % (n, (w1[idx] != w).sum())
        assert (st1[idx].view(np.uint32) == st.view(np.uint32)).all(), "output column %d: fp32 state differs" % n
    ctx.close()
