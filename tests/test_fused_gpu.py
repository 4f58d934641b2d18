"""GPU parity of the row-owning projections (adaptive normalisations fused into the GEMM epilogue, csrc/egg_gemm_fused.cuh)
and of the tensor-core attention (csrc/egg_attention_tc.cu), which run together wherever seq_len is a multiple of 128,
against the CPU oracle, against the two-kernel form of the same library, and -- at the benchmark's layer shapes --
against the reference's own kernels.  Everything here is integer work: bit-exact."""
import numpy as np
import pytest

from common import REF_CONFIGS, assert_losses_match_racy_reference, load_oracle, load_pkg, make_case, ref_binary, run_ref_mgpu

pytestmark = pytest.mark.gpu

SEED = 0x00C0FFEE


def _losses(pkg, cfg, model, data, seed, start, pop, wave, fused, attention_tc=False):
    ctx = pkg.Context(cfg, 0, wave)
    ctx.set_fused_epilogues(fused)          # False / True / 2 / 3: two-kernel, row-owning projections, + norm inside MLP-down, + LN2 inside the O projection
    ctx.set_attention_tensor_core(attention_tc)
    assert ctx.fused_epilogues_active() == int(fused)
    ctx.upload_model(model)
    ctx.set_dataset(data)
    ctx.eval_chunk(seed, start, 0, pop)
    out = ctx.read_losses(0, pop)
    ctx.close()
    return out


@pytest.mark.parametrize("hidden,layers,seq,pop,mask,kind", [
    (128, 1, 128, 8, 15, "init"),          # 128-column sub-tiles, one per row
    (256, 2, 128, 8, 3, "random"),         # 256-column sub-tiles, one per row; two layers chain x through the in-place projections
    (384, 1, 128, 6, 3, "random_all"),     # three 128-column sub-tiles in a ring of four TMEM slots; random norm gains and biases
    (512, 1, 256, 6, 3, "random"),         # the benchmark's layer shape: two 256-column sub-tiles, tiles of one member half
    (128, 1, 512, 4, 15, "random"),        # 512 tokens: four query blocks, the later ones with two key chunks (scores recomputed in pass B)
    (256, 1, 384, 4, 3, "random_all"),     # three query blocks: an odd number of key tiles in the last chunk
    (1024, 1, 128, 4, 3, "random_all"),    # a pair of thread blocks per row tile (2 x 512 columns), row maxima exchanged between them
    (768, 1, 256, 4, 15, "random"),        # a pair with 3 x 128 columns each
    (1024, 2, 256, 2, 3, "random"),        # pairs, two layers chained through the in-place projections
])
def test_fused_eval_matches_oracle(hidden, layers, seq, pop, mask, kind):
    pkg, O = load_pkg(), load_oracle()
    kw = dict(hidden_dim=hidden, n_layers=layers, seq_len=seq, population_size=pop, device_mask=mask)
    cfg, ocfg, model, data = make_case(kw, data_len=60000, model_kind=kind)
    want = O.eval_losses(ocfg, model, data, seq, SEED + 3, 0, pop)
    got = _losses(pkg, cfg, model, data, SEED + 3, seq, pop, 0, True)
    assert (got == want).all(), (got[:8], want[:8])
    got2 = _losses(pkg, cfg, model, data, SEED + 3, seq, pop, 0, 2)
    assert (got2 == want).all(), ("norm inside the MLP-down epilogue", got2[:8], want[:8])
    got3 = _losses(pkg, cfg, model, data, SEED + 3, seq, pop, 0, 3)
    assert (got3 == want).all(), ("LN2 inside the output projection as well", got3[:8], want[:8])
    assert (_losses(pkg, cfg, model, data, SEED + 3, seq, pop, 0, False) == want).all()
    assert (_losses(pkg, cfg, model, data, SEED + 3, seq, pop, 0, True, attention_tc=True) == want).all(), "tcgen05 attention"
    assert (_losses(pkg, cfg, model, data, SEED + 3, seq, pop, 0, True, attention_tc=2) == want).all(), "hybrid attention"


def test_fused_eval_many_units_per_block_and_ragged_waves():
    """More 128-row tiles than thread blocks, so every block walks several units (table double buffering, TMEM slot
    ring phases, box reuse, residual prefetch), with waves of different sizes including a short last one."""
    pkg, O = load_pkg(), load_oracle()
    kw = dict(hidden_dim=128, n_layers=1, seq_len=128, population_size=400, device_mask=15)
    cfg, ocfg, model, data = make_case(kw, data_len=200000, model_kind="random")
    want = O.eval_losses(ocfg, model, data, 256, SEED + 11, 0, 400)
    for wave in (0, 150):         # one wave of 400 members = 400 tiles (1200 Q/K/V units); then 150 + 150 + 100
        for level in (1, 2):
            got = _losses(pkg, cfg, model, data, SEED + 11, 256, 400, wave, level)
            assert (got == want).all(), "wave %d level %d: %d of 400 losses differ" % (wave, level, (got != want).sum())


def test_paired_blocks_walk_many_units():
    """H 1024: every 128-row tile is shared by a cluster of two thread blocks.  With 300 members there are more tiles
    than pairs, so every pair walks several units (alternating exchange buffers and barrier phases); the row-owning
    form must give the losses of the two-kernel form, whole and in ragged waves."""
    pkg = load_pkg()
    kw = dict(hidden_dim=1024, n_layers=2, seq_len=128, population_size=300, device_mask=3)
    cfg, ocfg, model, data = make_case(kw, data_len=200000, model_kind="random")
    want = _losses(pkg, cfg, model, data, SEED + 5, 128, 300, 0, False)
    for wave in (0, 128):
        for level in (1, 2):
            got = _losses(pkg, cfg, model, data, SEED + 5, 128, 300, wave, level)
            assert (got == want).all(), "wave %d level %d: %d of 300 losses differ" % (wave, level, (got != want).sum())


def test_fused_and_two_kernel_forms_agree_at_benchmark_shapes_and_with_reference_kernels():
    """H 512, 4 layers, 256 tokens (the benchmark's model) on 256 members: the row-owning form, the two-kernel form and
    the reference's own train_sequence_kernel give the same 256 losses; then four chained generations with updates
    stay bit-identical to the reference kernels (weights and fp32 state)."""
    tag = "med"
    if not ref_binary(tag):
        pytest.skip("oracle/_ref/ref_mgpu_med not built")
    pkg = load_pkg()
    from egg_c_b200 import synth
    kw = REF_CONFIGS[tag]
    cfg, ocfg, _, data = make_case(kw, data_len=400000)
    model = synth.random_model(cfg, 0, "uniform")
    pop, S = kw["population_size"], kw["seq_len"]
    a = _losses(pkg, cfg, model, data, SEED, 0, pop, 0, True)
    b = _losses(pkg, cfg, model, data, SEED, 0, pop, 0, False)
    assert (a == b).all()
    assert (_losses(pkg, cfg, model, data, SEED, 0, pop, 0, 2) == a).all(), "norm inside the MLP-down epilogue"
    assert (_losses(pkg, cfg, model, data, SEED, 0, pop, 0, True, attention_tc=True) == a).all(), "tcgen05 attention"
    assert (_losses(pkg, cfg, model, data, SEED, 0, pop, 0, True, attention_tc=2) == a).all(), "hybrid attention"
    ref = run_ref_mgpu(tag, model, data, SEED, 0, 0, pop)
    assert_losses_match_racy_reference(tag, model, data, SEED, 0, 0, a, ref["losses"])
    ctx = pkg.Context(cfg, 0, 100)          # ragged waves: 100 + 100 + 56 members
    assert ctx.fused_epilogues_active()
    ctx.upload_model(model)
    ctx.set_dataset(data)
    rmodel, ropt = model.copy(), None
    for step in range(3):
        ctx.eval_chunk(SEED + step, step * S, 0, pop)
        losses = ctx.read_losses(0, pop)
        r = run_ref_mgpu(tag, rmodel, data, SEED + step, step * S, 0, pop, lr=0.5, do_update=True, opt_state=ropt)
        assert_losses_match_racy_reference(tag, rmodel, data, SEED + step, step * S, 0, losses, r["losses"])
        ctx.write_fitness(r["fitness"], 0)              # the reference's own fitness: its raced losses cannot fork the two models
        n = ctx.apply_update(SEED + step, 0.5)
        assert n == r["updates"]
        rmodel, ropt = r["model"], r["opt"]
        assert (ctx.download_model() == rmodel).all()
        assert (ctx.download_opt_state() == ropt).all()
    ctx.close()
