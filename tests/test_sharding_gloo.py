"""world_size-2 run of the sharded generation on CPU ranks (gloo): each rank evaluates its pair-aligned
slice with the oracle, all-gathers fitness, applies the replicated update; every rank must end with the
same bytes as the single-process generation."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from common import ROOT, load_oracle, load_pkg, make_case

KW = dict(hidden_dim=128, n_layers=1, seq_len=16, population_size=16, device_mask=15)
SEED, LR = 77, 0.5


def _rank_main(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    O = load_oracle()
    load_pkg()
    from egg_c_b200 import sharding
    cfg, ocfg, model, data = make_case(KW, data_len=20000)
    opt = np.zeros(O.opt_bytes(ocfg), np.uint8)
    pop = KW["population_size"]
    for step in range(3):
        off, per = sharding.member_slice(rank, world, pop)
        losses = O.eval_losses(ocfg, model, data, step * KW["seq_len"], SEED + step, off, per)
        mine = torch.from_numpy(O.fitness(losses))
        parts = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        fit = torch.cat(parts).numpy()
        O.update(ocfg, model, opt, fit, SEED + step, LR)
    q.put((rank, model.tobytes(), opt.tobytes()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_generation_equals_single_process():
    O = load_oracle()
    cfg, ocfg, model, data = make_case(KW, data_len=20000)
    opt = np.zeros(O.opt_bytes(ocfg), np.uint8)
    pop = KW["population_size"]
    for step in range(3):
        losses = O.eval_losses(ocfg, model, data, step * KW["seq_len"], SEED + step, 0, pop)
        O.update(ocfg, model, opt, O.fitness(losses), SEED + step, LR)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, mb, ob in got:
        assert mb == model.tobytes(), "rank %d model differs" % rank
        assert ob == opt.tobytes(), "rank %d optimiser state differs" % rank


def _sharded_rank_main(rank, world, port, q):
    """The sharded update's data flow on CPU ranks: every rank keeps only the parameters the owner plan gives it from
    its own update, and the owners' bytes are broadcast -- what egg_set_update_sharding does with NCCL."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    O = load_oracle()
    pkg = load_pkg()
    from egg_c_b200 import sharding
    cfg, ocfg, model, data = make_case(KW, data_len=20000)
    owners, costs, offs, lens = pkg.update_owner_plan(cfg, world, spans=True)
    opt = np.zeros(O.opt_bytes(ocfg), np.uint8)
    pop = KW["population_size"]
    for step in range(3):
        off, per = sharding.member_slice(rank, world, pop)
        losses = O.eval_losses(ocfg, model, data, step * KW["seq_len"], SEED + step, off, per)
        mine = torch.from_numpy(O.fitness(losses))
        parts = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        fit = torch.cat(parts).numpy()
        before = model.copy()
        O.update(ocfg, model, opt, fit, SEED + step, LR)
        for i in range(len(owners)):            # a rank's own result counts only for the parameters it owns
            if owners[i] != rank:
                model[offs[i]:offs[i] + lens[i]] = before[offs[i]:offs[i] + lens[i]]
        for i in range(len(owners)):
            seg = torch.from_numpy(model[offs[i]:offs[i] + lens[i]].copy())
            dist.broadcast(seg, src=int(owners[i]))
            model[offs[i]:offs[i] + lens[i]] = seg.numpy()
    q.put((rank, model.tobytes()))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_update_data_flow_equals_single_process():
    O = load_oracle()
    pkg = load_pkg()
    cfg, ocfg, model, data = make_case(KW, data_len=20000)
    owners, costs, offs, lens = pkg.update_owner_plan(cfg, 2, spans=True)
    # the parameters tile the model: every byte belongs to exactly one of them, so broadcasting them moves everything
    cover = np.zeros(len(model), np.int32)
    for o, n in zip(offs, lens):
        cover[o:o + n] += 1
    assert (cover == 1).all()
    opt = np.zeros(O.opt_bytes(ocfg), np.uint8)
    pop = KW["population_size"]
    for step in range(3):
        losses = O.eval_losses(ocfg, model, data, step * KW["seq_len"], SEED + step, 0, pop)
        O.update(ocfg, model, opt, O.fitness(losses), SEED + step, LR)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_sharded_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, mb in got:
        assert mb == model.tobytes(), "rank %d model differs" % rank


def test_slices_are_pair_aligned_and_cover_population():
    load_pkg()
    from egg_c_b200 import sharding
    for world in (1, 2, 4, 8):
        pop = 40960 * world
        seen = []
        for r in range(world):
            off, per = sharding.member_slice(r, world, pop)
            assert off % 2 == 0 and per % 2 == 0
            assert sharding.pair_slice(r, world, pop) == (off // 2, per // 2)
            seen.append((off, per))
        assert seen[0][0] == 0 and sum(p for _, p in seen) == pop
        assert all(seen[i][0] + seen[i][1] == seen[i + 1][0] for i in range(world - 1))
    with pytest.raises(ValueError):
        sharding.member_slice(0, 4, 36)


def test_sharded_update_owner_plan_is_balanced_and_complete():
    """Every parameter has exactly one owner, every rank gets work, and the heaviest rank carries at most one largest
    parameter more than an even split (greedy longest-processing-time bound), at the benchmark and the d-eggs shapes."""
    pkg = load_pkg()
    for kw in (dict(hidden_dim=512, n_layers=4, seq_len=256), dict(hidden_dim=1024, n_layers=12, seq_len=512, use_muon=1),
               dict(hidden_dim=128, n_layers=1, seq_len=16, vocab_size=1024, ntt_mode=1)):
        cfg = pkg.default_config(**kw)
        for world in (1, 2, 4, 8):
            owners, costs = pkg.update_owner_plan(cfg, world)
            assert len(owners) == 12 * cfg.n_layers + 10 + (3 if cfg.ntt_mode else 0)
            assert owners.min() >= 0 and owners.max() < world
            load = np.bincount(owners, weights=costs, minlength=world)
            assert (load > 0).all()
            assert load.max() <= costs.sum() / world + costs.max()
            again, _ = pkg.update_owner_plan(cfg, world)
            assert (again == owners).all()
