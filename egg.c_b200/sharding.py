"""Population sharding over ranks: contiguous, pair-aligned slices (the reference batches members the
same way through global_pop_offset, full_cuda_train_transformer_adam_mgpu.cu:1523-1546).  Rank r of n
evaluates members [r*POP/n, (r+1)*POP/n) and owns fitness pairs [r*POP/2/n, (r+1)*POP/2/n); the only
exchange per generation is an all-gather of those fitness slices in rank order."""


def member_slice(rank, world, population_size):
    if population_size % (2 * world):
        raise ValueError("POPULATION_SIZE/2 = %d pairs do not divide over %d ranks" % (population_size // 2, world))
    per = population_size // world
    return rank * per, per


def pair_slice(rank, world, population_size):
    off, per = member_slice(rank, world, population_size)
    return off // 2, per // 2
