"""Seeded synthetic inputs with the shapes and value distributions the benchmark
configurations name: Zipf(s=1.1) bytes, uniform int8 weights in the reference's
packed layout, ternary weights, clamped-normal activations.  All draws come from
splitmix64 so that every consumer regenerates identical bytes."""
import numpy as np

_M64 = (1 << 64) - 1


def splitmix64(seed, n):
    """n successive splitmix64 outputs (uint64) starting from `seed`."""
    idx = np.arange(1, n + 1, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + idx * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return z


def uniform01(seed, n):
    return (splitmix64(seed, n) >> np.uint64(11)).astype(np.float64) * (1.0 / (1 << 53))


def zipf_bytes(seed, n, s=1.1):
    """i.i.d. bytes, P(rank r) ~ r^-s over the 256 values, byte = r-1 (inverse CDF)."""
    p = np.arange(1, 257, dtype=np.float64) ** (-s)
    cdf = np.cumsum(p / p.sum())
    u = uniform01(seed, n)
    return np.minimum(np.searchsorted(cdf, u, side="right"), 255).astype(np.uint8)


def zipf_tokens(seed, n, vocab, s=1.1):
    """i.i.d. uint32 tokens for a vocabulary other than 256: P(rank r) ~ r^-s, token = a fixed permutation of the
    rank (so that frequent tokens are spread over the whole index range, as a trained tokenizer's are)."""
    p = np.arange(1, vocab + 1, dtype=np.float64) ** (-s)
    cdf = np.cumsum(p / p.sum())
    u = uniform01(seed, n)
    rank = np.minimum(np.searchsorted(cdf, u, side="right"), vocab - 1)
    perm = np.argsort(splitmix64(0x70CE75, vocab), kind="stable")
    return perm[rank].astype(np.uint32)


def uniform_int8(seed, n, lo=-127, hi=127):
    span = np.uint64(hi - lo + 1)
    return ((splitmix64(seed, n) % span).astype(np.int64) + lo).astype(np.int8)


def ternary_int8(seed, n):
    """{-1,0,1} with P = (0.25, 0.5, 0.25)."""
    u = splitmix64(seed, n) & np.uint64(3)
    return np.where(u == 0, -1, np.where(u == 3, 1, 0)).astype(np.int8)


def normal_int8(seed, n, sigma=32.0):
    """clamp(round(N(0, sigma)), -127, 127) by Box-Muller on splitmix64."""
    m = (n + 1) // 2
    u1 = np.maximum(uniform01(seed, m), 1e-300)
    u2 = uniform01(seed ^ 0x5DEECE66D, m)
    r = np.sqrt(-2.0 * np.log(u1))
    z = np.concatenate([r * np.cos(2 * np.pi * u2), r * np.sin(2 * np.pi * u2)])[:n]
    return np.clip(np.rint(z * sigma), -127, 127).astype(np.int8)


def random_model(cfg, seed=0, kind="uniform", gains_random=False):
    """TransformerModel bytes: every byte of every matrix drawn i.i.d. (the packed
    layout is a permutation of the matrix, so drawing packed bytes directly is
    the same distribution).  Norm gains default to 16 and biases to 0, the
    reference's own initial values, unless gains_random."""
    import ctypes as C
    from . import model_bytes
    n = model_bytes(cfg)
    m = uniform_int8(seed, n) if kind == "uniform" else ternary_int8(seed, n)
    if not gains_random:
        H, V, L = cfg.hidden_dim, cfg.vocab_size, cfg.n_layers
        o = V * H
        m[o:o + H] = 0; o += H                       # emb_bias
        if cfg.ntt_mode:
            o += 3 * V * H                           # ntt_emb1..3
        m[o:o + H] = 16; o += H                      # ln_init
        m[o:o + H] = 0; o += H                       # ln_init_bias
        o += 4 * H * H
        m[o:o + 4 * H] = 0; o += 4 * H               # mlp_emb_bias_up
        o += 4 * H * H
        m[o:o + H] = 0; o += H                       # mlp_emb_bias_down
        m[o:o + L * H] = 16; o += L * H              # ln_1
        m[o:o + L * H] = 0; o += L * H               # ln_1_bias
        o += 4 * L * H * H                           # w_q..w_o
        m[o:o + L * H] = 16; o += L * H              # ln_2
        m[o:o + L * H] = 0; o += L * H               # ln_2_bias
        o += L * 4 * H * H
        m[o:o + L * 4 * H] = 0; o += L * 4 * H       # mlp_bias_up
        o += L * 4 * H * H
        m[o:o + L * H] = 0; o += L * H               # mlp_bias_down
        m[o:o + H] = 16; o += H                      # ln_f
        m[o:o + H] = 0; o += H                       # ln_f_bias
        assert o == n
    return m
