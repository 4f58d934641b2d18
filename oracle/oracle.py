"""ctypes binding of the CPU oracle (liboracle.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's cpu_baseline / reference legs, never by the library itself.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))


class EggConfig(C.Structure):
    """Mirror of struct egg_config (include/egg_b200.h); defaults are the
    reference's (full_cuda_train_transformer_adam_mgpu.cu:35-270)."""
    _fields_ = [(n, C.c_int32) for n in (
        "hidden_dim", "head_dim", "n_layers", "seq_len", "vocab_size", "population_size",
        "fixed_point", "sigma_shift", "sigma_shift_vector", "shift_attn", "shift_out",
        "shift_logit", "shift_mlp_up", "shift_mlp_down", "softmax_scale_bit", "rope_scale_bit",
        "device_mask", "device_gaussian", "host_mask", "use_same_data", "use_muon",
        "chunk_relative_loss")] + [
        ("softmax_exp_scale", C.c_double), ("adam_beta1", C.c_float), ("adam_beta2", C.c_float),
        ("adam_eps", C.c_float), ("adam_weight_decay", C.c_float), ("muon_momentum", C.c_float),
        ("muon_lr_scale", C.c_float), ("ntt_mode", C.c_int32)]


class GruConfig(C.Structure):
    """Mirror of struct egg_gru_config; defaults are full_trained_egg.c:10-21."""
    _fields_ = [(n, C.c_int32) for n in ("hidden_dim", "n_layers", "vocab_size", "seq_len", "population_size",
                                          "fixed_point", "sigma_shift", "update_threshold")]


def make_gru_config(**kw):
    d = dict(hidden_dim=512, n_layers=4, vocab_size=256, seq_len=4096, population_size=128, fixed_point=4, sigma_shift=4,
             update_threshold=160)
    for k in kw:
        if k not in d:
            raise KeyError(k)
    d.update(kw)
    return GruConfig(**d)


def make_config(**kw):
    d = dict(hidden_dim=256, head_dim=64, n_layers=4, seq_len=32, vocab_size=256,
             population_size=8192 * 2 * 4, fixed_point=4, sigma_shift=3, sigma_shift_vector=4,
             shift_attn=8, shift_out=9, shift_logit=8, shift_mlp_up=8, shift_mlp_down=10,
             softmax_scale_bit=18, rope_scale_bit=20, device_mask=15, device_gaussian=0,
             host_mask=15, use_same_data=0, use_muon=0, chunk_relative_loss=0,
             softmax_exp_scale=6.0, adam_beta1=0.9, adam_beta2=0.95, adam_eps=1e-8,
             adam_weight_decay=0.01, muon_momentum=0.85, muon_lr_scale=1.0, ntt_mode=0)
    for k in kw:
        if k not in d:
            raise KeyError(k)
    d.update(kw)
    return EggConfig(**d)


def build(force=False):
    so = os.path.join(_HERE, "liboracle.so")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(os.path.join(_HERE, "egg_oracle.c")):
        subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True, capture_output=True)
    return so


_lib = None


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(build())
        P = C.POINTER
        cfgp = P(EggConfig)
        L.oracle_hash_rng.restype = C.c_uint32
        L.oracle_hash_rng.argtypes = [C.c_uint32, C.c_uint32]
        L.oracle_noise.restype = C.c_int
        L.oracle_noise.argtypes = [cfgp, C.c_uint32, C.c_uint32]
        L.oracle_gen_noise_host.restype = C.c_int
        L.oracle_gen_noise_host.argtypes = [cfgp, P(C.c_uint32)]
        for f in (L.oracle_model_bytes, L.oracle_opt_bytes, L.oracle_scales_bytes):
            f.restype = C.c_int64
            f.argtypes = [cfgp]
        L.oracle_init_tables.argtypes = [cfgp, C.c_void_p, C.c_void_p, C.c_void_p]
        L.oracle_init_model.argtypes = [cfgp, C.c_void_p, C.c_uint32]
        L.oracle_repack_matrix.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        L.oracle_eval.argtypes = [cfgp, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                  C.c_uint32, C.c_int, C.c_int, C.c_void_p]
        L.oracle_fitness.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.oracle_window_transform.argtypes = [cfgp, C.c_void_p, C.c_int]
        L.oracle_generate.argtypes = [cfgp, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_uint32, C.c_float, C.c_float, C.c_float]
        L.oracle_update.restype = C.c_uint64
        L.oracle_update.argtypes = [cfgp, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_float, C.c_int]
        L.oracle_update_scaled.restype = C.c_uint64
        L.oracle_update_scaled.argtypes = [cfgp, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_float, C.c_int, C.c_void_p]
        L.oracle_vote_matrix.argtypes = [cfgp, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                         C.c_int, C.c_uint32, C.c_void_p]
        L.oracle_vote_columns.argtypes = [cfgp, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint32, C.c_void_p,
                                          C.c_int, C.c_void_p]
        L.oracle_adam_from_votes.restype = C.c_uint64
        L.oracle_adam_from_votes.argtypes = [cfgp, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_float, C.c_int]
        L.oracle_newton_schulz.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.oracle_projection.argtypes = [cfgp, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int,
                                        C.c_int, C.c_uint32, C.c_int, C.c_int, C.c_int, C.c_int]
        L.oracle_deggs_chunk_fitness.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_double, C.c_int, C.c_double, C.c_void_p, C.c_void_p]
        L.oracle_ternary_packed_size.restype = C.c_int64
        L.oracle_ternary_packed_size.argtypes = [C.c_int64]
        L.oracle_ternary_pack.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
        L.oracle_ternary_unpack.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
        gcp = P(GruConfig)
        L.oracle_gru_model_bytes.restype = C.c_int64
        L.oracle_gru_model_bytes.argtypes = [gcp]
        L.oracle_gru_init_model.argtypes = [gcp, C.c_void_p, C.c_uint32]
        L.oracle_gru_generation.argtypes = [gcp, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_uint32, C.c_int64,
                                            C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def hash_rng(s, idx):
    return lib().oracle_hash_rng(s & 0xFFFFFFFF, idx & 0xFFFFFFFF)


def noise(cfg, s, idx):
    return lib().oracle_noise(C.byref(cfg), s & 0xFFFFFFFF, idx & 0xFFFFFFFF)


def model_bytes(cfg):
    return lib().oracle_model_bytes(C.byref(cfg))


def opt_bytes(cfg):
    return lib().oracle_opt_bytes(C.byref(cfg))


def scales_bytes(cfg):
    return lib().oracle_scales_bytes(C.byref(cfg))


def init_tables(cfg):
    exp = np.zeros(256, np.int32)
    act = np.zeros(256, np.int8)
    rope = np.zeros(cfg.seq_len * cfg.head_dim, np.int32)
    lib().oracle_init_tables(C.byref(cfg), _p(exp), _p(act), _p(rope))
    return exp, act, rope


def init_model(cfg, seed=42):
    m = np.zeros(model_bytes(cfg), np.int8)
    lib().oracle_init_model(C.byref(cfg), _p(m), seed)
    return m


def eval_losses(cfg, model, dataset, start_idx, step_seed, pop_offset, count, scales=None):
    """dataset: uint8 tokens when cfg.vocab_size == 256, uint32 tokens otherwise (TokenType, mgpu.cu:58-66)."""
    want = np.uint8 if cfg.vocab_size == 256 else np.uint32
    assert dataset.dtype == want, "token width does not match vocab_size"
    out = np.zeros(count, np.int32)
    lib().oracle_eval(C.byref(cfg), _p(model), _p(scales), _p(dataset), len(dataset), start_idx,
                      step_seed & 0xFFFFFFFF, pop_offset, count, _p(out))
    return out


def window_transform(cfg, values):
    """The ntt_mode transform of one input window (int32 in, int32 out)."""
    d = np.ascontiguousarray(values, np.int32).copy()
    lib().oracle_window_transform(C.byref(cfg), _p(d), len(d))
    return d


def fitness(losses):
    f = np.zeros(len(losses) // 2, np.int32)
    lib().oracle_fitness(_p(np.ascontiguousarray(losses, np.int32)), _p(f), len(f))
    return f


FMA_NVCC = 34   # contraction pattern of the reference kernels under nvcc -fmad=true (see oracle_adam_step)


def update(cfg, model, opt_state, fit, step_seed, lr, fma_mode=FMA_NVCC):
    """In-place on model (int8) and opt_state (uint8 bytes); returns update count."""
    fit = np.ascontiguousarray(fit, np.int32)
    return int(lib().oracle_update(C.byref(cfg), _p(model), _p(opt_state), _p(fit), step_seed & 0xFFFFFFFF,
                                   C.c_float(lr), fma_mode))


def update_scaled(cfg, model, opt_state, fit, step_seed, lr, scales, fma_mode=FMA_NVCC):
    """d-eggs update: also steps the adaptive-noise overlays in `scales` (int8 array, in place)."""
    fit = np.ascontiguousarray(fit, np.int32)
    return int(lib().oracle_update_scaled(C.byref(cfg), _p(model), _p(opt_state), _p(fit), step_seed & 0xFFFFFFFF,
                                          C.c_float(lr), fma_mode, _p(scales)))


def vote_matrix(cfg, fit, rows_k, cols_n, off_a, off_b, seed_base, step_seed):
    fit = np.ascontiguousarray(fit, np.int32)
    v = np.zeros(rows_k * cols_n, np.int32)
    lib().oracle_vote_matrix(C.byref(cfg), _p(fit), len(fit), rows_k, cols_n, off_a, off_b, seed_base,
                             step_seed & 0xFFFFFFFF, _p(v))
    return v


def vote_columns(cfg, fit, rows_k, off_a, off_b, seed_base, step_seed, n_list):
    """Votes of the output columns n_list of one matrix: array [len(n_list)][rows_k]."""
    fit = np.ascontiguousarray(fit, np.int32)
    n_list = np.ascontiguousarray(n_list, np.int32)
    out = np.zeros((len(n_list), rows_k), np.int32)
    lib().oracle_vote_columns(C.byref(cfg), _p(fit), len(fit), rows_k, off_a, off_b, seed_base, step_seed & 0xFFFFFFFF,
                              _p(n_list), len(n_list), _p(out))
    return out


def adam_from_votes(cfg, w, state, vote, lr, fma_mode=FMA_NVCC):
    """In place on w (int8) and state (float32 [n][3]); returns the number of changed weights."""
    vote = np.ascontiguousarray(vote, np.int32)
    return int(lib().oracle_adam_from_votes(C.byref(cfg), _p(w), _p(state), _p(vote), vote.size, C.c_float(lr), fma_mode))


def newton_schulz(x):
    x = np.ascontiguousarray(x, np.float32).copy()
    lib().oracle_newton_schulz(_p(x), x.shape[0], x.shape[1])
    return x


def projection(cfg, x, w_packed, k_dim, n_dim, rows_per_member, seed, off_a, off_b, rank1_shift, out_shift):
    rows = x.size // k_dim
    y = np.zeros((rows, n_dim), np.int8)
    lib().oracle_projection(C.byref(cfg), _p(x), _p(w_packed), _p(y), rows, k_dim, n_dim, rows_per_member,
                            seed & 0xFFFFFFFF, off_a, off_b, rank1_shift, out_shift)
    return y


def repack(src_k_by_n):
    """[K][N] row-major int8 -> the reference's packed [K/4][N][4] bytes."""
    K, N = src_k_by_n.shape
    dst = np.zeros(K * N, np.int8)
    lib().oracle_repack_matrix(_p(dst), _p(np.ascontiguousarray(src_k_by_n, np.int8)), K, N)
    return dst


def ternary_pack(values):
    values = np.ascontiguousarray(values, np.int32)
    out = np.zeros(lib().oracle_ternary_packed_size(len(values)), np.uint8)
    lib().oracle_ternary_pack(_p(values), len(values), _p(out))
    return out


def ternary_unpack(packed, count):
    out = np.zeros(count, np.int32)
    lib().oracle_ternary_unpack(_p(np.ascontiguousarray(packed, np.uint8)), count, _p(out))
    return out


def deggs_chunk_fitness(losses, mean_filter=1, exponent=1.2, adaptive=1, alpha=0.1):
    losses = np.ascontiguousarray(losses, np.int32)
    fit = np.zeros(len(losses) // 2, np.int32)
    sl = np.zeros(1, np.int64)
    lib().oracle_deggs_chunk_fitness(_p(losses), len(losses), mean_filter, exponent, adaptive, alpha, _p(fit), _p(sl))
    return fit, int(sl[0])


# ---- the recurrent model of full_trained_egg.c
def gru_model_bytes(gcfg):
    return lib().oracle_gru_model_bytes(C.byref(gcfg))


def gru_state_bytes(gcfg):
    return gcfg.population_size * gcfg.n_layers * gcfg.hidden_dim


def gru_init_model(gcfg, seed=42):
    m = np.zeros(gru_model_bytes(gcfg), np.int8)
    lib().oracle_gru_init_model(C.byref(gcfg), _p(m), seed)
    return m


def gru_generation(gcfg, model, states, data, step_seed, start_idx, tokens, do_update=True):
    """In place on model and states; returns (losses[pop], fitness[pop/2])."""
    losses = np.zeros(gcfg.population_size, np.int32)
    fit = np.zeros(gcfg.population_size // 2, np.int32)
    lib().oracle_gru_generation(C.byref(gcfg), _p(model), _p(states), _p(data), len(data), step_seed & 0xFFFFFFFF, start_idx,
                                tokens, 1 if do_update else 0, _p(losses), _p(fit))
    return losses, fit


def generate(cfg, model, seed_tokens, gen_len, seed, temp=1.0, min_p=0.0, penalty=0.0):
    """Returns the seed tokens followed by gen_len sampled ones (uint8)."""
    buf = np.zeros(len(seed_tokens) + gen_len, np.uint8)
    buf[:len(seed_tokens)] = seed_tokens
    lib().oracle_generate(C.byref(cfg), _p(model), _p(buf), len(seed_tokens), gen_len, seed & 0xFFFFFFFF, temp, min_p, penalty)
    return buf
