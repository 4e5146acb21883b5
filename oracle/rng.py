"""CPU restatement of the device-side samplers.  TEST INFRASTRUCTURE ONLY.

Philox-4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11) in
NumPy, the inverse-CDF Poisson draw and the Bernoulli LGN draw exactly as ``csrc/v1g_rng.cu`` keys and
evaluates them.  The reference draws the same quantities with TensorFlow's stateless generators
(``v1_model_utils/models.py:865-887``, ``stim_dataset.py:182-193``); those streams belong to
TensorFlow 2.15 and are not restated, so parity with the reference's random numbers is unpinned -
what is pinned here is the generator (against its published known-answer vectors) and the CUDA
kernels against this file.
"""
import numpy as np

M0, M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
W0, W1 = np.uint32(0x9E3779B9), np.uint32(0xBB67AE85)
POISSON_TABLE = 32
STREAM_BKG, STREAM_LGN = 0x42, 0x4C


def philox4x32(ctr, key, rounds=10):
    """``ctr`` [..., 4] and ``key`` [..., 2] uint32 -> [..., 4] uint32."""
    c = [np.asarray(ctr[..., i], dtype=np.uint32).copy() for i in range(4)]
    k = [np.asarray(key[..., i], dtype=np.uint32).copy() for i in range(2)]
    mask = np.uint64(0xFFFFFFFF)
    with np.errstate(over="ignore"):
        for _ in range(rounds):
            p0 = M0 * c[0].astype(np.uint64)
            p1 = M1 * c[2].astype(np.uint64)
            hi0, lo0 = (p0 >> np.uint64(32)).astype(np.uint32), (p0 & mask).astype(np.uint32)
            hi1, lo1 = (p1 >> np.uint64(32)).astype(np.uint32), (p1 & mask).astype(np.uint32)
            c = [hi1 ^ c[1] ^ k[0], lo1, hi0 ^ c[3] ^ k[1], lo0]
            k = [(k[0] + W0).astype(np.uint32), (k[1] + W1).astype(np.uint32)]
    return np.stack(c, axis=-1)


def u01(w):
    """24 random bits as a float32 in [0, 1)."""
    return (np.asarray(w, dtype=np.uint32) >> np.uint32(8)).astype(np.float32) * np.float32(1.0 / 16777216.0)


def poisson_cdf(lam):
    p, c, out = np.exp(-np.float64(lam)), 0.0, []
    for k in range(POISSON_TABLE):
        c += p
        out.append(np.float32(min(c, 1.0)))
        p *= np.float64(lam) / (k + 1)
    out[-1] = np.float32(2.0)
    return np.asarray(out, dtype=np.float32)


def _words(ctr0, ctr1, ctr2, stream, key0, key1, sel):
    shape = np.broadcast(ctr0, ctr1, ctr2, sel, key0, key1).shape
    ctr = np.stack([np.broadcast_to(np.asarray(a, dtype=np.uint32), shape)
                    for a in (ctr0, ctr1, ctr2, np.uint32(stream))], axis=-1)
    key = np.stack([np.broadcast_to(np.asarray(a, dtype=np.uint32), shape) for a in (key0, key1)], axis=-1)
    r = philox4x32(ctr, key)
    return np.take_along_axis(r, np.broadcast_to(np.asarray(sel), shape)[..., None].astype(np.int64), axis=-1)[..., 0]


def bkg_counts(noise_seed, replica, first_step, batch, n_steps, n_bkg, lam):
    """counts[B, T, n_bkg] int32: key = (noise_seed + replica * 1000003, step), counter =
    (node // 4, trial, 0, stream), word node % 4, inverse CDF of Poisson(lam)."""
    key0 = np.uint32((int(noise_seed) + int(replica) * 1000003) & 0xFFFFFFFF)
    b = np.arange(batch, dtype=np.uint32)[:, None, None]
    t = (np.arange(n_steps, dtype=np.int64) + int(first_step)).astype(np.uint32)[None, :, None]
    j = np.arange(n_bkg, dtype=np.uint32)[None, None, :]
    w = _words(j >> np.uint32(2), b, np.uint32(0), STREAM_BKG, key0, t, j & np.uint32(3))
    u = u01(w)
    return (u[..., None] >= poisson_cdf(lam)).sum(-1).astype(np.int32)


def lgn_probability(rates):
    return (-np.expm1(-np.asarray(rates, dtype=np.float32) * np.float32(0.001))).astype(np.float32)


def lgn_uniforms(seed, batch, n_steps, n_lgn):
    """u[B, T, n_lgn] float32: key = the two halves of seed, counter = (unit // 4, step, trial, stream)."""
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    b = np.arange(batch, dtype=np.uint32)[:, None, None]
    t = np.arange(n_steps, dtype=np.uint32)[None, :, None]
    c = np.arange(n_lgn, dtype=np.uint32)[None, None, :]
    w = _words(c >> np.uint32(2), t, b, STREAM_LGN, np.uint32(seed & 0xFFFFFFFF), np.uint32(seed >> 32),
               c & np.uint32(3))
    return u01(w)


def lgn_spikes(rates, batch, seed):
    """x[B, T, n_lgn] uint8 = u < 1 - exp(-rate / 1000)."""
    rates = np.asarray(rates, dtype=np.float32)
    t_len, n_lgn = rates.shape[-2:]
    u = lgn_uniforms(seed, batch, t_len, n_lgn)
    return (u < lgn_probability(rates)).astype(np.uint8)
