"""LGN front end (movie -> firing rates): the oracle against vectors from the reference's own
``spatial_response`` / ``firing_rates_from_spatial`` (CPU), and the device front end against both (GPU).

Tolerances: float32 sums of up to 100 filter taps and 20 temporal taps in a different order from the
reference's convolutions; 2e-5 of the largest value in the compared array.
"""
import os

import numpy as np
import pytest
import torch

from oracle import lgn as oracle_lgn

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_lgn.npz")
TOL = 2e-5


def fixture_tables():
    z = np.load(GOLDEN)
    n_classes = sum(1 for k in z.files if k.startswith("gaussian_filter_"))
    tb = {k: z[k] for k in ("x", "y", "non_dominant_x", "non_dominant_y", "dom_temporal_kernels",
                            "non_dom_temporal_kernels", "amplitude", "non_dom_amplitude", "is_composite",
                            "spontaneous_firing_rates")}
    tb["gaussian_filters"] = [z[f"gaussian_filter_{c}"] for c in range(n_classes)]
    tb["spatial_range_indices"] = [z[f"spatial_range_indices_{c}"] for c in range(n_classes)]
    return z, tb


def close(got, want, tol=TOL):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape
    err = np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)
    assert err <= tol, err


@pytest.mark.parametrize("compat", [True, False])
def test_oracle_matches_reference_vectors(compat):
    z, tb = fixture_tables()
    tag = "" if compat else "_plain"
    dom, non_dom = oracle_lgn.spatial_response(torch.from_numpy(z["movie"]), tb, bmtk_compat=compat)
    close(dom, z["dom" + tag])
    close(non_dom, z["non_dom" + tag])
    rates = oracle_lgn.firing_rates_from_spatial(torch.from_numpy(z["dom" + tag]), torch.from_numpy(z["non_dom" + tag]), tb)
    close(rates, z["rates" + tag])
    assert (z["rates" + tag] >= 0).all() and (z["rates" + tag] == 0).any()      # the rectifier is exercised


def test_oracle_in_double_agrees_with_float():
    z, tb = fixture_tables()
    dom, non_dom = oracle_lgn.spatial_response(torch.from_numpy(z["movie"]).double(), tb)
    close(oracle_lgn.firing_rates_from_spatial(dom, non_dom, tb), z["rates"])


def random_tables(rng, n_units, height, width, sides, len_dom, len_non_dom):
    x = rng.uniform(0, width - 1, n_units).astype(np.float32)
    y = rng.uniform(0, height - 1, n_units).astype(np.float32)
    x[:4], y[:4] = [0, width - 1, 0, width - 1], [0, 0, height - 1, height - 1]
    cls = rng.integers(0, len(sides), n_units)
    cls[:len(sides)] = np.arange(len(sides))
    filters = []
    for side in sides:
        r = np.arange(side) - side // 2
        g = np.exp(-(r[:, None] ** 2 + r[None, :] ** 2) / (2 * (side / 6.0 + 0.2) ** 2))
        filters.append((g / g.sum()).astype(np.float32)[..., None, None])
    comp = (rng.random(n_units) < 0.3).astype(np.float32)
    return dict(x=x, y=y, non_dominant_x=np.clip(x + rng.normal(0, 4, n_units), 0, width - 1).astype(np.float32),
                non_dominant_y=np.clip(y + rng.normal(0, 4, n_units), 0, height - 1).astype(np.float32),
                gaussian_filters=filters, spatial_range_indices=[np.where(cls == c)[0].astype(np.int32) for c in range(len(sides))],
                dom_temporal_kernels=rng.normal(0, 0.2, (len_dom, n_units)).astype(np.float32),
                non_dom_temporal_kernels=(rng.normal(0, 0.2, (len_non_dom, n_units)) * comp).astype(np.float32),
                amplitude=rng.uniform(-3, 3, n_units).astype(np.float32),
                non_dom_amplitude=(rng.uniform(-3, 3, n_units) * comp).astype(np.float32), is_composite=comp,
                spontaneous_firing_rates=rng.uniform(0.5, 6, n_units).astype(np.float32))


def device_lgn(tb, height, width, compat=True):
    from v1_glif_model_b200.lgn import LGN
    return LGN(**tb, row_size=height, col_size=width, bmtk_compat=compat)


@pytest.mark.gpu
@pytest.mark.parametrize("compat", [True, False])
def test_device_matches_reference_vectors(compat):
    z, tb = fixture_tables()
    tag = "" if compat else "_plain"
    lgn = device_lgn(tb, *z["movie"].shape[1:], compat=compat)
    dom, non_dom = lgn.spatial_response(z["movie"], bmtk_compat=compat)
    close(dom.cpu(), z["dom" + tag])
    close(non_dom.cpu(), z["non_dom" + tag])
    close(lgn.firing_rates_from_spatial(z["dom" + tag], z["non_dom" + tag]).cpu(), z["rates" + tag])
    close(lgn.firing_rates(z["movie"][..., None]).cpu(), z["rates" + tag])           # [T, H, W, 1] as the reference takes it
    with pytest.raises(ValueError):
        lgn.spatial_response(z["movie"], bmtk_compat=not compat)


@pytest.mark.gpu
def test_device_matches_oracle_at_the_reference_frame_size():
    """120 x 240 frames (``lgn.py:115``), filters up to 27 taps wide, 2,000 units, a movie longer than
    the temporal kernels and not a multiple of the kernel's time tile."""
    rng = np.random.Generator(np.random.PCG64(3))
    height, width, n_units, n_frames = 120, 240, 2000, 77
    tb = random_tables(rng, n_units, height, width, (3, 7, 13, 27), 40, 33)
    movie = np.clip(rng.normal(0, 0.5, (n_frames, height, width)), -1, 1).astype(np.float32)
    dom, non_dom = oracle_lgn.spatial_response(torch.from_numpy(movie).double(), tb)
    want = oracle_lgn.firing_rates_from_spatial(dom, non_dom, tb)
    lgn = device_lgn(tb, height, width)
    got_dom, got_non_dom = lgn.spatial_response(movie)
    close(got_dom.cpu(), dom)
    close(got_non_dom.cpu(), non_dom)
    close(lgn.firing_rates(movie).cpu(), want)
    # frames shorter than the temporal kernels, and an empty movie
    close(lgn.firing_rates(movie[:5]).cpu(), want[:5])
    assert lgn.firing_rates(movie[:0]).shape == (0, n_units)


@pytest.mark.gpu
def test_movie_to_column_activity_through_the_rates():
    """Movie -> LGN rates -> rate-driven rollout of the column (spikes drawn on the device) equals the
    rollout over spikes sampled from the same rates and seed (``stim_dataset.py:170-193`` feeding
    ``models.py``'s cell)."""
    from util import make_cells
    cfg, dicts, orc, cell = make_cells("small", dampening_factor=0.5, pseudo_width=0.5,
                                       recurrent_dampening_factor=0.5, voltage_gradient_dampening=0.5)
    rng = np.random.Generator(np.random.PCG64(8))
    height, width, n_frames = 24, 40, 50
    tb = random_tables(rng, cell.input_dim, height, width, (3, 5, 9), 12, 9)
    tb["spontaneous_firing_rates"] *= 20.0                    # enough drive for the small column to fire
    movie = np.clip(rng.normal(0, 0.5, (n_frames, height, width)), -1, 1).astype(np.float32)
    rates = device_lgn(tb, height, width).firing_rates(movie)
    assert rates.shape == (n_frames, cell.input_dim) and float(rates.min()) >= 0.0
    x = cell.sample_lgn_spikes(rates, cfg.batch, seed=77)
    c = cell.sample_bkg_counts(cfg.batch, n_frames)
    z1, v1 = cell.rollout(x, c)
    z2, v2 = cell.rollout_rates(rates, 77, cfg.batch, bkg_counts=c)
    cell.synchronize()
    assert int(x.sum()) > 0 and int(z1.sum()) > 0
    assert torch.equal(z1, z2)
