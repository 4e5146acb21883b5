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
    from v1_glif_model_b200 import synth
    return synth.make_lgn_tables(n_units, height, width, sides, len_dom, len_non_dom, seed=int(rng.integers(1 << 30)))


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
@pytest.mark.parametrize("height,width", [(200, 240), (300, 320)])
def test_device_matches_oracle_for_frames_beyond_shared_memory(height, width):
    """Two 120 x 240 frames fit in one block's shared memory; a 200 x 240 frame fits alone and a 300 x 320
    frame does not fit at all (its pixels are then read from global memory)."""
    rng = np.random.Generator(np.random.PCG64(height))
    tb = random_tables(rng, 300, height, width, (5, 11), 9, 7)
    movie = np.clip(rng.normal(0, 0.5, (7, height, width)), -1, 1).astype(np.float32)
    dom, non_dom = oracle_lgn.spatial_response(torch.from_numpy(movie).double(), tb)
    got_dom, got_non_dom = device_lgn(tb, height, width).spatial_response(movie)
    close(got_dom.cpu(), dom)
    close(got_non_dom.cpu(), non_dom)


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
