"""CPU restatement of the reference's LGN front end.  TEST INFRASTRUCTURE ONLY.

Follows ``lgn_model/lgn.py``: ``temporal_filter`` (``:54-61``), ``transfer_function`` (``:63-65``),
``select_spatial`` (``:67-96``), ``LGN.spatial_response`` (``:481-517``) and
``LGN.firing_rates_from_spatial`` (``:519-528``) with torch CPU ops standing in for the TensorFlow
calls (``conv2d`` with padding SAME, ``gather_nd``, ``einsum``, ``depthwise_conv2d`` after front padding).
Pinned by ``tests/golden/reference_lgn.npz``, which ``tests/golden/run_reference_lgn.py`` produces by
running the reference's own two methods over the TensorFlow stand-in.
"""
import torch
import torch.nn.functional as F


def temporal_filter(all_spatial_responses, temporal_kernels):
    """Causal per-unit filter: ``out[t, u] = sum_j K[j, u] * s[t - (L - 1) + j, u]`` (zeros before the start)."""
    length, n_units = temporal_kernels.shape
    padded = F.pad(all_spatial_responses.t()[None], (length - 1, 0))                    # [1, U, T + L - 1]
    return F.conv1d(padded, temporal_kernels.t()[:, None, :], groups=n_units)[0].t()     # cross-correlation, [T, U]


def transfer_function(a):
    return (a >= 0).to(a.dtype) * a


def select_spatial(x, y, convolved_movie):
    """Bilinear sample of ``convolved_movie[T, H, W]`` at ``(x, y)`` -> ``[T, n]`` (``:67-96``)."""
    xf, yf, xc, yc = torch.floor(x).long(), torch.floor(y).long(), torch.ceil(x).long(), torch.ceil(y).long()
    m = convolved_movie.permute(1, 2, 0)
    ss = torch.stack([m[yf, xf], m[yc, xf], m[yf, xc], m[yc, xc]], 0)                  # [4, n, T]
    y_factor, x_factor = y - torch.floor(y), x - torch.floor(x)
    weights = torch.stack([(1 - x_factor) * (1 - y_factor), (1 - x_factor) * y_factor,
                           x_factor * (1 - y_factor), x_factor * y_factor], 0)
    return torch.einsum("int,in->tn", ss, weights)


def spatial_response(movie, tables, bmtk_compat=True):
    """``movie[T, H, W]`` -> ``(dominant, non_dominant)`` responses ``[T, n_units]`` (``:481-517``)."""
    dtype = movie.dtype
    frames = movie[:, None]                                                             # [T, 1, H, W]
    t = lambda a: torch.as_tensor(a, dtype=dtype)
    dom, non_dom, ids = [], [], []
    for g, indices in zip(tables["gaussian_filters"], tables["spatial_range_indices"]):
        g = t(g).reshape(g.shape[0], g.shape[1])[None, None]
        conv = F.conv2d(frames, g, padding="same")
        if bmtk_compat:
            conv = conv / F.conv2d(torch.ones_like(frames), g, padding="same")
        conv = conv[:, 0]
        idx = torch.as_tensor(indices, dtype=torch.int64)
        dom.append(select_spatial(t(tables["x"])[idx], t(tables["y"])[idx], conv))
        non_dom.append(select_spatial(t(tables["non_dominant_x"])[idx], t(tables["non_dominant_y"])[idx], conv))
        ids.append(idx)
    order = torch.argsort(torch.cat(ids))
    return torch.cat(dom, 1)[:, order], torch.cat(non_dom, 1)[:, order]


def firing_rates_from_spatial(dom, non_dom, tables):
    dtype = dom.dtype
    t = lambda a: torch.as_tensor(a, dtype=dtype)
    d = temporal_filter(dom, t(tables["dom_temporal_kernels"]))
    n = temporal_filter(non_dom, t(tables["non_dom_temporal_kernels"]))
    spont = t(tables["spontaneous_firing_rates"])
    return transfer_function(d * t(tables["amplitude"]) + spont) + \
        t(tables["is_composite"]) * transfer_function(n * t(tables["non_dom_amplitude"]) + spont)
