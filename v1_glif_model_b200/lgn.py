"""Host-side mirror of the reference's LGN front end (``lgn_model/lgn.py``): movie -> firing rates of
the LGN units on the GPU, with the method names of the reference's ``LGN`` class.

The reference builds its tables in ``LGN.__init__`` from BMTK filter objects and CSV/HDF5 files
(``lgn.py:115-478``) and caches them in two pickles; this class takes those tables as arrays (the
keys of the two cache files plus the per-unit class and the per-class Gaussian filters) and hands
them to ``libv1g.so``.  ``spatial_response`` and ``firing_rates_from_spatial`` are the two methods
the data pipeline calls (``stim_dataset.py:170-176``); :meth:`firing_rates` fuses them.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib


class LGN:
    def __init__(self, x, y, non_dominant_x, non_dominant_y, gaussian_filters, spatial_range_indices,
                 dom_temporal_kernels, non_dom_temporal_kernels, amplitude, non_dom_amplitude, is_composite,
                 spontaneous_firing_rates, row_size=120, col_size=240, bmtk_compat=True, device=None):
        """``gaussian_filters``: list of ``[k, k]`` (or ``[k, k, 1, 1]``) arrays, one per spatial size class;
        ``spatial_range_indices``: list of unit-index arrays, one per class (``lgn.py:398-437``);
        temporal kernels ``[taps, n_units]`` with the last tap on the current frame (``lgn.py:355-360``);
        positions in pixels, already scaled and clamped as in ``lgn.py:386-393``."""
        if not torch.cuda.is_available():
            raise RuntimeError("the LGN front end needs a CUDA device; there is no CPU fallback")
        self._lib = _lib.load()
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        torch.cuda.set_device(self.device)
        f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32)
        n = len(np.asarray(x))
        unit_class = np.full(n, -1, dtype=np.int32)
        for c, idx in enumerate(spatial_range_indices):
            unit_class[np.asarray(idx, dtype=np.int64)] = c
        if np.any(unit_class < 0):
            raise ValueError("every LGN unit must belong to one spatial size class")
        filters = [f32(np.asarray(g).reshape(np.asarray(g).shape[0], np.asarray(g).shape[1])) for g in gaussian_filters]
        sizes = np.array([g.shape[0] for g in filters], dtype=np.int32)
        flat = np.concatenate([g.reshape(-1) for g in filters]).astype(np.float32)
        kd, kn = f32(dom_temporal_kernels), f32(non_dom_temporal_kernels)
        keep = [sizes, flat, unit_class, f32(x), f32(y), f32(non_dominant_x), f32(non_dominant_y), kd, kn,
                f32(amplitude), f32(non_dom_amplitude), f32(is_composite), f32(spontaneous_firing_rates)]
        p = lambda a: a.ctypes.data
        tb = _lib.V1GLgnTables(n_units=n, height=int(row_size), width=int(col_size), n_classes=len(filters),
                               filter_sizes=p(keep[0]), filters=p(keep[1]), unit_class=p(keep[2]), x=p(keep[3]),
                               y=p(keep[4]), non_dominant_x=p(keep[5]), non_dominant_y=p(keep[6]),
                               len_dom=kd.shape[0], len_non_dom=kn.shape[0], dom_temporal_kernels=p(kd),
                               non_dom_temporal_kernels=p(kn), amplitude=p(keep[9]), non_dom_amplitude=p(keep[10]),
                               is_composite=p(keep[11]), spontaneous_firing_rates=p(keep[12]),
                               bmtk_compat=1 if bmtk_compat else 0)
        h = C.c_void_p()
        rc = self._lib.v1g_lgn_create(C.byref(tb), C.byref(h))
        if rc != _lib.OK:
            msg = self._lib.v1g_lgn_last_error(None).decode(errors="replace")
            raise ValueError(msg) if rc == _lib.EINVAL else _lib.V1GError(rc, msg)
        self._h, self.n_units, self.shape, self.bmtk_compat = h, n, (int(row_size), int(col_size)), bool(bmtk_compat)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.v1g_lgn_destroy(self._h)
            self._h = None

    def _run(self, movie, want_spatial, want_rates):
        movie = torch.as_tensor(movie, dtype=torch.float32, device=self.device)
        if movie.dim() == 4:
            movie = movie[..., 0]
        movie = movie.contiguous()
        assert tuple(movie.shape[1:]) == self.shape, f"frames must be {self.shape}, got {tuple(movie.shape[1:])}"
        t_len = movie.shape[0]
        spatial = torch.empty((2, t_len, self.n_units), dtype=torch.float32, device=self.device) if want_spatial else None
        rates = torch.empty((t_len, self.n_units), dtype=torch.float32, device=self.device) if want_rates else None
        ptr = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None
        rc = self._lib.v1g_lgn_firing_rates(self._h, ptr(movie), t_len, ptr(spatial), ptr(rates),
                                            C.c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc != _lib.OK:
            raise _lib.V1GError(rc, self._lib.v1g_lgn_last_error(self._h).decode(errors="replace"))
        return spatial, rates

    def spatial_response(self, movie, bmtk_compat=True):
        """``(all_spatial_responses, all_non_dom_spatial_responses)``, each ``[T, n_units]`` (``lgn.py:481-517``)."""
        if bool(bmtk_compat) != self.bmtk_compat:
            raise ValueError("the edge normalisation is folded into the stencils when the object is made: "
                             "pass bmtk_compat to the constructor")
        spatial, _ = self._run(movie, True, False)
        return spatial[0], spatial[1]

    def firing_rates(self, movie):
        """``firing_rates_from_spatial(*spatial_response(movie))`` in one call: ``[T, n_units]`` in Hz."""
        return self._run(movie, False, True)[1]

    def firing_rates_from_spatial(self, all_spatial_responses, all_non_dom_spatial_responses):
        """Temporal filters, amplitudes, spontaneous rates and rectification on given spatial responses
        (``lgn.py:519-528``): ``[T, n_units]`` in Hz."""
        spatial = torch.stack([torch.as_tensor(all_spatial_responses, dtype=torch.float32, device=self.device),
                               torch.as_tensor(all_non_dom_spatial_responses, dtype=torch.float32,
                                               device=self.device)]).contiguous()
        t_len = spatial.shape[1]
        rates = torch.empty((t_len, self.n_units), dtype=torch.float32, device=self.device)
        rc = self._lib.v1g_lgn_firing_rates(self._h, None, t_len, C.c_void_p(spatial.data_ptr()),
                                            C.c_void_p(rates.data_ptr()),
                                            C.c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc != _lib.OK:
            raise _lib.V1GError(rc, self._lib.v1g_lgn_last_error(self._h).decode(errors="replace"))
        return rates
