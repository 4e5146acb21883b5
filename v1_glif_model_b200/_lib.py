"""ctypes binding of ``libv1g.so`` (declarations follow ``include/v1g.h``).

There is no CPU fallback: if the library is missing, :func:`load` raises with the build command.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("V1G_LIB", os.path.join(HERE, "libv1g.so"))

OK, EINVAL, ECUDA, ENOMEM, ETIMEOUT, ESTATE, ERANGE = 0, -1, -2, -3, -4, -5, -6
SRC_REC, SRC_LGN, SRC_BKG = 0, 1, 2
FLAG_HARD_RESET, FLAG_PSEUDO_GAUSS = 1, 2
MAX_BATCH = 8


class V1GConfig(C.Structure):
    _fields_ = [("n_neurons", C.c_int32), ("n_receptors", C.c_int32), ("n_syn_types", C.c_int32),
                ("max_delay", C.c_int32), ("n_lgn", C.c_int32), ("n_bkg", C.c_int32),
                ("flags", C.c_int32), ("dt", C.c_float), ("dampening_factor", C.c_float),
                ("recurrent_dampening", C.c_float), ("voltage_gradient_dampening", C.c_float),
                ("gauss_std", C.c_float), ("pseudo_width", C.c_float), ("lr_scale", C.c_float),
                ("bkg_firing_rate", C.c_float)]


class V1GState(C.Structure):
    _fields_ = [("z_buf", C.c_void_p), ("v", C.c_void_p), ("r", C.c_void_p), ("asc", C.c_void_p),
                ("psc_rise", C.c_void_p), ("psc", C.c_void_p), ("noise_step", C.c_void_p)]


class V1GLgnTables(C.Structure):
    _fields_ = [("n_units", C.c_int32), ("height", C.c_int32), ("width", C.c_int32), ("n_classes", C.c_int32),
                ("filter_sizes", C.c_void_p), ("filters", C.c_void_p), ("unit_class", C.c_void_p),
                ("x", C.c_void_p), ("y", C.c_void_p), ("non_dominant_x", C.c_void_p), ("non_dominant_y", C.c_void_p),
                ("len_dom", C.c_int32), ("len_non_dom", C.c_int32), ("dom_temporal_kernels", C.c_void_p),
                ("non_dom_temporal_kernels", C.c_void_p), ("amplitude", C.c_void_p),
                ("non_dom_amplitude", C.c_void_p), ("is_composite", C.c_void_p),
                ("spontaneous_firing_rates", C.c_void_p), ("bmtk_compat", C.c_int32)]


class V1GLossSpec(C.Structure):
    _fields_ = [("rate_target", C.c_void_p), ("v_lo", C.c_void_p), ("rate_cost", C.c_float),
                ("voltage_cost", C.c_float), ("sync_cost", C.c_float), ("fano_target", C.c_float),
                ("sync_bin", C.c_int32), ("loss_scale", C.c_float),
                ("n_rate_groups", C.c_int32), ("n_rate_neurons", C.c_int32),
                ("rate_group_offsets", C.c_void_p), ("rate_group_neurons", C.c_void_p),
                ("rate_group_targets", C.c_void_p), ("rate_kappa", C.c_float),
                ("rate_pre_delay", C.c_int32), ("rate_post_delay", C.c_int32),
                ("n_sync_samples", C.c_int32), ("n_sync_members", C.c_int32),
                ("sync_sample_trial", C.c_void_p), ("sync_sample_offsets", C.c_void_p),
                ("sync_sample_neurons", C.c_void_p), ("n_sync_bins", C.c_int32),
                ("sync_bin_sizes", C.c_void_p), ("sync_bin_targets", C.c_void_p),
                ("sync_t_start", C.c_int32), ("sync_t_end", C.c_int32),
                ("osi_cost", C.c_float), ("n_osi_types", C.c_int32), ("osi_angle", C.c_void_p),
                ("osi_tuning_angle", C.c_void_p), ("osi_type_ids", C.c_void_p),
                ("osi_normalizer", C.c_void_p), ("osi_targets", C.c_void_p),
                ("dsi_targets", C.c_void_p), ("osi_type_counts", C.c_void_p),
                ("osi_pre_delay", C.c_int32), ("osi_post_delay", C.c_int32),
                ("voltage_mode", C.c_int32)]


class V1GCounters(C.Structure):
    _fields_ = [(n, C.c_ulonglong) for n in
                ("spikes", "rec_rows", "rec_events", "lgn_rows", "lgn_events", "bkg_rows",
                 "bkg_events", "bwd_rows", "bwd_events", "dw_events")]


_P = C.c_void_p
# name -> (restype, argtypes); every symbol include/v1g.h declares
SIGNATURES = {
    "v1g_create": (C.c_int, [C.POINTER(V1GConfig), C.POINTER(_P)]),
    "v1g_destroy": (C.c_int, [_P]),
    "v1g_last_error": (C.c_char_p, [_P]),
    "v1g_version": (C.c_char_p, []),
    "v1g_set_connectivity": (C.c_int, [_P, C.c_int, C.c_int64, _P, _P, C.c_int64]),
    "v1g_build_pre_ind_table": (C.c_int, [C.c_int64, _P, C.c_int64, _P, _P]),
    "v1g_get_pre_ind_table": (C.c_int, [_P, C.c_int, _P, _P]),
    "v1g_set_neuron_params": (C.c_int, [_P] * 9),
    "v1g_set_weights": (C.c_int, [_P, C.c_int, _P, _P]),
    "v1g_set_noise_seed": (C.c_int, [_P, C.c_int64, C.c_int32]),
    "v1g_sample_bkg_counts": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_int32, _P, _P]),
    "v1g_sample_lgn_spikes": (C.c_int, [_P, C.c_int32, C.c_int32, _P, C.c_int64, C.c_int64, _P, _P]),
    "v1g_rollout_fwd_rates": (C.c_int, [_P, C.c_int32, C.c_int32, _P, C.c_int64, C.c_int64, _P,
                                        C.POINTER(V1GState), _P, _P, C.c_int32, _P]),
    "v1g_lgn_create": (C.c_int, [C.POINTER(V1GLgnTables), C.POINTER(_P)]),
    "v1g_lgn_destroy": (C.c_int, [_P]),
    "v1g_lgn_last_error": (C.c_char_p, [_P]),
    "v1g_lgn_firing_rates": (C.c_int, [_P, _P, C.c_int32, _P, _P, _P]),
    "v1g_compact_spikes": (C.c_int, [_P, _P, C.c_int32, C.c_int64, _P, C.c_int64, _P, _P]),
    "v1g_compact_spikes_noalloc": (C.c_int, [_P, C.c_int32, C.c_int64, _P, C.c_int64, _P, _P]),
    "v1g_syn_currents_fwd": (C.c_int, [_P, C.c_int, _P, C.c_int32, _P, _P]),
    "v1g_syn_currents_bwd": (C.c_int, [_P, C.c_int, _P, _P, C.c_int32, _P, _P, _P]),
    "v1g_step_fwd": (C.c_int, [_P, C.c_int32, C.POINTER(V1GState), _P, C.POINTER(V1GState), _P, _P]),
    "v1g_step_bwd": (C.c_int, [_P, C.c_int32, C.POINTER(V1GState), _P, _P, _P, _P,
                               C.POINTER(V1GState), _P, _P]),
    "v1g_rollout_fwd": (C.c_int, [_P, C.c_int32, C.c_int32, _P, _P, C.POINTER(V1GState), _P, _P,
                                  C.c_int32, _P]),
    "v1g_rollout_fwd_host": (C.c_int, [_P, C.c_int32, C.c_int32, _P, _P, _P, _P, C.c_int32, _P]),
    "v1g_rollout_fwd_host_pipelined": (C.c_int, [_P, C.c_int32, C.c_int32, _P, _P, _P, C.c_int32, C.c_int32, _P]),
    "v1g_rollout_bwd": (C.c_int, [_P, C.POINTER(V1GLossSpec), _P, _P, _P, _P, _P, _P, _P]),
    "v1g_expadam_update": (C.c_int, [_P, _P, _P, _P, _P, C.c_int64, C.c_float, C.c_float,
                                     C.c_float, C.c_float, C.c_int64, C.c_float, _P]),
    "v1g_balance_slices": (C.c_int, [_P, _P, _P]),
    "v1g_train_layout": (C.c_int, [_P, _P]),
    "v1g_rollout_bwd_internal": (C.c_int, [_P, C.POINTER(V1GLossSpec), _P, _P, _P, _P, _P]),
    "v1g_expadam_update_internal": (C.c_int, [_P, _P, _P, _P, C.c_int32, C.c_float, C.c_float,
                                              C.c_float, C.c_float, C.c_int64, C.c_float, _P]),
    "v1g_weight_regularizer": (C.c_int, [_P, C.c_int32, _P, _P, C.c_int64, C.c_int32, _P, _P, _P, C.c_float,
                                         _P, _P, _P]),
    "v1g_get_internal_order": (C.c_int, [_P, C.c_int, _P]),
    "v1g_internal_weights": (C.c_int, [_P, C.c_int, C.POINTER(_P)]),
    "v1g_get_weights": (C.c_int, [_P, C.c_int, _P, _P]),
    "v1g_get_counters": (C.c_int, [_P, C.POINTER(V1GCounters)]),
    "v1g_synchronize": (C.c_int, [_P, _P]),
    "v1g_selftest_bounded_wait": (C.c_int, [_P, C.c_longlong, _P]),
    "v1g_set_option": (C.c_int, [_P, C.c_char_p, C.c_longlong]),
    "v1g_last_kernel_ms": (C.c_int, [_P, C.c_int, C.POINTER(C.c_float)]),
    "v1g_launch_count": (C.c_longlong, []),
    "v1g_get_phase_times": (C.c_int, [_P, _P, C.c_int32, C.POINTER(C.c_int32)]),
}

_lib = None


def load():
    """Open ``libv1g.so`` and attach the prototypes; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m v1_glif_model_b200.build` "
            "(nvcc, sm_100a). There is no CPU fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export the symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class V1GError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"libv1g error {code}: {msg}")
        self.code = code


def check(handle, rc):
    """Map a status code to the exception the reference would raise (ValueError for bad input)."""
    if rc == OK:
        return
    msg = load().v1g_last_error(handle).decode(errors="replace")
    if rc == EINVAL:
        raise ValueError(msg)
    raise V1GError(rc, msg)
