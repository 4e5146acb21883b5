"""Oracle restatement of the training losses.  TEST INFRASTRUCTURE ONLY.

These are the simplified losses of the benchmark configurations, modelled on the reference's
``VoltageRegularization`` (``v1_model_utils/loss_functions.py:1047-1119``), the population Fano
factor of ``SynchronizationLoss.pop_fano_tf`` (``loss_functions.py:964-981``) and a per-neuron
mean-rate regulariser (``loss_functions.py:873-889``), written with differentiable torch ops so
that autograd supplies the reference gradients.  All are multiplied by ``loss_scale``
(1/replicas, ``multi_training.py:427-429``).  ``rate_distribution_loss`` is the reference's own
firing-rate target in full; it is pinned against the reference's code by
``tests/golden/reference_rate_loss.npz``.
"""
import torch


def rate_loss(z, target, cost, loss_scale=1.0):
    """``cost * mean_n (mean_{b,t} z - target_n)^2`` with target in spikes per step."""
    m = z.mean(dim=(0, 1))
    return cost * loss_scale * torch.mean((m - target) ** 2)


def voltage_loss(v, v_lo, cost, loss_scale=1.0, mode="range"):
    """``cost * mean(relu(v - 1)^2 + relu(v_lo - v)^2)`` in scaled voltage units; with ``v_lo = 0``
    this is the reference's "range" penalty ``relu(|v - .5| - .5)^2`` and ``mode="threshold"`` is its
    ``(v - 1)^2`` (``VoltageRegularization``, ``loss_functions.py:1087-1119``)."""
    if mode == "threshold":
        pen = (v - 1.0) ** 2
    else:
        pen = torch.relu(v - 1.0) ** 2 + torch.relu(v_lo - v) ** 2
    return cost * loss_scale * pen.mean()


def sync_loss(z, bin_steps, cost, fano_target=1.0, loss_scale=1.0):
    """``cost * (mean_b Fano_b - target)^2``; Fano of the population count in ``bin_steps`` bins.

    Bins that do not fit are dropped (conv1d with stride = bin, padding VALID in the reference);
    variance is the biased one (``tf.math.reduce_variance``); the mean is floored at 1e-7.
    """
    b, t, _ = z.shape
    nbins = t // bin_steps
    if nbins < 1:
        return z.sum() * 0.0
    pop = z.sum(dim=2)[:, :nbins * bin_steps].reshape(b, nbins, bin_steps).sum(dim=2)
    mean = pop.mean(dim=1)
    var = ((pop - mean[:, None]) ** 2).mean(dim=1)
    fano = var / torch.clamp(mean, min=1e-7)
    return cost * loss_scale * (fano.mean() - fano_target) ** 2


def huber_quantile(u, tau, kappa):
    """Quantile-Huber penalty (``loss_functions.py:626-633``): ``|tau - [u <= 0]|`` times
    ``u^2 / (2 kappa)`` inside ``|u| <= kappa`` and ``|u| - kappa/2`` outside."""
    abs_u = u.abs()
    num = (tau - (u <= 0).to(u.dtype)).abs()
    return torch.where(abs_u <= kappa, num / (2 * kappa) * u ** 2, num * (abs_u - 0.5 * kappa))


def rate_distribution_loss(z, groups, cost, kappa=0.002, pre_delay=0, post_delay=0, loss_scale=1.0):
    """The reference's firing-rate target (``SpikeRateDistributionTarget.__call__``,
    ``loss_functions.py:873-889``, with ``compute_spike_rate_target_loss`` /
    ``compute_spike_rate_distribution_loss``, ``:635-681``).

    ``rates`` = mean of the spikes over batch and the steps ``[pre_delay, T - post_delay)``
    (``spike_trimming``, ``:604-611``).  For every population ``(neuron_ids, sorted_targets)`` the
    rates of its neurons are sorted and compared, rank by rank, with the sorted target sample:
    ``u_i = sorted_rate_i - target_i``, ``tau_i = (i + 1) / n``, penalty ``huber_quantile``; the
    penalties of all populations are summed and divided by the number of neurons covered.

    The reference shuffles a population's rates before sorting, so which of several neurons with
    EQUAL rates gets which rank is random there; here the sort is stable, i.e. equal rates keep
    the order of ``neuron_ids``.  The loss value does not depend on that choice, the gradient of
    tied neurons does.
    """
    t = z.shape[1]
    zt = z[:, pre_delay:t - post_delay if post_delay else t, :]
    rates = zt.mean(dim=(0, 1))
    total = z.sum() * 0.0
    count = 0
    for neuron_ids, targets in groups:
        if len(neuron_ids) == 0:
            continue
        ids = torch.as_tensor(neuron_ids, dtype=torch.long)
        tg = torch.as_tensor(targets, dtype=rates.dtype)
        srt = torch.sort(rates[ids], stable=True).values
        n = ids.numel()
        tau = (torch.arange(n, dtype=rates.dtype) + 1) / n
        total = total + huber_quantile(srt - tg, tau, kappa).sum()
        count += n
    return cost * loss_scale * total / max(count, 1)


def population_fano_loss(pop, bin_sizes, target_fanos, cost, eps=1e-7):
    """``cost * mean_k (target_k - Fano_k)^2`` for population counts ``pop[sample, step]``
    (``pop_fano_tf`` and the mean squared error of ``__call__``, ``loss_functions.py:964-981,
    1031-1044``): for every bin size smaller than half the window the counts are summed in
    non-overlapping bins (incomplete last bin dropped), Fano = biased variance / max(mean, eps)
    per sample, averaged over the samples."""
    w = pop.shape[1]
    terms = []
    for bs, tg in zip(bin_sizes, target_fanos):
        bs = int(bs)
        if not bs < w // 2:
            continue
        nb = w // bs
        c = pop[:, :nb * bs].reshape(pop.shape[0], nb, bs).sum(dim=2)
        mean = c.mean(dim=1)
        var = ((c - mean[:, None]) ** 2).mean(dim=1)
        fano = (var / torch.clamp(mean, min=eps)).mean()
        terms.append((float(tg) - fano) ** 2)
    if not terms:
        return pop.sum() * 0.0
    return cost * torch.stack(terms).mean()


def synchronization_loss(z, samples, bin_sizes, target_fanos, cost, t_start=0, t_end=None,
                         loss_scale=1.0, eps=1e-7):
    """The reference's synchrony target in full (``SynchronizationLoss.__call__``,
    ``loss_functions.py:983-1044``) for given samples.

    ``samples`` = list of ``(trial, neuron_ids)``: the population spike count of the neurons in
    trial (batch row) ``trial`` over the steps ``[t_start, t_end)`` enters ``population_fano_loss``.
    The reference draws trial, sample size and members at random in every call; here they are an
    input.
    """
    t_end = z.shape[1] if t_end is None else t_end
    zt = z[:, t_start:t_end, :]
    pop = torch.stack([zt[tr][:, torch.as_tensor(ids, dtype=torch.long)].sum(dim=1) for tr, ids in samples])
    return loss_scale * population_fano_loss(pop, bin_sizes, target_fanos, cost, eps)


def orientation_selectivity_loss(z, angle, tuning_angle, type_ids, osi_targets, dsi_targets, type_counts,
                                 cost, pre_delay=0, post_delay=0, normalizer=None, loss_scale=1.0,
                                 min_rate=0.0005):
    """The reference's population OSI/DSI target (``OrientationSelectivityLoss`` with
    ``method="crowd_osi"``: ``__call__``, ``crowd_osi_loss`` and ``_compute_osi_dsi_core``,
    ``loss_functions.py:1340-1440``).

    ``rates[b, n]`` = mean of the spikes over the steps ``[pre_delay, T - post_delay)``, optionally
    divided by ``max(normalizer[n], min_rate)``; ``delta[b, n] = (angle[b] - tuning_angle[n]) pi/180``.
    Per trial and cell type: ``den = max(mean_n rates, min_rate)``, ``osi = mean_n(rates cos 2 delta) /
    den``, ``dsi = mean_n(rates cos delta) / den`` (means over the neurons whose ``type_ids`` equal
    the type); both are averaged over the trials and the loss is
    ``cost * sum_type count_type ((osi - osi_target)^2 + (dsi - dsi_target)^2) / sum_type count_type``.
    """
    t = z.shape[1]
    zt = z[:, pre_delay:t - post_delay if post_delay else t, :]
    rates = zt.mean(dim=1)
    dt = rates.dtype
    if normalizer is not None:
        rates = rates / torch.clamp(torch.as_tensor(normalizer, dtype=dt), min=min_rate)
    delta = (torch.as_tensor(angle, dtype=dt)[:, None] - torch.as_tensor(tuning_angle, dtype=dt)[None, :]) \
        * (torch.pi / 180.0)
    ids = torch.as_tensor(type_ids, dtype=torch.long)
    n_types = len(osi_targets)
    onehot = torch.nn.functional.one_hot(ids, n_types).to(dt)            # [N, types]
    n_per = torch.clamp(onehot.sum(dim=0), min=1.0)

    def seg_mean(x):
        return (x @ onehot) / n_per                                      # [B, types]

    den = torch.clamp(seg_mean(rates), min=min_rate)
    osi = (seg_mean(rates * torch.cos(2.0 * delta)) / den).mean(dim=0)
    dsi = (seg_mean(rates * torch.cos(delta)) / den).mean(dim=0)
    cnt = torch.as_tensor(type_counts, dtype=dt)
    per_type = (osi - torch.as_tensor(osi_targets, dtype=dt)) ** 2 + (dsi - torch.as_tensor(dsi_targets, dtype=dt)) ** 2
    return cost * loss_scale * (per_type * cnt).sum() / cnt.sum()


def regularizer_groups(edge_type_ids):
    """``(idx, n_groups, order, row_splits)``: dense group index per synapse (``np.unique(...,
    return_inverse=True)``), and the synapse positions grouped by it with the original order kept
    inside a group (``_build_group_order_numba``, ``loss_functions.py:20-61``)."""
    import numpy as np
    _, idx = np.unique(np.asarray(edge_type_ids), return_inverse=True)
    n_groups = int(idx.max()) + 1 if idx.size else 0
    order = np.argsort(idx, kind="stable")
    row_splits = np.concatenate([[0], np.cumsum(np.bincount(idx, minlength=n_groups))])
    return idx.astype(np.int64), n_groups, order.astype(np.int64), row_splits.astype(np.int64)


def mean_stiff_regularizer(w, idx, n_groups, initial_weights, strength, relative=False):
    """``MeanStiffRegularizer`` (``loss_functions.py:171-220``): the mean weight per edge type against
    the mean of the initial weights; ``relative`` = ``penalize_relative_change`` (deviation divided by
    ``max(|initial mean|, 1e-4)``, root of the mean square)."""
    idx_t = torch.as_tensor(idx, dtype=torch.int64)
    w0 = torch.as_tensor(initial_weights, dtype=w.dtype)
    cnt = torch.zeros(n_groups, dtype=w.dtype).index_add(0, idx_t, torch.ones_like(w0))
    target = torch.zeros(n_groups, dtype=w.dtype).index_add(0, idx_t, w0) / cnt
    mean = torch.zeros(n_groups, dtype=w.dtype).index_add(0, idx_t, w) / torch.clamp(cnt, min=1.0)
    if relative:
        denom = torch.clamp(target.abs(), min=1e-4)
        return strength * torch.sqrt(torch.mean(((mean - target) / denom) ** 2))
    return strength * torch.mean((mean - target) ** 2)


def emd_regularizer(w, order, row_splits, initial_weights, strength):
    """``EarthMoversDistanceRegularizer`` (``loss_functions.py:536-601``): per edge type the mean
    absolute difference between the sorted current and the sorted initial weights, averaged over the
    types."""
    w0 = torch.as_tensor(initial_weights, dtype=w.dtype)
    order_t = torch.as_tensor(order, dtype=torch.int64)
    terms = []
    for g in range(len(row_splits) - 1):
        sel = order_t[int(row_splits[g]):int(row_splits[g + 1])]
        terms.append((torch.sort(w[sel]).values - torch.sort(w0[sel]).values).abs().mean())
    return strength * torch.stack(terms).mean()
