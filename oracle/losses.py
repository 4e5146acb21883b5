"""Oracle restatement of the training losses.  TEST INFRASTRUCTURE ONLY.

These are the simplified losses of the benchmark configurations, modelled on the reference's
``VoltageRegularization`` (``v1_model_utils/loss_functions.py:1047-1119``), the population Fano
factor of ``SynchronizationLoss.pop_fano_tf`` (``loss_functions.py:964-981``) and a per-neuron
mean-rate regulariser (``loss_functions.py:873-889``), written with differentiable torch ops so
that autograd supplies the reference gradients.  All are multiplied by ``loss_scale``
(1/replicas, ``multi_training.py:427-429``).
"""
import torch


def rate_loss(z, target, cost, loss_scale=1.0):
    """``cost * mean_n (mean_{b,t} z - target_n)^2`` with target in spikes per step."""
    m = z.mean(dim=(0, 1))
    return cost * loss_scale * torch.mean((m - target) ** 2)


def voltage_loss(v, v_lo, cost, loss_scale=1.0):
    """``cost * mean(relu(v - 1)^2 + relu(v_lo - v)^2)`` in scaled voltage units."""
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
