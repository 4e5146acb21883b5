"""Oracle of the Exponentiated-Adam dense update.  TEST INFRASTRUCTURE ONLY.

Follows ``ExponentiatedAdam.update_step``, dense branch
(``v1_model_utils/optimizers.py:267-289, 353-376``) and ``SignedConstraint``
(``v1_model_utils/models.py:419-427``) with torch CPU ops in fp32.
"""
import torch


def expadam_step(w, g, m, v, positive, lr, beta_1, beta_2, eps, step):
    dt = w.dtype
    local_step = torch.tensor(float(step), dtype=dt)
    b1 = torch.tensor(beta_1, dtype=dt)
    b2 = torch.tensor(beta_2, dtype=dt)
    alpha = torch.tensor(lr, dtype=dt) * torch.sqrt(1 - torch.pow(b2, local_step)) / (
        1 - torch.pow(b1, local_step))
    m = m + (g - m) * (1 - b1)
    v = v + (torch.square(g) - v) * (1 - b2)
    adam_grad = m / (torch.sqrt(v) + eps)
    sign_w = torch.sign(w)
    sign_w = torch.where(sign_w == 0, torch.ones_like(sign_w), sign_w)
    w = w * torch.exp(-alpha * adam_grad * sign_w)
    w = torch.where(positive, torch.relu(w), -torch.relu(-w))
    return w, m, v
