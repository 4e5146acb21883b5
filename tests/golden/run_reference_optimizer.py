"""Golden vectors for the Exp-Adam update from the reference's OWN optimizer code (run from the repo
root, in a container that has the reference tree):

    python tests/golden/run_reference_optimizer.py /path/to/V1_GLIF_model

Imports ``v1_model_utils/optimizers.py`` unmodified over ``tf_standin`` (whose ``Optimizer`` base
supplies slot variables, the iteration counter and the variable index that the Keras base class
would), builds ``ExponentiatedAdam(learning_rate, epsilon=1e-11)`` as ``create_optimizer`` does
(``optimizers.py:44-46``), and applies four dense ``update_step`` calls
(``optimizers.py:267-289, 353-376``) to a float32 weight vector with positive, negative and zero
entries, each followed by the ``SignedConstraint`` of ``v1_model_utils/models.py:419-427`` (Keras
applies a variable's constraint after the optimizer step).  Writes
``tests/golden/reference_expadam.npz``: initial weights, the gradients, and weights and both moments
after every step.  ``tests/test_oracle_pinning.py`` checks ``oracle/expadam.py`` against it.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

import tf_standin  # noqa: E402

LR, N, STEPS = 5e-3, 4096, 4


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("V1_GLIF_REFERENCE", "V1_GLIF_model")
    tf = tf_standin.install()
    tf_standin.set_policy_dtype(torch.float32)

    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, os.path.join(ref_root, rel))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[spec.name] = mod
        spec.loader.exec_module(mod)
        return mod
    opt_mod = load("reference_optimizers", os.path.join("v1_model_utils", "optimizers.py"))
    import tempfile
    os.environ.setdefault("NUMBA_CACHE_DIR", tempfile.mkdtemp(prefix="numba_cache_"))
    models = load("reference_models", os.path.join("v1_model_utils", "models.py"))

    rng = np.random.Generator(np.random.PCG64(11))
    w0 = (rng.lognormal(0.0, 1.0, N) * np.where(rng.random(N) < 0.8, 1.0, -1.0)).astype(np.float32)
    w0[:64] = 0.0                                  # zero weights: sign(0) = +1 keeps them at zero
    positive = w0 >= 0
    grads = (rng.normal(0.0, 1.0, (STEPS, N)) * rng.lognormal(-4.0, 2.0, (STEPS, N))).astype(np.float32)
    grads[1, 100:200] = 0.0
    var = tf.Variable(w0, trainable=True, dtype=torch.float32)
    constraint = models.SignedConstraint(torch.from_numpy(positive))
    opt = opt_mod.ExponentiatedAdam(learning_rate=LR, epsilon=1e-11)
    opt.build([var])
    ws, ms, vs = [], [], []
    for k in range(STEPS):
        with torch.no_grad():
            opt.update_step(torch.from_numpy(grads[k]), var)
            var.assign(constraint(var))
        opt.iterations += 1                        # apply_gradients increments after the updates
        slot = opt._index_dict[opt._var_key(var)]
        ws.append(var.detach().numpy().copy())
        ms.append(opt._momentums[slot].detach().numpy().copy())
        vs.append(opt._velocities[slot].detach().numpy().copy())
    out = os.path.join(HERE, "reference_expadam.npz")
    np.savez_compressed(out, w0=w0, positive=positive, grads=grads, lr=LR, beta_1=opt.beta_1,
                        beta_2=opt.beta_2, epsilon=opt.epsilon, w=np.stack(ws), m=np.stack(ms), v=np.stack(vs))
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
