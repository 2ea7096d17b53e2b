"""Checks a continuous-integration run switches on with ``--ci-test``.

* ``check_mtp_only_grad``: with draft-head training, a step's gradients must be non-zero for draft parameters and exactly
  zero for every policy parameter when the policy loss itself contributes nothing (the first step of a run whose
  advantages are all zero), i.e. the draft loss must not leak into the policy.
* ``check_mtp_loss``: the draft loss of a pretrained draft head stays below a bound.
Same role as slime/backends/megatron_utils/ci_utils.py:11-84 in the reference.
"""

from __future__ import annotations


def check_mtp_only_grad(model, step_id: int = 0) -> None:
    leaked, trained = [], []
    for name, p in model.named_parameters():
        g = getattr(p, "main_grad", None)
        if g is None:
            continue
        nonzero = bool(g.float().abs().sum() > 0)
        if name.startswith("mtp.") or ".mtp." in name:
            if nonzero:
                trained.append(name)
        elif nonzero:
            leaked.append(name)
    assert not leaked, f"step {step_id}: policy parameters received gradients although only the draft loss is active: {leaked[:5]}"
    assert trained, f"step {step_id}: no draft-head parameter received a gradient"


def check_mtp_loss(mtp_loss: float, max_mtp_loss: float = 1.0) -> None:
    assert mtp_loss < max_mtp_loss, f"draft-head loss {mtp_loss:.4f} is not below {max_mtp_loss}: the head was not loaded or is diverging"
