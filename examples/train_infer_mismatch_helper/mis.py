"""Entry point kept at the path launch scripts name
(``--custom-tis-function-path examples.train_infer_mismatch_helper.mis.compute_mis_weights_with_cp``);
the implementation is ``slime_b200.utils.mis``."""

from slime_b200.utils.mis import compute_mis_weights, compute_mis_weights_with_cp, mismatch_metrics  # noqa: F401
