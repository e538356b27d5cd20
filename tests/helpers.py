"""Shared helpers of the GPU parity tests: the same seeded tensors go to the CUDA library (through
the C ABI) and to the CPU oracle."""
import numpy as np
import torch

from oracle import oracle as orc


from oracle.from_synth import oracle_layer, rel_l2, to_np_weight  # noqa: F401,E402


def routing_agreement(gpu_idx, ref_idx, ref_logits, top_k, what, min_same):
    """Tokens whose top-k set differs from the f64 oracle's are allowed only where the oracle itself is
    on a knife edge: the gap between its k-th and (k+1)-th logit must be within the rounding of the
    logits.  Prints the count and the margins, asserts the share and the margins, returns the mask of
    agreeing tokens."""
    same = (np.asarray(gpu_idx) == np.asarray(ref_idx)).all(axis=1)
    n_diff = int((~same).sum())
    if n_diff:
        lg = np.sort(np.asarray(ref_logits, dtype=np.float64)[~same], axis=1)[:, ::-1]
        margins = lg[:, top_k - 1] - lg[:, top_k]
        print(f"{what}: top-k set differs from the oracle on {n_diff} of {len(same)} tokens; "
              f"oracle logit margin k-th vs (k+1)-th: max {margins.max():.3e}, median {np.median(margins):.3e}")
        # a token may flip only when its deciding logits are closer than the logit error bound
        assert margins.max() <= 1e-5, f"{what}: a token with a clear margin ({margins.max():.3e}) was routed differently"
    else:
        print(f"{what}: top-k sets identical to the oracle on all {len(same)} tokens")
    assert same.mean() >= min_same, f"{what}: top-k sets differ from the oracle on {n_diff} of {len(same)} tokens"
    return same


def reference_metrics(a, b):
    """The reference's own four numbers (src/moe/numerical.rs:30-90)."""
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    diff = np.abs(a - b)
    return {"max_abs_diff": float(diff.max()), "mean_abs_diff": float(diff.mean()),
            "rmse": float(np.sqrt((diff ** 2).mean())), "argmax_match": bool(a.argmax() == b.argmax())}
