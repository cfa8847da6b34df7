"""Shared helpers of the GPU engine tests."""
import numpy as np
import torch


def teacher_forced_gaps(mc, src, prompt, out):
    """For every generated token: (oracle max logit - oracle logit of that token) / logit std, with
    the oracle fed the engine's own tokens. 0 = the oracle agrees; small = a near tie."""
    from oxide_tech_llm_engine_b200.models.reference import ReferenceModel

    ref = ReferenceModel(mc, src)
    logits = ref.forward(list(prompt) + list(out[:-1]), all_logits=True)[len(prompt) - 1:]
    gaps = []
    for i, t in enumerate(out):
        row = logits[i]
        gaps.append(float((row.max() - row[t]) / row.std()))
    return gaps


def assert_consistent(mc, src, prompts, outs, tol=0.3, min_exact=0.6):
    all_gaps = []
    for p, o in zip(prompts, outs):
        all_gaps += teacher_forced_gaps(mc, src, p, o)
    g = np.asarray(all_gaps)
    assert g.max() < tol, f"a generated token is far from the oracle's choice: max gap {g.max():.3f}"
    assert (g == 0).mean() >= min_exact, f"only {(g == 0).mean():.2f} of tokens are the oracle's argmax"
