"""Plain CPU twin of the sampler: the same rule as the kernel, written the slow way.

The reference's rule (src/kernels/sampling.cu:128-210): temperature below 1e-5 is
argmax; else softmax(logits / T), the tokens sorted by probability, the shortest
prefix whose mass reaches top_p kept, and a uniform draw over the kept mass.  Here
the draw walks the kept tokens in index order (the reference walks them in sorted
order with an unseeded generator, so only the distribution is comparable), and
tokens tied with the last kept one are kept too.
"""
import torch


def plain_sample(logits: torch.Tensor, temperature: float, top_p: float, u: float):
    """Returns (token, margin): margin is the distance of the draw from the nearest
    edge of the chosen token's CDF interval, as a fraction of the kept mass."""
    lg = logits.double()
    if temperature < 1e-5:
        m = lg.max()
        return int((lg == m).nonzero()[0]), 1.0
    e = torch.exp((lg - lg.max()) / temperature)
    keep = torch.ones_like(e, dtype=torch.bool)
    if top_p < 1.0:
        srt, _ = torch.sort(e, descending=True)
        cum = torch.cumsum(srt, 0)
        k = int((cum >= top_p * e.sum()).nonzero()[0])
        keep = e >= srt[k]
    kept = torch.where(keep, e, torch.zeros_like(e))
    cdf = torch.cumsum(kept, 0)
    mass = float(cdf[-1])
    goal = u * mass
    idx = int((cdf > goal).nonzero()[0]) if bool((cdf > goal).any()) else int(keep.nonzero()[-1])
    lo = float(cdf[idx] - kept[idx])
    margin = min(goal - lo, float(cdf[idx]) - goal) / mass
    return idx, margin


def plain_repetition_penalty(logits: torch.Tensor, ids, penalty: float) -> torch.Tensor:
    """src/kernels/sampling.cuh:10-29: every DISTINCT id among ``ids`` has its logit divided
    by the penalty when positive and multiplied by it otherwise, once; ids outside the
    vocabulary are skipped; a penalty <= 1 does nothing."""
    out = logits.clone()
    if penalty <= 1.0:
        return out
    for t in set(int(i) for i in ids):
        if 0 <= t < out.numel():
            out[t] = out[t] / penalty if float(out[t]) > 0 else out[t] * penalty   # in the logits' own precision
    return out


def plain_log_prob(logits: torch.Tensor, target: int) -> float:
    """src/kernels/sampling.cu:213-247: (x_t - max) - log(sum exp(x - max)), here in double."""
    lg = logits.double()
    return float(lg[target] - lg.max() - torch.log(torch.exp(lg - lg.max()).sum()))
