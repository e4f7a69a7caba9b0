"""Which MSE shrink candidates a group may legitimately pick.

The reference compares per-group error sums that were accumulated in float32 and rounded to the
tensor's dtype.  The order of a float32 sum is not part of the reference's contract (its CPU and
CUDA reductions already differ), so a candidate whose exact error sum lies within the float32
summation error of a rounding midpoint of that dtype may round either way.  ``reachable`` replays
the search for one group under both roundings of every such candidate and returns the set of
(min, max) pairs the search can end with; an implementation is right if its pick is in that set."""
import itertools

import torch

import oracle
from oracle.observers import flatten_weight
from oracle.qparams import calculate_qparams
from oracle.quantize import _round_codes


def _round_to(dtype, v: float, up: bool):
    """The two neighbours of a float64 value in `dtype` (as floats): (nearest, other side)."""
    t = torch.tensor(v, dtype=torch.float64)
    a = t.to(dtype)
    if float(a) == v:
        return float(a), float(a)
    info = torch.finfo(dtype)
    b = torch.nextafter(a.float(), torch.tensor(float("inf") if float(a) < v else float("-inf"))).to(dtype) \
        if dtype == torch.float32 else None
    if b is None:
        # step one unit in the last place of `dtype` towards v
        bits = a.view(torch.int16).item()
        step = 1 if (float(a) < v) == (float(a) >= 0) else -1
        b = torch.tensor(bits + step, dtype=torch.int16).view(dtype)
    return float(a), float(b)


def candidate_errors(weight, spec, maxshrink=0.20, grid=100.0, norm=2.4, expand=1.0):
    """Exact (float64) per-candidate error sums [steps, *qparam_shape] and the candidates' (min, max)."""
    args = spec
    if args.strategy == "tensor_group" and args.scale_dtype is not None:
        args = args.model_copy(update={"scale_dtype": None})
    obs = flatten_weight(weight, args)
    mn = torch.amin(obs, dim=(0, -1)) * expand
    mx = torch.amax(obs, dim=(0, -1)) * expand
    errs, mns, mxs = [], [], []
    for i in range(int(maxshrink * grid)):
        p = 1 - i / grid
        smn, smx = mn * p, mx * p
        scale, zp = calculate_qparams(smn, smx, args, global_scale=None)
        s, z = scale.unsqueeze(-1), zp.unsqueeze(-1)
        v = obs / s + z.to(obs.dtype)
        q = _round_codes(v, args)
        fq = ((q.to(s.dtype) - z.to(s.dtype)) * s).to(obs.dtype)
        terms = (fq - obs).abs().pow(norm)
        errs.append(terms.double().sum(dim=(0, -1)))
        mns.append(smn)
        mxs.append(smx)
    return torch.stack(errs), torch.stack(mns), torch.stack(mxs), obs.shape[-1] * obs.shape[0]


def reachable(E, dtype, n_terms, patience_stop=None):
    """Indices of the candidates the search may end on for ONE group: E [steps] exact sums."""
    # error bound of a float32 sum of positive terms in any reasonable order (blocked / pairwise
    # sums grow with the block length, not with the term count)
    delta = min(n_terms, 256) * 2.0 ** -24
    options = []
    for e in E.tolist():
        near, other = _round_to(dtype, e, True)
        # the midpoint between the two neighbours
        mid = (near + other) / 2.0
        amb = near != other and abs(e - mid) <= delta * abs(e)
        options.append((near, other) if amb else (near,))
    amb_idx = [i for i, o in enumerate(options) if len(o) == 2]
    if len(amb_idx) > 14:
        raise AssertionError(f"{len(amb_idx)} ambiguous candidates in one group")
    picks = set()
    for choice in itertools.product(*[range(2) for _ in amb_idx]):
        vals = [o[0] for o in options]
        for k, i in zip(choice, amb_idx):
            vals[i] = options[i][k]
        best, best_i = float(torch.finfo(dtype).max), None
        for i, v in enumerate(vals):
            if patience_stop is not None and i >= patience_stop:
                break
            if v < best:
                best, best_i = v, i
        picks.add(best_i)
    return picks
