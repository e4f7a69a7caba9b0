import torch

from llm_compressor_b200.quant_args import QuantizationArgs


def args_from(d) -> QuantizationArgs:
    keys = ("num_bits", "type", "symmetric", "strategy", "group_size", "block_structure",
            "scale_dtype", "zp_dtype", "actorder", "observer", "observer_kwargs")
    kw = {k: d[k] for k in keys if k in d and d[k] is not None}
    return QuantizationArgs(**kw)


def bits_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    a, b = a.detach().cpu(), b.detach().cpu()
    if a.dtype != b.dtype or a.shape != b.shape:
        return False
    if a.dtype == torch.float8_e4m3fn:
        return torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    if a.is_floating_point():
        it = {2: torch.int16, 4: torch.int32}[a.element_size()]
        return torch.equal(a.contiguous().view(it), b.contiguous().view(it))
    return torch.equal(a, b)


def mismatch(a: torch.Tensor, b: torch.Tensor) -> float:
    """fraction of elements whose bit patterns differ"""
    a, b = a.detach().cpu(), b.detach().cpu()
    assert a.shape == b.shape and a.dtype == b.dtype, (a.shape, b.shape, a.dtype, b.dtype)
    if a.dtype == torch.float8_e4m3fn:
        a, b = a.view(torch.uint8), b.view(torch.uint8)
    elif a.is_floating_point():
        it = {2: torch.int16, 4: torch.int32}[a.element_size()]
        a, b = a.contiguous().view(it), b.contiguous().view(it)
    return float((a != b).float().mean())


def synth_weight(N, K, seed, dtype=torch.bfloat16, outliers=True):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g) * 0.02
    if outliers:
        n_out = max(1, (N * K) // 1000)
        idx = torch.randperm(N * K, generator=g)[:n_out]
        w.view(-1)[idx] = torch.randn(n_out, generator=g) * 0.5
    w[0, : min(128, K)] = 0.0
    if K > 9:
        w[1, 3] = 0.0
        w[1, 5] = -0.0
        w[2, 7] = -1e-6
        w[2, 9] = 1e-6
    return w.to(dtype)


def synth_acts(B, S, K, seed, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, S, K, generator=g)
    x = x * (0.25 + 2.0 * torch.rand(K, generator=g))
    return x.to(dtype)
