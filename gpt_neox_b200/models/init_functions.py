"""Weight-initialisation schemes selectable by ``init_method`` / ``output_layer_init_method``
(the nine of megatron/model/init_functions.py:187-225). Each factory returns ``init_(tensor)``."""
from __future__ import annotations

import math

import torch


def _scaled(fn, scale):
    def init_(t):
        fn(t)
        if scale != 1.0:
            with torch.no_grad():
                t.mul_(scale)
        return t
    return init_


def normal(sigma):
    return lambda t: torch.nn.init.normal_(t, mean=0.0, std=sigma)


def scaled_normal(sigma, num_layers, residuals_per_layer=2):
    """N(0, sigma / sqrt(residuals_per_layer * num_layers)): for matrices that write into the
    residual stream."""
    std = sigma / math.sqrt(residuals_per_layer * num_layers)
    return lambda t: torch.nn.init.normal_(t, mean=0.0, std=std)


def orthogonal(n_layers=1):
    gain = math.sqrt(2 / n_layers)

    def init_(t):
        if t.dim() < 2:
            raise ValueError("Only tensors with 2 or more dimensions are supported")
        with torch.no_grad():
            rows, cols = t.shape[0], t.numel() // t.shape[0]
            flat = torch.empty(rows, cols, dtype=torch.float32, device=t.device).normal_(0, 1)
            if rows < cols:
                flat = flat.t()
            q, r = torch.linalg.qr(flat)
            q = q * torch.diagonal(r).sign()
            if rows < cols:
                q = q.t()
            t.copy_(q.reshape(t.shape).to(t.dtype)).mul_(gain)
        return t
    return init_


def xavier_uniform():
    return lambda t: torch.nn.init.xavier_uniform_(t)


def xavier_normal():
    return lambda t: torch.nn.init.xavier_normal_(t)


def small_init(dim):
    """sqrt(2 / (5 d)) (Nguyen & Salazar 2019)."""
    std = math.sqrt(2 / (5 * dim))
    return lambda t: torch.nn.init.normal_(t, mean=0.0, std=std)


def wang_init(n_layers, dim):
    std = 2 / n_layers / math.sqrt(dim)
    return lambda t: torch.nn.init.normal_(t, mean=0.0, std=std)


def get_init_methods(args):
    """(init_method, output_layer_init_method) as callables; muP multiplies by ``mup_init_scale``."""
    def _get(name):
        if name == "normal":
            fn = normal(args.init_method_std)
        elif name == "scaled_normal":
            fn = scaled_normal(args.init_method_std, args.num_layers)
        elif name == "orthogonal":
            fn = orthogonal()
        elif name == "scaled_orthogonal":
            fn = orthogonal(args.num_layers)
        elif name == "xavier_uniform":
            fn = xavier_uniform()
        elif name == "xavier_normal":
            fn = xavier_normal()
        elif name == "wang_init":
            fn = wang_init(args.num_layers, args.hidden_size)
        elif name == "small_init":
            fn = small_init(args.hidden_size)
        elif name == "single_residual_scaled_normal":
            fn = scaled_normal(args.init_method_std, args.num_layers, residuals_per_layer=1)
        else:
            raise NotImplementedError(f"Unknown init method {name}")
        if getattr(args, "use_mup", False):
            if name in ("orthogonal", "scaled_orthogonal"):
                raise ValueError("Orthogonal init is not defined under muP; use a different init method")
            fn = _scaled(fn, args.mup_init_scale)
        return fn
    return _get(args.init_method), _get(args.output_layer_init_method)


# ------------------------------------------------------------------ the reference's factory names
def _named(factory):
    """``factory(..., use_mup_outer=False, mup_init_scale=1.0)`` -> ``init_(tensor, use_mup=use_mup_outer)``:
    the calling convention of megatron/model/init_functions.py:25-185."""
    def make(*args, use_mup_outer=False, mup_init_scale=1.0, **kwargs):
        plain = factory(*args, **kwargs)
        scaled = _scaled(plain, mup_init_scale)

        def init_(tensor, use_mup=use_mup_outer):
            return scaled(tensor) if use_mup else plain(tensor)
        return init_
    return make


init_method_normal = _named(normal)
scaled_init_method_normal = _named(lambda sigma, num_layers, num_residuals_per_layer=2:
                                   scaled_normal(sigma, num_layers, num_residuals_per_layer))
orthogonal_init_method = _named(orthogonal)
xavier_uniform_init_method = _named(xavier_uniform)
xavier_normal_init_method = _named(xavier_normal)
small_init_init_method = _named(small_init)
wang_init_method = _named(wang_init)
