"""Block-sparse attention patterns: ``local``, ``sparse_fixed``, ``sparse_variable``, ``bigbird``,
``bslongformer`` (the layouts the reference obtains from DeepSpeed's sparsity configs,
megatron/model/utils.py:261-361, driven by the ``sparsity_config`` dict).

A pattern is a boolean block layout ``[blocks, blocks]`` (True = the query block attends to the key block),
always intersected with causality (``attention="unidirectional"`` in every reference call).  It is expanded
to a token mask once and applied by the scaled-masked-softmax attention path, i.e. the *function* of the
sparse layers is reproduced; the FLOP savings of a block-sparse kernel are not (no Triton here, and a
tcgen05 block-sparse kernel is future work).
"""
from __future__ import annotations

import torch


def _window_ranges(nb, sizes):
    """Consecutive windows of the given block counts; the last size repeats."""
    out, start, i = [], 0, 0
    while start < nb:
        n = sizes[min(i, len(sizes) - 1)]
        out.append((start, min(start + n, nb)))
        start += n
        i += 1
    return out


def block_layout(attention_type: str, num_blocks: int, cfg: dict, seed: int = 0) -> torch.Tensor:
    """-> bool [num_blocks, num_blocks] (before causality)."""
    nb = num_blocks
    L = torch.zeros(nb, nb, dtype=torch.bool)
    r = torch.arange(nb)[:, None]
    c = torch.arange(nb)[None, :]
    if attention_type == "local":
        w = cfg.get("num_local_blocks", cfg.get("num_sliding_window_blocks", 4))
        L |= (c <= r) & (c >= r - w // 2)
    elif attention_type == "sparse_fixed":
        nl, ng = cfg.get("num_local_blocks", 4), cfg.get("num_global_blocks", 1)
        assert nl % ng == 0, "num_local_blocks must be divisible by num_global_blocks"
        for a, b in _window_ranges(nb, [nl]):
            L[a:b, a:b] = True                               # dense inside a local window
        first = nl - ng                                      # the last blocks of every window are global
        for a, _b in _window_ranges(nb, [nl]):
            g0, g1 = a + first, min(a + first + ng, nb)
            if g0 < nb:
                L[g0:, g0:g1] = True                         # later rows see the window's summary blocks
    elif attention_type == "sparse_variable":
        for a, b in _window_ranges(nb, list(cfg.get("local_window_blocks", [4]))):
            L[a:b, a:b] = True
        starts = list(cfg.get("global_block_indices", [0]))
        ends = cfg.get("global_block_end_indices", None)
        for i, g in enumerate(starts):
            e = (ends[i] if ends is not None else g + 1)
            if g < nb:
                L[:, g:min(e, nb)] = True
        _random_blocks(L, cfg.get("num_random_blocks", 0), seed)
    elif attention_type == "bigbird":
        w = cfg.get("num_sliding_window_blocks", 3)
        L |= (c - r).abs() <= w // 2
        g = cfg.get("num_global_blocks", 1)
        L[:g, :] = True
        L[:, :g] = True
        _random_blocks(L, cfg.get("num_random_blocks", 1), seed)
    elif attention_type == "bslongformer":
        w = cfg.get("num_sliding_window_blocks", 3)
        L |= (c - r).abs() <= w // 2
        starts = list(cfg.get("global_block_indices", [0]))
        ends = cfg.get("global_block_end_indices", None)
        for i, g in enumerate(starts):
            e = (ends[i] if ends is not None else g + 1)
            if g < nb:
                L[:, g:min(e, nb)] = True
                L[g:min(e, nb), :] = True
    else:
        raise ValueError(f"Attention type {attention_type} not recognized")
    return L


def _random_blocks(L, n, seed):
    if n <= 0:
        return
    g = torch.Generator().manual_seed(seed)
    nb = L.shape[0]
    for row in range(nb):
        hi = row + 1                                          # unidirectional: only earlier blocks
        picks = torch.randperm(hi, generator=g)[:n]
        L[row, picks] = True


def token_mask(attention_type: str, seq_len: int, cfg: dict, seed: int = 0) -> torch.Tensor:
    """-> bool [1, 1, seq, seq], True = masked out (the convention of the masked-softmax kernels)."""
    cfg = cfg or {}
    if cfg.get("different_layout_per_head", False):
        raise NotImplementedError("sparsity_config.different_layout_per_head is not supported")
    block = cfg.get("block", 16)
    nb = (seq_len + block - 1) // block
    lay = block_layout(attention_type, nb, cfg, seed)
    allowed = lay.repeat_interleave(block, 0).repeat_interleave(block, 1)[:seq_len, :seq_len]
    allowed &= torch.tril(torch.ones(seq_len, seq_len, dtype=torch.bool))
    return (~allowed)[None, None]
