"""Block-sparse 3-D attention for video DiTs: sliding tile attention (STA) and its selective extension (SSTA).

The latent canvas ``(t, h, w)`` is cut into tiles of ``tile_thw`` tokens; tokens are re-ordered so that a tile is a contiguous
block, and attention is computed between blocks only where a block mask allows it:

* STA   -- every query tile sees the key tiles inside a ``kernel_thw`` window around it (the window is shifted inwards at
  the borders so that every tile sees the same number of neighbours),
* SSTA  -- STA plus, per query tile, the ``topk`` key tiles whose mean key is most similar to the tile's mean query,
* text  -- trailing text blocks are visible to everyone and see everything.

Reference: mindspeed_mm/models/predictor/dits/hunyuanvideo15/ssta_attention.py (``tile`` :28, ``similarity_sampling`` :132,
``create_sta_3d_mask_optimize`` :335, ``create_ssta_3d_mask`` :418, ``ssta_3d_attention`` :500), where the masked product
itself is a vendor block-sparse kernel.  Here the selected key blocks of every query block are gathered and the
result is one packed variable-length attention call (query length = one block, key length = its selected blocks), so
the dense flash-attention kernel does the work and cost scales with the number of selected blocks.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


def _ceil_to(n: int, m: int) -> int:
    return (n + m - 1) // m * m


def tile_order(canvas: Sequence[int], tile: Sequence[int], device=None) -> torch.Tensor:
    """Permutation ``perm`` with ``x_tiled = x[perm]``: row-major canvas order -> tile-major order (tiles row-major, tokens
    inside a tile row-major).  ``canvas`` must be a multiple of ``tile`` on every axis."""
    t, h, w = canvas
    a, b, c = tile
    idx = torch.arange(t * h * w, device=device).view(t // a, a, h // b, b, w // c, c)
    return idx.permute(0, 2, 4, 1, 3, 5).reshape(-1)


def pad_canvas(x: torch.Tensor, canvas: Sequence[int], tile: Sequence[int], mode: str = "zero"):
    """x [B, t*h*w, ...] -> padded to tile multiples on every axis (zeros or a repeat of the last slice)."""
    t, h, w = canvas
    T, H, W = (_ceil_to(n, m) for n, m in zip(canvas, tile))
    if (T, H, W) == (t, h, w):
        return x, (t, h, w)
    B = x.shape[0]
    rest = x.shape[2:]
    g = x.view(B, t, h, w, *rest)
    for axis, (cur, want) in enumerate(zip((t, h, w), (T, H, W)), start=1):
        if want > cur:
            edge = g.narrow(axis, cur - 1, 1).expand(*[-1 if i != axis else want - cur for i in range(g.dim())])
            g = torch.cat([g, torch.zeros_like(edge) if mode == "zero" else edge], axis)
    return g.reshape(B, T * H * W, *rest), (T, H, W)


def sta_block_mask(tiles: Sequence[int], kernel: Sequence[int], device=None) -> torch.Tensor:
    """[n_tiles, n_tiles] bool: key tile j lies in the (border-clamped) window of query tile i."""
    nt, nh, nw = tiles
    n = nt * nh * nw
    ids = torch.arange(n, device=device)
    coords = torch.stack([ids // (nh * nw), (ids // nw) % nh, ids % nw], 1)              # [n, 3]
    mask = torch.ones(n, n, dtype=torch.bool, device=device)
    for ax, (cnt, k) in enumerate(zip(tiles, kernel)):
        half = k // 2
        centre = coords[:, ax].clamp(min=min(half, cnt - 1), max=max(cnt - 1 - half, 0))
        mask &= (centre[:, None] - coords[None, :, ax]).abs() <= half
    return mask


@torch.no_grad()
def select_blocks(q_mean: torch.Tensor, k_mean: torch.Tensor, topk: int) -> torch.Tensor:
    """q_mean / k_mean [..., n_blocks, D] -> bool [..., n_blocks, n_blocks] with the ``topk`` most similar key blocks set."""
    gate = q_mean.float() @ k_mean.float().transpose(-1, -2)
    k = min(topk, gate.shape[-1])
    idx = gate.topk(k, dim=-1).indices
    return torch.zeros_like(gate, dtype=torch.bool).scatter_(-1, idx, True)


def ssta_block_mask(q, k, block: int, tiles: Sequence[int], kernel: Sequence[int], topk: int, text_blocks: int = 0,
                    share_heads: bool = True) -> torch.Tensor:
    """q, k [B, S, N, D] in tile-major order (image blocks, then text blocks).  Returns bool [B, 1 or N, nb, nb]."""
    B, S, N, D = q.shape
    n_img = tiles[0] * tiles[1] * tiles[2]
    nb = n_img + text_blocks
    base = torch.zeros(nb, nb, dtype=torch.bool, device=q.device)
    base[:n_img, :n_img] = sta_block_mask(tiles, kernel, q.device)
    base[:, n_img:] = True
    base[n_img:, :] = True
    qm = q[:, : n_img * block].reshape(B, n_img, block, N, D).float().mean(2)            # [B, n_img, N, D]
    km = k[:, : n_img * block].reshape(B, n_img, block, N, D).float().mean(2)
    if share_heads:
        sel = select_blocks(qm.mean(2), km.mean(2), topk)[:, None]                       # [B, 1, n_img, n_img]
    else:
        sel = select_blocks(qm.transpose(1, 2), km.transpose(1, 2), topk)                # [B, N, n_img, n_img]
    mask = base[None, None].expand(B, sel.shape[1], nb, nb).clone()
    mask[:, :, :n_img, :n_img] |= sel
    return mask


def block_sparse_attention(q, k, v, mask: torch.Tensor, block: int, scale: Optional[float] = None):
    """q, k, v [B, S, N, D] with S = nb * block; ``mask`` bool [B, 1, nb, nb] (one mask for all heads).  Every query block
    attends to the key blocks its mask row selects."""
    from . import attention_varlen
    B, S, N, D = q.shape
    nb = S // block
    if mask.shape[1] != 1:
        # per-head masks: heads become batch entries
        outs = [block_sparse_attention(q[:, :, h:h + 1], k[:, :, h:h + 1], v[:, :, h:h + 1], mask[:, h:h + 1], block, scale)
                for h in range(N)]
        return torch.cat(outs, 2)
    m = mask[:, 0]                                                                       # [B, nb, nb]
    counts = m.sum(-1).reshape(-1)                                                       # selected key blocks per query block
    b_idx, qb_idx, kb_idx = m.nonzero(as_tuple=True)                                     # sorted by (batch, query block)
    tok = torch.arange(block, device=q.device)
    src = ((b_idx * nb + kb_idx) * block)[:, None] + tok                                 # [n_sel, block] rows of the [B*S] table
    kg = k.reshape(B * S, N, D)[src.reshape(-1)]
    vg = v.reshape(B * S, N, D)[src.reshape(-1)]
    cu_q = torch.arange(0, (B * nb + 1) * block, block, dtype=torch.int32, device=q.device)
    cu_k = torch.zeros(B * nb + 1, dtype=torch.int32, device=q.device)
    cu_k[1:] = torch.cumsum(counts * block, 0)
    max_k = int(counts.max()) * block
    o = attention_varlen(q.reshape(B * S, N, D), kg, vg, cu_q, cu_k, block, max_k, causal=False,
                         softmax_scale=scale if scale is not None else 1.0 / math.sqrt(D))
    return o.view(B, S, N, D)


def ssta_attention(q, k, v, canvas: Sequence[int], tile: Sequence[int] = (6, 8, 8), kernel: Sequence[int] = (1, 1, 1),
                   topk: int = 1, text_len: int = 0, mode: str = "ssta", pad: str = "zero", share_heads: bool = True,
                   scale: Optional[float] = None):
    """q, k, v [B, S, N, D], S = t*h*w + text_len, canvas tokens in row-major order followed by the text tokens.

    ``mode``: "sta" (window only), "ssta" (window + selected blocks), "dense".  Returns ``(out [B, S, N, D], density)`` where
    density is the fraction of block pairs that were computed.
    """
    if mode == "dense":
        from . import attention_dense
        return attention_dense(q, k, v, softmax_scale=scale), 1.0
    B, S, N, D = q.shape
    n_canvas = canvas[0] * canvas[1] * canvas[2]
    if n_canvas + text_len != S:
        raise ValueError(f"canvas {tuple(canvas)} + text {text_len} does not match sequence {S}")
    block = tile[0] * tile[1] * tile[2]
    parts = []
    for x in (q, k, v):
        img, padded = pad_canvas(x[:, :n_canvas], canvas, tile, pad)
        img = img[:, tile_order(padded, tile, x.device)]
        if text_len:
            txt = x[:, n_canvas:]
            extra = _ceil_to(text_len, block) - text_len
            if extra:
                txt = torch.cat([txt, txt[:, -1:].expand(-1, extra, -1, -1)], 1)
            img = torch.cat([img, txt], 1)
        parts.append(img)
    qt, kt, vt = parts
    tiles = tuple(p // m for p, m in zip(padded, tile))
    text_blocks = _ceil_to(text_len, block) // block if text_len else 0
    if mode == "sta":
        n_img = tiles[0] * tiles[1] * tiles[2]
        nb = n_img + text_blocks
        base = torch.ones(nb, nb, dtype=torch.bool, device=q.device)
        base[:n_img, :n_img] = sta_block_mask(tiles, kernel, q.device)
        mask = base[None, None].expand(B, 1, nb, nb)
    else:
        mask = ssta_block_mask(qt, kt, block, tiles, kernel, topk, text_blocks, share_heads)
    ot = block_sparse_attention(qt, kt, vt, mask, block, scale)
    n_pad = padded[0] * padded[1] * padded[2]
    inv = torch.empty(n_pad, dtype=torch.long, device=q.device)
    inv[tile_order(padded, tile, q.device)] = torch.arange(n_pad, device=q.device)
    img = ot[:, :n_pad][:, inv].view(B, *padded, N, D)[:, : canvas[0], : canvas[1], : canvas[2]].reshape(B, n_canvas, N, D)
    out = torch.cat([img, ot[:, n_pad:n_pad + text_len]], 1) if text_len else img
    return out, float(mask.float().mean())
