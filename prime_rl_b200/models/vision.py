"""Vision tower and multimodal glue of the Qwen3.5 family.

``VisionTower``: pixel patches ``[N, C * tp * p * p]`` (already cut by the processor; ``grid_thw``
gives frames / rows / columns of patches per image) -> patch projection + bilinearly interpolated
learned position embedding -> ``depth`` pre-LayerNorm blocks of bidirectional attention (per
frame, 2-D rotary over the patch's row and column) and a GELU MLP -> 2x2 spatial merge + MLP into
the language model's width. Patches arrive ordered so that the ``merge x merge`` neighbours that
are merged into one token are consecutive.

``mrope_position_ids``: three position axes (time, row, column) per token of a packed stream:
text tokens advance all three together; the tokens of an image share the time index and carry
their merged-grid row / column; the text after an image continues from the largest index used.
``mrope_angles`` interleaves the three axes over the rotary frequencies.

``MultimodalLM`` wraps a ``CausalLM``: image features replace the embeddings of the image
placeholder tokens and the decoder runs with the 3-axis positions.

Reference: src/prime_rl/trainer/models/qwen3_5/vision.py:17-263, rotary_embedding.py:60-171,
modeling_qwen3_5.py:201-310.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from pydantic import BaseModel

from .layers import SeqInfo


class VisionConfig(BaseModel):
    depth: int = 27
    hidden_size: int = 1152
    intermediate_size: int = 4304
    num_heads: int = 16
    in_channels: int = 3
    patch_size: int = 16
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2
    out_hidden_size: int = 3584
    num_position_embeddings: int = 2304
    initializer_range: float = 0.02


def _rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat([-x[..., h:], x[..., :h]], dim=-1)


class _Block(nn.Module):
    def __init__(self, c: VisionConfig, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.nh, self.hd = c.num_heads, c.hidden_size // c.num_heads
        self.norm1 = nn.LayerNorm(c.hidden_size, eps=1e-6, **kw)
        self.norm2 = nn.LayerNorm(c.hidden_size, eps=1e-6, **kw)
        self.attn = nn.ModuleDict({"qkv": nn.Linear(c.hidden_size, 3 * c.hidden_size, **kw),
                                   "proj": nn.Linear(c.hidden_size, c.hidden_size, **kw)})
        self.mlp = nn.ModuleDict({"linear_fc1": nn.Linear(c.hidden_size, c.intermediate_size, **kw),
                                  "linear_fc2": nn.Linear(c.intermediate_size, c.hidden_size, **kw)})

    def forward(self, x, frame_lens: list[int], cos, sin):
        n = x.shape[0]
        q, k, v = self.attn["qkv"](self.norm1(x)).view(n, 3, self.nh, self.hd).unbind(1)
        q = (q.float() * cos + _rotate_half(q.float()) * sin).to(x.dtype)
        k = (k.float() * cos + _rotate_half(k.float()) * sin).to(x.dtype)
        outs, t0 = [], 0
        for ln in frame_lens:                                   # bidirectional attention inside one frame
            sl = slice(t0, t0 + ln)
            o = F.scaled_dot_product_attention(q[sl].transpose(0, 1), k[sl].transpose(0, 1), v[sl].transpose(0, 1))
            outs.append(o.transpose(0, 1).reshape(ln, -1))
            t0 += ln
        x = x + self.attn["proj"](torch.cat(outs))
        return x + self.mlp["linear_fc2"](F.gelu(self.mlp["linear_fc1"](self.norm2(x)), approximate="tanh"))


class VisionTower(nn.Module):
    def __init__(self, config: VisionConfig, dtype=None, device=None):
        super().__init__()
        c, kw = config, dict(dtype=dtype, device=device)
        self.config = c
        self.patch_dim = c.in_channels * c.temporal_patch_size * c.patch_size ** 2
        # stored with the shape of the 3-D convolution the checkpoints hold; applied as one GEMM
        self.patch_embed = nn.ModuleDict({"proj": nn.Conv3d(c.in_channels, c.hidden_size,
                                                            (c.temporal_patch_size, c.patch_size, c.patch_size),
                                                            stride=(c.temporal_patch_size, c.patch_size, c.patch_size), **kw)})
        self.pos_embed = nn.Embedding(c.num_position_embeddings, c.hidden_size, **kw)
        self.side = math.isqrt(c.num_position_embeddings)
        self.blocks = nn.ModuleList([_Block(c, **kw) for _ in range(c.depth)])
        merged = c.hidden_size * c.spatial_merge_size ** 2
        self.merger = nn.ModuleDict({"norm": nn.LayerNorm(c.hidden_size, eps=1e-6, **kw),
                                     "linear_fc1": nn.Linear(merged, merged, **kw),
                                     "linear_fc2": nn.Linear(merged, c.out_hidden_size, **kw)})
        rd = c.hidden_size // c.num_heads // 2
        self.register_buffer("inv_freq", 1.0 / (10000.0 ** (torch.arange(0, rd, 2, dtype=torch.float32, device=device) / rd)),
                             persistent=False)

    def _merge_order(self, h: int, w: int, device):
        """Row / column of every patch in the order the processor emits them: blocks of
        ``merge x merge`` neighbours are consecutive."""
        m = self.config.spatial_merge_size
        br, bc = torch.arange(h // m, device=device), torch.arange(w // m, device=device)
        ir, ic = torch.arange(m, device=device), torch.arange(m, device=device)
        rows = (br[:, None, None, None] * m + ir[None, None, :, None]).expand(h // m, w // m, m, m).reshape(-1)
        cols = (bc[None, :, None, None] * m + ic[None, None, None, :]).expand(h // m, w // m, m, m).reshape(-1)
        return rows, cols

    def _positions(self, grid_thw: list[list[int]], device):
        """Learned position embedding interpolated bilinearly from the ``side x side`` table to each
        image's grid, and the (row, column) rotary angles, both in merge order."""
        embeds, angles = [], []
        for t, h, w in grid_thw:
            rows, cols = self._merge_order(h, w, device)
            ry = torch.linspace(0, self.side - 1, h, device=device)[rows]
            cx = torch.linspace(0, self.side - 1, w, device=device)[cols]
            y0, x0 = ry.floor().long(), cx.floor().long()
            y1, x1 = (y0 + 1).clamp_max(self.side - 1), (x0 + 1).clamp_max(self.side - 1)
            fy, fx = (ry - y0).unsqueeze(1), (cx - x0).unsqueeze(1)
            tab = self.pos_embed.weight
            e = (tab[y0 * self.side + x0] * (1 - fy) * (1 - fx) + tab[y0 * self.side + x1] * (1 - fy) * fx
                 + tab[y1 * self.side + x0] * fy * (1 - fx) + tab[y1 * self.side + x1] * fy * fx)
            embeds.append(e.to(tab.dtype).repeat(t, 1))
            ang = torch.cat([rows[:, None].float() * self.inv_freq, cols[:, None].float() * self.inv_freq], dim=1)
            angles.append(ang.repeat(t, 1))
        return torch.cat(embeds), torch.cat(angles)

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        """-> merged image tokens ``[sum(t * h * w) / merge^2, out_hidden_size]``."""
        grids = [[int(v) for v in g] for g in grid_thw.tolist()]
        w = self.patch_embed["proj"].weight
        x = F.linear(pixel_values.reshape(-1, self.patch_dim).to(w.dtype), w.reshape(w.shape[0], -1),
                     self.patch_embed["proj"].bias)
        pos, ang = self._positions(grids, x.device)
        x = x + pos
        ang = torch.cat([ang, ang], dim=-1)
        cos, sin = ang.cos().unsqueeze(1), ang.sin().unsqueeze(1)
        frame_lens = [h * w_ for t, h, w_ in grids for _ in range(t)]
        for blk in self.blocks:
            x = blk(x, frame_lens, cos, sin)
        m2 = self.config.spatial_merge_size ** 2
        x = self.merger["norm"](x).view(-1, m2 * self.config.hidden_size)
        return self.merger["linear_fc2"](F.gelu(self.merger["linear_fc1"](x)))


def mrope_position_ids(token_types: torch.Tensor, seq_lens: list[int], grid_thw: list[list[int]] | None,
                       merge: int) -> torch.Tensor:
    """``token_types [T]`` (0 = text, 1 = image placeholder) of a packed stream -> int64 ``[3, T]``
    (time, row, column), restarting at every document."""
    out = torch.zeros(3, token_types.shape[0], dtype=torch.long)
    types = token_types.tolist()
    grids = iter(grid_thw or [])
    off = 0
    for n in seq_lens:
        cur, i = 0, off
        while i < off + n:
            if types[i] == 0:
                out[:, i] = cur
                cur += 1
                i += 1
                continue
            if types[i] != 1:
                raise ValueError(f"unsupported multimodal token type {types[i]}")
            g = next(grids, None)
            if g is None:
                raise ValueError("more image token groups than rows of image_grid_thw")
            t, h, w = g[0], g[1] // merge, g[2] // merge
            cnt = t * h * w
            if any(types[j] != 1 for j in range(i, min(i + cnt, off + n))) or i + cnt > off + n:
                raise ValueError("image token group does not match image_grid_thw")
            out[0, i:i + cnt] = cur + torch.arange(t).repeat_interleave(h * w)
            out[1, i:i + cnt] = cur + torch.arange(h).repeat_interleave(w).repeat(t)
            out[2, i:i + cnt] = cur + torch.arange(w).repeat(h * t)
            cur += max(h, w)
            i += cnt
        off += n
    return out


def mrope_axis_of_frequency(num_freqs: int, section: tuple[int, int, int]) -> torch.Tensor:
    """Which position axis drives rotary frequency ``j`` (interleaved layout): ``j % 3 == 1`` and
    ``j < 3 * section[1]`` -> row, ``j % 3 == 2`` and ``j < 3 * section[2]`` -> column, else time."""
    j = torch.arange(num_freqs)
    axis = torch.zeros(num_freqs, dtype=torch.long)
    axis[(j % 3 == 1) & (j < 3 * section[1])] = 1
    axis[(j % 3 == 2) & (j < 3 * section[2])] = 2
    return axis


def mrope_angles(pos3: torch.Tensor, inv_freq: torch.Tensor, section: tuple[int, int, int]) -> torch.Tensor:
    """``pos3 [3, T]`` -> rotary angles ``[T, len(inv_freq)]``."""
    axis = mrope_axis_of_frequency(inv_freq.numel(), section).to(pos3.device)
    return pos3.float().t()[:, axis] * inv_freq.float()[None, :]


class MultimodalLM(nn.Module):
    """``language_model`` (a ``CausalLM``) + ``visual`` tower. Image features take the place of
    the embeddings at ``image_token_id`` positions; the decoder sees 3-axis positions through
    ``seq.mrope_angles`` (attention layers that find it use it instead of ``position_ids``)."""

    def __init__(self, language_model, vision: VisionConfig, image_token_id: int,
                 mrope_section: tuple[int, int, int] = (11, 11, 10), dtype=None, device=None):
        super().__init__()
        self.language_model = language_model
        self.visual = VisionTower(vision, dtype=dtype, device=device)
        self.image_token_id, self.mrope_section = image_token_id, tuple(mrope_section)

    @property
    def arch(self):
        return self.language_model.arch

    def forward(self, input_ids: torch.Tensor, seq: SeqInfo, pixel_values: torch.Tensor | None = None,
                image_grid_thw: torch.Tensor | None = None) -> torch.Tensor:
        ids = input_ids.reshape(-1)
        lm = self.language_model
        embeds = lm.model.embed_tokens(ids)
        is_image = ids == self.image_token_id
        if pixel_values is not None:
            feats = self.visual(pixel_values, image_grid_thw).to(embeds.dtype)
            if int(is_image.sum()) != feats.shape[0]:
                raise ValueError(f"{int(is_image.sum())} image tokens but {feats.shape[0]} image features")
            embeds = embeds.masked_scatter(is_image.unsqueeze(-1), feats)
        lens = (seq.cu_seqlens[1:] - seq.cu_seqlens[:-1]).tolist()
        grids = image_grid_thw.tolist() if image_grid_thw is not None else None
        pos3 = mrope_position_ids(is_image.long().cpu(), lens, grids, self.visual.config.spatial_merge_size).to(ids.device)
        rd = lm.arch.rotary_dim
        inv_freq = 1.0 / (lm.arch.rope_theta ** (torch.arange(0, rd, 2, dtype=torch.float32, device=ids.device) / rd))
        seq.mrope_angles = mrope_angles(pos3, inv_freq, self.mrope_section)
        return lm(ids, seq, inputs_embeds=embeds)

    def logprobs_entropy(self, *a, **kw):
        return self.language_model.logprobs_entropy(*a, **kw)
