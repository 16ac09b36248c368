"""Vision-language family (Qwen2-VL and Qwen2.5-VL architectures): a ViT tower whose merged patch embeddings replace the image placeholder
tokens of a decoder LM that runs multimodal rotary embedding (M-RoPE: temporal / height / width position streams).

* :class:`VisionTower` — patch embedding (the 3-D convolution over ``[C, T_p, P, P]`` written as one linear layer), pre-norm
  blocks with bidirectional attention inside each frame and 2-D rotary embedding, 2×2 patch merger into the LM width.
  Parameter names follow the Hugging Face checkpoint below ``visual.`` so the name mapping is a prefix.
* :func:`get_rope_index` — the 3-stream position ids of a token sequence with image blocks.
* :func:`mrope_tables` — per-token cos/sin ``[T, D/2]`` built from the three streams; the decoder's rotary kernel is reused by
  passing these as its tables with ``position = arange(T)``.
* :class:`VisionLanguageModel` — tower + :class:`~verl_b200.models.transformer.DecoderLM` on packed batches.

Reference: the Qwen2-VL patches of the reference (``verl/models/transformers/qwen2_vl.py:36-250``: rope index, Ulysses-aware
attention, embedding merge) and ``verl/utils/dataset/vision_utils.py`` for the inputs. The Qwen2.5-VL variant swaps in
RMSNorm, a gated SiLU MLP and window attention (:meth:`VisionTower._window_index`). Video inputs are not implemented.
"""

from __future__ import annotations

import dataclasses
from typing import Iterator, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from verl_b200.models.config import ModelConfig
from verl_b200.models.transformer import DecoderLM, PackedBatch

__all__ = ["VisionConfig", "VisionTower", "VisionLanguageModel", "get_rope_index", "mrope_tables"]


@dataclasses.dataclass(frozen=True)
class VisionConfig:
    depth: int = 32
    embed_dim: int = 1280
    num_heads: int = 16
    mlp_ratio: float = 4.0
    in_channels: int = 3
    patch_size: int = 14
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    hidden_size: int = 3584                 # width of the language model (output of the merger)
    image_token_id: int = 151655
    video_token_id: int = 151656
    vision_start_token_id: int = 151652
    mrope_section: tuple = (16, 24, 24)
    # Qwen2.5-VL tower: RMSNorm + gated SiLU MLP, attention inside windows of window_size pixels except in the listed blocks
    variant: str = "qwen2_vl"               # "qwen2_vl" | "qwen2_5_vl" | "qwen3_vl"
    intermediate_size: int = 0
    window_size: int = 0
    fullatt_block_indexes: tuple = ()
    # Qwen3-VL tower: learned position table interpolated to the image grid, biased patch embedding, tanh-GELU MLP, and "deep-stack"
    # mergers after the listed blocks whose outputs are added to the language model's stream after its first layers; the language
    # model's multimodal rotary embedding interleaves the three position streams over the frequencies instead of chunking them
    num_position_embeddings: int = 0
    deepstack_visual_indexes: tuple = ()
    mrope_interleaved: bool = False
    tokens_per_second: float = 0.0           # Qwen2.5-VL: temporal positions of a video advance by seconds-per-patch x this (0: by 1 per patch)

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size

    @classmethod
    def from_hf_dict(cls, d: dict, text: Optional[dict] = None) -> "VisionConfig":
        v = d.get("vision_config", {})
        rope = (text or d).get("rope_scaling") or (text or d).get("rope_parameters") or {}
        if d.get("model_type") == "qwen3_vl":
            return cls(depth=v.get("depth", 27), embed_dim=v.get("hidden_size", 1152), num_heads=v.get("num_heads", 16), in_channels=v.get("in_channels", 3),
                       patch_size=v.get("patch_size", 16), temporal_patch_size=v.get("temporal_patch_size", 2),
                       spatial_merge_size=v.get("spatial_merge_size", 2), hidden_size=v.get("out_hidden_size", (text or d).get("hidden_size", 4096)),
                       image_token_id=d.get("image_token_id", 151655), video_token_id=d.get("video_token_id", 151656),
                       vision_start_token_id=d.get("vision_start_token_id", 151652), mrope_section=tuple(rope.get("mrope_section", (24, 20, 20))),
                       variant="qwen3_vl", intermediate_size=v.get("intermediate_size", 4304), num_position_embeddings=v.get("num_position_embeddings", 2304),
                       deepstack_visual_indexes=tuple(v.get("deepstack_visual_indexes", (8, 16, 24))), mrope_interleaved=bool(rope.get("mrope_interleaved", True)))
        if d.get("model_type") == "qwen2_5_vl":
            return cls(depth=v.get("depth", 32), embed_dim=v.get("hidden_size", 1280), num_heads=v.get("num_heads", 16), in_channels=v.get("in_channels", 3),
                       patch_size=v.get("patch_size", 14), temporal_patch_size=v.get("temporal_patch_size", 2),
                       spatial_merge_size=v.get("spatial_merge_size", 2), hidden_size=v.get("out_hidden_size", (text or d).get("hidden_size", 3584)),
                       image_token_id=d.get("image_token_id", 151655), video_token_id=d.get("video_token_id", 151656),
                       vision_start_token_id=d.get("vision_start_token_id", 151652), mrope_section=tuple(rope.get("mrope_section", (16, 24, 24))),
                       variant="qwen2_5_vl", intermediate_size=v.get("intermediate_size", 3420), window_size=v.get("window_size", 112),
                       fullatt_block_indexes=tuple(v.get("fullatt_block_indexes", (7, 15, 23, 31))), tokens_per_second=float(v.get("tokens_per_second", 2)))
        return cls(depth=v.get("depth", 32), embed_dim=v.get("embed_dim", 1280), num_heads=v.get("num_heads", 16), mlp_ratio=v.get("mlp_ratio", 4.0),
                   in_channels=v.get("in_channels", v.get("in_chans", 3)), patch_size=v.get("patch_size", 14),
                   temporal_patch_size=v.get("temporal_patch_size", 2), spatial_merge_size=v.get("spatial_merge_size", 2),
                   hidden_size=v.get("hidden_size", (text or d).get("hidden_size", 3584)), image_token_id=d.get("image_token_id", 151655),
                   video_token_id=d.get("video_token_id", 151656), vision_start_token_id=d.get("vision_start_token_id", 151652),
                   mrope_section=tuple(rope.get("mrope_section", (16, 24, 24))))


def _rotate_half(x):
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat([-x2, x1], dim=-1)


class _VisionBlock(nn.Module):
    def __init__(self, cfg: VisionConfig, dtype, device):
        super().__init__()
        E, Hm = cfg.embed_dim, int(cfg.embed_dim * cfg.mlp_ratio)
        kw = dict(dtype=dtype, device=device)
        self.gated = cfg.variant == "qwen2_5_vl"
        self.v3 = cfg.variant == "qwen3_vl"
        self.attn = nn.Module()
        self.attn.qkv, self.attn.proj = nn.Linear(E, 3 * E, **kw), nn.Linear(E, E, **kw)
        self.mlp = nn.Module()
        if self.gated:
            I = cfg.intermediate_size
            self.norm1, self.norm2 = nn.RMSNorm(E, eps=1e-6, **kw), nn.RMSNorm(E, eps=1e-6, **kw)
            self.mlp.gate_proj, self.mlp.up_proj, self.mlp.down_proj = nn.Linear(E, I, **kw), nn.Linear(E, I, **kw), nn.Linear(I, E, **kw)
        elif self.v3:
            self.norm1, self.norm2 = nn.LayerNorm(E, eps=1e-6, **kw), nn.LayerNorm(E, eps=1e-6, **kw)
            self.mlp.linear_fc1, self.mlp.linear_fc2 = nn.Linear(E, cfg.intermediate_size, **kw), nn.Linear(cfg.intermediate_size, E, **kw)
        else:
            self.norm1, self.norm2 = nn.LayerNorm(E, eps=1e-6, **kw), nn.LayerNorm(E, eps=1e-6, **kw)
            self.mlp.fc1, self.mlp.fc2 = nn.Linear(E, Hm, **kw), nn.Linear(Hm, E, **kw)
        self.num_heads = cfg.num_heads

    def forward(self, x, cos, sin, seg_lens):
        N, E = x.shape
        H = self.num_heads
        q, k, v = self.attn.qkv(self.norm1(x)).reshape(N, 3, H, E // H).unbind(1)
        q = (q.float() * cos + _rotate_half(q.float()) * sin).to(x.dtype)
        k = (k.float() * cos + _rotate_half(k.float()) * sin).to(x.dtype)
        outs, s = [], 0
        for n in seg_lens:                  # bidirectional attention inside each frame, none across frames
            qs, ks, vs = (t[s:s + n].transpose(0, 1).unsqueeze(0) for t in (q, k, v))
            outs.append(F.scaled_dot_product_attention(qs, ks, vs).squeeze(0).transpose(0, 1).reshape(n, E))
            s += n
        x = x + self.attn.proj(torch.cat(outs, 0))
        y = self.norm2(x)
        if self.gated:
            return x + self.mlp.down_proj(F.silu(self.mlp.gate_proj(y)) * self.mlp.up_proj(y))
        if self.v3:
            return x + self.mlp.linear_fc2(F.gelu(self.mlp.linear_fc1(y), approximate="tanh"))
        h = self.mlp.fc1(y)
        return x + self.mlp.fc2(h * torch.sigmoid(1.702 * h))       # QuickGELU


class VisionTower(nn.Module):
    def __init__(self, cfg: VisionConfig, dtype=torch.bfloat16, device=None, seed: int = 0):
        super().__init__()
        self.cfg = cfg
        kw = dict(dtype=dtype, device=device)
        E, m2 = cfg.embed_dim, cfg.spatial_merge_size ** 2
        self.patch_embed = nn.Module()
        self.v3 = cfg.variant == "qwen3_vl"
        self.patch_embed.proj = nn.Linear(cfg.patch_dim, E, bias=self.v3, **kw)
        self.blocks = nn.ModuleList([_VisionBlock(cfg, dtype, device) for _ in range(cfg.depth)])
        self.merger = nn.Module()
        if self.v3:
            self.pos_embed = nn.Embedding(cfg.num_position_embeddings, E, **kw)

            def merger(post_shuffle: bool):
                mod = nn.Module()
                mod.norm = nn.LayerNorm(E * m2 if post_shuffle else E, eps=1e-6, **kw)
                mod.linear_fc1, mod.linear_fc2 = nn.Linear(E * m2, E * m2, **kw), nn.Linear(E * m2, cfg.hidden_size, **kw)
                return mod

            self.merger = merger(False)
            self.deepstack_merger_list = nn.ModuleList([merger(True) for _ in cfg.deepstack_visual_indexes])
        else:
            self.merger.ln_q = nn.RMSNorm(E, eps=1e-6, **kw) if cfg.variant == "qwen2_5_vl" else nn.LayerNorm(E, eps=1e-6, **kw)
            self.merger.mlp = nn.Sequential(nn.Linear(E * m2, E * m2, **kw), nn.GELU(), nn.Linear(E * m2, cfg.hidden_size, **kw))
        g = torch.Generator(device="cpu").manual_seed(seed + 7919)
        with torch.no_grad():
            for n, p in self.named_parameters():      # seeded, identical in every process: matrices N(0, 0.02²), biases 0, norms 1
                if p.dim() >= 2:
                    p.copy_((torch.randn(p.shape, generator=g) * 0.02).to(p.dtype))
                elif n.endswith(".bias"):
                    p.zero_()

    def _rot_pos(self, grid_thw: torch.Tensor) -> torch.Tensor:
        """(h, w) index of every patch in the processor's order: patches of one merge window are adjacent."""
        m = self.cfg.spatial_merge_size
        out = []
        for t, h, w in grid_thw.tolist():
            hp = torch.arange(h).unsqueeze(1).expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            wp = torch.arange(w).unsqueeze(0).expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            out.append(torch.stack([hp, wp], -1).repeat(t, 1))
        return torch.cat(out, 0)

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        """``pixel_values`` [N, C·T_p·P·P] flattened patches, ``grid_thw`` [n_images, 3] → [N / merge², hidden_size]."""
        cfg = self.cfg
        x = self.patch_embed.proj(pixel_values.to(self.patch_embed.proj.weight.dtype))
        D = cfg.embed_dim // cfg.num_heads
        pos = self._rot_pos(grid_thw.cpu()).to(x.device)
        inv = 1.0 / (10000.0 ** (torch.arange(0, D // 2, 2, dtype=torch.float32, device=x.device) / (D // 2)))
        ang = (pos[:, :, None].float() * inv[None, None, :]).flatten(1)              # [N, D/2]: (h freqs, w freqs)
        emb = torch.cat([ang, ang], -1)
        cos, sin = emb.cos()[:, None, :], emb.sin()[:, None, :]
        seg = [int(h * w) for t, h, w in grid_thw.tolist() for _ in range(int(t))]
        m2 = cfg.spatial_merge_size ** 2
        if self.v3:
            x = x + self._interpolated_positions(grid_thw.cpu()).to(x.dtype)
            E = cfg.embed_dim

            def merge(mod, t, post_shuffle):
                t = mod.norm(t.reshape(-1, E * m2)) if post_shuffle else mod.norm(t).reshape(-1, E * m2)
                return mod.linear_fc2(F.gelu(mod.linear_fc1(t)))

            deep = []
            for i, blk in enumerate(self.blocks):
                x = blk(x, cos, sin, seg)
                if i in cfg.deepstack_visual_indexes:
                    deep.append(merge(self.deepstack_merger_list[cfg.deepstack_visual_indexes.index(i)], x, True))
            self.last_deepstack = deep            # picked up by VisionLanguageModel.embed right after this call
            return merge(self.merger, x, False)
        if cfg.variant != "qwen2_5_vl":
            for blk in self.blocks:
                x = blk(x, cos, sin, seg)
            return self.merger.mlp(self.merger.ln_q(x).reshape(-1, cfg.embed_dim * m2))
        # windowed variant: merge groups are reordered window by window once; most blocks attend inside a window, the
        # listed ones inside the whole frame (in the window order, which attention does not care about); the merger's
        # output goes back to the original order
        win_index, win_seg = self._window_index(grid_thw.cpu())
        win_index = win_index.to(x.device)

        def reorder(t):
            return t.reshape(-1, m2, *t.shape[1:]).index_select(0, win_index).reshape(t.shape)

        x, cos, sin = reorder(x), reorder(cos), reorder(sin)
        for i, blk in enumerate(self.blocks):
            x = blk(x, cos, sin, seg if i in cfg.fullatt_block_indexes else win_seg)
        out = self.merger.mlp(self.merger.ln_q(x).reshape(-1, cfg.embed_dim * m2))
        return out.index_select(0, torch.argsort(win_index))

    def _interpolated_positions(self, grid_thw: torch.Tensor) -> torch.Tensor:
        """Learned position table (a square grid of ``sqrt(num_position_embeddings)`` points per side) read at the patch centres
        of each image by bilinear interpolation, in the processor's patch order (patches of one merge window adjacent)."""
        cfg = self.cfg
        side, m = int(cfg.num_position_embeddings ** 0.5), cfg.spatial_merge_size
        table = self.pos_embed.weight
        out = []
        for t, h, w in grid_thw.tolist():
            hs, ws = torch.linspace(0, side - 1, h), torch.linspace(0, side - 1, w)
            h0, w0 = hs.int(), ws.int()
            h1, w1 = (h0 + 1).clamp(max=side - 1), (w0 + 1).clamp(max=side - 1)
            dh, dw = (hs - h0)[:, None], (ws - w0)[None, :]
            acc = 0
            for hi, wi, wt in ((h0, w0, (1 - dh) * (1 - dw)), (h0, w1, (1 - dh) * dw), (h1, w0, dh * (1 - dw)), (h1, w1, dh * dw)):
                idx = (hi[:, None] * side + wi[None, :]).flatten().long().to(table.device)
                acc = acc + table.index_select(0, idx) * wt.flatten().to(table.device, table.dtype)[:, None]
            acc = acc.reshape(h // m, m, w // m, m, -1).permute(0, 2, 1, 3, 4).reshape(h * w, -1)
            out.append(acc.repeat(t, 1))
        return torch.cat(out, 0)

    def _window_index(self, grid_thw: torch.Tensor):
        """Order of the merge groups window by window (windows of ``window_size`` pixels, ragged at the right / bottom edge)
        and the number of PATCHES in each window, in that order."""
        cfg = self.cfg
        m = cfg.spatial_merge_size
        W = cfg.window_size // m // cfg.patch_size
        index, seg, base = [], [], 0
        for t, h, w in grid_thw.tolist():
            gh, gw = h // m, w // m
            idx = torch.arange(t * gh * gw).reshape(t, gh, gw)
            ph, pw = (W - gh % W) % W, (W - gw % W) % W
            idx = F.pad(idx, (0, pw, 0, ph), value=-1)
            nh, nw = (gh + ph) // W, (gw + pw) // W
            idx = idx.reshape(t, nh, W, nw, W).permute(0, 1, 3, 2, 4).reshape(t * nh * nw, W * W)
            for row in idx:
                keep = row[row >= 0]
                if keep.numel():
                    index.append(keep + base)
                    seg.append(int(keep.numel()) * m * m)
            base += t * gh * gw
        return torch.cat(index), seg


def get_rope_index(input_ids: torch.Tensor, image_grid_thw: Optional[torch.Tensor], cfg: VisionConfig,
                   attention_mask: Optional[torch.Tensor] = None, grid_t_scale: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, int]:
    """3-stream positions ``[3, L]`` of ONE sequence and the offset ``delta`` such that generated token ``j`` (0-based index
    in the unpadded sequence) sits at position ``j + delta`` in all three streams.

    Text tokens advance all streams together. An image block of ``t × h × w`` patches (``h, w`` in merged units) keeps the
    temporal stream at the block start and walks the height / width streams over the grid; the text after it continues
    from the largest position used so far + 1. Masked (padding) positions get 0. ``image_grid_thw`` lists the grids of images AND
    videos in token order; ``grid_t_scale`` (one factor per grid, default 1) is the number of positions the temporal stream of a
    video advances per temporal patch (Qwen2.5-VL: seconds per patch x tokens per second; truncated to integers like there)."""
    ids = input_ids if attention_mask is None else input_ids[attention_mask.bool()]
    L = ids.numel()
    m = cfg.spatial_merge_size
    pos = torch.zeros(3, L, dtype=torch.long)
    ids_l = ids.tolist()
    grids = image_grid_thw.tolist() if image_grid_thw is not None else []
    scales = grid_t_scale.tolist() if grid_t_scale is not None else [1.0] * len(grids)
    i, nxt, g = 0, 0, 0
    while i < L:
        if ids_l[i] in (cfg.image_token_id, cfg.video_token_id) and g < len(grids):
            t, h, w = grids[g]
            sc = float(scales[g])
            g += 1
            gh, gw = h // m, w // m
            n = t * gh * gw
            assert ids_l[i:i + n] == [ids_l[i]] * n, "image placeholder run does not match image_grid_thw"
            tt = (torch.arange(t).view(t, 1, 1).expand(t, gh, gw) * sc).long().flatten()
            hh = torch.arange(gh).view(1, gh, 1).expand(t, gh, gw).flatten()
            ww = torch.arange(gw).view(1, 1, gw).expand(t, gh, gw).flatten()
            pos[:, i:i + n] = torch.stack([tt, hh, ww]) + nxt
            nxt += max(int(tt.max()) + 1, gh, gw)
            i += n
        else:
            pos[:, i] = nxt
            nxt += 1
            i += 1
    delta = nxt - L
    if attention_mask is None:
        return pos, delta
    full = torch.zeros(3, input_ids.numel(), dtype=torch.long)
    full[:, attention_mask.bool()] = pos
    return full, delta


def mrope_tables(pos3: torch.Tensor, head_dim: int, theta: float, mrope_section, interleaved: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-token fp32 cos/sin ``[T, head_dim/2]``: frequency ``i`` reads the temporal, height or width stream according
    to ``mrope_section`` (their sizes add up to ``head_dim/2``): in three chunks [T.. | H.. | W..], or ``interleaved``
    (Qwen3-VL): T H W T H W ... for the first ``3 * section`` frequencies of each of H and W, temporal for the rest."""
    half = head_dim // 2
    assert sum(mrope_section) == half, (mrope_section, head_dim)
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=pos3.device) / head_dim))
    if interleaved:
        comp = torch.zeros(half, dtype=torch.long, device=pos3.device)
        for stream in (1, 2):
            comp[stream:mrope_section[stream] * 3:3] = stream
    else:
        comp = torch.repeat_interleave(torch.arange(3, device=pos3.device), torch.tensor(list(mrope_section), device=pos3.device))
    p = pos3.float().index_select(0, comp)                    # [half, T]: the stream each frequency follows
    ang = (p * inv[:, None]).t().contiguous()
    return ang.cos().contiguous(), ang.sin().contiguous()


class VisionLanguageModel(nn.Module):
    """``visual`` tower + ``language_model`` decoder. :meth:`forward` takes the decoder's packed batch plus the flattened
    patches of all images of the micro-batch (in token order) and the 3-stream positions of its tokens."""

    def __init__(self, cfg: ModelConfig, vcfg: Optional[VisionConfig] = None, dtype=torch.bfloat16, device=None, init: bool = True, seed: int = 0):
        super().__init__()
        if vcfg is None:
            v = dict(cfg.vision)
            vcfg = VisionConfig(**{**v, "mrope_section": tuple(v["mrope_section"])})
        self.cfg, self.vcfg = cfg, vcfg
        self.language_model = DecoderLM(cfg, dtype=dtype, device=device, init=init, seed=seed)
        self.visual = VisionTower(vcfg, dtype=dtype, device=device, seed=seed)

    @property
    def gradient_checkpointing(self):
        return self.language_model.gradient_checkpointing

    @gradient_checkpointing.setter
    def gradient_checkpointing(self, v):
        self.language_model.gradient_checkpointing = v

    # the engine drives a decoder through these members; they resolve to the language model
    @property
    def output_weight(self):
        return self.language_model.output_weight

    @property
    def layers(self):
        return self.language_model.layers

    @property
    def embed_tokens(self):
        return self.language_model.embed_tokens

    def _prepare(self, pb: PackedBatch) -> PackedBatch:
        mm = pb.mm
        if mm:
            pb.visual_embeds = self.embed(pb, mm.get("pixel_values"), mm.get("image_grid_thw"))
            pb.visual_token_ids = (self.vcfg.image_token_id, self.vcfg.video_token_id)
            if mm.get("mrope_positions") is not None:
                pb.rope_override = mrope_tables(mm["mrope_positions"].to(pb.input_ids.device), self.cfg.head_dim, self.cfg.rope_theta,
                                                self.vcfg.mrope_section, self.vcfg.mrope_interleaved)
            if self.vcfg.variant == "qwen3_vl" and pb.visual_embeds is not None:
                pb.deepstack_embeds = self.visual.last_deepstack
        return pb

    def forward_hidden(self, pb: PackedBatch, h_in=None):
        return self.language_model.forward_hidden(self._prepare(pb), h_in)

    def embed(self, pb: PackedBatch, pixel_values: Optional[torch.Tensor], image_grid_thw: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Rows for the image placeholder tokens of ``pb`` (``None`` for a text-only batch)."""
        if pixel_values is None or pixel_values.numel() == 0:
            return None
        vis = self.visual(pixel_values, image_grid_thw)
        n_tok = int(((pb.input_ids == self.vcfg.image_token_id) | (pb.input_ids == self.vcfg.video_token_id)).sum())
        assert vis.shape[0] == n_tok, f"{n_tok} image placeholder tokens but {vis.shape[0]} merged patch embeddings"
        return vis

    def forward(self, pb: PackedBatch, pixel_values=None, image_grid_thw=None, mrope_positions: Optional[torch.Tensor] = None, **kw):
        if pixel_values is not None or mrope_positions is not None:
            pb.mm = {"pixel_values": pixel_values, "image_grid_thw": image_grid_thw, "mrope_positions": mrope_positions}
        return self.language_model(self._prepare(pb), **kw)

    # ------------------------------------------------------------------ Hugging Face names
    def hf_named_tensors(self) -> Iterator[tuple[str, torch.Tensor]]:
        yield from self.language_model.hf_named_tensors()
        P = self.vcfg
        for n, p in self.visual.named_parameters():
            if n == "patch_embed.proj.weight":
                p = p.view(P.embed_dim, P.in_channels, P.temporal_patch_size, P.patch_size, P.patch_size)
            yield ("model.visual." if P.variant == "qwen3_vl" else "visual.") + n, p

    @torch.no_grad()
    def load_hf_stream(self, named_tensors) -> int:
        """Consume (hf_name, tensor) pairs (weight hand-off from a sharded trainer to a rollout copy)."""
        sd = {k: v for k, v in named_tensors}
        self.load_hf_state_dict(sd, strict=False)
        return len(sd)

    def load_hf_state_dict(self, sd: dict, strict: bool = True):
        sd = {(k[len("model."):] if k.startswith("model.visual.") else k): v for k, v in sd.items()}      # both checkpoint generations
        vis = {k[len("visual."):]: v for k, v in sd.items() if k.startswith("visual.")}
        own = dict(self.visual.named_parameters())
        missing = [k for k in own if k not in vis]
        if strict and missing:
            raise KeyError(f"missing vision tensors {missing[:5]} ...")
        with torch.no_grad():
            for k, v in vis.items():
                if k in own:
                    own[k].copy_(v.reshape(own[k].shape).to(own[k].dtype))
        lm = {k.replace("model.language_model.", "model."): v for k, v in sd.items() if not k.startswith("visual.")}
        self.language_model.load_hf_state_dict(lm, strict=strict)
