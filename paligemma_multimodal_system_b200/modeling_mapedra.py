"""Mapedra: a decoder-only language model whose layers mix tokens either by gated softmax attention or by decayed linear
("lightning") attention, served through the ragged-step engine (engine.py).

Block structure (x = fp32 residual stream; the sub-layers read x itself, norms sit on the sub-layer OUTPUTS):

    x <- x + gnorm(mixer(x)) * w1
    x <- x + gnorm(ff(x)) * w2                     (layers that have a feed-forward)
    x <- x + rms(side(x, token)) * w_side          (models with a per-token side table)
    logits = head(gnorm(x) * w_final)

gnorm = RMS norm in `norm.groups` consecutive parts of the vector, each with its own mean square.  Every size and every
model-dependent constant comes from config.json (`MapedraConfig`), tensor names from the checkpoint:

    embed, side.embed, final.norm, head, l<i>.norm1, l<i>.norm2, l<i>.mix.{q,k,v,g,o}, l<i>.mix.{q.norm,k.norm} (attention),
    l<i>.mix.norm (lightning), l<i>.mlp.{gate,up,down}, l<i>.side.{gate,proj,norm}
"""
import json
import os
from typing import Dict, List, Optional

import torch

from . import _lib, seq_ops
from .mixers import GatedSoftmaxAttention, GegluFeedForward, LightningAttention, TokenSideInput


class MapedraConfig:
    def __init__(self, cfg: dict):
        if cfg.get("architecture") != "Mapedra":
            raise ValueError("not a Mapedra config")
        self.raw = cfg
        self.vocab = int(cfg["vocab"])
        self.width = int(cfg["width"])
        self.embedding_scale = float(cfg.get("embedding", {}).get("scale", 1.0))
        self.norm_eps = float(cfg["norm"]["eps"])
        self.norm_groups = int(cfg["norm"].get("groups", 1))
        side = cfg.get("token_side")
        self.side_dim = int(side["dim"]) if side else 0
        self.layers: List[dict] = list(cfg["layers"])
        if self.width % self.norm_groups:
            raise ValueError("width must be a multiple of norm.groups")
        for i, l in enumerate(self.layers):
            if l["type"] not in ("attention", "lightning"):
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
            if l.get("mlp") and l["mlp"].get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {l['mlp'].get('kind')!r}")

    @classmethod
    def from_dir(cls, path):
        with open(os.path.join(path, "config.json")) as f:
            return cls(json.load(f))


class MapedraBlock:
    def __init__(self, c: MapedraConfig, i: int):
        l, m, D, eps = c.layers[i], c.layers[i]["mixer"], c.width, c.norm_eps
        if l["type"] == "attention":
            rot = m.get("rot") or {}
            self.mixer = GatedSoftmaxAttention(D, int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m.get("vdim", m["dim"])),
                                               m["scale"], m.get("softcap"), int(rot.get("dims", 0)), rot.get("base", 10000.0),
                                               rot.get("scaling"), eps)
        else:
            self.mixer = LightningAttention(D, int(m["heads"]), int(m["dim"]), int(m.get("vdim", m["dim"])), m["decay"], eps)
        self.ff = GegluFeedForward(D, int(l["mlp"]["ff"])) if l.get("mlp") else None
        self.side = TokenSideInput(D, c.side_dim, i) if c.side_dim else None
        self.i = i

    def load(self, take):
        p = f"l{self.i}."
        D = self.mixer.D
        self.norm1 = take(p + "norm1", (D,))
        self.mixer.load(take, p + "mix.")
        if self.ff is not None:
            self.norm2 = take(p + "norm2", (D,))
            self.ff.load(take, p + "mlp.")
        if self.side is not None:
            self.side.load(take, p + "side.")
            self.side_norm = take(p + "side.norm", (D,))

    def pack(self, prec):
        f32 = dict(device="cuda", dtype=torch.float32)
        self.norm1_d = self.norm1.to(**f32)
        self.mixer.pack(prec)
        if self.ff is not None:
            self.norm2_d = self.norm2.to(**f32)
            self.ff.pack(prec)
        if self.side is not None:
            self.side.pack(prec)
            self.side_norm_d = self.side_norm.to(**f32)


class MapedraForCausalLM:
    """Weights + the step function.  `step(batch, store, want_rows)` advances every entry of a ragged batch by its new
    tokens (keys / values and recurrent states are left in `store`) and returns fp32 logits of the wanted rows."""

    architecture = "Mapedra"

    def __init__(self, config: MapedraConfig, dtype: torch.dtype = torch.bfloat16):
        self.config = config
        self.prec = seq_ops.Precision(dtype)
        self.blocks = [MapedraBlock(config, i) for i in range(len(config.layers))]
        self.vocab_size = config.vocab
        self._packed = False

    # -- weights -------------------------------------------------------------------------------------------------------
    def load_weights(self, tensors: Dict[str, torch.Tensor]):
        """Every tensor must be used and have the shape the config implies; anything missing or left over raises."""
        c = self.config
        left = dict(tensors)

        def take(name, shape):
            if name not in left:
                raise KeyError(f"checkpoint lacks {name}")
            t = left.pop(name)
            if tuple(t.shape) != tuple(shape):
                raise ValueError(f"{name}: shape {tuple(t.shape)}, config implies {tuple(shape)}")
            return t

        self.embed = take("embed", (c.vocab, c.width))
        self.side_embed = take("side.embed", (c.vocab, c.side_dim * len(c.layers))) if c.side_dim else None
        for blk in self.blocks:
            blk.load(take)
        self.final_norm = take("final.norm", (c.width,))
        self.head = take("head", (c.vocab, c.width))
        if left:
            raise KeyError(f"checkpoint tensors without a place in the model: {sorted(left)[:8]}")
        self._packed = False
        return self

    def pack(self):
        _lib.require_device()
        dt = self.prec.dtype
        self.embed_d = self.embed.to("cuda", dt).contiguous()
        self.side_embed_d = self.side_embed.to("cuda", dt).contiguous() if self.side_embed is not None else None
        self.final_norm_d = self.final_norm.to("cuda", torch.float32)
        self.head_d = self.head.to("cuda", dt).contiguous()
        for blk in self.blocks:
            blk.pack(self.prec)
        torch.cuda.synchronize()
        self._packed = True

    def cache_layout(self):
        return [blk.mixer.cache_spec() for blk in self.blocks]

    # -- compute -------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, b: seq_ops.StepBatch, store, want_rows: Optional[torch.Tensor], trace: Optional[list] = None):
        """want_rows: int64 row indices (device) whose logits are returned as fp32 [n, vocab]; None / empty: no head."""
        if not self._packed:
            self.pack()
        c, prec = self.config, self.prec
        eps, groups = c.norm_eps, c.norm_groups
        x = seq_ops.embed_rows(b.tokens, self.embed_d, 0, c.width, c.embedding_scale)
        # the sub-layers read x in the activation type: in fp32 that is x itself, in bf16 a rounded copy each norm kernel leaves
        if prec.f32:
            xa = x
        else:
            xa = x.to(torch.bfloat16)
        for li, blk in enumerate(self.blocks):
            y = blk.mixer(xa, b, store, li, prec)
            seq_ops.group_rmsnorm_add(y, blk.norm1_d, x, None if prec.f32 else xa, groups, eps)
            if blk.ff is not None:
                y = blk.ff(xa, b, prec)
                seq_ops.group_rmsnorm_add(y, blk.norm2_d, x, None if prec.f32 else xa, groups, eps)
            if blk.side is not None:
                y = blk.side(xa, b, self.side_embed_d, prec)
                seq_ops.group_rmsnorm_add(y, blk.side_norm_d, x, None if prec.f32 else xa, 1, eps)
            if trace is not None:
                trace.append(x.clone())
        if want_rows is None or want_rows.numel() == 0:
            return None
        last = x.index_select(0, want_rows)
        hn = prec.empty(*last.shape)
        seq_ops.group_rmsnorm_add(last, self.final_norm_d, None, hn, groups, eps)
        return seq_ops.linear(hn, self.head_d, torch.empty(last.shape[0], c.vocab, device="cuda", dtype=torch.float32))


def load_mapedra(path: str, dtype: torch.dtype = torch.bfloat16) -> MapedraForCausalLM:
    from .utils import read_safetensors
    model = MapedraForCausalLM(MapedraConfig.from_dir(path), dtype)
    return model.load_weights(read_safetensors(os.path.join(path, "model.safetensors")))
