"""Pukerax: a decoder-only language model of latent-attention layers over a multi-stream residual, with dense or routed
squared-relu feed-forwards, served through the ragged-step engine (engine.py).

    streams x_1..x_S <- embedding row                                 (S = config `streams`; 1 without the key)
    sub-layer q of a layer:  u = sum_s a_s x_s;  y = f_q(norm(u));  x_t <- sum_s M[s, t] x_s + b_t y     (f_1 mixer, f_2 feed-forward)
    logits = head(norm(sum_s x_s))                                    norm(u) = u / sqrt(mean(u^2) + eps) * (1 + w)

Every size and model-dependent constant comes from config.json (`PukeraxConfig`), tensor names from the checkpoint:

    embed, final.norm, head, l<i>.norm1, l<i>.norm2, l<i>.hc{1,2}.{in,out,mix},
    l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,g,o}, l<i>.mlp.{up,down} (dense),
    l<i>.mlp.{router,correction,e<k>.up,e<k>.down,shared.up,shared.down} (routed)

The streams are fp32; the write-back of one sub-layer and the normalised read of the next are one kernel pass
(seq_ops.stream_mix_norm).
"""
import json
import os
from typing import Dict, List, Optional

import torch

from . import _lib, seq_ops
from .mixers import LatentAttention, RoutedFeedForward, SquaredReluFeedForward, StreamCoefficients


class PukeraxConfig:
    def __init__(self, cfg: dict):
        if cfg.get("architecture") != "Pukerax":
            raise ValueError("not a Pukerax config")
        self.raw = cfg
        self.vocab = int(cfg["vocab"])
        self.width = int(cfg["width"])
        self.norm_eps = float(cfg["norm"]["eps"])
        self.hyper = "streams" in cfg
        self.streams = int(cfg.get("streams", 1))
        if not 1 <= self.streams <= 16:
            raise ValueError("streams must be between 1 and 16")
        self.layers: List[dict] = list(cfg["layers"])
        for i, l in enumerate(self.layers):
            if l["type"] != "latent_attention":
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
            if l.get("mlp") and l["mlp"].get("kind", "dense") not in ("dense", "moe"):
                raise ValueError(f"layer {i}: unknown feed-forward kind {l['mlp'].get('kind')!r}")

    @classmethod
    def from_dir(cls, path):
        with open(os.path.join(path, "config.json")) as f:
            return cls(json.load(f))


def _feed_forward(width: int, mlp: Optional[dict]):
    if not mlp:
        return None
    if mlp.get("kind", "dense") == "dense":
        return SquaredReluFeedForward(width, int(mlp["ff"]))
    r = mlp["router"]
    groups = r.get("groups") or {}
    shared = mlp.get("shared")
    return RoutedFeedForward(width, int(r["experts"]), int(r.get("identity", 0)), int(r["top"]), int(groups.get("count", 1)),
                             int(groups.get("keep", groups.get("count", 1))), float(r.get("scale", 1.0)), int(mlp["expert"]["ff"]),
                             int(shared["ff"]) if shared else 0)


class PukeraxBlock:
    def __init__(self, c: PukeraxConfig, i: int):
        l, m = c.layers[i], c.layers[i]["mixer"]
        rot = m.get("rot") or {}
        rot_dim = int(m.get("rot_dim", 0))
        self.mixer = LatentAttention(c.width, int(m["heads"]), int(m["dim"]), rot_dim, int(m.get("vdim", m["dim"])), int(m["q_rank"]),
                                     int(m["kv_rank"]), m["scale"], int(rot.get("dims", rot_dim)), rot.get("base", 10000.0), c.norm_eps)
        self.ff = _feed_forward(c.width, l.get("mlp"))
        self.hc1 = StreamCoefficients(c.streams)
        self.hc2 = StreamCoefficients(c.streams) if self.ff is not None else None
        self.i, self.hyper, self.D = i, c.hyper, c.width

    def load(self, take):
        p = f"l{self.i}."
        self.norm1 = take(p + "norm1", (self.D,))
        self.mixer.load(take, p + "mix.")
        if self.hyper:
            self.hc1.load(take, p + "hc1.")
        if self.ff is not None:
            self.norm2 = take(p + "norm2", (self.D,))
            self.ff.load(take, p + "mlp.")
            if self.hyper:
                self.hc2.load(take, p + "hc2.")

    def pack(self, prec):
        # the norm weights are stored around zero: the kernels multiply by 1 + w (formed once, in fp32)
        self.norm1_d = 1.0 + self.norm1.to("cuda", torch.float32)
        self.mixer.pack(prec)
        self.hc1.pack()
        if self.ff is not None:
            self.norm2_d = 1.0 + self.norm2.to("cuda", torch.float32)
            self.ff.pack(prec)
            self.hc2.pack()

    def sublayers(self):
        """[(function of (h, batch, store, layer, prec), stream coefficients, norm weight)] in order."""
        subs = [(lambda h, b, store, li, prec: self.mixer(h, b, store, li, prec), self.hc1, self.norm1_d)]
        if self.ff is not None:
            subs.append((lambda h, b, store, li, prec: self.ff(h, b, prec), self.hc2, self.norm2_d))
        return subs


class PukeraxForCausalLM:
    """Weights + the step function.  `step(batch, store, want_rows)` advances every entry of a ragged batch by its new
    tokens (the latent rows are left in `store`) and returns fp32 logits of the wanted rows."""

    architecture = "Pukerax"

    def __init__(self, config: PukeraxConfig, dtype: torch.dtype = torch.bfloat16):
        self.config = config
        self.prec = seq_ops.Precision(dtype)
        self.blocks = [PukeraxBlock(config, i) for i in range(len(config.layers))]
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
        self.final_norm_d = 1.0 + self.final_norm.to("cuda", torch.float32)
        self.head_d = self.head.to("cuda", dt).contiguous()
        self.ones_d = torch.ones(self.config.streams, device="cuda", dtype=torch.float32)
        for blk in self.blocks:
            blk.pack(self.prec)
        self._subs = [(li, *s) for li, blk in enumerate(self.blocks) for s in blk.sublayers()]
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
        c, prec, eps = self.config, self.prec, self.config.norm_eps
        xs = seq_ops.embed_streams(b.tokens, self.embed_d, c.streams, c.width)
        ha = prec.empty(b.T, c.width)
        subs = self._subs
        seq_ops.stream_mix_norm(xs, read=subs[0][2].read, norm_w=subs[0][3], out_act=ha, eps=eps)
        for k, (li, fn, hc, _w) in enumerate(subs):
            y = fn(ha, b, store, li, prec)
            nxt = subs[k + 1] if k + 1 < len(subs) else None
            # the write-back of this sub-layer and the normalised read of the next one in one pass over the streams
            seq_ops.stream_mix_norm(xs, y, hc.mix, hc.write, read=nxt[2].read if nxt else None, norm_w=nxt[3] if nxt else None,
                                    out_act=ha if nxt else None, eps=eps)
            if trace is not None and (nxt is None or nxt[0] != li):
                trace.append(xs.sum(1))
        if want_rows is None or want_rows.numel() == 0:
            return None
        last = xs.index_select(0, want_rows)
        hn = prec.empty(last.shape[0], c.width)
        seq_ops.stream_mix_norm(last, read=self.ones_d, norm_w=self.final_norm_d, out_act=hn, eps=eps)
        return seq_ops.linear(hn, self.head_d, torch.empty(last.shape[0], c.vocab, device="cuda", dtype=torch.float32))


def load_pukerax(path: str, dtype: torch.dtype = torch.bfloat16) -> PukeraxForCausalLM:
    from .utils import read_safetensors
    model = PukeraxForCausalLM(PukeraxConfig.from_dir(path), dtype)
    return model.load_weights(read_safetensors(os.path.join(path, "model.safetensors")))
