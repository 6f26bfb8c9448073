"""Plain, slow fp32 restatement of the Mapedra decoder (test infrastructure only; the product path never imports it).

One function per mechanism, written from the design's equations in the notation below; every function works on one
sequence, token by token where the design is recurrent, and shares nothing with the kernels or their host wrappers.

  x_t           residual stream of token t (width D)
  rms(z)        z / sqrt(mean(z^2) + eps)
  layer         x <- x + gnorm1(mixer(x));  x <- x + gnorm2(ff(x)) (when the layer has a feed-forward);
                x <- x + rms(P (gelu(G x) * e_t)) * w_side   (e_t: the layer's slice of the token's side embedding)
  gnorm         the vector is cut into `groups` consecutive parts, each part is rms-normalised by itself, then * w

A "weights" argument is a dict name -> fp32 tensor with the checkpoint's tensor names; a "cfg" argument is the parsed
config.json.
"""
import math

import torch


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms(z, eps):
    return z / torch.sqrt((z * z).mean(-1, keepdim=True) + eps)


def group_norm(z, w, groups, eps):
    """z [..., D]: each of the `groups` consecutive parts divided by its own root mean square, whole times w."""
    shp = z.shape
    parts = z.reshape(*shp[:-1], groups, shp[-1] // groups)
    return rms(parts, eps).reshape(shp) * w


def rope_frequencies(rot):
    """f_i = base^(-2i/dims) with the long-wavelength rescaling: wavelengths below original/high keep f, above
    original/low get f/factor, between them a linear blend in original/wavelength."""
    dims = int(rot["dims"])
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = float(rot["base"]) ** (-2.0 * i / dims)
        if sc:
            wl = 2.0 * math.pi / f
            if wl < sc["original"] / sc["high"]:
                pass
            elif wl > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            else:
                s = (sc["original"] / wl - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return out


def rotate_interleaved(vec, p, freqs):
    """vec [..., dim]: the pairs (2i, 2i+1), i < len(freqs), are rotated by p * f_i; the remaining dimensions pass."""
    out = vec.clone()
    for i, f in enumerate(freqs):
        a = torch.tensor(float(p) * f, dtype=torch.float64)
        c, s = torch.cos(a).float(), torch.sin(a).float()
        u, v = vec[..., 2 * i], vec[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def attention_mixer(h, w, pre, m, eps):
    """h [T, D] -> [T, D].  Softmax attention with grouped key/value heads, per-head q/k norm before the rotation,
    weightless value norm, tanh soft cap on the scaled scores, causal, sigmoid output gate before the output projection."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    freqs = rope_frequencies(m["rot"])
    q = (h @ w[pre + "q"].T).view(T, H, dim)
    k = (h @ w[pre + "k"].T).view(T, G, dim)
    v = (h @ w[pre + "v"].T).view(T, G, vdim)
    gate = torch.sigmoid(h @ w[pre + "g"].T)
    q = rms(q, eps) * w[pre + "q.norm"]
    k = rms(k, eps) * w[pre + "k.norm"]
    v = rms(v, eps)
    for t in range(T):
        q[t] = rotate_interleaved(q[t], t, freqs)
        k[t] = rotate_interleaved(k[t], t, freqs)
    out = torch.zeros(T, H, vdim)
    cap = m.get("softcap")
    for t in range(T):
        for hd in range(H):
            g = hd // (H // G)
            s = (k[: t + 1, g] @ q[t, hd]) * m["scale"]
            if cap:
                s = cap * torch.tanh(s / cap)
            p = torch.softmax(s, 0)
            out[t, hd] = p @ v[: t + 1, g]
    return (out.reshape(T, H * vdim) * gate) @ w[pre + "o"].T


def lightning_mixer(h, w, pre, m, eps):
    """h [T, D] -> [T, D].  Per head S_t = a S_{t-1} + k_t v_t^T, o_t = S_t^T q_t with q, k, v = silu(projection); heads
    concatenated, rms-normalised together with a plain weight, gated by sigmoid(W_g h), projected."""
    T = h.shape[0]
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    silu = torch.nn.functional.silu
    q = silu(h @ w[pre + "q"].T).view(T, H, dim)
    k = silu(h @ w[pre + "k"].T).view(T, H, dim)
    v = silu(h @ w[pre + "v"].T).view(T, H, vdim)
    gate = torch.sigmoid(h @ w[pre + "g"].T)
    S = torch.zeros(H, dim, vdim)
    decay = torch.tensor(m["decay"], dtype=torch.float32).view(H, 1, 1)
    out = torch.zeros(T, H, vdim)
    for t in range(T):
        S = decay * S + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(out.reshape(T, H * vdim), eps) * w[pre + "norm"]
    return (o * gate) @ w[pre + "o"].T


def dense_ff(h, w, pre):
    return (gelu_tanh(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def side_input(x, tokens, w, i, dim, eps):
    """The per-layer token input: rms(P (gelu(G x) * e)) * w_side, e = columns [i*dim, (i+1)*dim) of the side table."""
    pre = f"l{i}.side."
    e = w["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    y = (gelu_tanh(x @ w[pre + "gate"].T) * e) @ w[pre + "proj"].T
    return rms(y, eps) * w[pre + "norm"]


MIXERS = {"attention": attention_mixer, "lightning": lightning_mixer}


def forward(cfg, w, tokens, return_layers=False):
    """tokens: list[int] -> fp32 logits [T, vocab] (and the residual stream after every layer)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    x = w["embed"][tokens] * cfg["embedding"]["scale"]
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        y = MIXERS[layer["type"]](x, w, pre + "mix.", layer["mixer"], eps)
        x = x + group_norm(y, w[pre + "norm1"], groups, eps)
        if layer.get("mlp"):
            x = x + group_norm(dense_ff(x, w, pre + "mlp."), w[pre + "norm2"], groups, eps)
        if cfg.get("token_side"):
            x = x + side_input(x, tokens, w, i, cfg["token_side"]["dim"], eps)
        layers.append(x.clone())
    logits = group_norm(x, w["final.norm"], groups, eps) @ w["head"].T
    return (logits, torch.stack(layers)) if return_layers else logits


def random_weights(cfg, seed=0, std=None):
    """fp32 weights (bf16-representable) with the checkpoint's tensor names for `cfg`; norm weights near one."""
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]

    def lin(o, i):
        return (torch.randn(o, i, generator=g) * (std or i ** -0.5)).bfloat16().float()

    def nw(n):
        return (1.0 + 0.1 * torch.randn(n, generator=g)).bfloat16().float()

    w = {"embed": (torch.randn(V, D, generator=g) * 0.05).bfloat16().float(), "final.norm": nw(D), "head": lin(V, D)}
    sd = cfg.get("token_side", {}).get("dim") if cfg.get("token_side") else None
    if sd:
        w["side.embed"] = torch.randn(V, sd * len(cfg["layers"]), generator=g).bfloat16().float()
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        w[p + "norm1"] = nw(D)
        if layer["type"] == "attention":
            w[p + "mix.q"] = lin(m["heads"] * m["dim"], D)
            w[p + "mix.k"] = lin(m["kv_heads"] * m["dim"], D)
            w[p + "mix.v"] = lin(m["kv_heads"] * m["vdim"], D)
            w[p + "mix.q.norm"], w[p + "mix.k.norm"] = nw(m["dim"]), nw(m["dim"])
            w[p + "mix.g"] = lin(m["heads"] * m["vdim"], D)
            w[p + "mix.o"] = lin(D, m["heads"] * m["vdim"])
        else:
            w[p + "mix.q"], w[p + "mix.k"] = lin(m["heads"] * m["dim"], D), lin(m["heads"] * m["dim"], D)
            w[p + "mix.v"], w[p + "mix.g"] = lin(m["heads"] * m["vdim"], D), lin(m["heads"] * m["vdim"], D)
            w[p + "mix.norm"] = nw(m["heads"] * m["vdim"])
            w[p + "mix.o"] = lin(D, m["heads"] * m["vdim"])
        if layer.get("mlp"):
            ff = layer["mlp"]["ff"]
            w[p + "norm2"] = nw(D)
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = lin(ff, D), lin(ff, D), lin(D, ff)
        if sd:
            w[p + "side.gate"], w[p + "side.proj"], w[p + "side.norm"] = lin(sd, D), lin(D, sd), nw(D)
    return w
