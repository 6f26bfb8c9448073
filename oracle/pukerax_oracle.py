"""Plain, slow fp32 restatement of the Pukerax decoder (test infrastructure only; the product path never imports it).

One function per mechanism, one sequence at a time, nothing shared with the kernels or their host wrappers.

  streams       the residual is S copies x_1..x_S of the embedding row; a sub-layer q reads u = sum_s a_s x_s, computes
                y = f(norm(u)) and every stream is rebuilt from the old ones: x_t <- sum_s M[s, t] x_s + b_t y
  norm(u)       u / sqrt(mean(u^2) + eps) * (1 + w)                      (weights stored around zero)
  latent attn   c_q = rms(W_dq h) * w_q, q = W_uq c_q = per head [plain | rotated];  W_dkv h = [c_raw | r],
                c = rms(c_raw) * w_c, r rotated (one key part for all heads);  k_h = [W_uk,h c | r], v_h = W_uv,h c;
                softmax over the causal keys, head output times sigmoid(W_g h)_h, then W_o
  feed-forward  W_down relu(W_up h)^2, dense or as routed experts with identity experts, a grouped choice and a shared expert

A "weights" argument is a dict name -> fp32 tensor with the checkpoint's tensor names; "cfg" is the parsed config.json.
"""
import math

import torch


def rms(z, eps):
    return z / torch.sqrt((z * z).mean(-1, keepdim=True) + eps)


def norm_one_plus(z, w, eps):
    return rms(z, eps) * (1.0 + w)


def rotate_interleaved(vec, p, base, dims):
    """vec [..., n >= dims]: pair (2i, 2i+1), i < dims/2, turned by the angle p * base^(-2i/dims); the rest passes."""
    out = vec.clone()
    for i in range(dims // 2):
        a = float(p) * float(base) ** (-2.0 * i / dims)
        c, s = math.cos(a), math.sin(a)
        u, v = vec[..., 2 * i], vec[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def latent_attention(h, w, pre, m, eps):
    """h [T, D] of ONE sequence (positions 0..T-1) -> [T, D].  Builds keys / values of every head explicitly."""
    T = h.shape[0]
    H, dim, rd, vd, R = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    base, rdims = float(m["rot"]["base"]), int(m["rot"]["dims"])
    cq = rms(h @ w[pre + "dq"].T, eps) * w[pre + "dq.norm"]
    q = (cq @ w[pre + "uq"].T).reshape(T, H, dim + rd)
    kv = h @ w[pre + "dkv"].T
    c = rms(kv[:, :R], eps) * w[pre + "dkv.norm"]
    r = kv[:, R:]
    kn = (c @ w[pre + "uk"].T).reshape(T, H, dim)
    v = (c @ w[pre + "uv"].T).reshape(T, H, vd)
    gate = torch.sigmoid(h @ w[pre + "g"].T)  # [T, H]
    out = torch.zeros(T, H, vd, dtype=h.dtype)
    rk = torch.stack([rotate_interleaved(r[j], j, base, rdims) for j in range(T)])
    for i in range(T):
        for hh in range(H):
            qr = rotate_interleaved(q[i, hh, dim:], i, base, rdims)
            s = (kn[: i + 1, hh] @ q[i, hh, :dim] + rk[: i + 1] @ qr) * float(m["scale"])
            p = torch.softmax(s, 0)
            out[i, hh] = (p[:, None] * v[: i + 1, hh]).sum(0) * gate[i, hh]
    return out.reshape(T, H * vd) @ w[pre + "o"].T


def relu2_ff(h, up, down):
    return torch.relu(h @ up.T) ** 2 @ down.T


def route(h, w, pre, r):
    """One token h [D] -> (chosen ids, weights).  Ids >= experts - identity ... are counted over experts + identity outputs."""
    n_all = int(r["experts"]) + int(r.get("identity", 0))
    s = torch.softmax(w[pre + "router"] @ h, 0)
    choice = s + w[pre + "correction"]
    groups = r.get("groups")
    if groups and int(groups["count"]) > 1:
        cnt, keep = int(groups["count"]), int(groups["keep"])
        per = n_all // cnt
        gscore = choice.reshape(cnt, per).max(1).values
        kept = torch.topk(gscore, keep).indices.tolist()
        mask = torch.full_like(choice, float("-inf")).reshape(cnt, per)
        for g in kept:
            mask[g] = 0.0
        choice = choice + mask.reshape(-1)
    ids = torch.topk(choice, int(r["top"])).indices
    wt = s[ids]
    wt = wt / (wt.sum() + 1e-20) * float(r["scale"])
    return ids.tolist(), wt


def moe_ff(h, w, pre, mlp):
    """h [T, D] -> [T, D]: routed experts (the last `identity` router outputs return h itself) plus the shared expert."""
    r = mlp["router"]
    n_real = int(r["experts"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        ids, wt = route(h[t], w, pre, r)
        for e, g in zip(ids, wt):
            if e >= n_real:
                out[t] += g * h[t]
            else:
                out[t] += g * relu2_ff(h[t][None], w[f"{pre}e{e}.up"], w[f"{pre}e{e}.down"])[0]
    if mlp.get("shared"):
        out = out + relu2_ff(h, w[pre + "shared.up"], w[pre + "shared.down"])
    return out


def feed_forward(h, w, pre, mlp):
    if mlp["kind"] == "dense":
        return relu2_ff(h, w[pre + "up"], w[pre + "down"])
    if mlp["kind"] == "moe":
        return moe_ff(h, w, pre, mlp)
    raise ValueError(mlp["kind"])


def hyper_sublayer(xs, w, pre, norm_w, eps, fn):
    """xs [T, S, D]; one sub-layer with its read vector a, write vector b and mixing matrix M[from, to]."""
    a, b, M = w[pre + "in"], w[pre + "out"], w[pre + "mix"]
    u = torch.einsum("s,tsd->td", a, xs)
    y = fn(norm_one_plus(u, norm_w, eps))
    return torch.einsum("sr,tsd->trd", M, xs) + b[None, :, None] * y[:, None, :]


def forward(w, cfg, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the stream sum after every layer when asked)."""
    eps = float(cfg["norm"]["eps"])
    S = int(cfg.get("streams", 1))
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    xs = x[:, None, :].repeat(1, S, 1)
    layers = []
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        if l["type"] != "latent_attention":
            raise ValueError(l["type"])
        mixer = lambda h, p=p, l=l: latent_attention(h, w, p + "mix.", l["mixer"], eps)
        if S > 1 or (p + "hc1.in") in w:
            xs = hyper_sublayer(xs, w, p + "hc1.", w[p + "norm1"], eps, mixer)
        else:
            xs = xs + mixer(norm_one_plus(xs[:, 0], w[p + "norm1"], eps))[:, None]
        if l.get("mlp"):
            ff = lambda h, p=p, l=l: feed_forward(h, w, p + "mlp.", l["mlp"])
            if S > 1 or (p + "hc2.in") in w:
                xs = hyper_sublayer(xs, w, p + "hc2.", w[p + "norm2"], eps, ff)
            else:
                xs = xs + ff(norm_one_plus(xs[:, 0], w[p + "norm2"], eps))[:, None]
        layers.append(xs.sum(1))
    logits = norm_one_plus(xs.sum(1), w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(layers)) if return_layers else logits


# ------------------------------------------------------------------------------------------------------------------
# random checkpoints for tests
# ------------------------------------------------------------------------------------------------------------------
def tensor_shapes(cfg):
    D, V, S = int(cfg["width"]), int(cfg["vocab"]), int(cfg.get("streams", 1))
    sh = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        H, dim, rd, vd, R, Q = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"))
        sh.update({p + "norm1": (D,), p + "mix.dq": (Q, D), p + "mix.dq.norm": (Q,), p + "mix.uq": (H * (dim + rd), Q),
                   p + "mix.dkv": (R + rd, D), p + "mix.dkv.norm": (R,), p + "mix.uk": (H * dim, R), p + "mix.uv": (H * vd, R),
                   p + "mix.g": (H, D), p + "mix.o": (D, H * vd)})
        if "streams" in cfg:
            sh.update({p + "hc1.in": (S,), p + "hc1.out": (S,), p + "hc1.mix": (S, S)})
        mlp = l.get("mlp")
        if mlp:
            sh[p + "norm2"] = (D,)
            if "streams" in cfg:
                sh.update({p + "hc2.in": (S,), p + "hc2.out": (S,), p + "hc2.mix": (S, S)})
            if mlp["kind"] == "dense":
                sh.update({p + "mlp.up": (int(mlp["ff"]), D), p + "mlp.down": (D, int(mlp["ff"]))})
            else:
                r = mlp["router"]
                n_all = int(r["experts"]) + int(r.get("identity", 0))
                sh.update({p + "mlp.router": (n_all, D), p + "mlp.correction": (n_all,)})
                for e in range(int(r["experts"])):
                    sh.update({f"{p}mlp.e{e}.up": (int(mlp["expert"]["ff"]), D), f"{p}mlp.e{e}.down": (D, int(mlp["expert"]["ff"]))})
                if mlp.get("shared"):
                    sh.update({p + "mlp.shared.up": (int(mlp["shared"]["ff"]), D), p + "mlp.shared.down": (D, int(mlp["shared"]["ff"]))})
    return sh


def random_weights(cfg, seed=0):
    """bf16-representable fp32 tensors.  Projections ~ 1/sqrt(fan-in), norm weights around zero (or one for the plain ones),
    stream matrices near the identity."""
    g = torch.Generator().manual_seed(seed)
    S = int(cfg.get("streams", 1))
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith(("dq.norm", "dkv.norm")):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name.endswith(("norm1", "norm2", "final.norm")):
            t = 0.2 * torch.randn(shape, generator=g)
        elif name.endswith("correction"):
            t = 0.05 * torch.randn(shape, generator=g)
        elif name.endswith((".in", ".out")):
            t = 1.0 / S + 0.3 * torch.randn(shape, generator=g) if name.endswith(".in") else 1.0 + 0.3 * torch.randn(shape, generator=g)
        elif name.endswith(".mix"):
            t = torch.eye(S) + 0.2 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif name.endswith("router"):
            t = 2.0 * torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out
