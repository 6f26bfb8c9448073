"""`bench.py --arch mapedra`: prefill and decode throughput of the Mapedra decoder at layer sizes of a real model (random
weights), beside the Gemma decoder of this package at equal width / heads / feed-forward / depth, plus a per-kernel table
(CUDA events, L2 flushed between launches) with each kernel's distance from its roofline and the like kernel of Gemma.

Rooflines use MEASURED_PEAKS.json (copy bandwidth, cuBLAS bf16 burst rate) when present.  Matrix products are the same
tcgen05 kernels in both models and are not listed again.
"""
import json
import os
import time

import torch

from . import _lib, seq_ops
from .cache import SequenceStore
from .engine import SequenceEngine
from .modeling_gemma import PAGE, GemmaConfig, GemmaForCausalLM, KVCache
from .modeling_mapedra import MapedraConfig, MapedraForCausalLM

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]) * 1e9, float(p["bf16_tflops"]) * 1e12, "measured"
    return 6650e9, 1590e12, "fallback"


def mapedra_config(width, heads, kv_heads, dim, ff, vocab, layers, every=4):
    """`every`-th layer softmax attention, the others lightning; feed-forward on every layer; a 64-wide token side table."""
    ls = []
    for i in range(layers):
        mlp = {"kind": "dense", "ff": ff}
        if (i + 1) % every == 0:
            ls.append({"type": "attention", "mlp": mlp,
                       "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "softcap": 50.0,
                                 "rot": {"base": 1e6, "dims": dim // 2, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}})
        else:
            ls.append({"type": "lightning", "mlp": mlp,
                       "mixer": {"heads": heads, "dim": dim, "vdim": dim, "decay": [1.0 - 2.0 ** (-5 - 3 * h / heads) for h in range(heads)]}})
    return {"architecture": "Mapedra", "vocab": vocab, "width": width, "embedding": {"scale": width ** 0.5}, "norm": {"eps": 1e-6, "groups": 4},
            "token_side": {"dim": 64}, "layers": ls}


def random_mapedra(cfg, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    c = MapedraConfig(cfg)
    model = MapedraForCausalLM(c, torch.bfloat16)
    shapes = {}

    def take(name, shape):
        shapes[name] = shape
        std = 1.0 if len(shape) == 1 else shape[-1] ** -0.5
        t = torch.randn(*shape, device="cuda", generator=g) * std
        return (t + 1.0 if len(shape) == 1 else t).to(torch.bfloat16)

    model.embed = take("embed", (c.vocab, c.width)) * 0.05
    model.side_embed = take("side.embed", (c.vocab, c.side_dim * len(c.layers))) if c.side_dim else None
    for blk in model.blocks:
        blk.load(take)
    model.final_norm, model.head = take("final.norm", (c.width,)), take("head", (c.vocab, c.width))
    model.pack()
    return model


def timed(fn, iters=5, warmup=2, flush=None):
    """Median device time of fn() in seconds; `flush` (a > L2 buffer) is rewritten before every timed launch."""
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.add_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e-3)
    return sorted(ts)[len(ts) // 2]


def run(args):
    _lib.require_device()
    torch.cuda.set_device(0)
    hbm, tflops, src = peaks()
    W, H, G, dh, F, V, L = args.width, args.heads, args.kv_heads, args.head_dim, args.ff, args.vocab, args.layers
    B_pre, S, B_dec, ctx = args.prefill_batch, args.seq_len, args.decode_batch, args.context
    flush = torch.zeros(64 * 1024 * 1024, device="cuda", dtype=torch.float32)  # 256 MB > L2
    out = {"metric": "mapedra_vs_gemma_tokens_per_s", "dtype": "bf16", "data": "synthetic", "peaks": src,
           "config": {"width": W, "heads": H, "kv_heads": G, "head_dim": dh, "ff": F, "vocab": V, "layers": L, "prefill": [B_pre, S],
                      "decode": [B_dec, ctx], "l2": "256 MB buffer rewritten before every timed launch"}}

    # ---------------------------------------------------------------- Mapedra end to end
    cfg = mapedra_config(W, H, G, dh, F, V, L)
    model = random_mapedra(cfg)
    n_att = sum(l["type"] == "attention" for l in cfg["layers"])
    eng = SequenceEngine(model, max_tokens=max(B_pre * S, B_dec * (ctx + PAGE)) + PAGE, num_slots=max(B_pre, B_dec))
    gen = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, V, (S,), generator=gen).tolist() for _ in range(B_pre)]

    def prefill():
        eng.step([(i, p, [S - 1]) for i, p in enumerate(prompts)], list(range(B_pre)))

    t = timed(prefill, iters=args.steps, warmup=args.warmup, flush=flush)
    out["mapedra_prefill_tok_s"] = B_pre * S / t
    # decode: B_dec sequences with `ctx` tokens each, then single-token steps
    long = [torch.randint(0, V, (ctx,), generator=gen).tolist() for _ in range(B_dec)]
    for i0 in range(0, B_dec, 8):
        eng.step([(("d", i), long[i], []) for i in range(i0, min(B_dec, i0 + 8))])

    def decode():
        eng.step([(("d", i), [7], [0]) for i in range(B_dec)])

    t = timed(decode, iters=max(args.steps, 8), warmup=args.warmup, flush=flush)
    out["mapedra_decode_tok_s"] = B_dec / t
    out["mapedra_decode_ms_per_step"] = t * 1e3
    for i in range(B_dec):
        eng.release(("d", i))

    # ---------------------------------------------------------------- Mapedra kernels
    prec, k = model.prec, {}
    att = next(b.mixer for b in model.blocks if hasattr(b.mixer, "G"))
    lin = next(b.mixer for b in model.blocks if hasattr(b.mixer, "decay"))
    li_att = next(i for i, b in enumerate(model.blocks) if hasattr(b.mixer, "G"))
    li_lin = next(i for i, b in enumerate(model.blocks) if hasattr(b.mixer, "decay"))
    store = eng.store

    def entries(n_seq, n_new, c0):
        es = []
        for i in range(n_seq):
            store.admit(("k", i))
            rec = store.reserve(("k", i), c0 + n_new)
            es.append(dict(tokens=[1] * n_new, ctx=c0, slot=rec.slot, pages=rec.pages))
        b = seq_ops.make_step_batch(es)
        return b

    def drop(n_seq):
        for i in range(n_seq):
            store.release(("k", i))

    for name, (n_seq, n_new, c0) in {"prefill": (B_pre, S, 0), "decode": (B_dec, 1, ctx)}.items():
        b = entries(n_seq, n_new, c0)
        T = b.T
        proj = torch.randn(T, att.w_in.shape[0], device="cuda").to(torch.bfloat16)
        q, o = prec.empty(T, H * dh), prec.empty(T, H * dh)
        kp, vp = store.k_pages[li_att], store.v_pages[li_att]
        kp.normal_()
        vp.normal_()
        gate = proj[:, (H + G) * dh + G * dh:]
        k[f"attn_prepare_{name}"] = dict(
            s=timed(lambda: seq_ops.attn_prepare(proj, b, att.freq_d, att.qn, att.kn, q, kp, vp, H, G, dh, dh, att.rot_dims, 1e-6, PAGE), flush=flush),
            bytes=T * (H + 2 * G) * dh * 2 * 2)
        pairs = n_seq * (n_new * c0 + n_new * (n_new + 1) // 2)
        k[f"attention_{name}"] = dict(
            s=timed(lambda: seq_ops.attn_ragged(q, kp, vp, gate, o, b, H, G, dh, dh, att.scale, att.softcap, PAGE), flush=flush),
            flops=4 * dh * H * pairs, bytes=n_seq * (c0 + n_new) * G * 2 * dh * 2 + 3 * T * H * dh * 2)
        projl = torch.randn(T, lin.w_in.shape[0], device="cuda").to(torch.bfloat16)
        ol = torch.empty(T, H * dh, device="cuda", dtype=torch.float32)
        k[f"lightning_{name}"] = dict(
            s=timed(lambda: seq_ops.linear_attn(projl, store.state[li_lin], lin.decay_d, ol, b, H, dh, dh), flush=flush),
            flops=T * H * 2 * (32 * dh + 32 * dh + 2 * dh * dh) if n_new > 1 else T * H * 4 * dh * dh,
            bytes=n_seq * H * dh * dh * 4 * 2 + T * H * dh * (3 * 2 + 4))
        attl = prec.empty(T, H * dh)
        k[f"lightning_norm_gate_{name}"] = dict(
            s=timed(lambda: seq_ops.rmsnorm_gate(ol, lin.norm, projl[:, 3 * H * dh:], attl, 1e-6), flush=flush), bytes=T * H * dh * (4 + 2 + 2))
        y, x, xa = torch.randn(T, W, device="cuda"), torch.randn(T, W, device="cuda"), prec.empty(T, W)
        w1 = torch.ones(W, device="cuda")
        k[f"group_norm_residual_{name}"] = dict(s=timed(lambda: seq_ops.group_rmsnorm_add(y, w1, x, xa, 4, 1e-6), flush=flush), bytes=T * W * (4 + 4 + 4 + 2))
        drop(n_seq)
    del eng, model, store
    torch.cuda.empty_cache()

    # ---------------------------------------------------------------- Gemma at equal size
    gc = GemmaConfig(hidden_size=W, intermediate_size=F, num_hidden_layers=L, num_attention_heads=H, num_key_value_heads=G, head_dim=dh,
                     vocab_size=V, rms_norm_eps=1e-6)
    gm = GemmaForCausalLM(gc, device="cuda", dtype=torch.bfloat16).eval()
    with torch.no_grad():
        for p in gm.parameters():
            if p.dim() == 2:
                p.normal_(0, p.shape[1] ** -0.5)
    gm.pack()
    L_ = _lib.lib()
    pos = torch.arange(S, device="cuda", dtype=torch.int32).repeat(B_pre)

    def g_prefill():
        h = torch.randn(B_pre * S, W, device="cuda")
        kv = KVCache()
        gm.prefill(h, pos, B_pre, S, kv, last_only=True)

    t = timed(g_prefill, iters=args.steps, warmup=args.warmup, flush=flush)
    out["gemma_prefill_tok_s"] = B_pre * S / t
    kv = KVCache()
    kv.allocate(B_dec, L, G, dh, ctx + PAGE)
    kv.k_pages.normal_()
    kv.v_pages.normal_()
    kv._set_len(ctx, L)
    kv.counters[0].fill_(ctx)
    kv.counters[1].fill_(ctx)
    kv.counters[2].fill_(ctx + 1)
    bufs = gm.decode_buffers(B_dec, private=True)

    def g_decode():
        bufs["h"].normal_()
        gm.decode_layers(bufs, kv, B_dec)

    t = timed(g_decode, iters=max(args.steps, 8), warmup=args.warmup, flush=flush)
    out["gemma_decode_tok_s"] = B_dec / t
    out["gemma_decode_ms_per_step"] = t * 1e3
    # Gemma kernels
    T = B_pre * S
    Wq = (H + 2 * G) * dh
    qkv = torch.randn(T, Wq, device="cuda").to(torch.bfloat16)
    qb, kb, vb = qkv, qkv[:, H * dh:], qkv[:, (H + G) * dh:]
    ao = torch.empty(T, H * dh, device="cuda", dtype=torch.bfloat16)
    Gq = H // G
    k["gemma_attention_prefill"] = dict(
        s=timed(lambda: _lib.check(L_.pg_attention_prefill(qb.data_ptr(), kb.data_ptr(), vb.data_ptr(), ao.data_ptr(), B_pre, G, S * Gq, S, dh, Gq,
                                                          S * Wq, Wq, dh, Gq * dh, S * Wq, Wq, dh, S * H * dh, H * dh, dh, Gq * dh, dh ** -0.5,
                                                          _lib.stream()), "attn"), flush=flush),
        flops=4 * dh * H * B_pre * S * S, bytes=T * Wq * 2 + T * H * dh * 2)
    qkvf = torch.randn(B_dec, Wq, device="cuda")
    ad = torch.empty(B_dec, H * dh, device="cuda", dtype=torch.bfloat16)
    k["gemma_attention_decode"] = dict(
        s=timed(lambda: _lib.check(L_.pg_attention_decode_fused(qkvf.data_ptr(), kv.counters[0].data_ptr(), kv.counters[2].data_ptr(),
                                                               gm._packed["inv_freq"].data_ptr(), kv.k_pages[0].data_ptr(), kv.v_pages[0].data_ptr(),
                                                               kv.page_table.data_ptr(), ad.data_ptr(), B_dec, H, G, dh, PAGE, kv.k_pages.shape[1],
                                                               kv.page_table.shape[1], dh ** -0.5, _lib.stream()), "attn_dec"), flush=flush),
        bytes=B_dec * (ctx + 1) * G * 2 * dh * 2)
    for name, rows in (("prefill", T), ("decode", B_dec)):
        hx, hn = torch.randn(rows, W, device="cuda"), torch.empty(rows, W, device="cuda", dtype=torch.bfloat16)
        w1 = torch.zeros(W, device="cuda")
        k[f"gemma_rmsnorm_{name}"] = dict(s=timed(lambda: _lib.rmsnorm(hx, w1, hn), flush=flush), bytes=rows * W * 6)
    for name, d in k.items():
        d["us"] = round(d.pop("s") * 1e6, 2)
        if "bytes" in d:
            d["hbm_frac"] = round(d["bytes"] / (d["us"] * 1e-6) / hbm, 4)
        if "flops" in d:
            d["tflops"] = round(d["flops"] / (d["us"] * 1e-6) / 1e12, 2)
            d["tensor_frac"] = round(d["flops"] / (d["us"] * 1e-6) / tflops, 5)
    out["kernels"] = k
    out["value"] = out["mapedra_decode_tok_s"]
    out["unit"] = "tokens/s"
    out["n_gpus"] = 1
    for key in list(out):
        if key.endswith("tok_s"):
            out[key] = round(out[key], 1)
    print(json.dumps(out), flush=True)
    return out
