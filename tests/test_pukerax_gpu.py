"""Pukerax through the framework (kernels, latent page pool, ragged steps, scheduler) against the plain fp32 oracle
(oracle/pukerax_oracle.py): every mechanism alone, then whole models under every way of cutting and batching the work."""
import copy
import json
import os
import struct
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import pukerax_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu

F32_TOL, BF16_TOL = 2e-4, 4e-2


def mixer_cfg(heads=3, dim=24, rot_dim=8, vdim=40, kv_rank=48, q_rank=40, base=5000.0, scale=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
            "rot": {"base": base, "dims": rot_dim}, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}


def dense(ff=80):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, identity=2, top=3, count=4, keep=2, scale=1.5, ff=24, shared=40):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}
    if count:
        m["router"]["groups"] = {"count": count, "keep": keep}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(mlp, **kw):
    return {"type": "latent_attention", "mixer": mixer_cfg(**kw), "mlp": mlp}


def make_cfg(layers, width=72, vocab=90, streams=3, eps=1e-5):
    cfg = {"architecture": "Pukerax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams:
        cfg["streams"] = streams
    return cfg


BASE_CFG = make_cfg([layer(dense()), layer(moe()), layer(None, heads=2, dim=16, rot_dim=16, vdim=16, kv_rank=24, q_rank=16),
                     layer(moe(experts=5, identity=0, top=2, count=0, shared=0, scale=1.0))])


def build(cfg, w, dtype):
    from paligemma_multimodal_system_b200.modeling_pukerax import PukeraxConfig, PukeraxForCausalLM
    return PukeraxForCausalLM(PukeraxConfig(cfg), dtype).load_weights({k: v.to(torch.bfloat16) for k, v in w.items()})


def engine_for(cfg, w, dtype, max_tokens=1024, slots=4):
    from paligemma_multimodal_system_b200.engine import SequenceEngine
    return SequenceEngine(build(cfg, w, dtype), max_tokens, slots)


def poison(engine):
    """Stale memory must never be read: pages start as huge values instead of zeros."""
    for t in engine.store.k_pages:
        if t is not None:
            t.fill_(1e4)


def rel_err(got, ref):
    got, ref = got.double().cpu(), ref.double()
    return float((got - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt())


def close(got, ref, dtype):
    """fp32: the whole tensor within F32_TOL.  bf16: nine rows in ten within BF16_TOL -- a routed layer may hand a token whose
    two best choice scores nearly tie to the other expert, which moves that token's row and nothing else."""
    if dtype == torch.float32:
        return rel_err(got, ref) < F32_TOL
    got, ref = got.double().cpu(), ref.double()
    rows = (got - ref).pow(2).mean(-1).sqrt() / ref.pow(2).mean(-1).sqrt()
    return float(rows.quantile(0.9)) < BF16_TOL and float(rows.median()) < BF16_TOL / 2


def toks(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def run_cut(engine, rid, tokens, cuts):
    """Feeds `tokens` in portions of the given sizes (the last size repeats); returns logits of every position."""
    out, pos, i = [], 0, 0
    while pos < len(tokens):
        k = min(cuts[min(i, len(cuts) - 1)], len(tokens) - pos)
        out.append(engine.step([(rid, tokens[pos:pos + k], list(range(k)))], [rid] if pos + k == len(tokens) else []))
        pos, i = pos + k, i + 1
    return torch.cat(out)


def _one_entry(spec, T, dtype, ctx=0):
    from paligemma_multimodal_system_b200 import seq_ops
    from paligemma_multimodal_system_b200.cache import SequenceStore
    store = SequenceStore([spec], max_tokens=(ctx + T + 63) // 64 * 64 + 128, num_slots=1, dtype=dtype)
    store.pool.take(2)  # the entry's pages do not start at page 0
    store.admit("a")
    rec = store.reserve("a", ctx + T)
    b = seq_ops.make_step_batch([dict(tokens=[0] * T, ctx=ctx, slot=rec.slot, pages=rec.pages)])
    return store, b


# ----------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ----------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("S,D", [(1, 40), (2, 33), (4, 96), (8, 130), (12, 64)])
@pytest.mark.parametrize("f32", [True, False])
def test_stream_write_back_and_normalised_read(S, D, f32):
    from paligemma_multimodal_system_b200 import seq_ops
    g = torch.Generator().manual_seed(S * 100 + D)
    T, eps = 9, 1e-5
    xs = torch.randn(T, S, D, generator=g)
    y = torch.randn(T, D, generator=g)
    w = {"h.in": torch.randn(S, generator=g), "h.out": torch.randn(S, generator=g), "h.mix": torch.eye(S) + 0.3 * torch.randn(S, S, generator=g)}
    a2, nw = torch.randn(S, generator=g), 0.3 * torch.randn(D, generator=g)
    # oracle: write back y through (mix, out), then the next read with a2 and its norm
    new = torch.einsum("sr,tsd->trd", w["h.mix"], xs) + w["h.out"][None, :, None] * y[:, None, :]
    ref_read = O.norm_one_plus(torch.einsum("s,tsd->td", a2, new), nw, eps)
    xd = xs.cuda().contiguous()
    out = torch.empty(T, D, device="cuda", dtype=torch.float32 if f32 else torch.bfloat16)
    seq_ops.stream_mix_norm(xd, y.cuda(), w["h.mix"].cuda().contiguous(), w["h.out"].cuda(), read=a2.cuda(), norm_w=(1.0 + nw).cuda(), out_act=out, eps=eps)
    assert torch.allclose(xd.cpu(), new, atol=1e-5, rtol=1e-5)
    assert rel_err(out.float(), ref_read) < (1e-5 if f32 else 5e-3)
    # read alone (first sub-layer of a step) leaves the streams untouched; write-back alone (last one) writes no read
    x2 = xs.cuda().contiguous()
    seq_ops.stream_mix_norm(x2, read=a2.cuda(), norm_w=(1.0 + nw).cuda(), out_act=out, eps=eps)
    assert torch.equal(x2.cpu(), xs)
    assert rel_err(out.float(), O.norm_one_plus(torch.einsum("s,tsd->td", a2, xs), nw, eps)) < (1e-5 if f32 else 5e-3)
    seq_ops.stream_mix_norm(x2, y.cuda(), w["h.mix"].cuda().contiguous(), w["h.out"].cuda())
    assert torch.allclose(x2.cpu(), new, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("kw", [dict(), dict(heads=5, dim=20, rot_dim=6, vdim=12, kv_rank=36, q_rank=28),
                                dict(heads=2, dim=64, rot_dim=32, vdim=64, kv_rank=128, q_rank=48, scale=0.05),
                                dict(heads=1, dim=8, rot_dim=2, vdim=8, kv_rank=8, q_rank=8)])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 3e-2)])
def test_latent_attention_alone(kw, dtype, tol):
    """The absorbed form over the one-row cache against explicit per-head keys and values; positions 0 .. T-1 in one portion and
    as a context of 70 cached tokens followed by a portion and a single token."""
    from paligemma_multimodal_system_b200 import seq_ops
    from paligemma_multimodal_system_b200.mixers import LatentAttention
    m, D, T, eps = mixer_cfg(**kw), 56, 101, 1e-5
    cfg = make_cfg([layer(None, **kw)], width=D)
    w = {k[len("l0.mix."):]: v for k, v in O.random_weights(cfg, seed=3).items() if k.startswith("l0.mix.")}
    g = torch.Generator().manual_seed(5)
    h = torch.randn(T, D, generator=g).to(torch.bfloat16).float()
    ref = O.latent_attention(h, {"m." + k: v for k, v in w.items()}, "m.", m, eps)
    mix = LatentAttention(D, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"], m["scale"], m["rot"]["dims"], m["rot"]["base"], eps)
    mix.load(lambda name, shape: w[name].to(torch.bfloat16), "")
    prec = seq_ops.Precision(dtype)
    mix.pack(prec)
    for cuts in ([T], [70, 30, 1]):
        store, _ = _one_entry(mix.cache_spec(), T, dtype)
        store.k_pages[0].fill_(1e4)
        outs, pos = [], 0
        rec = store.live["a"]
        for n in cuts:
            b = seq_ops.make_step_batch([dict(tokens=[0] * n, ctx=pos, slot=rec.slot, pages=rec.pages)])
            outs.append(mix(h[pos:pos + n].to(dtype).cuda().contiguous(), b, store, 0, prec))
            pos += n
        assert rel_err(torch.cat(outs), ref) < tol, cuts


@pytest.mark.parametrize("ctx,n", [(0, 200), (130, 70), (199, 1), (64, 1), (63, 2), (1100, 1), (1060, 40)])
@pytest.mark.parametrize("needle", [0, 1, 63, 64, 65, 127, 128, 1023, 1024])
def test_far_latent_row_at_page_borders_is_found(ctx, n, needle):
    """One cached row among hundreds is aligned with the last query and scaled up: the output of the last row must be that
    row's leading columns.  As a prompt portion and as a decoded token (long contexts split the keys over several CTAs)."""
    from paligemma_multimodal_system_b200 import seq_ops
    H, R, rot, total = 3, 40, 8, ctx + n
    kd = R + rot
    needle = min(needle, total - 1)
    g = torch.Generator().manual_seed(needle * 7 + n)
    store, b = _one_entry(("latent", kd), n, torch.float32, ctx=ctx)
    rows = torch.randn(total, kd, generator=g) * 0.1
    q = torch.randn(n, H, kd, generator=g) * 0.1
    q[-1] = torch.randn(H, kd, generator=g)
    rows[needle] = q[-1, 1] * 4 / q[-1, 1].norm()
    q[-1, 1] = q[-1, 1] * 8 / q[-1, 1].norm()
    pages = b.page_table[0].tolist()
    store.k_pages[0].fill_(1e4)
    for j in range(total):
        store.k_pages[0][pages[j // 64], j % 64] = rows[j].cuda()
    gate = torch.randn(n, H, generator=g)
    out = torch.empty(n, H * R, device="cuda", dtype=torch.float32)
    seq_ops.attn_ragged(q.reshape(n, H * kd).cuda().contiguous(), store.k_pages[0], store.k_pages[0], gate.cuda(), out, b, H, 1, kd, R, 1.0, 0.0, 64,
                        krow=kd, vrow=kd, gate_per_head=True)
    ref = torch.zeros(n, H, R)
    for i in range(n):
        s = torch.einsum("hd,jd->hj", q[i], rows[: ctx + i + 1])
        ref[i] = (torch.softmax(s, -1) @ rows[: ctx + i + 1, :R]) * torch.sigmoid(gate[i])[:, None]
    assert torch.allclose(out.cpu().view(n, H, R), ref, atol=2e-5, rtol=1e-4)
    w = torch.softmax(torch.einsum("d,jd->j", q[-1, 1], rows), 0)
    assert w[needle] > 0.99


@pytest.mark.parametrize("T,B,K,F,extra", [(1, 3, 64, 256, 32), (64, 32, 64, 256, 32), (130, 5, 256, 64, 0), (70, 2, 40, 24, 8), (9, 4, 20, 12, 6), (200, 3, 33, 17, 1)])
@pytest.mark.parametrize("f32", [False, True])
def test_per_head_products_on_column_slices(T, B, K, F, extra, f32):
    """out[:, b, :] = x[:, b, :K] w[b]^T with x and out column slices of wider per-head rows (the absorbed query and the value up
    projection); bf16 slices on 16-byte boundaries take the tensor-core kernel, the others plain FMAs."""
    from paligemma_multimodal_system_b200 import seq_ops
    dt = torch.float32 if f32 else torch.bfloat16
    g = torch.Generator().manual_seed(T + K)
    xw = torch.randn(T, B, K + extra, generator=g).to(dt)
    w = (torch.randn(B, F, K, generator=g) / K ** 0.5).to(dt)
    outw = torch.full((T, B, F + extra), 7.0, dtype=dt).cuda()
    xd = xw.cuda()
    seq_ops.linear_batched(xd[:, :, :K], w.cuda().contiguous(), outw[:, :, :F])
    ref = torch.einsum("tbk,bfk->tbf", xw[:, :, :K].double(), w.double())
    assert rel_err(outw[:, :, :F].float(), ref) < (1e-5 if f32 else 6e-3)
    assert bool((outw[:, :, F:] == 7.0).all())  # nothing written outside the slice


@pytest.mark.parametrize("R,rot", [(64, 32), (128, 32), (128, 64), (256, 32)])
@pytest.mark.parametrize("H,ctxs", [(3, [0, 63]), (16, [64, 700]), (40, [2100, 5]), (70, [129, 1023, 64])])
def test_tensor_core_latent_decode_keeps_fp32_probabilities(R, rot, H, ctxs):
    """Single-token entries in bf16 over the one-row cache: every head of a token against the same key tile, the values read
    from the key tile itself, long contexts split over CTAs.  One row per entry stands out (its weight must survive the three
    bf16 terms of the probabilities); compared with a float64 softmax over the same bf16 inputs."""
    from paligemma_multimodal_system_b200 import seq_ops
    from paligemma_multimodal_system_b200.cache import SequenceStore
    kd = R + rot
    assert (kd, R) in seq_ops.LATENT_MMA_SIZES
    g = torch.Generator().manual_seed(R + H)
    store = SequenceStore([("latent", kd)], max_tokens=sum((c + 64) // 64 * 64 for c in ctxs) + 64, num_slots=len(ctxs), dtype=torch.bfloat16)
    store.k_pages[0].fill_(1e4)
    store.pool.take(1)
    es, rows_all, qs = [], [], []
    for i, ctx in enumerate(ctxs):
        store.admit(i)
        rec = store.reserve(i, ctx + 1)
        rows = (torch.randn(ctx + 1, kd, generator=g) * 0.3).to(torch.bfloat16)
        q = (torch.randn(H, kd, generator=g) * 0.3).to(torch.bfloat16)
        needle = (ctx * 2) // 3
        rows[needle] = (q[H // 2].float() * 3 / q[H // 2].float().norm()).to(torch.bfloat16)
        q[H // 2] = (q[H // 2].float() * 6 / q[H // 2].float().norm()).to(torch.bfloat16)
        for j in range(ctx + 1):
            store.k_pages[0][rec.pages[j // 64], j % 64] = rows[j].cuda()
        es.append(dict(tokens=[0], ctx=ctx, slot=rec.slot, pages=rec.pages))
        rows_all.append(rows)
        qs.append(q)
    b = seq_ops.make_step_batch(es)
    E = len(ctxs)
    gate = torch.randn(E, H, generator=g).to(torch.bfloat16)
    out = torch.empty(E, H * R, device="cuda", dtype=torch.bfloat16)
    qd = torch.stack(qs).reshape(E, H * kd).cuda().contiguous()
    seq_ops.attn_ragged(qd, store.k_pages[0], store.k_pages[0], gate.cuda(), out, b, H, 1, kd, R, 0.7, 0.0, 64, krow=kd, vrow=kd, gate_per_head=True)
    plain = torch.empty_like(out)
    seq_ops.attn_ragged(qd, store.k_pages[0], store.k_pages[0], gate.cuda(), plain, b, H, 1, kd, R, 0.7, 0.0, 64, krow=kd, vrow=kd, gate_per_head=True,
                        tensor_cores=False)
    for i in range(E):
        s = (qs[i].double() @ rows_all[i].double().T) * 0.7
        ref = (torch.softmax(s, -1) @ rows_all[i][:, :R].double()) * torch.sigmoid(gate[i].double())[:, None]
        got = out[i].view(H, R).double().cpu()
        assert float((got - ref).abs().max()) < 6e-3 * max(1.0, float(ref.abs().max())), (i, ctxs[i])
        assert float((plain[i].view(H, R).double().cpu() - ref).abs().max()) < 6e-3 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("kw", [dict(n_all=8, n_real=6, top=3, count=4, keep=2), dict(n_all=20, n_real=17, top=4, count=5, keep=2),
                                dict(n_all=5, n_real=5, top=2, count=1, keep=1), dict(n_all=64, n_real=60, top=8, count=8, keep=3),
                                dict(n_all=7, n_real=4, top=7, count=1, keep=1), dict(n_all=12, n_real=12, top=1, count=6, keep=1)])
@pytest.mark.parametrize("negative", [False, True])
def test_router_choice_weights_and_counts(kw, negative):
    """Choice by probability + correction inside the kept groups, weights from the uncorrected probabilities.  With a strongly
    negative correction every choice score is below zero: a dropped group must count as minus infinity, not as zero."""
    from paligemma_multimodal_system_b200 import seq_ops
    n_all, n_real, top = kw["n_all"], kw["n_real"], kw["top"]
    g = torch.Generator().manual_seed(n_all * 31 + top)
    T, D = 37, n_all  # the oracle multiplies router @ h: an identity router makes h the logits
    z = torch.randn(T, n_all, generator=g) * 2.0
    corr = torch.randn(n_all, generator=g) * 0.1 - (3.0 if negative else 0.0)
    w = {"r.router": torch.eye(n_all), "r.correction": corr}
    r = {"experts": n_real, "identity": n_all - n_real, "top": top, "scale": 1.7, "groups": {"count": kw["count"], "keep": kw["keep"]}}
    ids, wts, counts = seq_ops.moe_route(z.cuda(), corr.cuda(), n_real, top, kw["count"], kw["keep"], 1.7)
    torch.cuda.synchronize()
    want_counts = [0] * n_real
    for t in range(T):
        rid, rw = O.route(z[t], w, "r.", r)
        assert ids[t].tolist() == rid, t
        assert torch.allclose(wts[t].cpu(), rw, atol=1e-6, rtol=1e-5)
        for e in rid:
            if e < n_real:
                want_counts[e] += 1
    assert counts.tolist() == want_counts


@pytest.mark.parametrize("mlp", [moe(), moe(experts=5, identity=0, top=2, count=0, shared=0, scale=1.0), moe(experts=12, identity=3, top=4, count=5, keep=3, ff=20),
                                 moe(experts=2, identity=6, top=4, count=2, keep=1, shared=8), dense(ff=50)])
@pytest.mark.parametrize("dtype,tol,T", [(torch.float32, 1e-5, 77), (torch.bfloat16, 2e-2, 77), (torch.float32, 1e-5, 1), (torch.bfloat16, 2e-2, 150)])
def test_feed_forwards_alone(mlp, dtype, tol, T):
    from paligemma_multimodal_system_b200 import seq_ops
    from paligemma_multimodal_system_b200.modeling_pukerax import _feed_forward
    D = 48
    cfg = make_cfg([layer(mlp)], width=D)
    w = {k[len("l0.mlp."):]: v for k, v in O.random_weights(cfg, seed=4).items() if k.startswith("l0.mlp.")}
    g = torch.Generator().manual_seed(T)
    h = torch.randn(T, D, generator=g).to(torch.bfloat16).float()
    ref = O.feed_forward(h, {"f." + k: v for k, v in w.items()}, "f.", mlp)
    ff = _feed_forward(D, mlp)
    ff.load(lambda name, shape: w[name].to(torch.bfloat16), "")
    prec = seq_ops.Precision(dtype)
    ff.pack(prec)
    got = ff(h.to(dtype).cuda().contiguous(), None, prec)
    assert rel_err(got, ref) < tol


@pytest.mark.parametrize("T", [40, 300])
def test_routed_experts_as_dense_runs_per_expert(T, monkeypatch):
    """Prompt-sized steps gather every expert's tokens into one run of rows and use the dense products; forced here at a small
    size, against the oracle and against the grouped kernel (same choice, bf16 rounding apart)."""
    from paligemma_multimodal_system_b200 import seq_ops
    from paligemma_multimodal_system_b200.mixers import RoutedFeedForward
    from paligemma_multimodal_system_b200.modeling_pukerax import _feed_forward
    D, mlp = 64, moe(experts=6, identity=2, top=3, count=4, keep=2, ff=32, shared=16)
    cfg = make_cfg([layer(mlp)], width=D)
    w = {k[len("l0.mlp."):]: v for k, v in O.random_weights(cfg, seed=14).items() if k.startswith("l0.mlp.")}
    g = torch.Generator().manual_seed(T)
    h = torch.randn(T, D, generator=g).to(torch.bfloat16).float()
    ref = O.feed_forward(h, {"f." + k: v for k, v in w.items()}, "f.", mlp)
    ff = _feed_forward(D, mlp)
    ff.load(lambda name, shape: w[name].to(torch.bfloat16), "")
    prec = seq_ops.Precision(torch.bfloat16)
    ff.pack(prec)
    hd = h.to(torch.bfloat16).cuda().contiguous()
    grouped = ff(hd, None, prec)
    monkeypatch.setattr(RoutedFeedForward, "DENSE_SEGMENT_ROWS", 0)
    assert ff._dense_segments(T, prec)
    dense_runs = ff(hd, None, prec)
    assert rel_err(dense_runs, ref) < 2e-2 and rel_err(dense_runs, grouped.cpu()) < 1e-2


def test_causal_edge_row_just_outside_is_not_seen():
    """Position i must see row i and not row i + 1: the later rows of the portion carry huge values in the cache by the time
    the attention runs (the whole portion is written first)."""
    w = O.random_weights(BASE_CFG, seed=2)
    tk = toks(80, BASE_CFG["vocab"], 6)
    ref = O.forward(w, BASE_CFG, tk)
    eng = engine_for(BASE_CFG, w, torch.float32)
    poison(eng)
    got = eng.step([("a", tk, list(range(80)))], ["a"])
    # a changed LAST token must leave every earlier position's logits bit-identical
    tk2 = tk[:-1] + [(tk[-1] + 1) % BASE_CFG["vocab"]]
    got2 = eng.step([("b", tk2, list(range(80)))], ["b"])
    assert torch.equal(got[:-1], got2[:-1]) and not torch.equal(got[-1], got2[-1])
    assert rel_err(got, ref) < F32_TOL


# ----------------------------------------------------------------------------------------------------------------------
# whole models
# ----------------------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def base():
    w = O.random_weights(BASE_CFG, seed=1)
    tk = toks(150, BASE_CFG["vocab"], 2)
    return w, tk, O.forward(w, BASE_CFG, tk)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)])
def test_whole_prompt_every_layer(base, dtype, tol):
    w, tk, ref = base
    eng = engine_for(BASE_CFG, w, dtype)
    poison(eng)
    trace = []
    got = eng.step([("a", tk, list(range(len(tk))))], ["a"], trace=trace)
    _, layers = O.forward(w, BASE_CFG, tk, return_layers=True)
    assert len(trace) == len(BASE_CFG["layers"])
    for i, x in enumerate(trace):
        assert close(x, layers[i], dtype), f"stream sum after layer {i}"
    assert close(got, ref, dtype)


@pytest.mark.parametrize("cuts", [[1], [2], [3, 5, 2], [31, 33], [32], [64, 1], [65, 2, 2, 1], [100, 7]])
def test_portions_and_token_by_token_equal_the_whole_prompt(base, cuts):
    w, tk, ref = base
    eng = engine_for(BASE_CFG, w, torch.float32)
    poison(eng)
    assert rel_err(run_cut(eng, "a", tk, cuts), ref) < F32_TOL


def test_portions_in_bf16(base):
    w, tk, ref = base
    eng = engine_for(BASE_CFG, w, torch.bfloat16)
    poison(eng)
    assert close(run_cut(eng, "a", tk, [37, 2, 64, 1]), ref, torch.bfloat16)


def test_unequal_batch_equals_each_alone_and_pages_are_reused(base):
    """Four live requests of different lengths, portions beside single tokens, in a pool that only holds them because finished
    requests give their pages and slots back; every request's logits equal its solo run."""
    w, _, _ = base
    V = BASE_CFG["vocab"]
    prompts = {i: toks(n, V, 10 + i) for i, n in enumerate([130, 70, 1, 45, 90, 64])}
    refs = {i: O.forward(w, BASE_CFG, p) for i, p in prompts.items()}
    eng = engine_for(BASE_CFG, w, torch.float32, max_tokens=6 * 64, slots=4)
    poison(eng)
    fed = {i: 0 for i in prompts}
    got = {i: [] for i in prompts}
    waiting, live, step = list(prompts), [], 0
    seen_pages = {}
    while waiting or live:
        while waiting and len(live) < 4 and sum((len(prompts[i]) + 63) // 64 for i in live + waiting[:1]) <= 6:
            live.append(waiting.pop(0))
        entries, end = [], []
        for k, i in enumerate(live):
            left = len(prompts[i]) - fed[i]
            n = 1 if (step + k) % 3 == 0 else min(left, [17, 2, 40][(step + k) % 3])
            n = min(n, left)
            entries.append((i, prompts[i][fed[i]:fed[i] + n], list(range(n))))
            fed[i] += n
            if fed[i] == len(prompts[i]):
                end.append(i)
        out = eng.step(entries, end)
        for i in live:
            if i in eng.store.live:
                seen_pages[i] = list(eng.store.live[i].pages)
        r = 0
        for i, tk, _ in entries:
            got[i].append(out[r:r + len(tk)])
            r += len(tk)
        live = [i for i in live if i not in end]
        step += 1
    for i in prompts:
        assert rel_err(torch.cat(got[i]), refs[i]) < F32_TOL, i
    all_pages = [p for ps in seen_pages.values() for p in ps]
    assert len(all_pages) > len(set(all_pages)), "no page was handed out twice"
    assert not eng.store.live and len(eng.store.pool.free) == 6


def test_long_decoding_across_page_borders(base):
    w, _, _ = base
    tk = toks(200, BASE_CFG["vocab"], 77)
    ref = O.forward(w, BASE_CFG, tk)
    for dtype, tol in ((torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)):
        eng = engine_for(BASE_CFG, w, dtype)
        poison(eng)
        assert close(run_cut(eng, "a", tk, [60, 1]), ref, dtype)  # 140 single-token steps: eager, captured, then replayed graphs


def test_long_context_decode_splits_keys_and_grows_the_page_table():
    cfg = make_cfg([layer(dense(32), heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=24, q_rank=16), layer(moe(ff=16, shared=16), heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=24, q_rank=16)],
                   width=32, vocab=50, streams=2)
    w = O.random_weights(cfg, seed=5)
    tk = toks(1200, 50, 9)
    ref = O.forward(w, cfg, tk)[-40:]
    eng = engine_for(cfg, w, torch.float32, max_tokens=1280, slots=1)
    poison(eng)
    got = run_cut(eng, "a", tk, [1160, 1])[-40:]
    assert rel_err(got, ref) < F32_TOL


def test_first_tokens_of_a_sequence(base):
    """One-token prompts, a one-token first portion, two-token portions from the start."""
    w, tk, ref = base
    eng = engine_for(BASE_CFG, w, torch.float32)
    poison(eng)
    one = eng.step([("x", tk[:1], [0])], ["x"])
    assert rel_err(one, ref[:1]) < F32_TOL
    assert rel_err(run_cut(eng, "y", tk[:9], [1, 2, 2, 1, 3]), ref[:9]) < F32_TOL
    assert rel_err(run_cut(eng, "z", tk[:8], [2]), ref[:8]) < F32_TOL


OTHER_SIZES = [
    # no stream key at all: the ordinary residual sum
    make_cfg([layer(dense(40)), layer(moe(shared=0))], width=40, vocab=33, streams=0),
    # one stream WITH coefficients, odd sizes everywhere, identity experts outnumber the real ones
    make_cfg([layer(moe(experts=2, identity=4, top=3, count=3, keep=2, ff=10, shared=6), heads=5, dim=10, rot_dim=6, vdim=14, kv_rank=18, q_rank=22)],
             width=34, vocab=41, streams=1),
    # eight streams, sizes the tensor-core kernels like, feed-forward missing on the first layer
    make_cfg([layer(None, heads=4, dim=64, rot_dim=32, vdim=64, kv_rank=64, q_rank=96), layer(dense(256), heads=4, dim=64, rot_dim=32, vdim=64, kv_rank=64, q_rank=96),
              layer(moe(experts=8, identity=0, top=2, count=2, keep=1, ff=64, shared=128), heads=2, dim=128, rot_dim=64, vdim=128, kv_rank=128, q_rank=64)],
             width=128, vocab=256, streams=8, eps=1e-6),
    # top = every output, one group
    make_cfg([layer(moe(experts=3, identity=1, top=4, count=1, keep=1, ff=12), heads=1, dim=32, rot_dim=4, vdim=8, kv_rank=16, q_rank=8)], width=24, vocab=20, streams=2),
]


@pytest.mark.parametrize("ci", range(len(OTHER_SIZES)))
@pytest.mark.parametrize("dtype,tol", [(torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)])
def test_other_sizes(ci, dtype, tol):
    cfg = OTHER_SIZES[ci]
    w = O.random_weights(cfg, seed=20 + ci)
    tk = toks(100, cfg["vocab"], ci)
    ref = O.forward(w, cfg, tk)
    eng = engine_for(cfg, w, dtype)
    poison(eng)
    assert close(run_cut(eng, "a", tk, [70, 2, 1, 1, 20, 1]), ref, dtype)
    two = [toks(n, cfg["vocab"], 50 + n) for n in (66, 30)]
    out = eng.step([(i, p, list(range(len(p)))) for i, p in enumerate(two)], [0, 1])
    assert close(out[:66], O.forward(w, cfg, two[0]), dtype) and close(out[66:], O.forward(w, cfg, two[1]), dtype)


def test_greedy_generation_through_the_scheduler():
    """engine.generate: more prompts than slots, a pool smaller than the sum of all requests, portions of 48 rows; the tokens
    equal the oracle's greedy continuation of each prompt alone."""
    cfg = make_cfg([layer(dense(48), heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=24, q_rank=16), layer(moe(ff=16, shared=16), heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=24, q_rank=16)],
                   width=48, vocab=60, streams=2)
    w = O.random_weights(cfg, seed=31)
    prompts = [toks(n, 60, 40 + n) for n in (70, 5, 33, 1, 90, 12)]
    new = 10
    eng = engine_for(cfg, w, torch.float32, max_tokens=5 * 64, slots=3)
    poison(eng)
    got = eng.generate(prompts, new, step_tokens=48)
    for p, g in zip(prompts, got):
        seq = list(p)
        for _ in range(new):
            lg = O.forward(w, cfg, seq)[-1]
            top2 = lg.topk(2).values
            assert float(top2[0] - top2[1]) > 1e-3, "test weights give a near tie"
            seq.append(int(lg.argmax()))
        assert g == seq[len(p):]
    assert not eng.store.live and len(eng.store.pool.free) == 5


def test_sampled_generation_stays_in_vocabulary_and_stops_at_eos():
    cfg = make_cfg([layer(moe(ff=16, shared=0), heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=24, q_rank=16)], width=48, vocab=60, streams=2)
    w = O.random_weights(cfg, seed=9)
    eng = engine_for(cfg, w, torch.bfloat16, max_tokens=256, slots=2)
    out = eng.generate([toks(20, 60, 1), toks(3, 60, 2), toks(40, 60, 3)], 10, do_sample=True, temperature=0.9, top_p=0.8, eos_token_id=7, seed=3)
    for g in out:
        assert 1 <= len(g) <= 10 and all(0 <= t < 60 for t in g)
        assert 7 not in g[:-1]


def test_registry_loads_a_checkpoint_folder(tmp_path):
    """config.json + model.safetensors on disk -> registry.load_model -> the same logits as the in-memory model."""
    from paligemma_multimodal_system_b200.engine import SequenceEngine
    from paligemma_multimodal_system_b200.registry import load_model
    cfg = copy.deepcopy(OTHER_SIZES[1])
    w = O.random_weights(cfg, seed=11)
    meta, blobs, off = {}, [], 0
    for name, t in w.items():
        raw = t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        meta[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    head = json.dumps(meta).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(head)) + head + b"".join(blobs))
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    tk = toks(50, cfg["vocab"], 5)
    eng = SequenceEngine(load_model(str(tmp_path), dtype=torch.float32), 128, 1)
    assert rel_err(eng.step([("a", tk, list(range(50)))], ["a"]), O.forward(w, cfg, tk)) < F32_TOL
