"""Mapedra through the framework (kernels, page pool, state slots, ragged steps, scheduler) against the plain fp32 oracle
(oracle/mapedra_oracle.py): every mechanism alone, then whole models under every way of cutting and batching the work."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import mapedra_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu

F32_TOL, BF16_TOL = 2e-4, 4e-2


def attn_layer(heads=4, kv_heads=2, dim=32, vdim=32, rot=16, ff=96, scaling=True, softcap=30.0, scale=None):
    rotd = {"base": 10000.0, "dims": rot}
    if scaling:
        rotd["scaling"] = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rotd,
                                           "scale": scale if scale is not None else dim ** -0.5, "softcap": softcap},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def light_layer(heads=2, dim=32, vdim=32, decay=(0.9, 0.99), ff=0):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def make_cfg(layers, width=96, vocab=80, groups=2, side=8, emb_scale=3.0, eps=1e-6):
    cfg = {"architecture": "Mapedra", "vocab": vocab, "width": width, "embedding": {"scale": emb_scale},
           "norm": {"eps": eps, "groups": groups}, "layers": layers}
    if side:
        cfg["token_side"] = {"dim": side}
    return cfg


BASE_CFG = make_cfg([attn_layer(), light_layer(), attn_layer(heads=4, kv_heads=4, ff=0), light_layer(heads=3, dim=16, vdim=48, decay=(1.0, 0.5, 0.97), ff=64)])


def build(cfg, w, dtype):
    from paligemma_multimodal_system_b200.modeling_mapedra import MapedraConfig, MapedraForCausalLM
    return MapedraForCausalLM(MapedraConfig(cfg), dtype).load_weights({k: v.to(torch.bfloat16) for k, v in w.items()})


def engine_for(cfg, w, dtype, max_tokens=1024, slots=4):
    from paligemma_multimodal_system_b200.engine import SequenceEngine
    return SequenceEngine(build(cfg, w, dtype), max_tokens, slots)


def poison(engine):
    """Stale memory must never be read: pages and states start as huge values instead of zeros."""
    st = engine.store
    for t in st.k_pages + st.v_pages + st.state:
        if t is not None:
            t.fill_(1e4)


def rel_err(got, ref):
    got, ref = got.double().cpu(), ref.double()
    d = got - ref
    return float(d.pow(2).mean().sqrt() / ref.pow(2).mean().sqrt())


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


# ----------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ----------------------------------------------------------------------------------------------------------------------
def _one_entry(spec, T, dtype, ctx=0):
    from paligemma_multimodal_system_b200.cache import SequenceStore
    from paligemma_multimodal_system_b200.seq_ops import make_step_batch
    store = SequenceStore([spec], 2048, 2, dtype)
    store.admit("a")
    rec = store.reserve("a", ctx + T)
    return store, make_step_batch([dict(tokens=[0] * T, ctx=ctx, slot=rec.slot, pages=rec.pages)])


@pytest.mark.parametrize("groups,D", [(1, 96), (2, 96), (4, 200), (3, 33)])
def test_grouped_rmsnorm_with_and_without_residual(groups, D):
    from paligemma_multimodal_system_b200 import seq_ops
    g = torch.Generator().manual_seed(groups)
    y, x, w = torch.randn(7, D, generator=g) * 3, torch.randn(7, D, generator=g), torch.randn(D, generator=g)
    ref = O.group_norm(y, w, groups, 1e-5)
    xd, act = x.cuda(), torch.empty(7, D, device="cuda", dtype=torch.bfloat16)
    seq_ops.group_rmsnorm_add(y.cuda(), w.cuda(), xd, act, groups, 1e-5)
    assert torch.allclose(xd.cpu(), x + ref, atol=1e-5, rtol=1e-5)
    assert torch.allclose(act.float().cpu(), (x + ref).bfloat16().float(), atol=1e-2, rtol=1e-2)
    bare = torch.empty(7, D, device="cuda", dtype=torch.float32)
    seq_ops.group_rmsnorm_add(y.cuda(), w.cuda(), None, bare, groups, 1e-5)
    assert torch.allclose(bare.cpu(), ref, atol=1e-5, rtol=1e-5)
    # a tiny eps matters when a group is all but zero: eps sits inside the root
    y0 = torch.zeros(1, D)
    seq_ops.group_rmsnorm_add(y0.cuda(), w.cuda(), None, bare[:1], groups, 1e-5)
    assert torch.isfinite(bare[:1]).all() and float(bare[:1].abs().max()) == 0.0


@pytest.mark.parametrize("shape", [(5, 16, 24), (70, 33, 130), (200, 72, 96)])
@pytest.mark.parametrize("f32", [True, False])
def test_plain_fma_gemm(shape, f32):
    from paligemma_multimodal_system_b200 import seq_ops
    T, F, K = shape
    g = torch.Generator().manual_seed(T)
    dt = torch.float32 if f32 else torch.bfloat16
    x, w = torch.randn(T, K, generator=g).to(dt), torch.randn(F, K, generator=g).to(dt)
    out = torch.empty(T, F, device="cuda", dtype=torch.float32)
    seq_ops.linear(x.cuda(), w.cuda(), out)
    ref = x.double() @ w.double().T
    assert rel_err(out, ref) < (2e-6 if f32 else 1e-5)


@pytest.mark.parametrize("kw", [dict(), dict(heads=6, kv_heads=2, dim=24, vdim=40, rot=24, scaling=False),
                                dict(heads=2, kv_heads=1, dim=80, vdim=16, rot=0, softcap=None), dict(heads=3, kv_heads=3, dim=16, vdim=16, rot=8, softcap=2.0)])
def test_attention_mixer_alone(kw):
    from paligemma_multimodal_system_b200.mixers import GatedSoftmaxAttention
    from paligemma_multimodal_system_b200.seq_ops import Precision
    layer = attn_layer(ff=0, **kw)
    cfg = make_cfg([layer], width=64, side=0)
    w = O.random_weights(cfg, seed=3)
    m = layer["mixer"]
    T = 150
    h = torch.randn(T, 64, generator=torch.Generator().manual_seed(1))
    ref = O.attention_mixer(h, w, "l0.mix.", m, 1e-6)
    mix = GatedSoftmaxAttention(64, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], m["softcap"], m["rot"]["dims"], m["rot"]["base"],
                                m["rot"].get("scaling"), 1e-6)
    mix.load(lambda name, shape: w[name], "l0.mix.")
    prec = Precision(torch.float32)
    mix.pack(prec)
    store, b = _one_entry(mix.cache_spec(), T, torch.float32)
    assert rel_err(mix(h.cuda(), b, store, 0, prec), ref) < F32_TOL


@pytest.mark.parametrize("kw", [dict(), dict(heads=3, dim=24, vdim=72, decay=(1.0, 0.3, 0.999)), dict(heads=1, dim=128, vdim=8, decay=(0.95,))])
@pytest.mark.parametrize("chunked", [False, True])
def test_lightning_mixer_alone(kw, chunked):
    from paligemma_multimodal_system_b200 import seq_ops
    from paligemma_multimodal_system_b200.mixers import LightningAttention
    layer = light_layer(**kw)
    cfg = make_cfg([layer], width=64, side=0)
    w = O.random_weights(cfg, seed=4)
    m = layer["mixer"]
    T = 100
    h = torch.randn(T, 64, generator=torch.Generator().manual_seed(2))
    ref = O.lightning_mixer(h, w, "l0.mix.", m, 1e-6)
    mix = LightningAttention(64, m["heads"], m["dim"], m["vdim"], m["decay"], 1e-6)
    mix.load(lambda name, shape: w[name], "l0.mix.")
    prec = seq_ops.Precision(torch.float32)
    mix.pack(prec)
    store, b = _one_entry(mix.cache_spec(), T, torch.float32)
    store.state[0].fill_(1e4)  # a fresh sequence must not read the slot's old state
    old = seq_ops.LINEAR_ATTN_CHUNK_MIN
    seq_ops.LINEAR_ATTN_CHUNK_MIN = 1 if chunked else 10 ** 9
    try:
        got = mix(h.cuda(), b, store, 0, prec)
    finally:
        seq_ops.LINEAR_ATTN_CHUNK_MIN = old
    assert rel_err(got, ref) < F32_TOL


def test_feed_forward_and_side_input_alone():
    from paligemma_multimodal_system_b200 import seq_ops
    from paligemma_multimodal_system_b200.mixers import GegluFeedForward, TokenSideInput
    cfg = make_cfg([attn_layer(ff=200), attn_layer(ff=64)], width=72, side=12, vocab=50)
    w = O.random_weights(cfg, seed=5)
    T = 40
    h = torch.randn(T, 72, generator=torch.Generator().manual_seed(3))
    tk = toks(T, 50, 9)
    store, b = _one_entry(None, T, torch.float32)
    b.tokens.copy_(torch.tensor(tk, dtype=torch.int32))
    for dt, tol in ((torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)):
        prec = seq_ops.Precision(dt)
        hd = h.bfloat16().float() if dt == torch.bfloat16 else h
        ff = GegluFeedForward(72, 200)
        ff.load(lambda name, shape: w[name], "l0.mlp.")
        ff.pack(prec)
        assert rel_err(ff(hd.cuda().to(dt), b, prec), O.dense_ff(hd, w, "l0.mlp.")) < tol
        side = TokenSideInput(72, 12, 1)
        side.load(lambda name, shape: w[name], "l1.side.")
        side.pack(prec)
        y = side(hd.cuda().to(dt), b, w["side.embed"].cuda().to(dt), prec)
        ref = (O.gelu_tanh(hd @ w["l1.side.gate"].T) * w["side.embed"][tk][:, 12:24]) @ w["l1.side.proj"].T
        assert rel_err(y, ref) < tol


# ----------------------------------------------------------------------------------------------------------------------
# attention over the paged cache with a key that stands out
# ----------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("ctx,n", [(0, 200), (130, 70), (199, 1), (64, 1), (63, 2), (1100, 1), (1060, 40)])
@pytest.mark.parametrize("needle", [0, 1, 63, 64, 65, 127, 128, 1023, 1024])
def test_far_key_at_page_borders_is_found(ctx, n, needle):
    """Among hundreds of random keys ONE (at `needle`) is aligned with the last query and scaled up: the output of the last row
    must be that key's value.  Run as a prompt portion (n > 1) and as a decoded token (n = 1, long contexts split the keys over
    several CTAs), needle on both sides of page edges."""
    from paligemma_multimodal_system_b200 import seq_ops
    H, G, dim, vdim, total = 2, 1, 32, 32, ctx + n
    needle = min(needle, total - 1)
    g = torch.Generator().manual_seed(needle * 7 + n)
    store, b = _one_entry(("kv", G * dim, G * vdim), n, torch.float32, ctx=ctx)
    k = torch.randn(total, dim, generator=g) * 0.1
    v = torch.randn(total, vdim, generator=g)
    q = torch.randn(n, H, dim, generator=g) * 0.1
    q[-1] = torch.randn(dim, generator=g)
    k[needle] = q[-1, 0] * 4 / q[-1, 0].norm()
    q[-1, 0] = q[-1, 0] * 8 / q[-1, 0].norm()
    pages = b.page_table[0].tolist()
    for j in range(total):
        store.k_pages[0][pages[j // 64], j % 64] = k[j].cuda()
        store.v_pages[0][pages[j // 64], j % 64] = v[j].cuda()
    out = torch.empty(n, H * vdim, device="cuda", dtype=torch.float32)
    seq_ops.attn_ragged(q.reshape(n, H * dim).cuda().contiguous(), store.k_pages[0], store.v_pages[0], None, out, b, H, G, dim, vdim, 1.0, 0.0, 64)
    ref = torch.zeros(n, H, vdim)
    for i in range(n):
        s = torch.einsum("hd,jd->hj", q[i], k[: ctx + i + 1])
        ref[i] = torch.softmax(s, -1) @ v[: ctx + i + 1]
    assert torch.allclose(out.cpu().view(n, H, vdim), ref, atol=2e-5, rtol=1e-4)
    assert (out.cpu().view(n, H, vdim)[-1, 0] - v[needle]).abs().max() < 1e-3  # the needle dominates


@pytest.mark.parametrize("dim,vdim,H,G", [(64, 64, 6, 2), (32, 32, 2, 2), (128, 128, 2, 1), (64, 128, 4, 1), (128, 64, 3, 3)])
@pytest.mark.parametrize("ctx,n", [(0, 150), (70, 61), (129, 2)])
def test_tensor_core_attention_keeps_fp32_probabilities(dim, vdim, H, G, ctx, n):
    """bf16 q / k / v through the tensor-core kernel against fp64 softmax attention of the same bf16 values: the error must be
    at the level of the bf16 OUTPUT rounding only (a bf16-rounded probability matrix would sit ten times higher on the
    flat rows this test makes), for every instantiated head size, with soft cap, gate, grouped heads and a cached context."""
    from paligemma_multimodal_system_b200 import seq_ops
    total = ctx + n
    g = torch.Generator().manual_seed(dim + n)
    store, b = _one_entry(("kv", G * dim, G * vdim), n, torch.bfloat16, ctx=ctx)
    k = (torch.randn(total, G, dim, generator=g) * 0.05).bfloat16()   # flat scores: hundreds of keys share the mass
    v = torch.randn(total, G, vdim, generator=g).bfloat16()
    q = torch.randn(n, H, dim, generator=g).bfloat16()
    gate = torch.randn(n, H * vdim, generator=g).bfloat16()
    pages = b.page_table[0].tolist()
    for j in range(total):
        store.k_pages[0][pages[j // 64], j % 64] = k[j].reshape(-1).cuda()
        store.v_pages[0][pages[j // 64], j % 64] = v[j].reshape(-1).cuda()
    outs = []
    for tc in (True, False):
        out = torch.empty(n, H * vdim, device="cuda", dtype=torch.bfloat16)
        seq_ops.attn_ragged(q.reshape(n, H * dim).cuda().contiguous(), store.k_pages[0], store.v_pages[0], gate.cuda(), out, b, H, G, dim, vdim,
                            0.3, 5.0, 64, decode_kernel=False, tensor_cores=tc)
        outs.append(out.float().cpu())
    ref = torch.zeros(n, H, vdim, dtype=torch.float64)
    for i in range(n):
        for h in range(H):
            kv = h // (H // G)
            s = (k[: ctx + i + 1, kv].double() @ q[i, h].double()) * 0.3
            s = 5.0 * torch.tanh(s / 5.0)
            ref[i, h] = torch.softmax(s, 0) @ v[: ctx + i + 1, kv].double()
    ref = (ref.reshape(n, H * vdim) * torch.sigmoid(gate.double())).float()
    for out in outs:
        assert torch.allclose(out, ref, atol=4e-3, rtol=1e-2)
    # before the final rounding both kernels carry fp32 probabilities: they agree to one bf16 ulp nearly everywhere
    assert float((outs[0] - outs[1]).abs().max()) <= 2 ** -7 * float(ref.abs().max())


def test_causal_edge_key_just_outside_is_not_seen():
    """A huge key one position AFTER a query must leave that query's output untouched, and one AT the query must take it over."""
    from paligemma_multimodal_system_b200 import seq_ops
    H, G, dim, vdim, n = 1, 1, 16, 16, 70
    g = torch.Generator().manual_seed(0)
    store, b = _one_entry(("kv", dim, vdim), n, torch.float32)
    k, v, q = torch.randn(n, dim, generator=g) * 0.1, torch.randn(n, vdim, generator=g), torch.randn(n, dim, generator=g)
    for edge in (31, 32, 63, 64):
        k[edge + 1] = q[edge] * 50  # visible to row edge + 1 only
    pages = b.page_table[0].tolist()
    for j in range(n):
        store.k_pages[0][pages[j // 64], j % 64] = k[j].cuda()
        store.v_pages[0][pages[j // 64], j % 64] = v[j].cuda()
    out = torch.empty(n, vdim, device="cuda", dtype=torch.float32)
    seq_ops.attn_ragged(q.cuda(), store.k_pages[0], store.v_pages[0], None, out, b, H, G, dim, vdim, 1.0, 0.0, 64)
    ref = torch.stack([torch.softmax(k[: i + 1] @ q[i], 0) @ v[: i + 1] for i in range(n)])
    assert torch.allclose(out.cpu(), ref, atol=2e-5, rtol=1e-4)


# ----------------------------------------------------------------------------------------------------------------------
# whole models
# ----------------------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def base():
    w = O.random_weights(BASE_CFG, seed=1)
    tk = toks(150, BASE_CFG["vocab"], 2)
    return w, tk, O.forward(BASE_CFG, w, tk)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)])
def test_whole_prompt_every_layer(base, dtype, tol):
    w, tk, ref = base
    eng = engine_for(BASE_CFG, w, dtype)
    poison(eng)
    trace = []
    got = eng.step([("a", tk, list(range(len(tk))))], ["a"], trace=trace)
    _, layers = O.forward(BASE_CFG, w, tk, return_layers=True)
    for i, x in enumerate(trace):
        assert rel_err(x, layers[i]) < tol, f"residual stream after layer {i}"
    assert rel_err(got, ref) < tol


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
    assert rel_err(run_cut(eng, "a", tk, [37, 2, 64, 1]), ref) < BF16_TOL


def test_unequal_batch_equals_each_alone_and_pages_slots_are_reused(base):
    """Four live requests of different lengths, portions beside single tokens, in a pool that only holds them because finished
    requests give their pages and slots back; every request's logits equal its solo run."""
    w, _, _ = base
    V = BASE_CFG["vocab"]
    prompts = {i: toks(n, V, 10 + i) for i, n in enumerate([130, 70, 1, 45, 90, 64])}
    refs = {i: O.forward(BASE_CFG, w, p) for i, p in prompts.items()}
    eng = engine_for(BASE_CFG, w, torch.float32, max_tokens=6 * 64, slots=4)
    poison(eng)
    fed = {i: 0 for i in prompts}
    got = {i: [] for i in prompts}
    waiting, live, step = list(prompts), [], 0
    used_slots, used_pages = [], []
    while waiting or live:
        while waiting and len(live) < 4 and sum((len(prompts[i]) + 63) // 64 for i in live + waiting[:1]) <= 6:
            live.append(waiting.pop(0))
        entries, end = [], []
        for j, i in enumerate(live):
            left = len(prompts[i]) - fed[i]
            k = min(left, [40, 1, 2, 17][(j + step) % 4])
            entries.append((i, prompts[i][fed[i]:fed[i] + k], list(range(k))))
            fed[i] += k
            if fed[i] == len(prompts[i]):
                end.append(i)
        out = eng.step(entries, end)
        for i in live:
            if i in eng.store.live:
                used_slots.append(eng.store.live[i].slot)
                used_pages += eng.store.live[i].pages
        r = 0
        for i, t, _ in entries:
            got[i].append(out[r:r + len(t)])
            r += len(t)
        live = [i for i in live if i not in end]
        step += 1
    assert len(used_slots) > len(set(used_slots)) and len(set(used_pages)) <= 6  # slots and pages really were handed out again
    assert not eng.store.live and len(eng.store.pool.free) == 6 and sorted(eng.store.free_slots) == [0, 1, 2, 3]
    for i in prompts:
        assert rel_err(torch.cat(got[i]), refs[i]) < F32_TOL, f"request {i}"


def test_long_decoding_across_page_borders(base):
    w, _, _ = base
    tk = toks(210, BASE_CFG["vocab"], 77)
    ref = O.forward(BASE_CFG, w, tk)
    eng = engine_for(BASE_CFG, w, torch.float32)
    poison(eng)
    assert rel_err(run_cut(eng, "a", tk, [40, 1]), ref) < F32_TOL  # 170 single-token steps over the borders at 64, 128, 192


def test_long_context_decode_splits_keys_and_grows_the_page_table():
    """A 1100-token prompt, then 40 single-token steps through the replayed decode graph: the decode attention runs with several
    key splits, the lightning state carries over 1100 tokens with a decay close to one."""
    cfg = make_cfg([attn_layer(heads=4, kv_heads=2, dim=64, vdim=64, rot=32, ff=0), light_layer(heads=2, dim=32, vdim=32, decay=(0.999, 0.97), ff=64)],
                   width=64, vocab=90, side=8)
    w = O.random_weights(cfg, seed=31)
    tk = toks(1140, 90, 5)
    ref = O.forward(cfg, w, tk)
    for dtype, tol in ((torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)):
        eng = engine_for(cfg, w, dtype, max_tokens=1152 + 64)
        poison(eng)
        head = eng.step([("a", tk[:1000], [999])])
        body = eng.step([("a", tk[1000:1100], list(range(100)))])
        tail = torch.cat([eng.step([("a", [t], [0])]) for t in tk[1100:]])
        assert rel_err(torch.cat([head, body, tail]), torch.cat([ref[999:1000], ref[1000:]])) < tol
        assert len(eng._decode_graphs) >= 1 and all(g["graph"] is not None for g in eng._decode_graphs.values() if g["seen"] >= 2)


def test_first_tokens_of_a_sequence(base):
    w, tk, ref = base
    eng = engine_for(BASE_CFG, w, torch.float32)
    poison(eng)
    one = eng.step([("x", tk[:1], [0])], ["x"])
    assert rel_err(one, ref[:1]) < F32_TOL
    two = eng.step([("y", tk[:2], [0, 1])], ["y"])
    assert rel_err(two, ref[:2]) < F32_TOL


OTHER_SIZES = [
    # one key/value head per query head, no rescaling, no soft cap, one norm group, unit embedding scale, no side table
    make_cfg([attn_layer(heads=2, kv_heads=2, dim=16, vdim=16, rot=16, scaling=False, softcap=None, ff=40)], width=48, vocab=33, groups=1, side=0, emb_scale=1.0),
    # a single shared key/value head, odd head sizes, a width the TMA kernels cannot take, side width not a multiple of 8
    make_cfg([attn_layer(heads=8, kv_heads=1, dim=24, vdim=40, rot=8, ff=100), light_layer(heads=5, dim=8, vdim=24, decay=(1, 0.9, 0.8, 0.7, 0.6))],
             width=100, vocab=101, groups=4, side=5),
    # lightning only, feed-forward on every layer, decay exactly one
    make_cfg([light_layer(heads=1, dim=64, vdim=64, decay=(1.0,), ff=128), light_layer(heads=4, dim=32, vdim=16, decay=(0.5, 0.5, 0.5, 0.5), ff=64)],
             width=64, vocab=64, groups=2, side=16),
    # head sizes outside the tensor-core instantiations, rotation over the whole head, three norm groups, wide lightning heads
    make_cfg([attn_layer(heads=4, kv_heads=2, dim=48, vdim=96, rot=48, ff=72), light_layer(heads=2, dim=128, vdim=128, decay=(0.99, 0.9), ff=0),
              attn_layer(heads=12, kv_heads=3, dim=16, vdim=8, rot=4, scaling=False, ff=0)], width=96, vocab=500, groups=3, side=24),
    # attention only, big heads, wide values
    make_cfg([attn_layer(heads=2, kv_heads=1, dim=128, vdim=160, rot=64, ff=0), attn_layer(heads=1, kv_heads=1, dim=96, vdim=32, rot=96, ff=256)],
             width=128, vocab=256, groups=8, side=8),
]


@pytest.mark.parametrize("ci", range(len(OTHER_SIZES)))
@pytest.mark.parametrize("dtype,tol", [(torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)])
def test_other_sizes(ci, dtype, tol):
    cfg = OTHER_SIZES[ci]
    w = O.random_weights(cfg, seed=20 + ci)
    tk = toks(90, cfg["vocab"], ci)
    ref = O.forward(cfg, w, tk)
    eng = engine_for(cfg, w, dtype, max_tokens=256)
    poison(eng)
    assert rel_err(eng.step([("a", tk, list(range(len(tk))))], ["a"]), ref) < tol
    assert rel_err(run_cut(eng, "b", tk, [33, 2, 1]), ref) < tol


def test_greedy_generation_through_the_scheduler():
    """engine.generate: more prompts than slots, a pool smaller than the sum of all requests, portions of 48 rows; the tokens
    equal the oracle's greedy continuation of each prompt alone."""
    cfg = make_cfg([attn_layer(), light_layer(ff=64)], width=64, vocab=60)
    w = O.random_weights(cfg, seed=8, std=0.3)
    prompts = [toks(n, 60, 40 + n) for n in (70, 5, 33, 1, 90, 12)]
    new = 12
    eng = engine_for(cfg, w, torch.float32, max_tokens=5 * 64, slots=3)
    poison(eng)
    got = eng.generate(prompts, new, step_tokens=48)
    for p, g in zip(prompts, got):
        seq = list(p)
        for _ in range(new):
            lg = O.forward(cfg, w, seq)[-1]
            top2 = lg.topk(2).values
            assert float(top2[0] - top2[1]) > 1e-3, "test weights give a near tie"
            seq.append(int(lg.argmax()))
        assert g == seq[len(p):]
    assert not eng.store.live and len(eng.store.pool.free) == 5


def test_sampled_generation_stays_in_vocabulary_and_stops_at_eos():
    cfg = make_cfg([attn_layer(ff=0), light_layer()], width=64, vocab=60)
    w = O.random_weights(cfg, seed=9)
    eng = engine_for(cfg, w, torch.bfloat16, max_tokens=256, slots=2)
    out = eng.generate([toks(20, 60, 1), toks(3, 60, 2), toks(40, 60, 3)], 10, do_sample=True, temperature=0.9, top_p=0.8, eos_token_id=7, seed=3)
    for g in out:
        assert 1 <= len(g) <= 10 and all(0 <= t < 60 for t in g)
        assert 7 not in g[:-1]


def test_registry_loads_a_checkpoint_folder(tmp_path):
    """config.json + model.safetensors on disk -> registry.load_model -> the same logits as the in-memory model."""
    import json
    import struct
    from paligemma_multimodal_system_b200.engine import SequenceEngine
    from paligemma_multimodal_system_b200.registry import load_model
    cfg = make_cfg([light_layer(ff=64), attn_layer(ff=0)], width=64, vocab=40)
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
    tk = toks(50, 40, 5)
    eng = SequenceEngine(load_model(str(tmp_path), dtype=torch.float32), 128, 1)
    assert rel_err(eng.step([("a", tk, list(range(50)))], ["a"]), O.forward(cfg, w, tk)) < F32_TOL
