"""Host-side parts of the Pukerax path (no GPU): config parsing, the cache layout a latent-attention model asks for, the
registry entry, and the oracle's own consistency (the absorbed form of latent attention against explicit heads; the router's
group limit against a brute-force choice)."""
import itertools
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import pukerax_oracle as O  # noqa: E402
from paligemma_multimodal_system_b200.cache import SequenceStore  # noqa: E402


def _cfg(streams=2):
    mixer = {"heads": 3, "dim": 12, "rot_dim": 4, "vdim": 10, "kv_rank": 20, "q_rank": 14, "rot": {"base": 777.0, "dims": 4}, "scale": 0.25}
    moe = {"kind": "moe", "expert": {"ff": 8}, "shared": {"ff": 6},
           "router": {"experts": 4, "identity": 2, "top": 2, "scale": 1.3, "groups": {"count": 3, "keep": 2}}}
    cfg = {"architecture": "Pukerax", "vocab": 30, "width": 24, "norm": {"eps": 1e-5},
           "layers": [{"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": 16}},
                      {"type": "latent_attention", "mixer": mixer, "mlp": moe}, {"type": "latent_attention", "mixer": mixer, "mlp": None}]}
    if streams:
        cfg["streams"] = streams
    return cfg


def test_config_and_cache_layout():
    from paligemma_multimodal_system_b200.modeling_pukerax import PukeraxConfig, PukeraxForCausalLM
    c = PukeraxConfig(_cfg())
    assert (c.vocab, c.width, c.streams, c.hyper, len(c.layers)) == (30, 24, 2, True, 3)
    assert PukeraxConfig(_cfg(streams=0)).streams == 1 and not PukeraxConfig(_cfg(streams=0)).hyper
    m = PukeraxForCausalLM(c, torch.float32)
    assert m.cache_layout() == [("latent", 24)] * 3  # one row of kv_rank + rot_dim per token and layer, nothing per head
    bad = _cfg()
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(ValueError):
        PukeraxConfig(bad)
    bad = _cfg()
    bad["layers"][1]["mlp"]["kind"] = "sparse"
    with pytest.raises(ValueError):
        PukeraxConfig(bad)
    with pytest.raises(ValueError):
        PukeraxConfig(dict(_cfg(), streams=17))


def test_weight_loading_checks_names_and_shapes():
    from paligemma_multimodal_system_b200.modeling_pukerax import PukeraxConfig, PukeraxForCausalLM
    cfg = _cfg()
    w = O.random_weights(cfg, seed=1)
    PukeraxForCausalLM(PukeraxConfig(cfg), torch.float32).load_weights(w)
    miss = dict(w)
    del miss["l1.mlp.correction"]
    with pytest.raises(KeyError):
        PukeraxForCausalLM(PukeraxConfig(cfg), torch.float32).load_weights(miss)
    extra = dict(w, **{"l2.mlp.up": torch.zeros(3, 3)})
    with pytest.raises(KeyError):
        PukeraxForCausalLM(PukeraxConfig(cfg), torch.float32).load_weights(extra)
    wrong = dict(w, **{"l0.mix.uk": torch.zeros(3 * 12, 21)})
    with pytest.raises(ValueError):
        PukeraxForCausalLM(PukeraxConfig(cfg), torch.float32).load_weights(wrong)
    # without the stream key the checkpoint has no stream coefficients
    w0 = O.random_weights(_cfg(streams=0), seed=1)
    assert not any(".hc" in k for k in w0)
    PukeraxForCausalLM(PukeraxConfig(_cfg(streams=0)), torch.float32).load_weights(w0)


def test_latent_store_keeps_one_page_tensor_per_layer():
    st = SequenceStore([("latent", 24), None], max_tokens=3 * 64, num_slots=2, dtype=torch.float32, device="cpu")
    assert st.k_pages[0].shape == (3, 64, 24) and st.v_pages[0] is None and st.state[0] is None and st.k_pages[1] is None
    with pytest.raises(ValueError):
        SequenceStore([("rows", 3)], max_tokens=64, num_slots=1, dtype=torch.float32, allocate=False)


def test_registry_knows_the_architecture():
    from paligemma_multimodal_system_b200 import registry
    assert "pukerax" in registry.known_architectures()
    assert registry.architecture_of({"architecture": "Pukerax"}) == "Pukerax"


def test_oracle_absorbed_form_equals_explicit_heads():
    """(W_uk^T q_plain) . c == q_plain . (W_uk c), and W_uv applied after the weighted sum of the latent rows."""
    cfg = _cfg()
    m, eps = cfg["layers"][0]["mixer"], 1e-5
    w = O.random_weights(cfg, seed=2)
    g = torch.Generator().manual_seed(0)
    T, H, dim, rd, vd, R = 9, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    h = torch.randn(T, cfg["width"], generator=g)
    ref = O.latent_attention(h, w, "l0.mix.", m, eps)
    p = "l0.mix."
    cq = O.rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(T, H, dim + rd)
    kv = h @ w[p + "dkv"].T
    c = O.rms(kv[:, :R], eps) * w[p + "dkv.norm"]
    r = torch.stack([O.rotate_interleaved(kv[j, R:], j, m["rot"]["base"], m["rot"]["dims"]) for j in range(T)])
    uk, uv = w[p + "uk"].reshape(H, dim, R), w[p + "uv"].reshape(H, vd, R)
    gate = torch.sigmoid(h @ w[p + "g"].T)
    out = torch.zeros(T, H, vd)
    for i in range(T):
        for hh in range(H):
            ql = uk[hh].T @ q[i, hh, :dim]
            qr = O.rotate_interleaved(q[i, hh, dim:], i, m["rot"]["base"], m["rot"]["dims"])
            s = (c[: i + 1] @ ql + r[: i + 1] @ qr) * m["scale"]
            out[i, hh] = uv[hh] @ (torch.softmax(s, 0) @ c[: i + 1]) * gate[i, hh]
    assert torch.allclose(out.reshape(T, H * vd) @ w[p + "o"].T, ref, atol=1e-5, rtol=1e-4)


def test_oracle_rotation_is_relative():
    """q rotated by i and k rotated by j give a product that depends on i - j only."""
    g = torch.Generator().manual_seed(3)
    a, b = torch.randn(8, generator=g), torch.randn(8, generator=g)
    d1 = O.rotate_interleaved(a, 17, 1000.0, 6) @ O.rotate_interleaved(b, 11, 1000.0, 6)
    d2 = O.rotate_interleaved(a, 106, 1000.0, 6) @ O.rotate_interleaved(b, 100, 1000.0, 6)
    assert abs(float(d1 - d2)) < 1e-4
    assert torch.equal(O.rotate_interleaved(a, 5, 1000.0, 6)[6:], a[6:])  # dimensions past rot.dims pass unchanged


def test_oracle_router_against_brute_force():
    """The chosen set maximises the sum of choice scores over all sets of `top` outputs inside `keep` groups chosen by their
    best member; with every choice score negative a dropped group still never wins."""
    g = torch.Generator().manual_seed(4)
    n_all, cnt, keep, top = 12, 4, 2, 3
    r = {"experts": 10, "identity": 2, "top": top, "scale": 2.0, "groups": {"count": cnt, "keep": keep}}
    for trial in range(20):
        w = {"r.router": torch.eye(n_all), "r.correction": torch.randn(n_all, generator=g) * 0.05 - (2.0 if trial % 2 else 0.0)}
        z = torch.randn(n_all, generator=g)
        ids, wt = O.route(z, w, "r.", r)
        s = torch.softmax(z, 0)
        choice = s + w["r.correction"]
        gbest = choice.reshape(cnt, -1).max(1).values
        kept = set(sorted(range(cnt), key=lambda k: -float(gbest[k]))[:keep])
        eligible = [i for i in range(n_all) if i // (n_all // cnt) in kept]
        best = max(itertools.combinations(eligible, top), key=lambda c: sum(float(choice[i]) for i in c))
        assert set(ids) == set(best)
        assert abs(float(wt.sum()) - 2.0) < 1e-5 and torch.allclose(wt, s[ids] / s[ids].sum() * 2.0)


def test_oracle_single_stream_without_coefficients_is_the_plain_residual():
    cfg = _cfg(streams=0)
    w = O.random_weights(cfg, seed=6)
    tk = [3, 7, 1, 29, 0, 12]
    one = dict(cfg, streams=1)
    w1 = dict(w)
    for i, l in enumerate(cfg["layers"]):
        for q in (1, 2) if l["mlp"] else (1,):
            w1[f"l{i}.hc{q}.in"], w1[f"l{i}.hc{q}.out"], w1[f"l{i}.hc{q}.mix"] = torch.ones(1), torch.ones(1), torch.ones(1, 1)
    assert torch.allclose(O.forward(w, cfg, tk), O.forward(w1, one, tk), atol=1e-5)
