"""Host-side parts of the ragged-step engine (no GPU): step planning, page and slot bookkeeping, config parsing, the
safetensors reader, the registry, and the oracle's own consistency (its mixers against closed forms)."""
import json
import math
import os
import struct
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import mapedra_oracle as O  # noqa: E402
from paligemma_multimodal_system_b200.cache import PagePool, SequenceStore  # noqa: E402
from paligemma_multimodal_system_b200.serving import StepScheduler, TokenRequest  # noqa: E402


def test_page_pool_hands_out_lowest_first_and_refuses_double_free():
    p = PagePool(5)
    a = p.take(2)
    b = p.take(2)
    assert a == [0, 1] and b == [2, 3]
    p.give(a)
    assert p.take(3) == [0, 1, 4]
    with pytest.raises(MemoryError):
        p.take(1)
    p.give(b)
    with pytest.raises(RuntimeError):
        p.give(b)


def test_sequence_store_bookkeeping_without_tensors():
    st = SequenceStore([("kv", 8, 8), ("state", (1, 2, 2)), None], max_tokens=4 * 64, num_slots=2, dtype=torch.float32, allocate=False)
    a = st.admit("a")
    st.reserve("a", 65)
    assert a.slot == 0 and a.pages == [0, 1] and a.length == 0
    st.commit("a", 65)
    st.reserve("a", 63)       # 128 tokens still fit two pages
    assert a.pages == [0, 1]
    st.reserve("a", 64)       # 129 do not
    assert a.pages == [0, 1, 2]
    b = st.admit("b")
    assert b.slot == 1
    with pytest.raises(MemoryError):
        st.admit("c")
    st.reserve("b", 1)
    with pytest.raises(MemoryError):
        st.reserve("b", 65)
    st.release("a")
    c = st.admit("c")
    st.reserve("c", 130)
    assert c.slot == 0 and c.pages == [0, 1, 2]  # the freed slot and pages are used again
    with pytest.raises(KeyError):
        st.admit("c")


def test_step_scheduler_mixes_decode_rows_and_portions():
    s = StepScheduler(num_slots=2, num_pages=4, page=64, step_tokens=50, eos_token_id=9)
    s.submit(TokenRequest(0, list(range(70)), 3))     # 2 pages
    s.submit(TokenRequest(1, [5, 6], 2))               # 1 page
    s.submit(TokenRequest(2, list(range(100)), 30))    # 3 pages: waits for request 0's pages
    plan = s.plan()
    assert [(r.rid, len(t), smp) for r, t, smp in plan] == [(0, 50, False)]
    s.advance(plan[0][0], 50, None)
    plan = s.plan()  # request 0's last 20 rows, request 1's whole prompt beside it
    assert [(r.rid, len(t), smp) for r, t, smp in plan] == [(0, 20, True), (1, 2, True)]
    assert not s.advance(plan[0][0], 20, 4)
    assert not s.advance(plan[1][0], 2, 4)
    plan = s.plan()  # both decode one token each; request 2 still queued (slots full)
    assert [(r.rid, t, smp) for r, t, smp in plan] == [(0, [4], True), (1, [4], True)]
    assert not s.advance(plan[0][0], 1, 8)
    assert s.advance(plan[1][0], 1, 8)        # budget 2 reached
    plan = s.plan()  # slot free, but 2 + 3 pages > 4: request 2 keeps waiting
    assert [(r.rid, t) for r, t, _ in plan] == [(0, [8])]
    assert s.advance(plan[0][0], 1, 9) and s.finished[0] == [4, 8, 9]  # EOS appended, then stop
    plan = s.plan()
    assert [(r.rid, len(t)) for r, t, _ in plan] == [(2, 50)] and s.pages_out == 3
    with pytest.raises(ValueError):
        s.submit(TokenRequest(3, list(range(300)), 1))


def test_config_parsing_and_registry(tmp_path):
    from paligemma_multimodal_system_b200 import registry
    from paligemma_multimodal_system_b200.modeling_mapedra import MapedraConfig, MapedraForCausalLM
    cfg = {"architecture": "Mapedra", "vocab": 11, "width": 8, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5, "groups": 2},
           "token_side": {"dim": 3},
           "layers": [{"type": "lightning", "mixer": {"heads": 2, "dim": 4, "vdim": 6, "decay": [0.5, 0.25]}, "mlp": None},
                      {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 2, "scale": 0.5, "softcap": 10.0,
                                                      "rot": {"base": 100.0, "dims": 2}}, "mlp": {"kind": "dense", "ff": 12}}]}
    c = MapedraConfig(cfg)
    assert (c.vocab, c.width, c.norm_groups, c.side_dim, len(c.layers)) == (11, 8, 2, 3, 2)
    m = MapedraForCausalLM(c, torch.float32)
    assert m.cache_layout() == [("state", (2, 4, 6)), ("kv", 4, 2)]
    w = O.random_weights(cfg, seed=0)
    m.load_weights(w)
    with pytest.raises(KeyError):
        m.load_weights({k: v for k, v in w.items() if k != "l1.mix.k.norm"})
    with pytest.raises(KeyError):
        m.load_weights(dict(w, extra=torch.zeros(1)))
    with pytest.raises(ValueError):
        m.load_weights(dict(w, head=torch.zeros(11, 9)))
    with pytest.raises(ValueError):
        MapedraConfig(dict(cfg, layers=[{"type": "conv", "mixer": {}}]))
    assert registry.architecture_of(cfg) == "Mapedra" and "mapedra" in registry.known_architectures()
    assert registry.architecture_of({"architectures": ["PaliGemmaForConditionalGeneration"]}).lower() in registry.known_architectures()
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Nope"}))
    with pytest.raises(ValueError):
        registry.load_model(str(tmp_path))


def test_safetensors_reader(tmp_path):
    from paligemma_multimodal_system_b200.utils import read_safetensors
    a = torch.randn(3, 5).bfloat16()
    b = torch.arange(7, dtype=torch.int32)
    ra, rb = a.view(torch.int16).numpy().tobytes(), b.numpy().tobytes()
    meta = {"__metadata__": {"k": "v"}, "a": {"dtype": "BF16", "shape": [3, 5], "data_offsets": [0, len(ra)]},
            "b": {"dtype": "I32", "shape": [7], "data_offsets": [len(ra), len(ra) + len(rb)]}}
    head = json.dumps(meta).encode()
    f = tmp_path / "m.safetensors"
    f.write_bytes(struct.pack("<Q", len(head)) + head + ra + rb)
    t = read_safetensors(str(f))
    assert torch.equal(t["a"], a) and torch.equal(t["b"], b) and set(t) == {"a", "b"}
    f.write_bytes(struct.pack("<Q", len(head)) + head + ra)  # truncated data
    with pytest.raises(ValueError):
        read_safetensors(str(f))


def test_oracle_lightning_matches_the_closed_form():
    """o_t = sum_{j <= t} a^(t-j) (q_t . k_j) v_j -- the recurrence unrolled."""
    cfg = {"architecture": "Mapedra", "vocab": 8, "width": 16, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6, "groups": 1},
           "layers": [{"type": "lightning", "mixer": {"heads": 2, "dim": 4, "vdim": 6, "decay": [0.9, 1.0]}, "mlp": None}]}
    w = O.random_weights(cfg, seed=1)
    h = torch.randn(12, 16, generator=torch.Generator().manual_seed(0))
    m = cfg["layers"][0]["mixer"]
    silu = torch.nn.functional.silu
    q, k = silu(h @ w["l0.mix.q"].T).view(12, 2, 4), silu(h @ w["l0.mix.k"].T).view(12, 2, 4)
    v = silu(h @ w["l0.mix.v"].T).view(12, 2, 6)
    o = torch.zeros(12, 2, 6)
    for t in range(12):
        for j in range(t + 1):
            for hd in range(2):
                o[t, hd] += m["decay"][hd] ** (t - j) * (q[t, hd] @ k[j, hd]) * v[j, hd]
    ref = (O.rms(o.reshape(12, 12), 1e-6) * w["l0.mix.norm"] * torch.sigmoid(h @ w["l0.mix.g"].T)) @ w["l0.mix.o"].T
    assert torch.allclose(O.lightning_mixer(h, w, "l0.mix.", m, 1e-6), ref, atol=1e-5, rtol=1e-4)


def test_oracle_rotation_is_relative_and_partial():
    """Scores of rotated q, k depend on the position difference only, and dimensions past rot.dims are untouched."""
    f = O.rope_frequencies({"base": 100.0, "dims": 4})
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(8, generator=g), torch.randn(8, generator=g)
    s1 = O.rotate_interleaved(q, 17, f) @ O.rotate_interleaved(k, 5, f)
    s2 = O.rotate_interleaved(q, 112, f) @ O.rotate_interleaved(k, 100, f)
    assert abs(float(s1 - s2)) < 1e-4
    assert torch.equal(O.rotate_interleaved(q, 9, f)[4:], q[4:])
    r = O.rotate_interleaved(torch.tensor([1.0, 0.0, 0, 0, 0, 0, 0, 0]), 1, f)   # (u, v) -> (u cos - v sin, v cos + u sin)
    assert torch.allclose(r[:2], torch.tensor([torch.cos(torch.tensor(1.0)), torch.sin(torch.tensor(1.0))]))


def test_rotary_frequencies_with_and_without_rescaling():
    from paligemma_multimodal_system_b200.mixers import rotary_frequencies
    for rot in ({"base": 10000.0, "dims": 16}, {"base": 5e5, "dims": 32, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 128}},
                {"base": 100.0, "dims": 8, "scaling": {"factor": 2.0, "low": 2.0, "high": 4.0, "original": 40}}):
        got = rotary_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
        ref = torch.tensor(O.rope_frequencies(rot), dtype=torch.float64)
        assert torch.allclose(got, ref, rtol=1e-12, atol=0)
        if "scaling" in rot:  # all three branches occur
            wl, sc = 2 * math.pi / torch.tensor([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)]), rot["scaling"]
            assert (wl < sc["original"] / sc["high"]).any() and (wl > sc["original"] / sc["low"]).any()
            assert ((wl >= sc["original"] / sc["high"]) & (wl <= sc["original"] / sc["low"])).any()
