"""Tazadra without a GPU: configuration round trip and errors by key, tensor names, the
plain mechanisms against closed forms, and what the design asks of the cache (values of
their own size, a state of several tensors, a free extent of a stored tensor)."""
import copy
import math

import pytest
import torch

import plain_tazadra as P
from tazadra_models import CONFIGS, MIXED, ODD, make_model, load_weights, read_config

F = torch.float64


def test_configuration_round_trip_and_spec():
    from nnis_b200.config import config_from_dict
    for cfg in CONFIGS.values():
        typed = config_from_dict(cfg)
        assert config_from_dict(typed.to_dict()).to_dict() == typed.to_dict()
        spec = typed.to_spec()
        assert [l.block for l in spec.layers] == ["branch_norm"] * len(cfg["layers"])
        for i, (entry, layer) in enumerate(zip(spec.schedule, cfg["layers"])):
            assert entry.cache_of == layer["mixer"].get("kv_from")
            assert ("ffn" in spec.layers[i].parts) == (layer["mlp"] is not None)
            assert spec.layers[i].params["residual_mult"] == cfg["residual_mult"]
    spec = config_from_dict(MIXED).to_spec()
    att = spec.layers[3].part("mixer")
    assert att.kind == "sink_attention" and att["kv"] == "shared" and att["chunk"] == 24 and att["softcap"] == 0.0
    assert spec.layers[0].part("mixer")["position"]["scaling"]["original"] == 64
    assert spec.head["softcap"] == 20.0 and config_from_dict(ODD).to_spec().head["softcap"] == 0.0


@pytest.mark.parametrize("change, word", [
    (lambda c: c.update(architecture="Other"), "architecture"),
    (lambda c: c["layers"][0].update(type="conv"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"].update(heads=5), "multiple"),
    (lambda c: c["layers"][0]["mixer"].update(dim=23), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(high=1.0), "differ"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "earlier"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "keys and values"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=8), "differs"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "exceeds"),
    (lambda c: c["layers"][1]["mlp"].pop("limit"), "limit"),
    (lambda c: c["layers"][2]["mixer"].update(state=0), "state"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_configuration_errors_name_the_key(change, word):
    from nnis_b200.config import ConfigError, config_from_dict
    cfg = copy.deepcopy(MIXED)
    change(cfg)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(cfg)


def test_tensor_names_and_the_free_extent(tmp_path):
    from nnis_b200.config import config_from_dict
    from nnis_b200.engine.model import DecoderModel
    from nnis_b200.weights.loader import shape_fits
    want = DecoderModel.weight_specs_of(config_from_dict(MIXED).to_spec())
    for name in ("embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q.norm", "l0.mix.k.norm", "l0.mix.sink",
                 "l0.mix.g", "l0.mlp.router", "l0.mlp.e5.gate", "l1.mix.mu.w", "l1.mix.w0", "l1.mix.u", "l1.mlp.up",
                 "l2.mix.conv", "l2.mix.conv.b", "l2.mix.A_log", "l2.mix.dt.b", "l2.mix.D", "l3.mix.q", "l4.norm1"):
        assert name in want, name
    for name in ("l3.mix.k", "l3.mix.v", "l3.mix.k.norm", "l0.mix.q.weight"):
        assert name not in want, name
    assert want["l4.norm2"].role == "unused"  # (a layer without a feed-forward neither reads nor misses it)
    assert want["l0.mix.v"].shape == (2 * 16, 96) and want["l0.mix.g"].shape == (4, 96)
    assert want["l2.mix.x"].shape == (6 + 2 * 12, 80) and want["l2.mix.conv"].shape == (80, 3)
    assert want["l1.mix.u"].shape == (3, 16) and want["l1.mix.w1"].shape == (12, 96)
    # a configuration that does not name the decay's inner size takes the stored tensor's
    cfg = copy.deepcopy(MIXED)
    del cfg["layers"][1]["mixer"]["decay_rank"]
    free = DecoderModel.weight_specs_of(config_from_dict(cfg).to_spec())
    assert free["l1.mix.w1"].shape == (-1, 96) and free["l1.mix.w2"].shape == (48, -1)
    assert shape_fits((12, 96), (-1, 96)) and not shape_fits((12, 95), (-1, 96)) and not shape_fits((0, 96), (-1, 96))
    from nnis_b200.weights import write_random_model
    with pytest.raises(ValueError, match="extent"):
        write_random_model(cfg, 1, str(tmp_path / "m"))


def test_the_cache_gives_values_their_own_size_and_states_of_several_tensors():
    from nnis_b200.cache import CacheManager, KVRequest, StateRequest
    requests = [KVRequest(2, 24, 0, True, 16), None, StateRequest((3, 4, 4), extra=(((7,), torch.float32),)),
                KVRequest(2, 24, 0, True, 16), KVRequest(2, 24), StateRequest((5, 2), extra=(((2, 5), torch.float32),))]
    cache = CacheManager(requests, torch.float32, torch.device("cpu"), 640, 4, 1 << 20)
    assert len(cache.groups) == 2  # values of 16 and values of 24 do not share storage
    a, b, c = cache.view(0), cache.view(3), cache.view(4)
    assert a.group == b.group != c.group and tuple(a.k.shape[1:]) == (2, 64, 24) and tuple(a.v.shape[1:]) == (2, 64, 16)
    assert tuple(c.v.shape[1:]) == (2, 64, 24) and cache.view(1) is None
    s, t = cache.view(2), cache.view(5)
    assert tuple(s.state.shape) == (4, 3, 4, 4) and tuple(s.extra[0].shape) == (4, 7) and tuple(t.extra[0].shape) == (4, 2, 5)
    slot = cache.acquire()
    for x in (s.state, s.extra[0], t.state, t.extra[0]):
        x[slot].fill_(3.0)
    kept = cache.snapshot(slot)
    s.extra[0][slot].fill_(5.0)
    cache.restore(kept)
    assert float(s.extra[0][slot].max()) == 3.0
    cache.release(slot)
    assert cache.acquire() == slot
    assert all(float(x[slot].abs().max()) == 0.0 for x in (s.state, s.extra[0], t.state, t.extra[0]))
    assert cache.kv_bytes_per_token() == (2 * 2 * (24 + 16) + 2 * (24 + 24)) * 4


# ---- the plain mechanisms against closed forms ----------------------------------------------
def test_plain_rotation_turns_neighbours_and_keeps_the_rest():
    x = torch.arange(2 * 1 * 6, dtype=F).reshape(2, 1, 6) + 1
    freq = torch.tensor([0.5], dtype=F)
    y = P.rotate_pairs(x, torch.tensor([0, 3]), freq)
    assert torch.equal(y[0], x[0]) and torch.equal(y[1, 0, 2:], x[1, 0, 2:])
    c, s = math.cos(1.5), math.sin(1.5)
    assert torch.allclose(y[1, 0, :2], torch.tensor([7 * c - 8 * s, 8 * c + 7 * s], dtype=F))
    assert abs(float((y[1, 0, :2] ** 2).sum()) - (49 + 64)) < 1e-9


def _attention_weights(T, chunk, sink, cap=None, scale=1.0):
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 1, "scale": scale, "rot": {"dims": 0, "base": 10.0}}
    if chunk:
        m["mask"] = {"size": chunk}
    if cap:
        m["softcap"] = cap
    w = {"a.q": torch.zeros(2, 2, dtype=F), "a.q.norm": torch.ones(2, dtype=F), "a.sink": torch.tensor([sink], dtype=F),
         "a.g": torch.zeros(1, 2, dtype=F), "a.o": torch.ones(1, 1, dtype=F)}
    probes = {}
    h = torch.ones(T, 2, dtype=F)
    P.attention(h, w, "a", m, 1e-6, torch.arange(T), torch.ones(T, 1, 2, dtype=F), torch.ones(T, 1, 1, dtype=F), False,
                probes)
    return probes["weights"][0], probes["sink"][0]


def test_plain_attention_chunks_count_from_zero_and_the_sink_counts_once():
    weights, sink = _attention_weights(7, 3, 0.0)
    # scores are all zero: a query shares its weight evenly between its chunk's keys so far and the sink
    for i in range(7):
        seen = i % 3 + 1
        assert torch.allclose(weights[i], torch.tensor([1.0 / (seen + 1) if i - i % 3 <= j <= i else 0.0 for j in range(7)],
                                                       dtype=F))
        assert abs(float(sink[i]) - 1.0 / (seen + 1)) < 1e-12
    weights, sink = _attention_weights(4, 0, math.log(3.0))
    assert abs(float(sink[3]) - 3.0 / 7.0) < 1e-12 and abs(float(weights[3].sum()) - 4.0 / 7.0) < 1e-12


def test_plain_wkv_is_the_decayed_sum_with_a_bonus_for_the_current_token():
    torch.manual_seed(0)
    T, W, H, d = 6, 4, 1, 3
    w = {f"a.mu.{s}": torch.zeros(W, dtype=F) for s in "rkvgw"}
    for p in "rkvg":
        w[f"a.{p}"] = torch.randn(H * d, W, dtype=F)
    w.update({"a.w1": torch.zeros(2, W, dtype=F), "a.w2": torch.zeros(H * d, 2, dtype=F),
              "a.w0": torch.log(-torch.log(torch.tensor([0.5, 0.9, 0.99], dtype=F))), "a.u": torch.tensor([[2.0, 0.0, -1.0]], dtype=F),
              "a.norm": torch.ones(H * d, dtype=F), "a.o": torch.eye(H * d, dtype=F)})
    h = torch.randn(T, W, dtype=F)
    got = P.wkv(h, w, "a", {"heads": H, "dim": d}, 1e-9, False)
    r, k, v = (h @ w[f"a.{p}"].T for p in "rkv")
    decay = torch.tensor([0.5, 0.9, 0.99], dtype=F)
    for t in range(T):
        o = sum((r[t] * decay ** (t - 1 - j) * k[j]).sum() * v[j] for j in range(t)) + (r[t] * w["a.u"][0] * k[t]).sum() * v[t]
        want = o / torch.sqrt((o * o).mean() + 1e-9) * P.silu(h[t] @ w["a.g"].T)
        assert torch.allclose(got[t], want, atol=1e-9)
    # the token shift: with mu = 1 every stream reads the token before, and the first token reads zeros
    for s in "rkvgw":
        w[f"a.mu.{s}"] = torch.ones(W, dtype=F)
    shifted = P.wkv(h, w, "a", {"heads": H, "dim": d}, 1e-9, False)
    assert float(shifted[0].abs().max()) == 0.0
    assert torch.allclose(shifted[1:], P.wkv(torch.cat([h[:-1]]), {**w, **{f"a.mu.{s}": torch.zeros(W, dtype=F) for s in "rkvgw"}},
                                             "a", {"heads": H, "dim": d}, 1e-9, False), atol=1e-9)


def test_plain_selective_scan_is_the_weighted_sum_over_the_past():
    torch.manual_seed(1)
    T, W, I, N, R, taps = 5, 3, 2, 2, 1, 3
    w = {"a.in": torch.randn(2 * I, W, dtype=F), "a.conv": torch.randn(I, taps, dtype=F), "a.conv.b": torch.randn(I, dtype=F),
         "a.x": torch.randn(R + 2 * N, I, dtype=F), "a.dt": torch.randn(I, R, dtype=F), "a.dt.b": torch.randn(I, dtype=F),
         "a.A_log": torch.randn(I, N, dtype=F), "a.D": torch.randn(I, dtype=F), "a.o": torch.eye(I, dtype=F)}
    h = torch.randn(T, W, dtype=F)
    got = P.mamba1(h, w, "a", {"inner": I, "state": N, "dt_rank": R, "conv": taps}, False)
    xz = h @ w["a.in"].T
    x_in, z = xz[:, :I], xz[:, I:]
    x = torch.stack([sum(w["a.conv"][:, j] * (x_in[t - (taps - 1 - j)] if t - (taps - 1 - j) >= 0 else 0) for j in range(taps))
                     + w["a.conv.b"] for t in range(T)])
    x = P.silu(x)
    dbc = x @ w["a.x"].T
    dt = torch.log1p(torch.exp(dbc[:, :R] @ w["a.dt"].T + w["a.dt.b"]))
    A = -torch.exp(w["a.A_log"])
    for t in range(T):
        y = torch.zeros(I, dtype=F)
        for j in range(t + 1):
            carried = torch.exp(A * dt[j + 1:t + 1].sum(dim=0)[:, None])  # [I, N]
            y += (carried * (dt[j] * x[j])[:, None] * dbc[j, R:R + N][None, :] * dbc[t, R + N:][None, :]).sum(dim=1)
        y = (y + w["a.D"] * x[t]) * P.silu(z[t])
        assert torch.allclose(got[t], y, atol=1e-9)


def test_plain_feed_forwards():
    w = {"a.gate": torch.tensor([[1.0], [1.0], [1.0]], dtype=F), "a.up": torch.tensor([[1.0], [-1.0], [0.5]], dtype=F),
         "a.down": torch.eye(3, dtype=F)}
    got = P.dense_ff(torch.tensor([[5.0]], dtype=F), w, "a", {"limit": 2.0}, False)[0]
    g = 2.0 / (1 + math.exp(-1.702 * 2.0))
    assert torch.allclose(got, torch.tensor([g * 3.0, g * -1.0, g * 3.0], dtype=F))
    low = P.dense_ff(torch.tensor([[-5.0]], dtype=F), w, "a", {"limit": 2.0}, False)[0]
    gl = -5.0 / (1 + math.exp(1.702 * 5.0))  # the gate has no lower limit
    assert torch.allclose(low, torch.tensor([gl * -1.0, gl * 3.0, gl * -1.0], dtype=F))
    # experts: sigmoid scores of the chosen, not renormalised, on the expert's input
    mlp = {"router": {"experts": 3, "top": 2}}
    w = {"m.router": torch.tensor([[1.0, 0.0], [3.0, 0.0], [2.0, 0.0]], dtype=F)}
    for e in range(3):
        w.update({f"m.e{e}.gate": torch.tensor([[1.0 + e, 0.0]], dtype=F), f"m.e{e}.up": torch.tensor([[0.0, 1.0]], dtype=F),
                  f"m.e{e}.down": torch.tensor([[1.0], [0.0]], dtype=F)})
    h = torch.tensor([[1.0, 2.0]], dtype=F)
    ids, val, gap = P.router(h, w, "m", mlp)
    assert ids.tolist() == [[1, 2]] and torch.allclose(val, torch.sigmoid(torch.tensor([[3.0, 2.0]], dtype=F)))
    assert abs(float(gap) - (1 / (1 + math.exp(-2.0)) - 1 / (1 + math.exp(-1.0)))) < 1e-12
    got = P.moe_ff(h, w, "m", mlp, False)[0, 0]
    want = sum(float(P.silu(torch.tensor((1.0 + e) * s, dtype=F))) * (2.0 * s)
               for e, s in ((1, 1 / (1 + math.exp(-3.0))), (2, 1 / (1 + math.exp(-2.0)))))
    assert abs(float(got) - want) < 1e-12


def test_plain_forward_runs_every_configuration_and_prefixes_agree(tmp_path):
    """Causality: the logits of a prefix are the logits of the whole at those positions."""
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        d = make_model(str(tmp_path / name), cfg, seed=i)
        w = load_weights(d, False)
        toks = [(7 * j + i) % cfg["vocab"] for j in range(30)]
        whole = P.forward(read_config(d), w, toks)
        part = P.forward(read_config(d), w, toks[:17])
        assert torch.isfinite(whole).all() and torch.allclose(whole[:17], part, atol=1e-9), name


def test_a_layer_without_feed_forward_tolerates_a_stored_second_norm(tmp_path):
    """The folder may hold the second norm of a layer that has no feed-forward: it is neither read nor
    missed, and any other stranger is still refused."""
    from safetensors.torch import load_file, save_file
    from nnis_b200.config import read_config as typed_config
    from nnis_b200.engine.model import DecoderModel
    from nnis_b200.weights.loader import WeightError, check_weights
    import os
    d = make_model(str(tmp_path / "m"), MIXED, seed=1)
    wanted = DecoderModel.weight_specs_of(typed_config(d).to_spec())
    assert wanted["l4.norm2"].role == "unused" and "l3.norm2" in wanted and wanted["l3.norm2"].role == "vector"
    path = os.path.join(d, "model.safetensors")
    w = load_file(path)
    assert "l4.norm2" not in w
    check_weights(d, wanted)
    w["l4.norm2"] = torch.ones(96, dtype=torch.bfloat16)
    save_file(w, path)
    check_weights(d, wanted)
    w["l4.norm3"] = torch.ones(96, dtype=torch.bfloat16)
    save_file(w, path)
    with pytest.raises(WeightError, match="unexpected"):
        check_weights(d, wanted)
