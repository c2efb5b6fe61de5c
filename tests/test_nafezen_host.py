"""Nafezen without a GPU: configuration, the model's tensor names, random model
folders, and the plain implementation's mechanisms against closed forms."""
import json
import math
import os

import pytest
import torch

import plain_nafezen as P
from nafezen_models import CONFIGS, MIXED, ODD, make_model

F = torch.float64


def test_config_reads_back_and_names_tensors(tmp_path):
    from nnis_b200.config import config_from_dict, read_config
    from nnis_b200.engine.model import DecoderModel
    for name, raw in CONFIGS.items():
        cfg = config_from_dict(raw)
        assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
        spec = cfg.to_spec()
        assert spec.architecture == "Nafezen" and len(spec.layers) == len(raw["layers"])
        names = DecoderModel.weight_specs_of(spec)
        assert {"embed", "embed.norm", "final.norm", "l0.norm1"} <= set(names)
        assert not any(n.endswith(".weight") for n in names)
    names = DecoderModel.weight_specs_of(config_from_dict(MIXED).to_spec())
    assert names["l0.mix.dkv"].shape == (48 + 8, 96) and names["l0.mix.uq"].shape == (3 * 40, 40)
    assert names["l1.mlp.e4.down"].shape == (96, 56) and names["l1.mlp.shared.sg"].shape == (1, 96)
    assert names["l1.mix.g"].shape == (120, 96) and "l2.mlp.shared.up" not in names
    assert not any(n.startswith("l3.mlp") for n in names)
    d = make_model(str(tmp_path / "m"), ODD, seed=3)
    assert read_config(d).to_dict() == config_from_dict(ODD).to_dict()


@pytest.mark.parametrize("change, text", [
    (lambda c: c.update(architecture="Other"), "unknown architecture"),
    (lambda c: c["norm"].update(groups=5), "does not divide"),
    (lambda c: c["layers"][0].update(type="window"), "not a mixer"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "one number per head"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mlp"].update(kind="conv"), "not known"),
    (lambda c: c.pop("vocab"), "vocab"),
])
def test_config_errors_name_the_key(change, text):
    from nnis_b200.config import ConfigError, config_from_dict
    raw = json.loads(json.dumps(MIXED))
    change(raw)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(raw)


def test_loader_reports_every_fault_of_a_folder(tmp_path):
    from safetensors.torch import load_file, save_file
    from nnis_b200.config import read_config
    from nnis_b200.engine.model import DecoderModel
    from nnis_b200.weights.loader import WeightError, check_weights
    d = make_model(str(tmp_path / "m"), MIXED, seed=1)
    wanted = DecoderModel.weight_specs_of(read_config(d).to_spec())
    assert check_weights(d, wanted)["recognized_tensors"] == len(wanted)
    path = os.path.join(d, "model.safetensors")
    w = load_file(path)
    del w["l1.mlp.router.b"]
    w["l0.mix.uk"] = w["l0.mix.uk"][:, :-1].contiguous()
    w["l9.extra"] = torch.zeros(2)
    save_file(w, path)
    with pytest.raises(WeightError) as e:
        check_weights(d, wanted)
    assert "l1.mlp.router.b" in str(e.value) and "l0.mix.uk" in str(e.value) and "l9.extra" in str(e.value)


def test_command_line_writes_and_validates_a_model_folder(tmp_path):
    from nnis_b200.cli.main import main
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(ODD))
    out = tmp_path / "model"
    assert main(["random-model", "--config", str(cfg), "--seed", "9", "--out", str(out)]) == 0
    report = tmp_path / "report.json"
    assert main(["validate", "--model", str(out), "--json", "--output", str(report)]) == 0
    seen = json.loads(report.read_text())
    assert seen["ready"] and seen["architecture"] == "Nafezen" and seen["layers"] == 3


# ---- the plain implementation's mechanisms against closed forms ---------------------
def test_plain_grouped_norm():
    x = torch.randn(5, 12, dtype=F)
    w = torch.randn(12, dtype=F)
    y = P.grouped_rms_norm(x, w, 1e-5, 3)
    for r in range(5):
        for g in range(3):
            part = x[r, 4 * g:4 * g + 4]
            want = part / math.sqrt(float((part * part).mean()) + 1e-5) * w[4 * g:4 * g + 4]
            assert torch.allclose(y[r, 4 * g:4 * g + 4], want, atol=1e-12)
    assert torch.allclose(P.grouped_rms_norm(x, w, 1e-5, 1), P.rms_norm(x, w, 1e-5))


def test_plain_rotation_turns_the_first_dims_only():
    x = torch.randn(7, 2, 10, dtype=F)
    y = P.rotate(x, 100.0, 6)
    assert torch.equal(y[..., 6:], x[..., 6:]) and torch.allclose(y[0], x[0])
    for i in range(3):
        a = 5 * 100.0 ** (-2 * i / 6)
        u, v = x[5, 1, i], x[5, 1, i + 3]
        assert abs(float(y[5, 1, i]) - float(u * math.cos(a) - v * math.sin(a))) < 1e-5
        assert abs(float(y[5, 1, i + 3]) - float(v * math.cos(a) + u * math.sin(a))) < 1e-5
    # a rotation keeps the dot product of a pair rotated at the same distance
    q, k = torch.randn(9, 1, 8, dtype=F), torch.randn(9, 1, 8, dtype=F)
    same = lambda t: q[0:1].expand(9, 1, 8) if t == "q" else k[0:1].expand(9, 1, 8)
    rq, rk = P.rotate(same("q").clone(), 50.0, 8), P.rotate(same("k").clone(), 50.0, 8)
    assert abs(float((rq[7] * rk[5]).sum() - (rq[4] * rk[2]).sum())) < 1e-5


def test_plain_retention_is_the_decayed_sum():
    torch.manual_seed(0)
    t, width = 9, 16
    m = {"heads": 2, "dim": 4, "vdim": 6, "decay": [0.5, 0.9], "rot": {"base": 10.0, "dims": 2}}
    w = {"x.q": torch.randn(8, width), "x.k": torch.randn(8, width), "x.v": torch.randn(12, width),
         "x.g": torch.randn(12, width), "x.o": torch.eye(12)}
    h = torch.randn(t, width, dtype=F)
    got = P.retention(h, w, "x.", m, 1e-6, False)
    q = P.rotate((h @ w["x.q"].to(F).t()).reshape(t, 2, 4), 10.0, 2)
    k = P.rotate((h @ w["x.k"].to(F).t()).reshape(t, 2, 4), 10.0, 2) * 4 ** -0.5
    v = (h @ w["x.v"].to(F).t()).reshape(t, 2, 6)
    g = h @ w["x.g"].to(F).t()
    g = g * torch.sigmoid(g)
    for i in (0, 3, 8):
        for hd in range(2):
            o = sum(m["decay"][hd] ** (i - s) * float(q[i, hd] @ k[s, hd]) * v[s, hd] for s in range(i + 1))
            o = o / torch.sqrt((o * o).mean() + 1e-6)
            assert torch.allclose(got[i, 6 * hd:6 * hd + 6], o * g[i, 6 * hd:6 * hd + 6], atol=1e-9)


def test_plain_latent_attention_first_token_and_causality():
    torch.manual_seed(1)
    from nafezen_models import latent
    m = latent(2, 4, 2, 3, 5, 6)
    width = 8
    w = {"x.dq": torch.randn(5, width), "x.dq.norm": torch.ones(5), "x.uq": torch.randn(12, 5),
         "x.dkv": torch.randn(8, width), "x.dkv.norm": torch.rand(6) + 0.5, "x.uk": torch.randn(8, 6),
         "x.uv": torch.randn(6, 6), "x.o": torch.eye(6)}
    h = torch.randn(6, width, dtype=F)
    full = P.latent_attention(h, w, "x.", m, 1e-6, False)
    # the first token sees itself only: its output is its own value
    c = P.rms_norm((h[0:1] @ w["x.dkv"].to(F).t())[:, :6], w["x.dkv.norm"], 1e-6)
    assert torch.allclose(full[0], (c @ w["x.uv"].to(F).t())[0], atol=1e-9)
    # later tokens do not change earlier outputs
    assert torch.allclose(P.latent_attention(h[:4], w, "x.", m, 1e-6, False), full[:4], atol=1e-9)


def test_plain_experts_weigh_the_chosen_only():
    torch.manual_seed(2)
    from nafezen_models import moe
    width, mlp = 6, moe(4, 2, 5, shared=3)
    w = {"x.router": torch.randn(4, width), "x.router.b": torch.randn(4), "x.shared.up": torch.randn(3, width),
         "x.shared.down": torch.randn(width, 3), "x.shared.sg": torch.randn(1, width)}
    for e in range(4):
        w[f"x.e{e}.up"], w[f"x.e{e}.down"] = torch.randn(5, width), torch.randn(width, 5)
    h = torch.randn(3, width, dtype=F)
    got = P.moe_ff(h, w, "x.", mlp, False)
    for n in range(3):
        z = h[n] @ w["x.router"].to(F).t() + w["x.router.b"].to(F)
        order = sorted(range(4), key=lambda e: -float(z[e]))[:2]
        p = torch.softmax(z[order], 0)
        want = sum(p[j] * (torch.relu(h[n] @ w[f"x.e{e}.up"].to(F).t()) ** 2) @ w[f"x.e{e}.down"].to(F).t()
                   for j, e in enumerate(order))
        sh = (torch.relu(h[n] @ w["x.shared.up"].to(F).t()) ** 2) @ w["x.shared.down"].to(F).t()
        want = want + torch.sigmoid(h[n] @ w["x.shared.sg"].to(F)[0]) * sh
        assert torch.allclose(got[n], want, atol=1e-9)


def test_cache_groups_without_values_and_state_areas():
    from nnis_b200.cache import CacheManager, KVRequest, StateRequest
    cache = CacheManager([KVRequest(1, 56, 0, values=False), StateRequest((3, 24, 40)),
                          KVRequest(1, 56, 0, values=False), KVRequest(2, 16, 0)],
                         torch.float32, torch.device("cpu"), max_tokens=256, max_slots=3, max_positions=1 << 20)
    assert len(cache.groups) == 2 and cache.view(0).v is None and cache.view(3).v is not None
    assert cache.view(0).group == cache.view(2).group and tuple(cache.view(0).k.shape) == (4, 1, 64, 56)
    assert cache.kv_bytes_per_token() == (2 * 56 + 2 * 2 * 16) * 4
    a = cache.acquire()
    cache.view(1).state[a].fill_(1.0)
    cache.reserve([a], [70])
    cache.commit([a], [70])
    snap = cache.snapshot(a)
    cache.view(1).state[a].fill_(2.0)
    cache.restore(snap)
    assert float(cache.view(1).state[a].max()) == 1.0
    cache.release(a)
    b = cache.acquire()
    assert b == a and float(cache.view(1).state[b].abs().max()) == 0.0  # a slot used again starts at zero
    cache.release(b)
    cache.check()
