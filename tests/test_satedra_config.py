"""Satedra without a GPU: the configuration reader and its checks, the model's spec (tensor names, which run reads
whose cache, the window a shared cache is kept for), the table of stretched rotary frequencies against the plain
implementation's, and the plain implementation against an independent restatement of its own attention."""
import copy
import json
import math

import pytest
import torch

import plain_satedra as P
from mini_rsglang_b200.errors import InvalidRequest
from mini_rsglang_b200.models import config_from_dict, model_spec_for


def attention(heads=3, dim=24, rot_dim=8, vdim=20, kv_rank=40, scale=0.3, size=20, base=10000.0, dims=None, scaling=None, kv_from=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
             "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if size:
        mixer["mask"] = {"size": size}
    if scaling:
        mixer["rot"]["scaling"] = scaling
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer}


def moe(ff=36, experts=5, identity=1, top=2, scale=1.5, shared=28):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


STRETCH = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}
RAW = {"architecture": "Satedra", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "logit_scale": 0.7, "layers": [
    dict(attention(size=20, scaling=STRETCH), mlp={"kind": "dense", "ff": 100}),
    dict(attention(size=33, scaling=STRETCH, kv_from=0, heads=2, dim=16, vdim=24), mlp=moe()),
    dict(attention(size=9), mlp=None),
    dict(attention(size=0, kv_from=2), mlp=moe(identity=0, top=1, shared=0))]}


def test_reads_every_key_and_writes_them_back():
    config = config_from_dict(copy.deepcopy(RAW))
    assert config.model_type == "satedra" and config.vocab_size == 211 and config.width == 72 and config.logit_scale == 0.7
    assert config.layers[1]["mixer"]["kv_from"] == 0 and config.layers[2]["mlp"] is None
    assert config.layers[3]["mlp"]["router"]["identity"] == 0 and "shared" not in config.layers[3]["mlp"]
    assert config.eos_ids() == []
    again = config_from_dict(json.loads(json.dumps(config.to_dict())))
    assert again.to_dict() == config.to_dict()


@pytest.mark.parametrize("path,value", [
    (("layers", 1, "mixer", "kv_from"), 1), (("layers", 1, "mixer", "kv_from"), 2), (("layers", 1, "mixer", "kv_rank"), 48),
    (("layers", 0, "mixer", "rot", "dims"), 7), (("layers", 0, "mixer", "rot", "dims"), 10), (("layers", 1, "mlp", "router", "top"), 7),
    (("layers", 0, "mlp", "kind"), "sparse"), (("layers", 0, "type"), "attention"), (("layers", 2, "mixer", "mask", "size"), 0),
    (("norm", "eps"), 0.0), (("layers", 0, "mixer", "heads"), 0), (("layers", 1, "mlp", "expert", "ff"), 0)])
def test_refuses_what_does_not_fit(path, value):
    raw = copy.deepcopy(RAW)
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(InvalidRequest):
        config_from_dict(raw)


def test_spec_names_runs_and_cache_windows():
    spec = model_spec_for(config_from_dict(copy.deepcopy(RAW)))
    names = {s.name: tuple(s.shape) for s in spec.weight_specs()}
    assert names["embed"] == (211, 72) and names["head"] == (211, 72) and names["final.norm.b"] == (72,)
    assert names["l0.mix.dkv"] == (48, 72) and names["l0.mix.dkv.norm"] == (40,) and names["l0.mix.q"] == (3 * 32, 72)
    assert "l1.mix.dkv" not in names and names["l1.mix.uk"] == (2 * 16, 40) and names["l1.mix.uv"] == (2 * 24, 40)
    assert names["l1.mix.g"] == (2, 72) and names["l1.mix.o"] == (72, 48)
    assert names["l1.mlp.router"] == (6, 72) and names["l1.mlp.correction"] == (6,) and names["l1.mlp.e4.down"] == (72, 36)
    assert "l1.mlp.e5.gate" not in names and names["l1.mlp.shared.sg"] == (1, 72) and names["l1.mlp.shared.up"] == (28, 72)
    assert "l2.norm2" not in names and "l2.mlp.gate" not in names and "l3.mlp.shared.gate" not in names
    assert [(e.layer, e.cache_of) for e in spec.run_order] == [(0, None), (1, 0), (2, None), (3, 2)]
    mixers = [layer.parts["mixer"].params for layer in spec.layers]
    assert [m["window"] for m in mixers] == [20, 33, 9, 0]
    assert [m["cache_window"] for m in mixers] == [33, 33, 0, 0]       # the widest window that reads the cache; none: every key
    assert [m["shares_cache"] for m in mixers] == [False, True, False, True]


@pytest.mark.parametrize("dims,base,scaling", [(8, 10000.0, STRETCH), (48, 200000.0, {"factor": 6.0, "original": 1024, "fast": 24.0, "slow": 1.5}),
                                               (16, 100.0, {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 0.5}), (6, 50.0, None), (2, 10.0, STRETCH)])
def test_rotary_table_is_the_plain_one(dims, base, scaling):
    from mini_rsglang_b200.parts.base import POSITION_ENCODINGS, PartSpec

    params = {"rotary_dim": dims, "theta": base}
    params.update(scaling or {})
    part = POSITION_ENCODINGS.build(PartSpec("yarn_rope", params), "x")
    want, magnitude = P.yarn_frequencies(dims, base, scaling)
    assert torch.allclose(part.frequencies(), want, rtol=1e-14, atol=0)
    assert part.magnitude == pytest.approx(magnitude, rel=1e-15)
    if scaling:
        plain = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
        assert (want <= plain * (1 + 1e-12)).all() and (want >= plain / scaling["factor"] * (1 - 1e-12)).all()
        assert magnitude == pytest.approx(0.1 * math.log(scaling["factor"]) + 1.0)


def test_plain_attention_in_the_latent_space_equals_the_one_with_keys_and_values():
    """The identity that the engine's kernels rest on, checked on the plain implementation alone: scores and sums
    taken against the latent, with the up-projections moved to the query and to the result, give the same output."""
    torch.manual_seed(5)
    c = attention(heads=3, dim=8, rot_dim=4, vdim=6, kv_rank=10, size=5, scaling=STRETCH)["mixer"]
    T, W = 17, 12
    w = {"m.q": torch.randn(3 * 12, W).double(), "m.dkv": torch.randn(14, W).double(), "m.dkv.norm": torch.rand(10).double() + 0.5,
         "m.uk": torch.randn(3 * 8, 10).double(), "m.uv": torch.randn(3 * 6, 10).double(), "m.g": torch.randn(3, W).double(),
         "m.o": torch.randn(W, 18).double()}
    h = torch.randn(T, W).double()
    kept = P.latent_keys(h, w, "m.", c, 1e-5, torch.arange(T))
    want = P.latent_attention(h, w, "m.", c, 1e-5, kept)
    latent, key_rot = kept
    f, magnitude = P.yarn_frequencies(4, 10000.0, STRETCH)
    q = (h @ w["m.q"].T).view(T, 3, 12)
    rows = torch.cat([latent, key_rot], dim=1)
    heads = []
    for head in range(3):
        q_latent = q[:, head, :8] @ w["m.uk"].view(3, 8, 10)[head]
        q_row = torch.cat([q_latent, P.rotate(q[:, head, 8:], torch.arange(T), f, magnitude)], dim=1)
        s = torch.where(P.window_mask(T, 5), q_row @ rows.T * c["scale"], torch.tensor(-math.inf, dtype=torch.float64))
        mixed = torch.softmax(s, dim=-1) @ latent
        heads.append(mixed @ w["m.uv"].view(3, 6, 10)[head].T * torch.sigmoid(h @ w["m.g"].T)[:, head:head + 1])
    got = torch.cat(heads, dim=1) @ w["m.o"].T
    assert (got - want).abs().max() < 1e-10
