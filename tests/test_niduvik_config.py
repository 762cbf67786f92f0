"""Niduvik without a GPU: its configuration as config.json has it, the parts and tensor names that the registry makes of
it, the distance buckets against the plain implementation, seeded random models, and the plain implementation's own
consistency (a window that covers everything equals no window; kept tokens change what a far query sees)."""
import json
import os

import pytest
import torch

import plain_niduvik as P
from mini_rsglang_b200.errors import InvalidRequest
from mini_rsglang_b200.models import config_from_dict, load_config, model_spec_for
from mini_rsglang_b200.weights import write_random_model
from mini_rsglang_b200.weights.safetensors_io import SafetensorsFile

RAW = {"architecture": "Niduvik", "vocab": 50, "width": 24, "norm": {"eps": 1e-5}, "layers": [
    {"type": "mamba2", "mixer": {"heads": 2, "vdim": 8, "state": 6, "groups": 1, "conv": 3, "norm_groups": 2}, "mlp": None},
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 10, "scale": 0.4, "softcap": 5.0, "bias_max": 20,
                                    "bias_rows": 6, "v_mix": True, "mask": {"size": 7, "keep_first": 2}},
     "mlp": {"kind": "dense", "ff": 40, "limit": 1.0}},
    {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 12, "vdim": 10, "scale": 0.3, "softcap": 9.0, "bias_max": 20,
                                    "bias_rows": 6, "v_mix": True, "mask": {"size": 5, "keep_first": 0}}, "mlp": None}]}


def test_config_is_read_as_the_file_has_it_and_written_back():
    config = config_from_dict(RAW)
    assert config.model_type == "niduvik" and config.vocab_size == 50 and config.width == 24 and config.eos_ids() == []
    assert config.layers[1]["mixer"]["mask"] == {"size": 7, "keep_first": 2} and config.layers[0]["mlp"] is None
    assert config_from_dict(json.loads(json.dumps(config.to_dict()))).to_dict() == config.to_dict()
    for path, value in ((("layers", 0, "type"), "lstm"), (("layers", 1, "mixer", "kv_heads"), 3), (("layers", 1, "mlp", "kind"), "routed"),
                        (("norm",), None), (("layers", 0, "mixer", "norm_groups"), 3)):
        broken = json.loads(json.dumps(RAW))
        at = broken
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(InvalidRequest):
            config_from_dict(broken)


def test_spec_names_the_checkpoints_tensors_and_leaves_the_table_rows_to_the_file():
    spec = model_spec_for(config_from_dict(RAW))
    names = {w.name: tuple(w.shape) for w in spec.weight_specs()}
    assert names["embed"] == (50, 24) and names["final.norm"] == (24,) and "head.weight" not in names
    assert names["l0.mix.in"] == (2 * 16 + 2 * 6 + 2, 24) and names["l0.mix.conv"] == (16 + 12, 3) and "l0.norm2" not in names
    assert names["l1.mix.q"] == (24, 24) and names["l1.mix.v.b"] == (20,) and names["l1.mix.rel"] == (6, 4)
    assert names["l1.mix.vmix"] == () and names["l1.mix.g"] == (4, 24) and names["l1.mlp.down"] == (24, 40)
    without = json.loads(json.dumps(RAW))
    for layer in without["layers"][1:]:
        del layer["mixer"]["bias_rows"]
    assert {w.name: tuple(w.shape) for w in model_spec_for(config_from_dict(without)).weight_specs()}["l1.mix.rel"] == (-1, 4)
    mixers = [layer.parts["mixer"] for layer in spec.layers]
    assert mixers[1].params["value_mix_source"] and not mixers[2].params["value_mix_source"]


def test_distance_buckets():
    from mini_rsglang_b200.parts.attention_biased import distance_buckets

    for rows, far in ((32, 120.0), (12, 50.0), (7, 30.0), (4, 9.0), (2, 5.0), (32, 400.0), (9, 1000.5)):
        table = distance_buckets(rows, far)
        for n in range(len(table) + 40):
            assert table[min(n, len(table) - 1)] == P.distance_bucket(n, rows, far), (rows, far, n)


def test_random_model_folder_loads_and_the_plain_implementation_runs_it(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), config_from_dict(RAW), seed=3)
    assert load_config(folder).to_dict() == config_from_dict(RAW).to_dict()
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    weights = {k: t.read() for k, t in SafetensorsFile(os.path.join(folder, "model.safetensors")).tensors.items()}
    tokens = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5, 8, 9, 7, 9, 3]
    logits, streams = P.forward(config, weights, tokens)
    assert logits.shape == (16, 50) and streams.shape == (3, 16, 24) and torch.isfinite(logits).all()
    again, _ = P.forward(config, weights, tokens[:9])
    assert torch.allclose(again, logits[:9], atol=1e-12), "a position's logits depend on later tokens"


def test_plain_window_and_kept_tokens():
    torch.manual_seed(0)
    T_, H, G, d = 30, 2, 1, 4
    q, k, rel = torch.randn(T_, H, d).double(), torch.randn(T_, G, d).double(), torch.randn(6, H).double()
    everything = P.attention_scores(q, k, rel, 0.5, 4.0, 20.0, T_ + 1, 0)
    assert torch.isfinite(everything[:, 20, :21]).all() and torch.isinf(everything[:, 20, 21:]).all()
    windowed = P.attention_scores(q, k, rel, 0.5, 4.0, 20.0, 5, 2)
    seen = [j for j in range(T_) if torch.isfinite(windowed[0, 20, j])]
    assert seen == [0, 1, 16, 17, 18, 19, 20]
    assert torch.equal(windowed[:, 20, seen], everything[:, 20, seen]), "kept tokens keep their true distances"
    p = P.sink_softmax(windowed)
    assert (p.sum(-1) < 1).all() and torch.allclose(p[0, 0, 0], torch.exp(windowed[0, 0, 0]) / (1 + torch.exp(windowed[0, 0, 0])))


def test_chunks_of_the_recurrence_are_chosen_from_shapes():
    from mini_rsglang_b200.kernels import ssm_chunk_length

    assert ssm_chunk_length(8, 8, 64, 128, 64, 148) == 0             # decoded tokens
    assert ssm_chunk_length(300, 1, 64, 128, 64, 148) == 0           # a short portion
    assert ssm_chunk_length(2048, 1, 64, 128, 64, 148) == 256
    n = ssm_chunk_length(2048, 1, 4, 32, 48, 148)
    assert n == 128
    assert ssm_chunk_length(2048, 32, 4, 32, 48, 148) == 0           # many short portions


def test_window_group_keeps_the_pages_of_the_first_positions():
    """A window of 6 positions with the first 5 kept, pages of 4: logical pages 0 and 1 stay for the request's whole life,
    the pages between them and the window go back to the pool as the request grows, and every page comes back at its end."""
    from mini_rsglang_b200.cache.manager import CacheGroup, CacheManager

    m = CacheManager([CacheGroup("window", 6, 9, keep_first=5)], page_size=4, max_slots=2)
    assert m.worst_case_pages(0, 1000, 1) == 2 + 1 + 2             # the window's span, and the two kept pages
    m.open(1)
    held = []
    for length in range(1, 33):
        m.extend(1, length)
        m.trim(1, length)
        table = m.table(1)
        assert (table[:min(2, len(table))] >= 0).all(), "a kept page was given back"
        first_key = max(0, length - 6 + 1)
        for page, physical in enumerate(table):
            needed = page < 2 or (page + 1) * 4 > first_key
            assert (physical >= 0) == needed, (length, page, table)
        held.append(int((table >= 0).sum()))
        m.check_integrity()
    assert max(held) <= 5 and m.free_pages(0) == 9 - held[-1]
    m.close(1)
    assert m.free_pages(0) == 9
    with pytest.raises(InvalidRequest):
        CacheManager([CacheGroup("full", 0, 9, keep_first=5)], page_size=4, max_slots=2)
