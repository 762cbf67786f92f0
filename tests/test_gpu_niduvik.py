"""Niduvik on the GPU against the plain implementation (`plain_niduvik.py`): every mechanism's kernel alone, then
whole models of several small shapes through `bin/trace_run` in every cutting (whole, a decoded tail, portions
down to two tokens, requests mixed in a pool so small that pages and state slots are used again), in float32 and
bfloat16, and greedy generation through the engine's entry point and scheduler.  Where random weights would hide a
fault (a far key, a kept first token, a window's edge), queries and keys are scaled so that one score stands out."""
import functools
import json
import os

import pytest
import torch

import plain_niduvik as P
import trace_tools as T

pytestmark = pytest.mark.gpu


def attention_layer(heads, kv_heads, dim, vdim, size, keep_first, v_mix, rows, far=50.0, scale=0.3, softcap=8.0):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                           "softcap": softcap, "bias_max": far, "bias_rows": rows, "v_mix": v_mix,
                                           "mask": {"size": size, "keep_first": keep_first}}}


def recurrent_layer(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


# X: a recurrence first, an attention layer that does not blend values before the two that do, groups of 2 and of 1
# query heads a key head, a layer without feed-forward at both kinds, page size 4.
SHAPE_X = {"architecture": "Niduvik", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "layers": [
    dict(recurrent_layer(3, 20, 24, 1, 4, 3), mlp=dense(100, 1.5)),
    dict(attention_layer(6, 3, 24, 40, 20, 3, False, 12), mlp=None),
    dict(attention_layer(6, 3, 24, 40, 20, 3, True, 12), mlp=dense(100, 1.5)),
    dict(attention_layer(3, 3, 32, 40, 9, 1, True, 7, far=30.0, softcap=3.0), mlp=dense(64, 0.7)),
    dict(recurrent_layer(4, 16, 8, 4, 2, 1), mlp=None)]}
# Y: values that a model may happen to make equal or 1: no kept tokens, a window longer than any request, a window
# of one, one tap (no convolution state), one part in the norm, key and value heads of one size, one head.
SHAPE_Y = {"architecture": "Niduvik", "vocab": 97, "width": 48, "norm": {"eps": 1e-6}, "layers": [
    dict(attention_layer(2, 2, 16, 16, 1000, 0, True, 4, far=9.0), mlp=dense(48, 4.0)),
    dict(recurrent_layer(2, 24, 40, 2, 1, 1), mlp=dense(80, 2.5)),
    dict(attention_layer(1, 1, 48, 8, 1, 0, False, 32, far=400.0, softcap=50.0), mlp=None),
    dict(attention_layer(4, 2, 8, 16, 33, 40, True, 4, far=9.0), mlp=dense(48, 4.0)),
    dict(recurrent_layer(1, 64, 16, 1, 3, 4), mlp=dense(80, 2.5))]}
SHAPES = {"X": (SHAPE_X, 4), "Y": (SHAPE_Y, 16)}
LENGTHS = {"X": [70, 45, 33, 100, 130, 64, 37, 90], "Y": [1, 7, 17, 40, 129, 65, 96, 50]}
MODES = ("whole", "decode_tail", "portions", "mixed")
SHARPEN = 6.0          # q and k projections scaled by this: scores grow 36-fold and attention becomes peaked


def write_model(folder, raw, seed, sharpen=1.0):
    from mini_rsglang_b200.models import config_from_dict
    from mini_rsglang_b200.weights import write_random_model, write_safetensors
    from mini_rsglang_b200.weights.safetensors_io import SafetensorsFile

    write_random_model(folder, config_from_dict(raw), seed=seed, dtype=torch.bfloat16)
    if sharpen != 1.0:
        path = os.path.join(folder, "model.safetensors")
        tensors = {k: t.read() for k, t in SafetensorsFile(path).tensors.items()}
        for name in tensors:
            if name.endswith(".mix.q") or name.endswith(".mix.k"):
                tensors[name] = (tensors[name].float() * sharpen).to(tensors[name].dtype)
        write_safetensors(path, tensors)
    return folder


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: write_model(str(tmp_path_factory.mktemp(f"niduvik_{name}")), raw, 31 + i, SHARPEN)
            for i, (name, (raw, _)) in enumerate(SHAPES.items())}


def load_plain(folder):
    from mini_rsglang_b200.weights.safetensors_io import SafetensorsFile

    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    weights = {k: t.read() for k, t in SafetensorsFile(os.path.join(folder, "model.safetensors")).tensors.items()}
    return config, weights


@functools.lru_cache(maxsize=None)
def plain_logits(folder, name):
    config, weights = load_plain(folder)
    reqs = T.requests_for(config["vocab"], LENGTHS[name], seed=200 + ord(name))
    return reqs, {r: P.forward(config, weights, tokens)[0] for r, tokens in reqs.items()}


_results = {}


def replay(folder, name, dtype, tmp_path_factory):
    key = (name, dtype)
    if key in _results:
        return _results[key]
    reqs, want = plain_logits(folder, name)
    raw, page = SHAPES[name]
    mixed, peak = T.trace_mixed(reqs, seed=7)
    traces = {"whole": T.trace_whole(reqs), "decode_tail": T.trace_decode_tail(reqs),
              "portions": T.trace_portions(reqs, seed=5), "mixed": mixed}
    max_tokens = max(peak, max(T.rounded(len(t)) for t in reqs.values()))
    assert sum(T.rounded(len(t)) for t in reqs.values()) > max_tokens, "the pool must force pages to be used again"
    run = T.TraceRun(folder, dtype, str(tmp_path_factory.mktemp(f"out_{name}_{dtype}")), max_tokens, extra=("--page-size", str(page)))
    out, first = {}, 0
    for mode in MODES:
        trace = T.renumber(traces[mode], first, f"{mode}-")
        first += len(trace.steps)
        rows = []
        for step, places in zip(trace.steps, trace.rows):
            got = run.step(step, raw["vocab"])
            if places:
                rows.append((step["step"], got, torch.stack([want[r][p] for r, p in places]), places))
        out[mode] = rows
    assert run.close() == 0
    _results[key] = out
    return out


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["X", "Y"])
def test_replay_matches_plain(folders, tmp_path_factory, name, dtype, mode):
    rows = replay(folders[name], name, dtype, tmp_path_factory)[mode]
    assert rows
    for step, got, want, _ in rows:
        T.check_rows(got, want, dtype, f"{name} {dtype} {mode} step {step}")


@pytest.mark.parametrize("name", ["X", "Y"])
def test_float32_logits_do_not_depend_on_the_cutting_bit_for_bit(folders, tmp_path_factory, name):
    """Prefill against token-by-token decoding, portions of every size, batches against each request alone, pages
    and slots used again: on the 32-bit path every kernel's sum for a row runs in an order that the row alone
    decides, so the bits agree."""
    result = replay(folders[name], name, "float32", tmp_path_factory)
    whole = {place: row for _, got, _, places in result["whole"] for row, place in zip(got, places)}
    compared = 0
    for mode in MODES[1:]:
        differing = []
        for step, got, _, places in result[mode]:
            for row, place in zip(got, places):
                if not torch.equal(row, whole[place]):
                    differing.append((step, place, (row - whole[place]).abs().max().item()))
                compared += 1
        assert not differing, f"{name} {mode}: {len(differing)} rows differ from the whole run, first {differing[:3]}"
    assert compared > 50


# ----------------------------------------------------------------------------------------------------------------
# each mechanism alone
# ----------------------------------------------------------------------------------------------------------------
DEV = "cuda:0"


def test_norm_after_a_branch_and_the_next_norm_in_one_kernel():
    from mini_rsglang_b200 import kernels

    torch.manual_seed(1)
    for width in (72, 320, 1001):
        stream = torch.randn(9, width, device=DEV) * 3
        branch = torch.randn(9, width, device=DEV) * 50
        post, nxt = torch.rand(width, device=DEV) + 0.5, torch.rand(width, device=DEV) + 0.5
        want_stream = stream.double().cpu() + P.rms_norm(branch.double().cpu(), post.double().cpu(), 1e-5)
        want_rows = P.rms_norm(want_stream, nxt.double().cpu(), 1e-6)
        for dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 8e-3)):
            s, out = stream.clone(), torch.empty(9, width, dtype=dtype, device=DEV)
            kernels.postnorm_add_norm(s, branch, post, 1e-5, nxt, 1e-6, out)
            assert (s.double().cpu() - want_stream).abs().max() < 2e-6 * want_stream.abs().max()
            assert (out.double().cpu() - want_rows).abs().max() < tol * want_rows.abs().max()
        s = stream.clone()
        kernels.postnorm_add_norm(s, branch, post, 1e-5, None, 0.0, None)           # the sum alone
        assert (s.double().cpu() - want_stream).abs().max() < 2e-6 * want_stream.abs().max()


def test_clamped_gated_unit():
    from mini_rsglang_b200 import kernels

    torch.manual_seed(2)
    gate_up = torch.randn(7, 2 * 50, device=DEV) * 4          # many values beyond the limit on both sides
    want = P.clamped_glu(gate_up[:, :50].double().cpu(), gate_up[:, 50:].double().cpu(), 1.5)
    out = torch.empty(7, 50, device=DEV)
    kernels.glu_clamped(gate_up, out, 1.5, 1.702)
    assert (out.double().cpu() - want).abs().max() < 1e-5
    out16 = torch.empty(7, 50, dtype=torch.bfloat16, device=DEV)
    kernels.glu_clamped(gate_up.bfloat16(), out16, 1.5, 1.702)
    want16 = P.clamped_glu(gate_up[:, :50].bfloat16().double().cpu(), gate_up[:, 50:].bfloat16().double().cpu(), 1.5)
    assert (out16.double().cpu() - want16).abs().max() < 0.03


def test_distance_buckets_are_the_plain_ones():
    from mini_rsglang_b200.parts.attention_biased import distance_buckets

    for rows, far in ((32, 120.0), (12, 50.0), (7, 30.0), (4, 9.0), (2, 5.0), (32, 400.0)):
        table = distance_buckets(rows, far)
        assert table[-1] == rows - 1 and all(b < rows - 1 for b in table[:-1]) or rows == 2
        for n in range(len(table) + 50):
            assert table[min(n, len(table) - 1)] == P.distance_bucket(n, rows, far), (rows, far, n)


def run_attention(dtype, T_, H, G, d, e, size, keep, rows, far, cap, scale, page, q, k, v, rel, gate, seed, kernel="simt"):
    """The attention kernels on one sequence whose pages lie scattered in a larger pool: `kernel` "simt" (one warp a row),
    "rows", "keys" or "split" (the tensor-core kernel over tiles of 64 rows, of 16 rows, of 16 rows with three CTAs a tile)."""
    from mini_rsglang_b200 import kernels
    from mini_rsglang_b200.parts.attention_biased import distance_buckets

    gen = torch.Generator().manual_seed(seed)
    pages = -(-T_ // page)
    pool = pages + 5
    table = torch.randperm(pool, generator=gen)[:pages].to(torch.int32)
    k_cache = torch.full((pool, G, page, d), 7.0, dtype=dtype, device=DEV)         # other pages hold values that would show
    v_cache = torch.full((pool, G, page, e), -9.0, dtype=dtype, device=DEV)
    slots = torch.tensor([int(table[p // page]) * page + p % page for p in range(T_)], dtype=torch.int32, device=DEV)
    proj = torch.cat([q.reshape(T_, -1), k.reshape(T_, -1), v.reshape(T_, -1), gate], dim=1).float().to(DEV).contiguous()
    q_out = torch.empty(T_, H * d, dtype=dtype, device=DEV)
    gate_out = torch.empty(T_, H, dtype=torch.float32, device=DEV)
    kernels.qkv_bias_store(proj, None, q_out, k_cache, v_cache, slots, H, G, d, e, gate_out=gate_out)
    bias = rel.float()[torch.tensor(distance_buckets(rows, far))].to(DEV).contiguous()
    out = torch.empty(T_, H * e, dtype=dtype, device=DEV)
    positions = torch.arange(T_, dtype=torch.int32, device=DEV)
    if kernel == "simt":
        kernels.attention_biased_simt(q_out, k_cache, v_cache, positions, torch.zeros(T_, dtype=torch.int32, device=DEV),
                                      table.view(1, -1).to(DEV), out, H, G, d, e, scale, cap, size, keep, bias, gate_out, True)
    else:
        per = (64 if kernel == "rows" else 16) // (H // G)          # "split": tiles of 16 rows whose key blocks three CTAs share
        tiles = torch.tensor([[0, first, min(per, T_ - first), 0] for first in range(0, T_, per)] + [[0, 0, 0, 0]],
                             dtype=torch.int32, device=DEV)                  # and an entry without tokens, as padded lists have
        kernels.attention_biased_mma(q_out, k_cache, v_cache, positions, table.view(1, -1).to(DEV), tiles, out, H, G, d, e, scale,
                                     cap, size, keep, bias, gate_out, True, narrow=kernel != "rows", splits=3 if kernel == "split" else 1)
    return out.double().cpu().view(T_, H, e)


def plain_attention(q, k, v, rel, gate, scale, cap, far, size, keep):
    s = P.attention_scores(q, k, rel, scale, cap, far, size, keep)
    p = P.sink_softmax(s)
    H, G = q.shape[1], k.shape[1]
    out = torch.stack([p[h] @ v[:, h // (H // G)] for h in range(H)], dim=1)
    return out * torch.sigmoid(gate)[:, :, None]


@pytest.mark.parametrize("H,G,d,e,size,keep,rows,far,page", [
    (4, 2, 24, 40, 20, 3, 12, 50.0, 4), (3, 3, 32, 8, 9, 1, 7, 30.0, 16), (2, 1, 16, 16, 1000, 0, 4, 9.0, 8),
    (1, 1, 48, 72, 1, 0, 32, 200.0, 4), (6, 2, 8, 130, 33, 40, 6, 20.0, 16), (2, 2, 256, 256, 64, 5, 16, 100.0, 16)])
def test_attention_kernel_random(H, G, d, e, size, keep, rows, far, page):
    T_ = 150
    torch.manual_seed(H * 100 + d)
    q, k, v = torch.randn(T_, H, d).double(), torch.randn(T_, G, d).double(), torch.randn(T_, G, e).double()
    rel, gate = torch.randn(rows, H).double(), torch.randn(T_, H).double()
    scale, cap = 0.7 / d ** 0.5, 5.0
    want = plain_attention(q, k, v, rel, gate, scale, cap, far, size, keep)
    got = run_attention(torch.float32, T_, H, G, d, e, size, keep, rows, far, cap, scale, page, q, k, v, rel, gate, 3)
    assert (got - want).abs().max() < 2e-5 * max(1.0, want.abs().max().item())
    q16, k16, v16 = (x.bfloat16().double() for x in (q, k, v))
    want16 = plain_attention(q16, k16, v16, rel, gate, scale, cap, far, size, keep)
    got16 = run_attention(torch.bfloat16, T_, H, G, d, e, size, keep, rows, far, cap, scale, page, q, k, v, rel, gate, 4)
    assert (got16 - want16).abs().max() < 0.02 * max(1.0, want16.abs().max().item())


@pytest.mark.parametrize("kernel", ["rows", "keys", "split"])
@pytest.mark.parametrize("H,G,d,e,size,keep,rows,far,page", [
    (4, 2, 32, 48, 20, 3, 12, 50.0, 4), (3, 3, 96, 32, 9, 1, 7, 30.0, 16), (2, 1, 16, 16, 1000, 0, 4, 9.0, 8),
    (8, 2, 128, 128, 64, 5, 16, 100.0, 16), (2, 2, 256, 256, 33, 40, 6, 20.0, 16), (20, 1, 16, 32, 70, 3, 8, 40.0, 16),
    (1, 1, 48, 16, 1, 0, 32, 200.0, 4)])
def test_tensor_core_attention_kernel_random(kernel, H, G, d, e, size, keep, rows, far, page):
    if kernel != "rows" and H // G > 16:
        pytest.skip("tiles of 16 rows hold groups of up to 16 query heads")
    T_ = 200
    torch.manual_seed(H * 100 + d)
    q, k, v = torch.randn(T_, H, d), torch.randn(T_, G, d), torch.randn(T_, G, e)
    rel, gate = torch.randn(rows, H).double(), torch.randn(T_, H).double()
    scale, cap = 0.7 / d ** 0.5, 5.0
    q16, k16, v16 = (x.bfloat16().double() for x in (q, k, v))
    want = plain_attention(q16, k16, v16, rel, gate, scale, cap, far, size, keep)
    got = run_attention(torch.bfloat16, T_, H, G, d, e, size, keep, rows, far, cap, scale, page, q, k, v, rel, gate, 4, kernel)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() < 0.02 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("kernel", ["simt", "rows", "keys", "split"])
@pytest.mark.parametrize("size,keep,page", [(20, 3, 4), (64, 6, 16), (17, 0, 8), (33, 40, 16), (100, 70, 16)])
def test_attention_kernel_sees_exactly_its_window_and_first_tokens(kernel, size, keep, page):
    """A query whose one key stands out (its score hits the cap, the others lie far below): the key just inside the
    window, just outside it, the last kept first token, the first token that is not kept, a far kept token, keys at page
    borders.  With a wrong edge the output is another token's value."""
    T_, H, G, d, e, rows, far = 210, 2, 1, 16, 16, 8, 40.0
    torch.manual_seed(size)
    i = T_ - 1
    dtype, tol = (torch.float32, 1e-5) if kernel == "simt" else (torch.bfloat16, 0.03)
    targets = sorted({i - size + 1, i - size, max(keep - 1, 0), keep, 0, i, (i - size + 1) // page * page, (i // page) * page - 1,
                      63, 64, 127, 128} & set(range(T_)))
    for target in targets:
        q, k = 0.01 * torch.randn(T_, H, d).double(), 0.01 * torch.randn(T_, G, d).double()
        v = torch.randn(T_, G, e).double()
        direction = torch.randn(d).double()
        direction /= direction.norm()
        q[i] = 30.0 * direction
        k[target, 0] = 30.0 * direction
        if dtype is torch.bfloat16:
            q, k, v = (x.bfloat16().double() for x in (q, k, v))
        rel, gate = 0.1 * torch.randn(rows, H).double(), torch.randn(T_, H).double()
        want = plain_attention(q, k, v, rel, gate, 1.0, 12.0, far, size, keep)
        got = run_attention(dtype, T_, H, G, d, e, size, keep, rows, far, 12.0, 1.0, page, q, k, v, rel, gate, target, kernel)
        seen = P.visible(i, target, size, keep)
        alone = (want[i, 0] / torch.sigmoid(gate[i, 0]) - v[target, 0]).abs().max()
        assert (alone < 1e-2) == seen, f"target {target}: the plain implementation itself does not single the key out"
        assert (got - want).abs().max() < tol, f"key {target} (seen: {seen}) with window {size}, kept {keep}"


def recurrence_inputs(T_, heads, P_, N, G, taps, seed):
    gen = torch.Generator().manual_seed(seed)
    channels = heads * P_ + 2 * G * N
    width = heads * P_ + channels + heads
    proj = torch.randn(T_, width, generator=gen)
    return proj, channels, dict(conv=torch.randn(channels, taps, generator=gen) * 0.5, conv_b=torch.randn(channels, generator=gen) * 0.5,
                                dt_bias=torch.randn(heads, generator=gen), a_log=torch.randn(heads, generator=gen) * 0.5 - 2.0,
                                d=torch.randn(heads, generator=gen), norm=torch.rand(heads * P_, generator=gen) + 0.5)


@pytest.mark.parametrize("heads,P_,N,G,taps,parts", [(3, 20, 24, 1, 4, 3), (4, 16, 8, 4, 2, 1), (2, 24, 40, 2, 1, 1), (1, 64, 130, 1, 3, 4),
                                                     (8, 64, 128, 2, 4, 2)])
@pytest.mark.parametrize("chunk", [0, 16])
def test_recurrence_kernels_in_portions_with_slots_used_again(heads, P_, N, G, taps, parts, chunk):
    """Convolution, recurrence and the gated norm in parts against the plain functions: two sequences side by side, cut
    into portions of 1 to 40 tokens (also shorter than the convolution), in state slots that held another sequence's
    state before; the recurrence in one go (chunk 0) and in chunks of 16 rows that run side by side."""
    from mini_rsglang_b200 import kernels

    lengths, cuts = [97, 61], [[40, 1, 2, 1, 1, 33, 19], [1, 1, 3, 56]]
    inner = heads * P_
    slots = 3
    state = torch.full((slots, (taps - 1) * (inner + 2 * G * N) + heads * N * P_), 11.0, device=DEV)      # stale contents
    data = [recurrence_inputs(n, heads, P_, N, G, taps, 50 + s) for s, n in enumerate(lengths)]
    w = data[0][2]
    channels = data[0][1]
    dev = {k: t.to(DEV).contiguous() for k, t in w.items()}
    want = []
    for proj, _, _ in data:
        p = proj.double()
        xbc = P.silu(P.causal_conv(p[:, inner:inner + channels], w["conv"].double(), w["conv_b"].double()))
        n = p.shape[0]
        y = P.selective_scan(xbc[:, :inner].view(n, heads, P_), xbc[:, inner:inner + G * N].view(n, G, N),
                             xbc[:, inner + G * N:].view(n, G, N), p[:, inner + channels:], w["dt_bias"].double(),
                             w["a_log"].double(), w["d"].double())
        want.append(P.gated_part_norm(y.reshape(n, inner), p[:, :inner], w["norm"].double(), parts, 1e-5))
    got = [torch.zeros(n, inner, dtype=torch.float64) for n in lengths]
    done = [0, 0]
    conv_state = state[:, :(taps - 1) * channels].view(slots, taps - 1, channels)
    ssm_state = state[:, (taps - 1) * channels:].view(slots, heads, N, P_)
    use_slots = [2, 0]
    step = 0
    while any(done[s] < lengths[s] for s in range(2)):
        batch = [(s, cuts[s][step]) for s in range(2) if step < len(cuts[s])]
        step += 1
        rows = torch.cat([data[s][0][done[s]:done[s] + n] for s, n in batch]).to(DEV).contiguous()
        positions = torch.cat([torch.arange(done[s], done[s] + n) for s, n in batch]).to(torch.int32).to(DEV)
        seq_of = torch.cat([torch.full((n,), b) for b, (s, n) in enumerate(batch)]).to(torch.int32).to(DEV)
        starts = [0]
        for _, n in batch:
            starts.append(starts[-1] + n)
        q_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
        slot_of = torch.tensor([use_slots[s] for s, _ in batch], dtype=torch.int32, device=DEV)
        xbc = torch.empty(rows.shape[0], channels, device=DEV)
        kernels.causal_conv_silu(rows, inner, dev["conv"], dev["conv_b"], conv_state, positions, seq_of, q_start, slot_of, xbc)
        y = torch.zeros(rows.shape[0], inner, device=DEV)
        kernels.ssm_scan(xbc, rows[:, inner + channels:], dev["dt_bias"], dev["a_log"], dev["d"], ssm_state, positions, q_start,
                         slot_of, y, heads, G, N, P_, chunk_len=chunk)
        out = torch.empty(rows.shape[0], inner, device=DEV)
        kernels.gated_part_norm(y, rows[:, :inner], dev["norm"], 1e-5, out, parts)
        for b, (s, n) in enumerate(batch):
            got[s][done[s]:done[s] + n] = out[starts[b]:starts[b + 1]].double().cpu()
            done[s] += n
    for s in range(2):
        assert (got[s] - want[s]).abs().max() < 2e-4 * max(1.0, want[s].abs().max().item()), f"sequence {s}"
    assert (state[1] == 11.0).all(), "a slot that no sequence holds was written"


def test_recurrence_keeps_a_far_token():
    """A slowly decaying head carries one early token's input over hundreds of steps of single tokens: the state is
    kept in float32 and handed on from step to step."""
    from mini_rsglang_b200 import kernels

    heads, P_, N, G, T_ = 1, 8, 4, 1, 400
    inner, channels = heads * P_, heads * P_ + 2 * G * N
    xbc = torch.zeros(T_, channels, dtype=torch.float64)
    xbc[5, :inner] = torch.arange(1, P_ + 1, dtype=torch.float64)          # the token to remember
    xbc[5, inner:inner + N] = 1.0                                          # written along every state row
    xbc[T_ - 1, inner + N:] = 1.0                                          # and read back at the very end
    dt_raw = torch.full((T_, heads), -3.0, dtype=torch.float64)
    dt_bias, a_log, d = torch.zeros(heads).double(), torch.full((heads,), -4.0).double(), torch.zeros(heads).double()
    want = P.selective_scan(xbc[:, :inner].view(T_, heads, P_), xbc[:, inner:inner + N].view(T_, G, N),
                            xbc[:, inner + N:].view(T_, G, N), dt_raw, dt_bias, a_log, d).reshape(T_, inner)
    assert want[T_ - 1].abs().min() > 0.01
    state = torch.full((2, heads, N, P_), 5.0, device=DEV)
    got = torch.zeros(T_, inner, device=DEV)
    for t in range(T_):
        y = torch.zeros(1, inner, device=DEV)
        kernels.ssm_scan(xbc[t:t + 1].float().to(DEV), dt_raw[t:t + 1].float().to(DEV), dt_bias.float().to(DEV), a_log.float().to(DEV),
                         d.float().to(DEV), state, torch.tensor([t], dtype=torch.int32, device=DEV),
                         torch.tensor([0, 1], dtype=torch.int32, device=DEV), torch.tensor([1], dtype=torch.int32, device=DEV),
                         y, heads, G, N, P_)
        got[t] = y[0]
    assert (got.double().cpu() - want).abs().max() < 2e-4 * want.abs().max(), (got.double().cpu() - want).abs().max()


# ----------------------------------------------------------------------------------------------------------------
# the engine's own entry point and scheduler
# ----------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(folders, dtype):
    """Prompts of unequal lengths, more requests than state slots, prompt portions under a small token budget beside
    decoded tokens, 40 generated tokens each (the window of layer 3 of X passes over decoded tokens): every token is the
    plain implementation's arg-max, or within rounding of it."""
    from mini_rsglang_b200 import RuntimeConfig, SamplingParams
    from mini_rsglang_b200.engine import EngineHandle

    folder = folders["X"]
    config, weights = load_plain(folder)
    prompts = [T.requests_for(config["vocab"], [n], seed=300 + n)["r0"] for n in (3, 50, 1, 77, 20, 31)]
    engine = EngineHandle.load(folder, 0, config=RuntimeConfig(max_seq_len=160, prefill_budget=24, max_running=3, page_size=4),
                               dtype=dtype, num_pages=120)
    results = engine.generate_many(prompts, SamplingParams(max_tokens=40, ignore_eos=True))
    engine.shutdown()
    for prompt, result in zip(prompts, results):
        assert len(result.token_ids) == 40
        tokens = list(prompt)
        for token in result.token_ids:
            logits = P.forward(config, weights, tokens)[0][-1]
            best = int(logits.argmax())
            gap = (logits[best] - logits[token]).item()
            limit = 2e-5 if dtype == "float32" else 0.02 * logits.abs().max().item()
            assert token == best or gap <= limit, f"{dtype}: engine chose {token}, plain {best}, gap {gap}"
            tokens.append(token)
