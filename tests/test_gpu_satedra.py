"""Satedra on the GPU against the plain implementation (`plain_satedra.py`): every mechanism's kernel alone, then
whole models of several small shapes through `bin/trace_run` in every cutting (whole, a decoded tail, portions
down to two tokens, requests mixed in a pool so small that pages are used again), in float32 and bfloat16, and
greedy generation through the engine's entry point and scheduler.  Where random weights would hide a fault (a far
key, a window's edge, a page border), queries and keys are made so that one score stands out.

Routing in whole models: in float32 the router chooses freely (the engine's float32 scores and the plain
implementation's float64 ones order the experts alike unless two scores agree to six digits).  In bfloat16 a
rounded input may turn a close call, which is no fault, so the bfloat16 models carry corrections that are far
apart: the choice is then the same set of experts for every token, while weights, experts, identity experts and
the shared expert still run on every token's own scores; free routing in bfloat16 is covered kernel by kernel."""
import functools
import json
import math
import os

import pytest
import torch

import plain_satedra as P
import trace_tools as T

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def attention(heads, dim, rot_dim, vdim, kv_rank, size, scale=0.3, base=10000.0, dims=None, scaling=None, kv_from=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
             "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if size:
        mixer["mask"] = {"size": size}
    if scaling:
        mixer["rot"]["scaling"] = scaling
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer}


def moe(ff, experts, identity, top, scale, shared):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


STRETCH = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}
# X: sizes that no tensor-core kernel takes (the CUDA-core kernels in both dtypes): every per-head size different, three
# heads, a layer that reads another's cache with a wider window than the owner's and other head sizes, a layer without
# feed-forward, experts without a shared one and with one choice, a layer that sees every key, plain rotary positions
# beside stretched ones, fewer rotated elements than the rotated part holds, page size 4.
SHAPE_X = {"architecture": "Satedra", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "logit_scale": 0.7, "layers": [
    dict(attention(3, 24, 8, 20, 40, 20, scaling=STRETCH), mlp=moe(36, 5, 1, 2, 1.5, 28)),
    dict(attention(2, 12, 8, 28, 40, 33, scaling=STRETCH, kv_from=0), mlp={"kind": "dense", "ff": 100}),
    dict(attention(3, 24, 12, 20, 44, 9, dims=8), mlp=None),
    dict(attention(5, 8, 12, 8, 44, 0, dims=8, kv_from=2), mlp=moe(20, 3, 0, 1, 1.0, 0)),
    dict(attention(1, 40, 6, 30, 18, 1000, base=50.0), mlp=moe(24, 2, 3, 3, 2.5, 40))]}
# Y: sizes of the tensor-core kernels (multiples of 16 and 8), values that a model may happen to make equal or 1: one
# head, a window of one, a window longer than any request, one expert, every expert chosen, identity experts alone,
# a logit scale of 1, groups of 4 and of 20 heads (tiles of 16 rows hold up to 16), page size 16.
SHAPE_Y = {"architecture": "Satedra", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}, "logit_scale": 1.0, "layers": [
    dict(attention(4, 16, 16, 16, 64, 24, scaling={"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}), mlp=moe(32, 4, 2, 3, 2.0, 48)),
    dict(attention(20, 16, 16, 8, 64, 24, scaling={"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}, kv_from=0), mlp=moe(16, 1, 0, 1, 1.0, 16)),
    dict(attention(1, 32, 32, 48, 32, 1), mlp=moe(8, 0, 2, 2, 1.0, 0)),
    dict(attention(2, 8, 16, 24, 48, 1000, base=300.0), mlp={"kind": "dense", "ff": 72}),
    dict(attention(4, 16, 16, 16, 48, 40, base=300.0, kv_from=3), mlp=moe(24, 3, 0, 3, 0.5, 0))]}
SHAPES = {"X": (SHAPE_X, 4), "Y": (SHAPE_Y, 16)}
LENGTHS = {"X": [70, 45, 33, 100, 130, 64, 37, 90], "Y": [1, 7, 17, 40, 129, 65, 96, 50]}
MODES = ("whole", "decode_tail", "portions", "mixed")
SHARPEN = 6.0          # q, the key up-projection and the rotated key's rows scaled by this: attention becomes peaked


def write_model(folder, raw, seed, fixed_choice):
    """A seeded random model, its attention sharpened.  `fixed_choice`: corrections far apart (the experts' order is
    theirs); else corrections of the size of the scores' differences."""
    from mini_rsglang_b200.models import config_from_dict
    from mini_rsglang_b200.weights import write_random_model, write_safetensors
    from mini_rsglang_b200.weights.safetensors_io import SafetensorsFile

    write_random_model(folder, config_from_dict(raw), seed=seed, dtype=torch.bfloat16)
    path = os.path.join(folder, "model.safetensors")
    tensors = {k: t.read() for k, t in SafetensorsFile(path).tensors.items()}
    gen = torch.Generator().manual_seed(seed)
    for name, t in tensors.items():
        layer = int(name.split(".")[0][1:]) if name.startswith("l") and name[1].isdigit() else None
        if name.endswith(".mix.q") or name.endswith(".mix.uk"):
            tensors[name] = (t.float() * SHARPEN).to(t.dtype)
        elif name.endswith(".mix.dkv"):
            rank = raw["layers"][layer]["mixer"]["kv_rank"]
            scaled = t.float()
            scaled[rank:] *= SHARPEN
            tensors[name] = scaled.to(t.dtype)
        elif name.endswith(".mlp.router"):
            tensors[name] = (t.float() * 25.0).to(t.dtype)              # scores that differ from token to token
        elif name.endswith(".mlp.correction"):
            order = torch.randperm(t.numel(), generator=gen).float()
            tensors[name] = (order * 3.0 if fixed_choice else torch.randn(t.numel(), generator=gen) * 0.05).to(t.dtype)
    write_safetensors(path, tensors)
    return folder


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {(name, fixed): write_model(str(tmp_path_factory.mktemp(f"satedra_{name}_{int(fixed)}")), raw, 41 + i, fixed)
            for i, (name, (raw, _)) in enumerate(SHAPES.items()) for fixed in (False, True)}


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
    return reqs, {r: P.forward(config, weights, tokens) for r, tokens in reqs.items()}


_results = {}


def replay(folders, name, dtype, tmp_path_factory):
    key = (name, dtype)
    if key in _results:
        return _results[key]
    folder = folders[(name, dtype == "bfloat16")]
    reqs, want = plain_logits(folder, name)
    raw, page = SHAPES[name]
    mixed, peak = T.trace_mixed(reqs, seed=7)
    traces = {"whole": T.trace_whole(reqs), "decode_tail": T.trace_decode_tail(reqs, tail=40),
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
    """Prefill against token-by-token decoding (the tail of 40 tokens lets the windows of 9, 20, 24 and 33 pass over
    decoded tokens), portions of every size, batches against each request alone, pages used again."""
    rows = replay(folders, name, dtype, tmp_path_factory)[mode]
    assert rows
    for step, got, want, _ in rows:
        T.check_rows(got, want, dtype, f"{name} {dtype} {mode} step {step}")


@pytest.mark.parametrize("name", ["X", "Y"])
def test_float32_logits_do_not_depend_on_the_cutting(folders, tmp_path_factory, name):
    """The same position whole, decoded, in portions and mixed with other requests on pages used again: within the
    rounding of float32 sums (the batched library products may sum in another order for another number of rows)."""
    result = replay(folders, name, "float32", tmp_path_factory)
    whole = {place: row for _, got, _, places in result["whole"] for row, place in zip(got, places)}
    compared = 0
    for mode in MODES[1:]:
        for step, got, _, places in result[mode]:
            for row, place in zip(got, places):
                assert (row - whole[place]).abs().max() <= 2e-5 * max(1.0, whole[place].abs().max().item()), (mode, step, place)
                compared += 1
    assert compared > 50


# ----------------------------------------------------------------------------------------------------------------
# each mechanism alone
# ----------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("width", [72, 320, 1001, 4100])
def test_layer_norm_with_bias_and_residual_sum(width):
    from mini_rsglang_b200 import kernels

    torch.manual_seed(width)
    stream = torch.randn(9, width, device=DEV) * 3 + 1.5              # a mean that a norm without centring would keep
    weight, bias = torch.rand(width, device=DEV) + 0.5, torch.randn(width, device=DEV)
    for dtype, tol in ((torch.float32, 3e-6), (torch.bfloat16, 8e-3)):
        delta = (torch.randn(9, width, device=DEV) * 2).to(dtype)
        total = stream.double().cpu() + delta.double().cpu()
        want = P.layer_norm(total, weight.double().cpu(), bias.double().cpu(), 1e-5)
        s, out = stream.clone(), torch.empty(9, width, dtype=dtype, device=DEV)
        kernels.add_layernorm(s, delta, weight, bias, 1e-5, out)
        assert (s.double().cpu() - total).abs().max() < 1e-6 * total.abs().max()
        assert (out.double().cpu() - want).abs().max() < tol * want.abs().max()
        rows = torch.tensor([7, 0, 7, 3], dtype=torch.int32, device=DEV)          # some rows, the sum not kept
        s, out = stream.clone(), torch.empty(4, width, dtype=dtype, device=DEV)
        kernels.add_layernorm(s, delta, weight, bias, 1e-5, out, rows, write_back=False)
        assert torch.equal(s, stream)
        assert (out.double().cpu() - want[rows.cpu().long()]).abs().max() < tol * want.abs().max()
        s, out = stream.clone(), torch.empty(9, width, dtype=dtype, device=DEV)
        kernels.add_layernorm(s, None, weight, bias, 1e-5, out)                  # no branch to add
        alone = P.layer_norm(stream.double().cpu(), weight.double().cpu(), bias.double().cpu(), 1e-5)
        assert (out.double().cpu() - alone).abs().max() < tol * alone.abs().max()


@pytest.mark.parametrize("H,d,r,R,rotary,scaling,keeps,gated", [
    (3, 24, 8, 40, 8, STRETCH, True, True), (2, 12, 12, 44, 8, None, True, False), (5, 8, 6, 18, 6, STRETCH, False, True),
    (1, 40, 32, 144, 32, {"factor": 6.0, "original": 1024, "fast": 24.0, "slow": 1.5}, True, True), (4, 16, 4, 16, 0, None, True, True)])
def test_latent_rows_rotation_and_gates(H, d, r, R, rotary, scaling, keeps, gated):
    """The kernel after the fused projection against the plain norm and rotation: positions near 0 and far out, cache
    rows at scattered slots, a token that keeps nothing (slot -1), a layer that keeps no cache at all."""
    from mini_rsglang_b200 import kernels

    torch.manual_seed(H * 10 + r)
    tokens, page, pool = 13, 4, 9
    width = H * (d + r) + (R + r if keeps else 0) + (H if gated else 0)
    proj = torch.randn(tokens, width)
    positions = torch.tensor([0, 1, 2, 3, 63, 64, 65, 1000, 4095, 4096, 50001, 7, 8], dtype=torch.int32)
    slots = torch.randperm(pool * page)[:tokens].to(torch.int32)
    slots[5] = -1
    f, magnitude = P.yarn_frequencies(rotary, 10000.0, scaling) if rotary else (torch.zeros(0, dtype=torch.float64), 1.0)
    latent_w = torch.rand(R) + 0.5
    p64 = proj.double()
    q = p64[:, :H * (d + r)].view(tokens, H, d + r)
    want_q_rot = P.rotate(q[..., d:], positions, f, magnitude, torch.float32) if rotary else q[..., d:]      # angles in 32-bit, as the design has them
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 1e-2)):
        q_plain = torch.empty(H, tokens, d, dtype=dtype, device=DEV)
        q_rows = torch.zeros(tokens, H, R + r, dtype=dtype, device=DEV)
        cache = torch.full((pool, 1, page, R + r), 7.0, dtype=dtype, device=DEV)
        gate = torch.empty(tokens, H, device=DEV) if gated else None
        kernels.latent_prepare(proj.to(DEV), latent_w.to(DEV) if keeps else None, 1e-5, f.float().to(DEV) if rotary else None, magnitude,
                               positions.to(DEV), slots.to(DEV) if keeps else None, q_plain, q_rows, cache if keeps else None, gate,
                               H, d, r, R, rotary, keeps)
        assert (q_plain.double().cpu().transpose(0, 1) - q[..., :d]).abs().max() < tol * 4
        assert (q_rows.double().cpu()[..., R:] - want_q_rot).abs().max() < tol * 6
        assert (q_rows[..., :R] == 0).all()
        if gated:
            assert (gate.double().cpu() - torch.sigmoid(p64[:, -H:])).abs().max() < 1e-6
        flat = cache.double().cpu().view(pool * page, R + r)
        if keeps:
            low = p64[:, H * (d + r):H * (d + r) + R + r]
            want_rows = torch.cat([P.rms_norm(low[:, :R], latent_w.double(), 1e-5),
                                   P.rotate(low[:, R:], positions, f, magnitude, torch.float32) if rotary else low[:, R:]], dim=1)
            for t in range(tokens):
                if slots[t] >= 0:
                    assert (flat[slots[t]] - want_rows[t]).abs().max() < tol * 6, t
            untouched = sorted(set(range(pool * page)) - {int(s) for s in slots if s >= 0})
            assert (flat[untouched] == 7.0).all()
        else:
            assert (flat == 7.0).all()


def plain_latent_attention(q_rows, rows, gate, R, scale, window):
    """Attention in the latent space: scores against whole rows, sums over the rows' first R elements."""
    T_, H, _ = q_rows.shape
    seen = P.window_mask(T_, window)
    out = torch.empty(T_, H, R, dtype=torch.float64)
    for h in range(H):
        s = torch.where(seen, q_rows[:, h] @ rows.T * scale, torch.tensor(-math.inf, dtype=torch.float64))
        out[:, h] = torch.softmax(s, dim=-1) @ rows[:, :R] * (gate[:, h:h + 1] if gate is not None else 1.0)
    return out


def run_latent_attention(dtype, q_rows, rows, gate, R, scale, window, page, seed, kernel, give_back=0):
    """The attention kernels on one sequence whose pages lie scattered in a larger pool.  `kernel`: "simt" (one warp a
    row), "rows", "keys" or "split" (the tensor-core kernel over tiles of 64 rows, of 16 rows, of 16 rows with three CTAs
    a tile).  `give_back`: so many of the first pages are -1 in the table, as a window that has passed leaves them."""
    from mini_rsglang_b200 import kernels

    T_, H, row = q_rows.shape
    gen = torch.Generator().manual_seed(seed)
    pages = -(-T_ // page)
    pool = pages + 5
    table = torch.randperm(pool, generator=gen)[:pages].to(torch.int32)
    cache = torch.full((pool, 1, page, row), 7.0, dtype=dtype, device=DEV)          # other pages hold values that would show
    flat = cache.view(pool * page, row)
    index = torch.tensor([int(table[p // page]) * page + p % page for p in range(T_)], device=DEV)
    flat[index] = rows.to(dtype).to(DEV)
    table[:give_back] = -1
    q = q_rows.to(dtype).to(DEV).reshape(T_, H * row).contiguous()
    g = gate.float().to(DEV).contiguous() if gate is not None else None
    out = torch.empty(T_, H * R, dtype=dtype, device=DEV)
    positions = torch.arange(T_, dtype=torch.int32, device=DEV)
    if kernel == "simt":
        kernels.attention_biased_simt(q, cache, None, positions, torch.zeros(T_, dtype=torch.int32, device=DEV), table.view(1, -1).to(DEV),
                                      out, H, 1, row, R, scale, window=window, gate=g)
    else:
        per = (64 if kernel == "rows" else 16) // H
        tiles = torch.tensor([[0, first, min(per, T_ - first), 0] for first in range(0, T_, per)] + [[0, 0, 0, 0]],
                             dtype=torch.int32, device=DEV)                  # and an entry without tokens, as padded lists have
        kernels.attention_biased_mma(q, cache, None, positions, table.view(1, -1).to(DEV), tiles, out, H, 1, row, R, scale,
                                     window=window, gate=g, narrow=kernel != "rows", splits=3 if kernel == "split" else 1)
    return out.double().cpu().view(T_, H, R)


@pytest.mark.parametrize("H,R,r,window,page", [(3, 40, 8, 20, 4), (2, 44, 12, 9, 16), (5, 18, 6, 0, 8), (1, 130, 30, 1, 4), (6, 512, 64, 33, 16),
                                               (7, 300, 33, 64, 16), (2, 1024, 128, 40, 16)])
def test_latent_attention_kernel_random(H, R, r, window, page):
    T_ = 150
    torch.manual_seed(H * 100 + R)
    q_rows, rows, gate = torch.randn(T_, H, R + r).double(), torch.randn(T_, R + r).double(), torch.rand(T_, H).double()
    scale = 0.7 / (R + r) ** 0.5
    want = plain_latent_attention(q_rows, rows, gate, R, scale, window)
    got = run_latent_attention(torch.float32, q_rows, rows, gate, R, scale, window, page, 3, "simt")
    assert (got - want).abs().max() < 2e-5 * max(1.0, want.abs().max().item())
    q16, rows16 = q_rows.bfloat16().double(), rows.bfloat16().double()
    want16 = plain_latent_attention(q16, rows16, gate, R, scale, window)
    got16 = run_latent_attention(torch.bfloat16, q_rows, rows, gate, R, scale, window, page, 4, "simt")
    assert (got16 - want16).abs().max() < 0.02 * max(1.0, want16.abs().max().item())


@pytest.mark.parametrize("kernel", ["rows", "keys", "split"])
@pytest.mark.parametrize("H,R,r,window,page", [(4, 64, 16, 24, 16), (20, 64, 16, 24, 16), (1, 32, 32, 1, 4), (2, 48, 16, 0, 8), (6, 112, 32, 90, 16),
                                               (16, 256, 32, 70, 16), (3, 16, 0, 33, 16)])
def test_tensor_core_latent_attention_kernel_random(kernel, H, R, r, window, page):
    if kernel != "rows" and H > 16:
        pytest.skip("tiles of 16 rows hold up to 16 heads")
    T_ = 200
    torch.manual_seed(H * 100 + R)
    q_rows, rows, gate = torch.randn(T_, H, R + r), torch.randn(T_, R + r), torch.rand(T_, H).double()
    scale = 0.7 / (R + r) ** 0.5
    want = plain_latent_attention(q_rows.bfloat16().double(), rows.bfloat16().double(), gate, R, scale, window)
    got = run_latent_attention(torch.bfloat16, q_rows, rows, gate if H != 2 else None, R, scale, window, page, 4, kernel)
    if H == 2:
        want = plain_latent_attention(q_rows.bfloat16().double(), rows.bfloat16().double(), None, R, scale, window)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() < 0.02 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("kernel", ["simt", "rows", "keys", "split"])
@pytest.mark.parametrize("window,page,T_", [(20, 4, 210), (64, 16, 210), (17, 8, 210), (96, 16, 210), (0, 16, 700), (1, 16, 70)])
def test_latent_attention_sees_exactly_its_window(kernel, window, page, T_):
    """The last query's one key stands out (the others score far below): the key just inside the window, just outside
    it, the query's own, the very first, keys at page and block borders, and without a window a key hundreds of tokens
    back.  The pages that the window has passed are given back.  With a wrong edge the output is another token's row."""
    H, R, r = 2, 16, 16
    torch.manual_seed(window)
    i = T_ - 1
    dtype, tol = (torch.float32, 1e-5) if kernel == "simt" else (torch.bfloat16, 0.03)
    first_seen = i - window + 1 if window else 0
    targets = sorted({first_seen, first_seen - 1, i, i - 1, 0, 3, first_seen // page * page, first_seen // page * page - 1,
                      (i // page) * page - 1, (i // page) * page, 63, 64, 127, 128} & set(range(T_)))
    earliest = max(first_seen - 31, 0)                                 # rows from here on are compared: the last tiles of every kernel
    give_back = max(earliest - window + 1, 0) // page if window else 0  # pages that none of them sees
    for target in targets:
        q_rows, rows = 0.01 * torch.randn(T_, H, R + r).double(), 0.01 * torch.randn(T_, R + r).double()
        rows[:, :R] += torch.randn(T_, R).double()                     # values that tell the tokens apart ...
        q_rows[..., :R] = 0.0                                          # ... and do not enter the scores
        direction = torch.randn(r).double()
        direction /= direction.norm()
        q_rows[i, :, R:] = 30.0 * direction
        rows[target, R:] = 30.0 * direction
        if dtype is torch.bfloat16:
            q_rows, rows = q_rows.bfloat16().double(), rows.bfloat16().double()
        gate = torch.rand(T_, H).double()
        want = plain_latent_attention(q_rows, rows, gate, R, 1.0, window)
        got = run_latent_attention(dtype, q_rows, rows, gate, R, 1.0, window, page, target, kernel, give_back)
        seen = first_seen <= target <= i
        alone = (want[i, 0] / gate[i, 0] - rows[target, :R]).abs().max()
        assert (alone < 1e-2) == seen, f"target {target}: the plain implementation itself does not single the key out"
        assert (got[earliest:] - want[earliest:]).abs().max() < tol, f"key {target} (seen: {seen}) with window {window}"


@pytest.mark.parametrize("experts,identity,top,scale,sigmoid", [(5, 1, 2, 1.5, False), (11, 2, 4, 1.7, False), (1, 0, 1, 1.0, False),
                                                                (0, 3, 2, 1.0, False), (70, 0, 40, 0.5, False), (6, 0, 2, 1.0, True)])
def test_router_choice_and_weights(experts, identity, top, scale, sigmoid):
    from mini_rsglang_b200 import kernels

    torch.manual_seed(experts * 10 + top)
    tokens, all_experts = 37, experts + identity
    logits = (torch.randn(tokens, all_experts + 1) * 3).to(DEV)
    correction = torch.randn(all_experts).to(DEV)
    chosen = torch.empty(tokens, top, dtype=torch.int32, device=DEV)
    weights = torch.empty(tokens, top, device=DEV)
    shared = torch.empty(tokens, device=DEV)
    kernels.moe_route(logits, correction, chosen, weights, shared, all_experts, top, scale, sigmoid_scores=sigmoid)
    z = logits.double().cpu()
    if sigmoid:
        scores = torch.sigmoid(z[:, :all_experts])
        want_chosen = torch.topk(scores + correction.double().cpu(), top, dim=-1).indices
        picked = torch.gather(scores, 1, want_chosen)
        want_weights = picked / (picked.sum(dim=-1, keepdim=True) + 1e-20) * scale
    else:
        w = {"router": torch.eye(all_experts, dtype=torch.float64), "correction": correction.double().cpu()}
        want_chosen, want_weights = P.route(z[:, :all_experts], w, "", {"top": top, "scale": scale})
    assert torch.equal(chosen.cpu().long(), want_chosen)               # in the order of their choice scores
    assert (weights.double().cpu() - want_weights).abs().max() < 1e-5 * scale
    assert (shared.double().cpu() - torch.sigmoid(z[:, all_experts])).abs().max() < 1e-6
    kernels.moe_route(logits[:, :all_experts].contiguous(), None, chosen, weights, None, all_experts, top, scale, sigmoid_scores=sigmoid)
    if not sigmoid:
        w["correction"] = torch.zeros(all_experts, dtype=torch.float64)
        assert torch.equal(chosen.cpu().long(), P.route(z[:, :all_experts], w, "", {"top": top, "scale": scale})[0])


@pytest.mark.parametrize("kernel", ["simt", "rows", "mma", "tc"])
@pytest.mark.parametrize("tokens,width,inner,experts,top,crowd", [(50, 72, 36, 5, 2, False), (1, 64, 24, 3, 3, False), (200, 64, 32, 4, 2, True),
                                                                  (9, 136, 200, 7, 1, False), (300, 192, 64, 10, 3, False), (700, 136, 192, 5, 2, True),
                                                                  (40, 264, 128, 3, 1, False)])
def test_expert_products_over_the_lists(kernel, tokens, width, inner, experts, top, crowd):
    """Both products over the expert lists against the plain gated unit, pair by pair, on the CUDA cores (the kernel for
    every size and the one for few rows an expert), with mma.sync and with tcgen05: experts that nobody chose, an expert that nearly every token chose (several tiles), identity experts among
    the choices (their rows of the output stay as they were), sizes that fill no tile, gate and up rows in blocks of 64 where
    the inner size allows."""
    from mini_rsglang_b200 import kernels

    tensor_cores = kernel in ("mma", "tc")
    block = 64 if inner % 64 == 0 else 0
    if kernel == "rows" and (width % 8 or inner % 8):
        pytest.skip("the product for few rows takes rows of a multiple of 16 bytes")
    if kernel == "mma" and (width % 8 or inner % 8):
        pytest.skip("the tensor-core product takes rows on 16-byte boundaries")
    if kernel == "tc" and (width % 8 or not block):
        pytest.skip("the product for many rows takes blocks of 64 gate and up rows")
    torch.manual_seed(tokens + width)
    identity = 2
    scores = torch.rand(tokens, experts + identity)
    scores[:, 1 % experts] -= 5.0                                          # an expert without tokens
    if crowd:
        scores[:, 0] += 5.0
    chosen = torch.topk(scores, top, dim=-1).indices.to(torch.int32)
    gate_up, down = torch.randn(experts, 2 * inner, width) / width ** 0.5, torch.randn(experts, width, inner) / inner ** 0.5
    h = torch.randn(tokens, width)
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
        if tensor_cores and dtype is torch.float32:
            continue
        hd, gu, dn = (t.to(dtype).to(DEV).contiguous() for t in (h, gate_up, down))
        laid = gu
        if block:              # blocks of 64 gate rows, each followed by its up rows
            laid = torch.stack([gu[:, :inner].view(experts, -1, block, width), gu[:, inner:].view(experts, -1, block, width)], dim=2) \
                .reshape(experts, 2 * inner, width).contiguous()
        y = torch.full((tokens * top, width), 5.0, dtype=dtype, device=DEV)
        kernels.moe_experts(hd, chosen.to(DEV), laid, dn, y, experts, kernel=kernel, block=block)
        y = y.double().cpu().view(tokens, top, width)
        h64, gu64, dn64 = hd.double().cpu(), gu.double().cpu(), dn.double().cpu()
        for t in range(tokens):
            for c in range(top):
                e = int(chosen[t, c])
                if e >= experts:
                    assert (y[t, c] == 5.0).all()
                    continue
                w = {"gate": gu64[e, :inner], "up": gu64[e, inner:], "down": dn64[e]}
                want = P.gated_unit(h64[t:t + 1], w, "")[0]
                assert (y[t, c] - want).abs().max() < tol * max(1.0, want.abs().max().item()), (t, c, e)


def test_weighted_sum_of_choices_with_identity_and_shared_expert():
    from mini_rsglang_b200 import kernels

    torch.manual_seed(9)
    tokens, width, top, experts = 21, 72, 3, 4
    chosen = torch.stack([torch.randperm(experts + 2)[:top] for _ in range(tokens)]).to(torch.int32)
    weights, gate = torch.rand(tokens, top), torch.rand(tokens)
    y, h, shared = torch.randn(tokens * top, width), torch.randn(tokens, width), torch.randn(tokens, width)
    want = torch.zeros(tokens, width, dtype=torch.float64)
    for t in range(tokens):
        for c in range(top):
            want[t] += weights[t, c].double() * (y[t * top + c].double() if chosen[t, c] < experts else h[t].double())
    out = torch.empty(tokens, width, device=DEV)
    kernels.moe_combine(y.to(DEV), h.to(DEV), None, chosen.to(DEV), weights.to(DEV), None, out, experts)
    assert (out.double().cpu() - want).abs().max() < 1e-5
    kernels.moe_combine(y.to(DEV), h.to(DEV), shared.to(DEV), chosen.to(DEV), weights.to(DEV), gate.to(DEV), out, experts)
    assert (out.double().cpu() - (want + gate.double()[:, None] * shared.double())).abs().max() < 1e-5
    only_identity = torch.full((tokens, top), experts, dtype=torch.int32)
    kernels.moe_combine(None, h.to(DEV), None, only_identity.to(DEV), weights.to(DEV), None, out, 0)
    assert (out.double().cpu() - weights.double().sum(dim=1, keepdim=True) * h.double()).abs().max() < 1e-5


# ----------------------------------------------------------------------------------------------------------------
# the engine's own entry point and scheduler
# ----------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(folders, dtype):
    """Prompts of unequal lengths, more requests than run at a time, prompt portions under a small token budget beside
    decoded tokens, 40 generated tokens each (the windows of 9, 20 and 33 pass over decoded tokens): every token is the
    plain implementation's arg-max, or within rounding of it."""
    from mini_rsglang_b200 import RuntimeConfig, SamplingParams
    from mini_rsglang_b200.engine import EngineHandle

    folder = folders[("X", dtype == "bfloat16")]
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
            logits = P.forward(config, weights, tokens)[-1]
            best = int(logits.argmax())
            gap = (logits[best] - logits[token]).item()
            limit = 2e-5 if dtype == "float32" else 0.02 * logits.abs().max().item()
            assert token == best or gap <= limit, f"{dtype}: engine chose {token}, plain {best}, gap {gap}"
            tokens.append(token)


def test_command_line_generates_the_plain_tokens(folders):
    """`bin/mini-rsglang generate` on a Satedra folder: the architecture is found by config.json, prefix sharing (on by
    default on the command line) is switched off with a note because the model keeps windows of keys, and the tokens are
    the plain implementation's."""
    import subprocess
    import sys

    folder = folders[("X", False)]
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    cmd = [sys.executable, os.path.join(T.ROOT, "bin", "mini-rsglang"), "--model", folder, "--dtype", "float32", "--page-size", "4",
           "--max-seq-len", "128", "--num-pages", "40", "generate", "--token-ids", ",".join(map(str, prompt)), "--max-tokens", "12",
           "--ignore-eos", "--json"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    assert "prefix sharing is off" in proc.stderr
    events = [json.loads(line) for line in proc.stdout.splitlines() if line.startswith("{")]
    tokens = [e["Token"]["token_id"] for e in events if "Token" in e]
    done = events[-1]["Finished"]
    assert done["reason"] == "length" and done["prompt_tokens"] == len(prompt) and done["completion_tokens"] == 12
    config, weights = load_plain(folder)
    sequence = list(prompt)
    for token in tokens:
        logits = P.forward(config, weights, sequence)[-1]
        best = int(logits.argmax())
        assert token == best or (logits[best] - logits[token]).item() <= 2e-5, (token, best)
        sequence.append(token)
