"""The Rolevik decoder in the engine against the plain implementation (tests/plain/plain_rolevik.py): each mechanism alone
with inputs made so that one key, a chunk's edge, a carried state, one expert or an identity expert decides the result,
whole prompts, prompts cut into portions, token-by-token decoding across cache pages and chunks, unequal batches, slots,
pages and states used again, long decoding from CUDA graphs, and greedy generation through the public entry point."""

import json
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from plain import plain_rolevik as pr
from tiny import TOLERANCE, random_tokens, scaled_error
from tiny_rolevik import RLV, dense, make_folder, model, moe, parallel, plain_logits_and_sure, rglru
from tiny_rolevik import plain_logits as plain_logits_alone

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F = torch.float64


def _engine(folder, dtype, max_tokens=2048, **more):
    from models_b200.engine.loading import engine_from_folder

    return engine_from_folder(folder, dtype, max_tokens, **more)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("rolevik")
    return {name: make_folder(raw, seed=61 + i, root=root) for i, (name, raw) in enumerate(RLV.items())}


def plain_logits(folder, tokens):
    """The plain logits [T, vocab + 1]: the last column says (1 or 0) whether every router decision up to and with that
    token was clear of a close call.  It rides along through the tests' slicing and stacking; `_close` takes it off."""
    logits, sure = plain_logits_and_sure(folder, tokens)
    return torch.cat([logits, sure.to(logits.dtype)[:, None]], dim=-1)


def _close(got, want, dtype):
    """float32: every position within five times the common bound, all but one in fifty within the bound itself and the median
    within a quarter of it.  bfloat16: a router decision that is a close call in the plain
    implementation may fall the other way after 8-bit roundings; that token then differs by a whole expert, and the later
    ones of its sequence, which read it through the cache and the recurrent states, by a good part of that.  So the
    positions before a sequence's first close call stay within five times the bound, at most one in eight of them beyond the
    bound itself; over all positions the median stays within the bound and every position is sane."""
    got, want = torch.as_tensor(got, dtype=F).cpu(), torch.as_tensor(want, dtype=F).cpu()
    if got.dim() == 1:
        got, want = got[None], want[None]
    sure = torch.ones(want.shape[0], dtype=torch.bool)
    if want.shape[-1] == got.shape[-1] + 1:
        want, sure = want[:, :-1], want[:, -1] > 0.5
    assert got.shape == want.shape, (got.shape, want.shape)
    errors = (got - want).abs().amax(-1) / want.abs().max().clamp_min(1e-30)
    bound = TOLERANCE[dtype]
    if dtype == "float32":
        # (a norm sits on every sublayer's RESULT: where a result happens to be small against its spread, the norm enlarges
        # its rounding; such a position lies at ten times the median and still far below any real fault)
        ok = bool((errors < 5 * bound).all()) and int((errors >= bound).sum()) <= max(1, errors.numel() // 50) and float(errors.median()) < bound / 4
    else:
        ok = bool((errors[sure] < 5 * bound).all()) and int((errors[sure] >= bound).sum()) <= max(1, int(sure.sum()) // 8) \
            and bool((errors < 1.0).all()) and float(errors.median()) < bound
    if not ok:
        print("positions", errors.numel(), "sure", int(sure.sum()), "median", float(errors.median()),
              "largest", [(int(i), round(float(errors[i]), 6), bool(sure[i])) for i in errors.argsort(descending=True)[:12]])
    return ok


def _rounded(t, dtype):
    return t.to(dtype).to(F)


# ----------------------------------------------------------------------------------- mechanisms alone

def _pools(T, G, D, Dv, page_size, device, dtype, shuffle_seed=0):
    """Fresh pools (full of NaN) with the sequence's pages in a shuffled order: pools, page table, slot mapping, positions."""
    pages = -(-T // page_size)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(shuffle_seed)) + 1
    k_pool = torch.full((pages + 1, G, page_size, D), float("nan"), dtype=dtype, device=device)
    v_pool = torch.full((pages + 1, G, page_size, Dv), float("nan"), dtype=dtype, device=device)
    positions = torch.arange(T, dtype=torch.int32)
    mapping = (order[positions // page_size].to(torch.int32) * page_size + positions % page_size).to(torch.int32).to(device)
    return k_pool, v_pool, order.to(torch.int32)[None, :].contiguous().to(device), mapping, positions.to(device)


def _plain_attend(q, k, v, scale, chunk):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] float64 -> [T, H, Dv]: softmax attention inside chunks counted from 0."""
    T, H, _ = q.shape
    G = k.shape[1]
    seen = pr.chunk_visible(T, chunk if chunk else T)
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T * scale).masked_fill(~seen, float("-inf"))
        out[:, h] = torch.softmax(s, -1) @ v[:, g]
    return out


def _attend(q, k, v, scale, chunk, dtype, device, q_len, kernel, page_size=64):
    """The same through the cache-write kernel and one form of the attention kernel; the last `q_len` tokens are the step."""
    from models_b200.kernels import ops

    T, H, D = q.shape
    G, Dv = k.shape[1], v.shape[2]
    k_pool, v_pool, table, mapping, positions = _pools(T, G, D, Dv, page_size, device, dtype)
    qd, kd, vd = (t.reshape(T, -1).to(dtype).to(device).contiguous() for t in (q, k, v))
    first = T - q_len
    for lo, hi in ((0, first), (first, T)):
        if hi > lo:
            ops.project_norm_rotate_store(qd[lo:hi], kd[lo:hi], vd[lo:hi], None, None, None, None, None, 1e-6, positions[lo:hi], None, None,
                                          0, False, k_pool, v_pool, mapping[lo:hi], H, G, D, Dv)
    out = torch.empty((q_len, H * Dv), dtype=dtype, device=device)
    cu_q = torch.tensor([0, q_len], dtype=torch.int32, device=device)
    kv_lens = torch.tensor([T], dtype=torch.int32, device=device)
    ops.gated_attention(qd[first:], out, k_pool, v_pool, table, cu_q, kv_lens, q_len, H, G, D, Dv, "softmax", scale, block=chunk or 0, kernel=kernel)
    return out.double().cpu().reshape(q_len, H, Dv)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,target,chunk", [
    (700, 3, None),      # far away among hundreds, no chunks
    (700, 640, 64),      # the first key of the query's chunk
    (700, 639, 64),      # the key just before it: invisible
    (700, 600, 100),     # a chunk's first key inside a page
    (700, 599, 100),     # and the one before it
    (130, 128, 128),     # a chunk that starts with a page
    (130, 127, 128),
    (257, 255, 5),       # chunks smaller than the kernels' tiles
    (257, 254, 5),
    (40, 39, 7),         # the query's own position
    (70, 0, 1000),       # the sequence's first key, one chunk for everything
    (66, 64, 1),         # chunks of one position: every query sees itself alone
])
def test_one_key_decides_inside_and_outside_a_chunk(cuda_device, tokens, target, chunk, dtype):
    """One key is made to stand out for the last query (its score towers over the others): if it is visible the result is its
    value, if it lies before the query's chunk it must not be seen at all.  Every form of the kernel, against the plain one."""
    g = torch.Generator().manual_seed(tokens * 31 + target)
    H, G, D, Dv = 4, 2, 32, 16
    q = _rounded(torch.randn(tokens, H, D, generator=g, dtype=F) * 0.5, dtype)
    k = _rounded(torch.randn(tokens, G, D, generator=g, dtype=F) * 0.5, dtype)
    v = _rounded(torch.randn(tokens, G, Dv, generator=g, dtype=F), dtype)
    direction = torch.randn(D, generator=g, dtype=F)
    direction /= direction.norm()
    q[-1] = _rounded(direction * 6.0 + q[-1] * 0.1, dtype)
    k[target] = _rounded(direction * 6.0, dtype)
    want = _plain_attend(q, k, v, 0.5, chunk)
    last = tokens - 1
    visible = target <= last and (chunk is None or target // chunk == last // chunk)
    if visible and target != last:
        assert float((want[-1, 0] - v[target, 0]).abs().max()) < 0.05  # the test's own premise: that key takes all the weight
    bound = 2e-5 if dtype == torch.float32 else 2e-2
    forms = [("rows", tokens), ("rows", 3), ("decode", 1)] + ([("tc", tokens), ("tc", 70 if tokens > 70 else 9)] if dtype == torch.bfloat16 else [])
    for kernel, q_len in forms:
        got = _attend(q, k, v, 0.5, chunk, dtype, cuda_device, q_len, kernel)
        assert scaled_error(got, want[tokens - q_len:]) < bound, (kernel, q_len)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot,chunk", [(4, 2, 16, 8, 8, 5), (3, 1, 20, 12, 10, 100), (1, 1, 8, 40, 0, None),
                                                              (6, 3, 18, 14, 18, 7), (8, 2, 64, 128, 32, 96), (2, 2, 32, 32, 32, 64)])
def test_projection_norm_rotation_and_chunks_at_other_sizes(cuda_device, heads, kv_heads, dim, vdim, rot, chunk, dtype):
    """Biases, ONE norm over all query heads and one over all key heads, rotation of the first `rot` coordinates from a
    position far from 0, through a prompt step and through single-token steps, against the plain arithmetic."""
    from models_b200.kernels import ops

    T, start = 150, (1000 if chunk else 0)  # (without chunks every earlier position is visible: the sequence starts at 0)
    g = torch.Generator().manual_seed(heads * 100 + dim)
    eps = 1e-5
    rnd = lambda *shape: torch.randn(*shape, generator=g, dtype=F)  # noqa: E731
    q, k, v = _rounded(rnd(T, heads * dim), dtype), _rounded(rnd(T, kv_heads * dim), dtype), _rounded(rnd(T, kv_heads * vdim), dtype)
    bq, bk, bv = rnd(heads * dim).float(), rnd(kv_heads * dim).float(), rnd(kv_heads * vdim).float()
    gq, gk = (1 + 0.3 * rnd(heads * dim)).float(), (1 + 0.3 * rnd(kv_heads * dim)).float()
    positions = torch.arange(start, start + T)
    qn = pr.rotate_half(pr.rms_norm(q + bq.double(), gq.double(), eps).view(T, heads, dim), positions, rot, 777.0)
    kn = pr.rotate_half(pr.rms_norm(k + bk.double(), gk.double(), eps).view(T, kv_heads, dim), positions, rot, 777.0)
    vn = (v + bv.double()).view(T, kv_heads, vdim)
    seen = pr.chunk_visible(T, chunk if chunk else 10 ** 9, start)
    want = torch.zeros(T, heads, vdim, dtype=F)
    for h in range(heads):
        s = (qn[:, h] @ kn[:, h // (heads // kv_heads)].T * 0.3).masked_fill(~seen, float("-inf"))
        want[:, h] = torch.softmax(s, -1) @ vn[:, h // (heads // kv_heads)]
    # the engine's side: the sequence's positions start..start+T live in pages start/64 ...; the earlier pages are never read
    page = 64
    pages = -(-(start + T) // page)
    order = torch.randperm(pages, generator=g) + 1
    # (what the step does not write holds large numbers: a key read from before the query's chunk would take all the weight)
    k_pool = torch.full((pages + 1, kv_heads, page, dim), 50.0, dtype=dtype, device=cuda_device)
    v_pool = torch.full((pages + 1, kv_heads, page, vdim), 50.0, dtype=dtype, device=cuda_device)
    table = order.to(torch.int32)[None, :].contiguous().to(cuda_device)
    pos32 = positions.to(torch.int32).to(cuda_device)
    mapping = (order[positions // page].to(torch.int32) * page + (positions % page).to(torch.int32)).to(torch.int32).to(cuda_device)
    half = rot // 2
    cos = sin = None
    if rot:
        freq = torch.tensor([777.0 ** (-2.0 * i / rot) for i in range(half)], dtype=F).float()
        angle = (torch.arange(start + T, dtype=torch.float32)[:, None] * freq[None, :]).double()
        cos, sin = torch.cos(angle).float().contiguous().to(cuda_device), torch.sin(angle).float().contiguous().to(cuda_device)
    dev = lambda t: t.to(cuda_device).contiguous()  # noqa: E731
    qd, kd, vd = dev(q.to(dtype)), dev(k.to(dtype)), dev(v.to(dtype))
    # the chunk that holds `start` began before the step: its earlier keys are not in the cache, so the comparison starts at
    # the first chunk that begins inside the step
    first_whole = (-(-start // chunk)) * chunk - start if chunk else 0
    out_rows = []
    prompt = 100
    for lo, hi in [(0, prompt)] + [(i, i + 1) for i in range(prompt, T)]:
        qs = qd[lo:hi].clone()
        ops.project_norm_rotate_store(qs, kd[lo:hi], vd[lo:hi], dev(bq), dev(bk), dev(bv), dev(gq), dev(gk), eps, pos32[lo:hi], cos, sin, rot, False,
                                      k_pool, v_pool, mapping[lo:hi], heads, kv_heads, dim, vdim)
        out = torch.empty((hi - lo, heads * vdim), dtype=dtype, device=cuda_device)
        cu_q = torch.tensor([0, hi - lo], dtype=torch.int32, device=cuda_device)
        kv_lens = torch.tensor([start + hi], dtype=torch.int32, device=cuda_device)
        ops.gated_attention(qs, out, k_pool, v_pool, table, cu_q, kv_lens, hi - lo, heads, kv_heads, dim, vdim, "softmax", 0.3, block=chunk or 0)
        out_rows.append(out.double().cpu())
    got = torch.cat(out_rows).reshape(T, heads, vdim)
    bound = 2e-5 if dtype == torch.float32 else 3e-2
    assert scaled_error(got[first_whole:], want[first_whole:]) < bound


def _fake_batch(lengths, slots, device):
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + n)
    return SimpleNamespace(cu_q=torch.tensor(cu, dtype=torch.int32, device=device), slots=torch.tensor(slots, dtype=torch.int32, device=device),
                           max_q_len=max(lengths))


def _part(kind, spec, tensors, dtype, device):
    from models_b200.parts import RunContext, Runtime, build_part

    part = build_part("mixer", spec, Runtime(device, dtype, max_positions=64))
    part.load({n: t.to(torch.bfloat16 if dtype == "bfloat16" else torch.float32) for n, t in tensors.items()})
    request = part.state_request()
    state = torch.zeros((5,) + tuple(request.shape), dtype=torch.float32, device=device)
    return part, RunContext(run=0, state=state)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,taps", [(2, 1, 16, 24, 4), (3, 3, 8, 8, 2), (1, 1, 32, 32, 1), (6, 2, 18, 10, 5), (4, 2, 64, 128, 4),
                                                         (2, 2, 100, 40, 3)])
def test_gated_delta_rule_ragged_carried_and_in_portions(cuda_device, heads, kv_heads, dim, vdim, taps, dtype):
    """Three sequences of unequal lengths in one step, then more tokens for two of them (a long portion, and single tokens):
    the state S and the convolutions' last inputs are carried per slot; a slot used again starts from zero."""
    from models_b200.config.specs import GatedDeltaSpec

    W = 48
    g = torch.Generator().manual_seed(heads * 1000 + dim + taps)
    names = {r: "m." + r for r in ("q", "k", "v", "o", "a", "b", "A_log", "dt_bias", "norm")}
    names.update(gate="m.g", q_conv="m.q.conv", k_conv="m.k.conv", v_conv="m.v.conv")
    spec = GatedDeltaSpec(W, heads, kv_heads, dim, vdim, taps, 1e-6, 1e-5, names)
    rnd = lambda *shape: torch.randn(*shape, generator=g)  # noqa: E731
    w = {"m.q": rnd(kv_heads * dim, W) * 0.3, "m.k": rnd(kv_heads * dim, W) * 0.3, "m.v": rnd(heads * vdim, W) * 0.3,
         "m.q.conv": rnd(kv_heads * dim, taps) * 0.6, "m.k.conv": rnd(kv_heads * dim, taps) * 0.6, "m.v.conv": rnd(heads * vdim, taps) * 0.6,
         "m.b": rnd(heads, W) * 0.4, "m.a": rnd(heads, W) * 0.4, "m.A_log": torch.rand(heads, generator=g) * 3 - 3,
         "m.dt_bias": torch.rand(heads, generator=g) * 3 - 2, "m.norm": 1 + 0.2 * rnd(vdim), "m.g": rnd(heads * vdim, W) * 0.3,
         "m.o": rnd(W, heads * vdim) * 0.2}
    w = {n: t.to(torch.bfloat16).float() for n, t in w.items()}
    part, run = _part("gated_delta", spec, w, dtype, cuda_device)
    td = TORCH[dtype]
    c = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim}
    full = [_rounded(rnd(n, W).double(), td) for n in (150, 37, 9)]
    want = [pr.gated_delta_rule(x, w, "m.", c, 1e-5) for x in full]
    bound = 3e-5 if dtype == "float32" else 3e-2

    def step(pieces, slots):
        xn = torch.cat(pieces).to(td).to(cuda_device)
        return part.forward(xn, _fake_batch([p.shape[0] for p in pieces], slots, cuda_device), run).double().cpu()

    out = step([full[0][:20], full[1][:30], full[2][:1]], [3, 0, 2])
    assert scaled_error(out, torch.cat([want[0][:20], want[1][:30], want[2][:1]])) < bound
    out = step([full[2][1:9], full[0][20:140]], [2, 3])  # portions that start inside the sequences
    assert scaled_error(out, torch.cat([want[2][1:9], want[0][20:140]])) < bound
    rows = [step([full[0][i:i + 1], full[1][30 + i - 140:31 + i - 140]], [3, 0]) for i in range(140, 147)]  # token by token
    assert scaled_error(torch.cat(rows), torch.cat([torch.cat([want[0][i:i + 1], want[1][30 + i - 140:31 + i - 140]]) for i in range(140, 147)])) < bound
    run.state[2].zero_()  # what opening a slot does
    assert scaled_error(step([full[1][:5]], [2]), want[1][:5]) < bound


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,blocks,taps", [(48, 3, 3), (40, 1, 1), (72, 6, 4), (33, 3, 2), (256, 2, 4)])
def test_rglru_ragged_carried_and_in_portions(cuda_device, width, blocks, taps, dtype):
    """The same for the recurrent block; lambda spans recurrences that forget at once and ones that barely forget (a state lost
    at a portion's start then shows), and the steps are long enough for the walk in runs and short enough for the single walk."""
    from models_b200.config.specs import RglruSpec

    W = 40
    g = torch.Generator().manual_seed(width * 10 + taps)
    per = width // blocks
    names = {r: "m." + r for r in ("y", "x", "conv", "o", "lam")}
    names.update(y_bias="m.y.b", x_bias="m.x.b", conv_bias="m.conv.b", gate_a="m.ra", gate_a_bias="m.ra.b", gate_i="m.ri", gate_i_bias="m.ri.b")
    spec = RglruSpec(W, width, blocks, taps, 8.0, names)
    rnd = lambda *shape: torch.randn(*shape, generator=g)  # noqa: E731
    w = {"m.y": rnd(width, W) * 0.3, "m.y.b": rnd(width) * 0.3, "m.x": rnd(width, W) * 0.3, "m.x.b": rnd(width) * 0.3,
         "m.conv": rnd(width, taps) * 0.6, "m.conv.b": rnd(width) * 0.3, "m.ra": rnd(blocks, per, per) * 0.4, "m.ra.b": rnd(blocks, per) * 0.5,
         "m.ri": rnd(blocks, per, per) * 0.4, "m.ri.b": rnd(blocks, per) * 0.5, "m.lam": torch.rand(width, generator=g) * 8 - 7,
         "m.o": rnd(W, width) * 0.2}
    w = {n: t.to(torch.bfloat16).float() for n, t in w.items()}
    part, run = _part("rglru", spec, w, dtype, cuda_device)
    td = TORCH[dtype]
    c = {"width": width, "blocks": blocks}
    full = [_rounded(rnd(n, W).double(), td) for n in (300, 37, 9)]
    want = [pr.rglru_mixer(x, w, "m.", c) for x in full]
    bound = 3e-5 if dtype == "float32" else 3e-2

    def step(pieces, slots):
        xn = torch.cat(pieces).to(td).to(cuda_device)
        return part.forward(xn, _fake_batch([p.shape[0] for p in pieces], slots, cuda_device), run).double().cpu()

    out = step([full[0][:20], full[1][:30], full[2][:1]], [3, 0, 2])
    assert scaled_error(out, torch.cat([want[0][:20], want[1][:30], want[2][:1]])) < bound
    out = step([full[2][1:3], full[0][20:290]], [2, 3])
    assert scaled_error(out, torch.cat([want[2][1:3], want[0][20:290]])) < bound
    rows = [step([full[0][i:i + 1], full[1][i - 260:i - 259]], [3, 0]) for i in range(290, 297)]
    assert scaled_error(torch.cat(rows), torch.cat([torch.cat([want[0][i:i + 1], want[1][i - 260:i - 259]]) for i in range(290, 297)])) < bound
    run.state[2].zero_()
    assert scaled_error(step([full[1][:5]], [2]), want[1][:5]) < bound


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,identity,top,groups,width,ff,shared,tokens", [
    (6, 2, 2, (4, 2), 64, 40, 24, 70), (6, 2, 2, (4, 2), 64, 40, 24, 3), (5, 3, 3, (2, 2), 72, 36, 16, 200), (3, 1, 4, (1, 1), 50, 20, None, 9),
    (4, 0, 1, (1, 1), 64, 24, None, 130), (8, 4, 2, (3, 2), 256, 128, 64, 600), (7, 0, 3, (7, 4), 56, 12, 8, 33), (12, 20, 4, (32, 5), 64, 16, None, 40)])
def test_scored_router_groups_identity_and_shared_experts(cuda_device, experts, identity, top, groups, width, ff, shared, tokens, dtype):
    """The feed-forward alone, in the three forms the step's size picks; the weights are made so that identity experts are
    chosen often, and tokens whose decision is a close call are left out of the bfloat16 comparison."""
    from models_b200.config.specs import ClampedExpertSpec, RoutedFeedForwardSpec
    from models_b200.parts import Runtime, build_part

    g = torch.Generator().manual_seed(experts * 100 + tokens)
    total = experts + identity
    names = {"router": "f.router", "correction": "f.correction"}
    for r in ("gate", "up", "down"):
        names["expert_" + r] = "f.e{expert}." + r
        names["shared_" + r] = "f.shared." + r
    plain = lambda n: ClampedExpertSpec(n, float("inf"), 1.0, up_offset=0.0)  # noqa: E731
    spec = RoutedFeedForwardSpec(width, experts, top, plain(ff), plain(shared) if shared else None, names, rule="scored", correction=True,
                                 groups=groups[0], keep_groups=groups[1], weight_scale=1.7, identity_experts=identity, shared_gated=False)
    rnd = lambda *shape: torch.randn(*shape, generator=g)  # noqa: E731
    w = {"f.router": rnd(total, width) * 0.4, "f.correction": rnd(total) * 0.1}
    for e in range(experts):
        w.update({f"f.e{e}.gate": rnd(ff, width) * 0.2, f"f.e{e}.up": rnd(ff, width) * 0.2, f"f.e{e}.down": rnd(width, ff) * 0.2})
    if shared:
        w.update({"f.shared.gate": rnd(shared, width) * 0.2, "f.shared.up": rnd(shared, width) * 0.2, "f.shared.down": rnd(width, shared) * 0.2})
    w = {n: t.to(torch.bfloat16).float() for n, t in w.items()}
    td = TORCH[dtype]
    part = build_part("feed_forward", spec, Runtime(cuda_device, dtype))
    part.load({n: t.to(td) for n, t in w.items()})
    x = _rounded(rnd(tokens, width).double(), td)
    c = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": 1.7,
                                                        "groups": {"count": groups[0], "keep": groups[1]}}}
    if shared:
        c["shared"] = {"ff": shared}
    want = pr.moe_ff(x, w, "f.", c)
    chosen, _, margin = pr.route(x, w, "f.", c)
    if identity:
        assert int((chosen >= experts).sum()) > 0  # identity experts do get chosen
    got = part.forward_wide(x.to(td).to(cuda_device)).double().cpu()
    sure = margin > (1e-4 if dtype == "float32" else 0.03)
    assert int(sure.sum()) >= tokens // 3
    assert scaled_error(got[sure], want[sure]) < (2e-5 if dtype == "float32" else 3e-2)
    # the choices themselves
    from models_b200.kernels import ops
    ids, weights = ops.router_topk(x.to(td).to(cuda_device), part.router, top, scored=True, correction=part.correction, groups=groups[0],
                                   keep=groups[1], weight_scale=1.7)
    assert torch.equal(ids.cpu().long()[sure], chosen[sure])


@pytest.mark.parametrize("width,rows", [(50, 3), (256, 70), (64, 1), (2048, 5)])
def test_norm_on_the_result_scale_and_add(cuda_device, width, rows):
    """x += scale * LN(y) for one result and for the mean of two RMS-normed ones, rows far from zero mean, and the copy."""
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(width + rows)
    rnd = lambda *shape: torch.randn(*shape, generator=g)  # noqa: E731
    x, a, b = rnd(rows, width), rnd(rows, width) * 3 + 5, rnd(rows, width) * 0.1
    weight, scale, ga, gb = 1 + 0.2 * rnd(width), rnd(width), 1 + 0.2 * rnd(width), 1 + 0.2 * rnd(width)
    dev = lambda t: t.to(cuda_device).contiguous()  # noqa: E731
    eps = 1e-5
    for pair in (False, True):
        y = 0.5 * (pr.rms_norm(a.double(), ga.double(), eps) + pr.rms_norm(b.double(), gb.double(), eps)) if pair else a.double()
        want = x.double() + scale.double() * pr.layer_norm(y, weight.double(), eps)
        xd = dev(x.clone())
        copy = ops.outnorm_add(xd, dev(a), dev(weight), dev(scale), eps, b=dev(b) if pair else None, gain_a=dev(ga) if pair else None,
                               gain_b=dev(gb) if pair else None, copy_dtype=torch.bfloat16)
        assert scaled_error(xd.cpu(), want) < 1e-5
        assert torch.equal(copy.cpu(), xd.cpu().to(torch.bfloat16))
    got = ops.pair_norm_mean(dev(a), dev(b), dev(ga), dev(gb), eps)
    assert scaled_error(got.cpu(), 0.5 * (pr.rms_norm(a.double(), ga.double(), eps) + pr.rms_norm(b.double(), gb.double(), eps))) < 1e-5


# ----------------------------------------------------------------------------------- whole models

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(RLV))
def test_whole_prompt_every_position(cuda_device, folders, name, dtype):
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype)
    for n, seed in ((1, 1), (2, 5), (7, 2), (70, 3), (200, 4)):
        tokens = random_tokens(RLV[name]["vocab"], n, seed)
        slot = engine.open_slot()
        logits = engine.step([StepEntry(slot, tokens, list(range(n)))])
        engine.release_slot(slot)
        assert _close(logits, plain_logits(folders[name], tokens), dtype), (name, dtype, n)
    engine.cache.check()


@pytest.mark.parametrize("name", sorted(RLV))
def test_residual_stream_after_every_layer(cuda_device, folders, name):
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], "float32")
    tokens = random_tokens(RLV[name]["vocab"], 90, 6)
    seen = []
    engine.model.observer = lambda run, x: seen.append(x.double().cpu())
    slot = engine.open_slot()
    engine.step([StepEntry(slot, tokens, [89])])
    expected = []
    plain_logits_alone(folders[name], tokens, expected)
    assert len(seen) == len(expected) == len(RLV[name]["layers"])
    for run, (got, want) in enumerate(zip(seen, expected)):
        assert scaled_error(got, want) < 1e-5, run


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(RLV))
def test_prompt_then_token_by_token(cuda_device, folders, name, dtype):
    """A short prompt, then 130 tokens one by one: the decode form of the attention crosses cache pages and chunk edges, and
    both recurrences with their convolutions are carried through every step."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype)
    n, head = 150, 20
    tokens = random_tokens(RLV[name]["vocab"], n, 7)
    expected = plain_logits(folders[name], tokens)
    slot = engine.open_slot()
    rows = [engine.step([StepEntry(slot, tokens[:head], [head - 1])])]
    for i in range(head, n):
        rows.append(engine.step([StepEntry(slot, [tokens[i]], [0])]))
    assert _close(torch.cat(rows), expected[head - 1:], dtype)
    engine.cache.check()
    engine.release_slot(slot)
    assert all(g.pages.held == 0 for g in engine.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "D"])
def test_token_by_token_from_the_first_token(cuda_device, folders, name, dtype):
    """No prompt step at all: the first tokens of a sequence go through the decode kernels (one key; states and convolutions
    that start at zero)."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype)
    tokens = random_tokens(RLV[name]["vocab"], 70, 17)
    expected = plain_logits(folders[name], tokens)
    slot = engine.open_slot()
    rows = [engine.step([StepEntry(slot, [t], [0])]) for t in tokens]
    assert _close(torch.cat(rows), expected, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,portions", [("A", [2, 3, 17, 64, 1, 2, 90, 21]), ("B", [64, 64, 2, 70]), ("C", [130, 2, 68]),
                                           ("D", [5, 2, 2, 129, 62])])
def test_prompt_in_portions(cuda_device, folders, name, portions, dtype):
    """A portion starts inside a sequence and inside a chunk: its recurrences go on from the stored states, its convolutions
    from the stored inputs (also when the portion is shorter than the convolution), its queries see the chunk's earlier keys."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype)
    tokens = random_tokens(RLV[name]["vocab"], sum(portions), 8)
    expected = plain_logits(folders[name], tokens)
    slot = engine.open_slot()
    at, rows = 0, []
    for count in portions:
        rows.append(engine.step([StepEntry(slot, tokens[at:at + count], list(range(count)))]).clone())
        if dtype == "float32":
            assert _close(rows[-1], expected[at:at + count], dtype), (at, count)
        at += count
    assert _close(torch.cat(rows), expected, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(RLV))
def test_unequal_batches_and_slots_used_again(cuda_device, folders, name, dtype):
    """Four prompts of unequal lengths in one step, decoded together while the shorter ones end; then new requests take the
    freed slots and pages (their states must start at zero, their pages hold old keys and values)."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype, max_tokens=1024)
    vocab = RLV[name]["vocab"]
    for round_index in range(2):
        lengths, prompts = [1, 33, 140, 70], [1, 20, 131, 66]
        full = [random_tokens(vocab, n + 12, 10 * round_index + i) for i, n in enumerate(lengths)]
        expected = [plain_logits(folders[name], t) for t in full]
        slots = [engine.open_slot() for _ in full]
        out = engine.step([StepEntry(s, t[:p], [0, p - 1]) for s, t, p in zip(slots, full, prompts)])
        want = torch.stack([expected[i][r] for i, p in enumerate(prompts) for r in (0, p - 1)])
        assert _close(out, want, dtype), round_index
        live = list(range(4))
        at = list(prompts)
        got_rows, want_rows = [], []
        while live:
            out = engine.step([StepEntry(slots[i], [full[i][at[i]]], [0]) for i in live])
            for row, i in enumerate(live):
                got_rows.append(out[row].clone())
                want_rows.append(expected[i][at[i]])
                at[i] += 1
            for i in [i for i in live if at[i] == len(full[i])]:
                engine.release_slot(slots[i])
                live.remove(i)
        assert _close(torch.stack(got_rows), torch.stack(want_rows), dtype), round_index
        engine.cache.check()
    assert engine.cache.slots.held == 0 and all(g.pages.held == 0 for g in engine.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_from_graphs(cuda_device, folders, name, dtype):
    """Three sequences decoded for 330 steps from captured steps, over several pages and many chunks; one sequence ends on the
    way and another takes its slot (and must not inherit its states or its keys)."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype, max_tokens=4096)
    engine.enable_decode_graphs(4)
    vocab = RLV[name]["vocab"]
    full = [random_tokens(vocab, n, 20 + i) for i, n in enumerate((340, 200, 150, 120))]
    expected = [plain_logits(folders[name], t) for t in full]
    prompts = [5, 70, 1, 30]
    slots = {i: engine.open_slot() for i in range(3)}
    engine.step([StepEntry(slots[i], full[i][:prompts[i]], []) for i in range(3)])
    at = {i: prompts[i] for i in range(3)}
    got_rows, want_rows = [], []
    while at:
        live = sorted(at)
        out = engine.decode([slots[i] for i in live], [full[i][at[i]] for i in live])
        for row, i in enumerate(live):
            if at[i] % 7 == 0 or at[i] > len(full[i]) - 3:
                got_rows.append(out[row].clone())
                want_rows.append(expected[i][at[i]])
            at[i] += 1
            if at[i] == len(full[i]):
                engine.release_slot(slots.pop(i))
                del at[i]
                if i == 2:  # a new request in the freed slot, from its prompt
                    slots[3] = engine.open_slot()
                    engine.step([StepEntry(slots[3], full[3][:prompts[3]], [])])
                    at[3] = prompts[3]
    assert _close(torch.stack(got_rows), torch.stack(want_rows), dtype)
    assert engine.decode_graphs.captured  # the steps did come from captures
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["rglru", "parallel"])
def test_models_of_one_kind_of_layer(cuda_device, tmp_path, kind, dtype):
    """Only recurrent blocks (no cache group at all, state alone) or only parallel layers: prompts of one length class four
    times over, then tokens one by one from captured decode steps."""
    from models_b200.engine import StepEntry

    layers = {"rglru": [rglru(48, 2, 4, dense(48)), rglru(24, 3, 2, None)],
              "parallel": [parallel((4, 2, 16, 8, 0.25, 10, (16, 1e4)), (2, 2, 16, 16, 4), moe(4, 2, 2, 2.0, (3, 2), 24)),
                           parallel((2, 1, 32, 32, 0.2, 3, (8, 300.0)), (4, 1, 8, 8, 2), None)]}[kind]
    raw = model(120, 64, 1e-5, 1.0, 0.5, layers)
    folder = make_folder(raw, 90, tmp_path)
    engine = _engine(folder, dtype, 1024)
    engine.enable_decode_graphs(4)
    assert (len(engine.cache.groups) == 0) == (kind == "rglru")
    for seed in range(4):
        tokens = random_tokens(120, 140, seed)
        want = plain_logits(folder, tokens)
        slot = engine.open_slot()
        rows = [engine.step([StepEntry(slot, tokens[:100], [99])])]
        for t in tokens[100:]:
            rows.append(engine.decode([slot], [t]).clone())
        assert _close(torch.cat(rows), want[99:], dtype), seed
        engine.release_slot(slot)
    engine.cache.check()


RLV_MID = model(1000, 384, 1e-6, 0.8, 0.6, [
    parallel((6, 3, 48, 80, 0.144, 96, (24, 30000.0)), (4, 2, 48, 80, 3), moe(24, 8, 5, 1.8, (8, 3), 96, 160)),
    rglru(200, 5, 3, dense(640)),
    parallel((5, 1, 40, 24, 0.16, 250, (40, 1000.0)), (6, 6, 24, 40, 4), dense(512)),
    rglru(384, 3, 4, moe(10, 0, 2, 1.0, (2, 1), 128)),
])


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_mid_sized_model_long_prompts_and_batches(cuda_device, tmp_path, dtype):
    """Sizes between the small configurations and the benchmark's (heads of 48 and 40, values of 80 and 24, 32 router outputs in
    8 groups, chunks of 96 and 250): a prompt of 700 tokens whole, then decoded across chunk edges; three unequal prompts in one
    step (1, 300 and 650 tokens), then decoded together while the short one ends."""
    from models_b200.engine import StepEntry

    folder = make_folder(RLV_MID, 77, tmp_path, std=0.08)
    engine = _engine(folder, dtype, max_tokens=4096)
    vocab = RLV_MID["vocab"]
    tokens = random_tokens(vocab, 740, 5)
    expected = plain_logits(folder, tokens)
    want_rows = [0, 95, 96, 97, 249, 250, 251, 383, 384, 500, 699]
    slot = engine.open_slot()
    rows = [engine.step([StepEntry(slot, tokens[:700], want_rows)])]
    for i in range(700, 740):
        rows.append(engine.step([StepEntry(slot, [tokens[i]], [0])]))
    assert _close(torch.cat(rows), torch.cat([expected[want_rows], expected[700:]]), dtype)
    engine.release_slot(slot)
    lengths, prompts = [9, 330, 680], [1, 300, 650]
    full = [random_tokens(vocab, n, 30 + i) for i, n in enumerate(lengths)]
    wanted = [plain_logits(folder, t) for t in full]
    slots = [engine.open_slot() for _ in full]
    out = engine.step([StepEntry(s, t[:p], [p - 1]) for s, t, p in zip(slots, full, prompts)])
    got, want = [out], [torch.stack([wanted[i][p - 1] for i, p in enumerate(prompts)])]
    live, at = [0, 1, 2], list(prompts)
    while live:
        out = engine.step([StepEntry(slots[i], [full[i][at[i]]], [0]) for i in live])
        got.append(out.clone())
        want.append(torch.stack([wanted[i][at[i]] for i in live]))
        for i in list(live):
            at[i] += 1
            if at[i] == len(full[i]):
                engine.release_slot(slots[i])
                live.remove(i)
    assert _close(torch.cat(got), torch.cat(want), dtype)
    engine.cache.check()


def test_logits_do_not_depend_on_the_batch_or_the_cut(cuda_device, folders):
    """float32: the same position through a whole prompt, through portions, and inside a batch differs by rounding only."""
    from models_b200.engine import StepEntry

    for name in ("A", "C"):
        engine = _engine(folders[name], "float32")
        vocab = RLV[name]["vocab"]
        a, b = random_tokens(vocab, 100, 31), random_tokens(vocab, 37, 32)
        slot = engine.open_slot()
        whole = engine.step([StepEntry(slot, a, [99])])
        engine.release_slot(slot)
        s1, s2 = engine.open_slot(), engine.open_slot()
        engine.step([StepEntry(s2, b[:30], []), StepEntry(s1, a[:64], [])])
        engine.step([StepEntry(s1, a[64:99], []), StepEntry(s2, b[30:], [])])
        cut = engine.step([StepEntry(s1, a[99:], [0])])
        assert scaled_error(cut, whole) < 5e-6, name


def test_greedy_generation_through_the_entry_point(cuda_device, folders):
    import models_b200

    folder = folders["A"]
    prompts = [random_tokens(RLV["A"]["vocab"], n, 50 + n) for n in (3, 40, 11)]
    steps = 40
    config, weights = pr.read_model_folder(folder)
    expected, margins = [], []
    for prompt in prompts:
        tokens, out, margin = list(prompt), [], []
        for _ in range(steps):
            logits = pr.forward(config, weights, tokens)[-1]
            top = torch.topk(logits, 2).values
            margin.append(float(top[0] - top[1]))
            out.append(int(torch.argmax(logits)))
            tokens.append(out[-1])
        expected.append(out)
        margins.append(margin)
    for dtype in DTYPES:
        generator = models_b200.load_model(folder, dtype=dtype, max_batch=4, context=256)
        results = generator.generate_batch(prompts, models_b200.SamplingOptions(temperature=0.0, max_tokens=steps))
        for result, want, margin in zip(results, expected, margins):
            for i, (a, b) in enumerate(zip(result.tokens, want)):
                if a != b:
                    assert dtype == "bfloat16" and margin[i] < 0.05, (dtype, i, result.tokens, want)
                    break
        generator.close()


def test_trace_replay_program(cuda_device, folders, tmp_path):
    """bin/trace_run on a Rolevik folder: two prompts in one step, then decoded together from captured steps."""
    name = "D"
    vocab = RLV[name]["vocab"]
    a, b = random_tokens(vocab, 90, 1), random_tokens(vocab, 12, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []}]
    for i in range(20):
        entries = [{"id": "a", "tokens": [a[70 + i]], "want": [0]}]
        if i < 7:
            entries.append({"id": "b", "tokens": [b[5 + i]], "want": [0]})
        steps.append({"step": i + 1, "entries": entries, "end": (["b"] if i == 6 else []) + (["a"] if i == 19 else [])})
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ea, eb = plain_logits(folders[name], a), plain_logits(folders[name], b)
    for dtype in DTYPES:
        proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(folders[name]), "--dtype", dtype,
                               "--out", str(out), "--max-tokens", "102"],
                              input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
        assert proc.returncode == 0, proc.stderr[-2000:]
        first = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, vocab)
        got = [first[0], first[1], first[2]]
        want = [ea[0], ea[69], eb[4]]
        for i in range(20):
            rows = np.fromfile(out / f"{i + 1}.f32", dtype="<f4").reshape(-1, vocab)
            got.append(rows[0])
            want.append(ea[70 + i])
            if i < 7:
                got.append(rows[1])
                want.append(eb[5 + i])
        assert _close(np.stack(got), torch.stack(want), dtype), dtype
