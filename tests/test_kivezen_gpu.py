"""The Kivezen decoder in the engine against the plain implementation (tests/plain/plain_kivezen.py): each kernel alone
with inputs made so that one key, the sink, the cap, one expert or one stream decides the result, whole prompts, prompts
cut into portions, token-by-token decoding across cache pages, unequal batches, slots, pages and states used again, long
decoding from CUDA graphs, and greedy generation through the public entry point."""

import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from plain import plain_kivezen as pk
from tiny import TOLERANCE, random_tokens, scaled_error
from tiny_kivezen import KVZ, attention, dense, lightning, make_folder, moe, plain_logits

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
F = torch.float64


def _engine(folder, dtype, max_tokens=2048, **more):
    from models_b200.engine.loading import engine_from_folder

    return engine_from_folder(folder, dtype, max_tokens, **more)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("kivezen")
    return {name: make_folder(raw, seed=41 + i, root=root) for i, (name, raw) in enumerate(KVZ.items())}


def _close(got, want, dtype):
    """float32: every position within the common bound.  bfloat16: a router logit that is a close call in the plain
    implementation may fall the other way after 8-bit roundings, and that token (and, faintly, the later ones that attend
    to it) then differs by a whole expert; so at most one position in eight may be beyond the bound, none beyond five times
    it -- a wrong mechanism shows at every position."""
    got, want = torch.as_tensor(got, dtype=F).cpu(), torch.as_tensor(want, dtype=F).cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    if got.dim() == 1:
        got, want = got[None], want[None]
    errors = (got - want).abs().amax(-1) / want.abs().max().clamp_min(1e-30)
    bound = TOLERANCE[dtype]
    if dtype == "float32":
        return bool((errors < bound).all())
    return bool((errors < 5 * bound).all()) and int((errors >= bound).sum()) <= max(1, errors.numel() // 8)


def _rounded(t, dtype):
    return t.to(dtype).to(F)


# ----------------------------------------------------------------------------------- kernels alone

def _pools(T, G, D, Dv, page_size, device, dtype, shuffle_seed=0):
    """Fresh pools with the sequence's pages in a shuffled order: pools, page table, slot mapping, positions."""
    pages = -(-T // page_size)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(shuffle_seed)) + 1
    k_pool = torch.full((pages + 1, G, page_size, D), float("nan"), dtype=dtype, device=device)
    v_pool = torch.full((pages + 1, G, page_size, Dv), float("nan"), dtype=dtype, device=device)
    positions = torch.arange(T, dtype=torch.int32)
    mapping = (order[positions // page_size].to(torch.int32) * page_size + positions % page_size).to(torch.int32).to(device)
    return k_pool, v_pool, order.to(torch.int32)[None, :].contiguous().to(device), mapping, positions.to(device)


def _tables(dims, base, scaling, positions, device):
    """float32 cos / sin tables [positions, dims / 2] as the plain frequencies give them."""
    f, magnitude = pk.pair_frequencies(dims, base, scaling)
    angle = (torch.arange(positions, dtype=torch.float32)[:, None] * f.float()[None, :]).double()
    return ((torch.cos(angle) * magnitude).float().contiguous().to(device), (torch.sin(angle) * magnitude).float().contiguous().to(device),
            f, magnitude)


def _capped_attend(q, k, v, rot, vrot_base, temperature, scale, cap, sink, dtype, device, page_size=64, q_len=None, kernel=None,
                   eps=1e-5):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] (float64, already rounded to `dtype`) through rotate_norm_store and the
    attention kernel; the last `q_len` tokens are the step (the earlier ones are stored by a step of their own)."""
    from models_b200.kernels import ops

    T, H, D = q.shape
    G, Dv = k.shape[1], v.shape[2]
    q_len = T if q_len is None else q_len
    k_pool, v_pool, table, mapping, positions = _pools(T, G, D, Dv, page_size, device, dtype)
    cos = sin = vcos = vsin = None
    dims = 0
    if rot is not None:
        dims = rot[0]
        cos, sin, _, _ = _tables(dims, rot[1], rot[2] if len(rot) > 2 else None, T, device) if dims else (None, None, None, None)
    if vrot_base:
        vcos, vsin, _, _ = _tables(Dv, vrot_base, None, T, device)
    qd, kd, vd = (t.reshape(T, -1).to(dtype).to(device).contiguous() for t in (q, k, v))
    temp = None if temperature is None else temperature.float().to(device).contiguous()
    out = torch.empty((q_len, H * Dv), dtype=dtype, device=device)
    first = T - q_len
    if first:
        ops.rotate_norm_store(qd[:first].clone(), kd[:first], vd[:first], positions[:first], cos, sin, dims, True, True, eps, vcos, vsin,
                              Dv if vrot_base else 0, k_pool, v_pool, mapping[:first], H, G, D, Dv)
    qs = qd[first:].clone()
    ops.rotate_norm_store(qs, kd[first:], vd[first:], positions[first:], cos, sin, dims, True, True, eps, vcos, vsin,
                          Dv if vrot_base else 0, k_pool, v_pool, mapping[first:], H, G, D, Dv)
    cu_q = torch.tensor([0, q_len], dtype=torch.int32, device=device)
    kv_lens = torch.tensor([T], dtype=torch.int32, device=device)
    ops.gated_attention(qs, out, k_pool, v_pool, table, cu_q, kv_lens, q_len, H, G, D, Dv, "softmax", scale, head_scale=temp,
                        softcap=cap or 0.0, sink=sink, turn_cos=vcos, turn_sin=vsin, kernel=kernel)
    return out.double().cpu().reshape(q_len, H, Dv)


def _plain_capped_attend(q, k, v, rot, vrot_base, temperature, scale, cap, sink, eps=1e-5):
    T, H, D = q.shape
    G, Dv = k.shape[1], v.shape[2]
    positions = torch.arange(T, dtype=F)
    if rot is not None and rot[0]:
        f, magnitude = pk.pair_frequencies(rot[0], rot[1], rot[2] if len(rot) > 2 else None)
        q, k = pk.rotate_interleaved(q, positions, f, magnitude, torch.float32), pk.rotate_interleaved(k, positions, f, magnitude, torch.float32)
    q, k = pk.rms_norm(q, None, eps), pk.rms_norm(k, None, eps)
    if vrot_base:
        vf, _ = pk.pair_frequencies(Dv, vrot_base)
        v = pk.rotate_interleaved(v, positions, vf, 1.0, torch.float32)
    heads = []
    for h in range(H):
        g = h // (H // G)
        s = pk.capped_scores(q[:, h], k[:, g], scale, 1.0 if temperature is None else temperature[h], cap)
        if sink:
            p = pk.sink_softmax(s)
        else:
            p = torch.softmax(s.masked_fill(~torch.ones(T, T, dtype=torch.bool).tril(), -math.inf), dim=-1)
        heads.append(p @ v[:, g])
    o = torch.stack(heads, dim=1)
    if vrot_base:
        o = pk.rotate_interleaved(o, -positions, vf, 1.0, torch.float32)
    return o


KERNEL_TOLERANCE = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot,page", [
    (1, 1, 8, 8, None, 32), (6, 2, 20, 12, (10, 3000.0, (2.0, 32, 8.0, 2.0)), 64), (3, 3, 40, 72, (40, 50.0), 128),
    (4, 1, 64, 128, (32, 1e5, (4.0, 128, 16.0, 1.0)), 64), (2, 2, 18, 14, (0, 100.0), 64), (8, 4, 32, 160, (16, 1e4), 64)])
def test_capped_attention_sizes_rotation_cap_sink_in_every_form(cuda_device, heads, kv_heads, dim, vdim, rot, page, dtype):
    """Random heads: a whole prompt (the tensor-core form where it applies, and the form with a warp per row), a prompt's last
    portion, and one decoded token (keys cut into runs), with pages in a shuffled order."""
    g = torch.Generator().manual_seed(heads * 100 + dim)
    T = 203
    q, k, v = (_rounded(torch.randn(T, h, d, generator=g, dtype=F), dtype) for h, d in ((heads, dim), (kv_heads, dim), (kv_heads, vdim)))
    temperature = torch.rand(heads, generator=g, dtype=F) + 0.5
    base = rot[1] if rot is not None else 0.0
    for cap, sink in ((4.0, True), (None, False), (40.0, True)):
        want = _plain_capped_attend(q, k, v, rot, base, temperature, 0.3, cap, sink)
        scale = float(want.abs().max())
        for q_len, kernel in ((T, None), (T, "rows"), (75, None), (2, None), (1, None)):
            got = _capped_attend(q, k, v, rot, base, temperature, 0.3, cap, sink, dtype, cuda_device, page, q_len, kernel)
            assert float((got - want[T - q_len:]).abs().max()) / scale < KERNEL_TOLERANCE[dtype], (cap, sink, q_len, kernel)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,target", [(700, 3), (700, 0), (130, 63), (130, 64), (65, 64), (321, 255), (40, 39)])
def test_one_far_key_decides_and_the_sink_takes_the_rest(cuda_device, tokens, target, dtype):
    """Every key is orthogonal to the query except key `target`, whose score is large: the result is that key's value
    (turned back to the distance between the two positions) times exp(s) / (1 + (n - 1) + exp(s)) -- the sink and the
    other keys weigh 1 each.  Without the sink the denominator is one less.  Prompt and decoded token."""
    D, Dv = 16, 8
    q = torch.zeros(tokens, 1, D, dtype=F)
    k = torch.zeros(tokens, 1, D, dtype=F)
    q[:, 0, 0] = 1.0
    k[:, 0, 1] = 1.0
    k[target, 0, 0], k[target, 0, 1] = 1.0, 0.0
    g = torch.Generator().manual_seed(tokens + target)
    v = _rounded(torch.randn(tokens, 1, Dv, generator=g, dtype=F), dtype)
    # unit norm makes q.k = D for the target and 0 for the others; scale 0.5 -> score 8, cap 6 -> 6 tanh(8/6)
    for sink in (True, False):
        want = _plain_capped_attend(q, k, v, None, 77.0, None, 0.5, 6.0, sink)
        s = 6.0 * math.tanh(8.0 / 6.0)
        n = tokens  # the last query sees all keys
        share = math.exp(s) / ((1.0 if sink else 0.0) + (n - 1) + math.exp(s)) if target < tokens else 0.0
        assert want[-1, 0].norm() > 0.5 * share * v[target, 0].norm()  # the plain result is indeed that key's value, mostly
        for q_len in (tokens, 1):
            got = _capped_attend(q, k, v, None, 77.0, None, 0.5, 6.0, sink, dtype, cuda_device, 64, q_len)
            assert float((got[-1] - want[-1]).abs().max()) / float(want[-1].abs().max()) < KERNEL_TOLERANCE[dtype], (sink, q_len)
    # and the sink alone: with every score at -cap the weights are tiny and the result nearly vanishes
    q2 = q.clone()
    q2[:, 0, 0] = -1.0
    k2 = torch.zeros_like(k)
    k2[:, 0, 0] = 1.0
    with_sink = _capped_attend(q2, k2, v, None, 0.0, None, 0.5, 6.0, True, dtype, cuda_device, 64, 1)
    without = _capped_attend(q2, k2, v, None, 0.0, None, 0.5, 6.0, False, dtype, cuda_device, 64, 1)
    mean = v[:, 0].mean(0)
    weight = tokens * math.exp(-s) / (1.0 + tokens * math.exp(-s))
    assert float((with_sink[0, 0] - weight * mean).abs().max()) < 2e-2 * float(mean.abs().max()) + 1e-4
    assert float((without[0, 0] - mean).abs().max()) < 2e-2 * float(mean.abs().max()) + 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotated_values_come_back_by_the_distance(cuda_device, dtype):
    """A query that sees one key only (its own, by a huge score): the value goes in rotated by j and comes out turned back by
    i = j, so the result is the value itself; and one far key: the value comes out turned by j - i."""
    D, Dv, T = 8, 12, 150
    q = torch.zeros(T, 1, D, dtype=F)
    k = torch.zeros(T, 1, D, dtype=F)
    for t in range(T):  # key t points along coordinate t % D with a sign pattern that makes only q_t . k_t large
        q[t, 0, t % D] = 1.0
        k[t, 0, t % D] = 1.0 if t % (2 * D) < D else -1.0
        q[t, 0, t % D] = k[t, 0, t % D]
    g = torch.Generator().manual_seed(3)
    v = _rounded(torch.randn(T, 1, Dv, generator=g, dtype=F), dtype)
    want = _plain_capped_attend(q, k, v, None, 20.0, None, 4.0, None, False)
    for q_len in (T, 1):
        got = _capped_attend(q, k, v, None, 20.0, None, 4.0, None, False, dtype, cuda_device, 64, q_len)
        assert float((got - want[T - q_len:]).abs().max()) / float(want.abs().max()) < KERNEL_TOLERANCE[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("streams,width,tokens", [(1, 50, 3), (2, 256, 70), (3, 64, 1), (8, 72, 33)])
def test_reading_and_writing_the_streams(cuda_device, streams, width, tokens, dtype):
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(streams * 7 + width)
    x = torch.randn(tokens, streams, width, generator=g, dtype=F)
    read, out = torch.randn(streams, generator=g, dtype=F), torch.randn(streams, generator=g, dtype=F)
    mix = torch.randn(streams, streams, generator=g, dtype=F)
    gain = 1.0 + 0.1 * torch.randn(width, generator=g, dtype=F)
    y = _rounded(torch.randn(tokens, width, generator=g, dtype=F), dtype)
    dev = lambda t: t.float().contiguous().to(cuda_device)  # noqa: E731
    xd = dev(x.reshape(tokens, streams * width))
    u = torch.einsum("s,tsd->td", read, x.float().double())
    got = ops.hyper_read_norm(xd, dev(read), dev(gain), 1e-5, dtype)
    assert scaled_error(got, pk.rms_norm(u, gain, 1e-5)) < KERNEL_TOLERANCE[dtype]
    wide = torch.zeros(tokens, width + 8, dtype=dtype, device=cuda_device)
    wide[:, 8:] = y.to(dtype).to(cuda_device)
    ops.hyper_write(xd, wide[:, 8:], dev(out), dev(mix))
    want = torch.einsum("sr,tsd->trd", mix.float().double(), x.float().double()) + out.float().double()[None, :, None] * y[:, None, :]
    assert scaled_error(xd.reshape(tokens, streams, width), want) < 2e-6
    assert scaled_error(ops.stream_sum(xd, width), want.sum(1)) < 2e-6
    copies = ops.stream_copies(dev(y), streams).reshape(tokens, streams, width)
    assert all(torch.equal(copies[:, s], dev(y)) for s in range(streams))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,width,ff,tokens", [(6, 2, 64, 40, 1), (12, 4, 256, 80, 300), (3, 3, 50, 33, 77), (5, 1, 72, 36, 130),
                                                         (40, 8, 128, 64, 9)])
def test_routed_experts(cuda_device, experts, top, width, ff, tokens, dtype):
    """Router choices (ties to the lower index), the softmax over the chosen logits, the grouped products with few and many
    rows per expert (experts nobody chose among them), the clamps, and the shared expert behind its gate."""
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(experts * 10 + top)
    x = _rounded(torch.randn(tokens, width, generator=g, dtype=F), dtype)
    router = _rounded(torch.randn(experts, width, generator=g, dtype=F) * 0.3, dtype)
    if experts > 3:
        router[experts - 1] = router[1]  # a tie: the lower index is chosen first
        router[2] = -3.0 * x[0] if tokens > 1 else router[2]  # an expert the first token never picks
    names = {}
    for e in range(experts):
        names[f"e{e}.gate"], names[f"e{e}.up"] = (_rounded(torch.randn(ff, width, generator=g, dtype=F) * 0.4, dtype) for _ in range(2))
        names[f"e{e}.down"] = _rounded(torch.randn(width, ff, generator=g, dtype=F) * 0.2, dtype)
    names["router"] = router
    dev = lambda t: t.to(dtype).contiguous().to(cuda_device)  # noqa: E731
    xd = dev(x)
    chosen, weights = ops.router_topk(xd, dev(router), top)
    want_chosen, want_weights = pk.route(x, router, top)
    assert torch.equal(chosen.cpu().long(), want_chosen)
    assert scaled_error(weights, want_weights) < 1e-5
    limit = 0.8
    plan = ops.route_sort(chosen, experts)
    stack = lambda role: dev(torch.stack([names[f"e{e}.{role}"] for e in range(experts)]))  # noqa: E731
    for tensor_cores in (True, False):
        mid = ops.expert_first_product(xd, stack("gate"), stack("up"), plan, limit, pk.SWISH_SLOPE, tensor_cores)
        slot_out = ops.expert_second_product(mid, stack("down"), plan, tensor_cores)
        got = ops.expert_combine(slot_out, weights)
        mlp = {"router": {"experts": experts, "top": top}, "expert": {"limit": limit}}
        want = pk.routed_feed_forward(x, names, "", mlp)
        assert scaled_error(got, want) < KERNEL_TOLERANCE[dtype], tensor_cores
    shared = torch.randn(tokens, width, generator=g, dtype=F)
    score = _rounded(torch.randn(tokens, 1, generator=g, dtype=F), dtype)
    got = ops.expert_combine(slot_out, weights, shared.float().contiguous().to(cuda_device), dev(score))
    assert scaled_error(got, want + pk.sigmoid(score) * shared.float().double()) < KERNEL_TOLERANCE[dtype]
    gate, up = (_rounded(torch.randn(tokens, ff, generator=g, dtype=F) * 2, dtype) for _ in range(2))
    both = dev(torch.cat([gate, up], dim=1))
    out = torch.empty((tokens, ff), dtype=dtype, device=cuda_device)
    ops.clamped_swish(both[:, :ff], both[:, ff:], out, limit, pk.SWISH_SLOPE)
    gl, ul = torch.clamp(gate, max=limit), torch.clamp(up, -limit, limit)
    assert scaled_error(out, gl * pk.sigmoid(pk.SWISH_SLOPE * gl) * (ul + 1.0)) < KERNEL_TOLERANCE[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("run_length", [0, 16, 7])
@pytest.mark.parametrize("heads,dim,vdim,decay", [(2, 16, 24, [0.9, 0.999]), (1, 32, 32, [1.0]), (3, 10, 6, [0.5, 0.0, 0.99]),
                                                  (4, 64, 128, [0.97, 0.99, 0.999, 0.9])])
def test_lightning_ragged_and_carried(cuda_device, heads, dim, vdim, decay, run_length, dtype):
    """The retention kernel in its lightning form (silu on q, k, v; raw results; one norm over all heads; sigmoid gate): three
    sequences of unequal lengths in one step, the second continuing from a stored state."""
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(heads + dim)
    lengths = [37, 1, 90]
    T = sum(lengths)
    W = heads * (2 * dim + 2 * vdim)
    proj = _rounded(torch.randn(T, W, generator=g, dtype=F), dtype)
    gain = 1.0 + 0.1 * torch.randn(heads * vdim, generator=g, dtype=F)
    start = torch.randn(heads, dim, vdim, generator=g, dtype=F).float().double()
    at = [0, heads * dim, 2 * heads * dim, 2 * heads * dim + heads * vdim]
    pd = proj.to(dtype).contiguous().to(cuda_device)
    q, k = pd[:, at[0]:at[1]], pd[:, at[1]:at[2]]
    v, gate = pd[:, at[2]:at[3]], pd[:, at[3]:]
    state = torch.zeros(5, heads, dim, vdim, dtype=torch.float32, device=cuda_device)
    state[3] = start.float().to(cuda_device)
    slots = torch.tensor([1, 3, 0], dtype=torch.int32, device=cuda_device)
    cu = torch.tensor([0, 37, 38, 128], dtype=torch.int32, device=cuda_device)
    positions = torch.cat([torch.arange(n) for n in lengths]).to(torch.int32).to(cuda_device)
    raw = torch.empty(T, heads * vdim, dtype=torch.float32, device=cuda_device)
    out = torch.empty(T, heads * vdim, dtype=dtype, device=cuda_device)
    ops.retention_scan(q, k, v, None, positions, None, None, 0, torch.tensor(decay, dtype=torch.float32, device=cuda_device), 1.0, 1e-5,
                       state, slots, cu, heads, dim, vdim, None, 1.0, max(lengths), run_length=run_length, input_activation="silu",
                       raw_out=raw)
    ops.group_norm_gate(raw, gain.float().to(cuda_device), gate, out, 1e-5, "sigmoid")
    row = 0
    for n, slot, begin in zip(lengths, (1, 3, 0), (None, start, None)):
        part = proj[row:row + n]
        qs, ks = (pk.silu(part[:, a:b]).reshape(n, heads, dim) for a, b in ((at[0], at[1]), (at[1], at[2])))
        vs = pk.silu(part[:, at[2]:at[3]]).reshape(n, heads, vdim)
        heads_out, finals = zip(*[pk.lightning_recurrence(qs[:, h], ks[:, h], vs[:, h], decay[h], None if begin is None else begin[h])
                                  for h in range(heads)])
        o = torch.stack(heads_out, dim=1).reshape(n, heads * vdim)
        want = pk.rms_norm(o, gain, 1e-5) * pk.sigmoid(part[:, at[3]:])
        assert scaled_error(out[row:row + n], want) < KERNEL_TOLERANCE[dtype], slot
        assert scaled_error(state[slot], torch.stack(finals)) < 2e-5, slot
        row += n
