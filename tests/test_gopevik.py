"""The Gopevik decoder: its mechanisms one by one against `plain_gopevik`, then whole models through the
engine's step function, scheduler and entry points.  The plain implementation shares nothing with the
package; it runs in float64 on bfloat16-rounded random weights."""
import ctypes
import math
import os

import pytest
import torch

import gopevik_models
import plain_gopevik as plain
from helpers import assert_close, assert_rows_close, engine_model, run_portions, run_whole, write_model_folder

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# bfloat16 rows against the float64 plain implementation (relative RMSE, relative largest difference, cosine):
# a factor of two above the worst rows these models measure (0.089 / 0.24 / 0.9961: with a few values per norm
# group and heads of 8 a single rounding weighs far more than in a wide model).  A wrong key, a lost state or a
# missing sink moves a row by its whole size; the float32 runs of the same tests are the sharp ones.
BF16 = dict(rmse=0.18, max=0.5, cosine=0.992)


def tokens_for(config, count, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, config["vocab"], (count,), generator=g).tolist()


def plain_logits(config, weights, tokens):
    return plain.forward(config, weights, tokens, torch.float64).float()


# ----------------------------------------------------------------------------- without a GPU
def test_config_and_plan_name_every_tensor():
    from mini_llm_runtime_b200 import models  # noqa: F401
    from mini_llm_runtime_b200.config.registry import config_from_dict, plan_for
    from mini_llm_runtime_b200.engine.structure import expected_weights
    for name in gopevik_models.ALL:
        config = gopevik_models.get(name)
        weights = gopevik_models.random_weights(config, 1)
        expected = expected_weights(plan_for(config_from_dict(config)))
        assert set(expected) == set(weights)
        for key, spec in expected.items():
            assert tuple(spec.shape) == tuple(weights[key].shape), key


@pytest.mark.parametrize("path,value,message", [
    (("width",), None, "width"),
    (("norm", "groups"), 5, "equal parts"),
    (("layers", 0, "type"), "moe", "parallel"),
    (("layers", 1, "mixer", "left", "kv_heads"), 3, "share"),
    (("layers", 1, "mixer", "right", "decay"), [0.5], "decay"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 30, "dims"),
    (("layers", 0, "mlp", "kind"), "experts", "dense"),
])
def test_config_errors_name_the_key(path, value, message):
    from mini_llm_runtime_b200 import models  # noqa: F401
    from mini_llm_runtime_b200.config.base import ConfigError
    from mini_llm_runtime_b200.config.registry import config_from_dict
    config = gopevik_models.get("small_a")
    at = config
    for key in path[:-1]:
        at = at[key]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError, match=message):
        config_from_dict(config)


def test_plain_retention_is_the_weighted_sum_of_outer_products():
    g = torch.Generator().manual_seed(5)
    T, H, D, Dv = 9, 2, 4, 3
    q, k, v = (torch.randn(T, H, n, generator=g, dtype=torch.float64) for n in (D, D, Dv))
    decay = [0.5, 0.9]
    out, _ = plain.retention(q, k, v, decay)
    for h in range(H):
        for t in range(T):
            want = sum(decay[h] ** (t - j) * (q[t, h] @ k[j, h]) * v[j, h] for j in range(t + 1))
            assert torch.allclose(out[t, h], want, atol=1e-12)


def test_plain_delta_rule_stores_and_recalls_a_pair():
    # With g = 1 and beta = 1, writing (k, v) and asking with q = k returns v (k a unit vector).
    k = torch.tensor([[[0.6, 0.8]]], dtype=torch.float64)
    v = torch.tensor([[[2.0, -1.0, 0.5]]], dtype=torch.float64)
    out = plain.gated_delta_rule(k, k, v, torch.ones(1, 1, dtype=torch.float64), torch.ones(1, 1, dtype=torch.float64))
    assert torch.allclose(out[0, 0], v[0, 0])


def test_plain_sink_takes_the_weight_when_every_score_is_low():
    q = torch.full((1, 1, 2), 10.0, dtype=torch.float64)
    k = torch.full((1, 1, 2), -10.0, dtype=torch.float64)
    v = torch.ones(1, 1, 3, dtype=torch.float64)
    out = plain.chunk_sink_attention(q, k, v, torch.arange(1), 1.0, None)
    assert out.abs().max() < 1e-40


# ----------------------------------------------------------------------------- kernels alone
def _call(module, fn, *args):
    from mini_llm_runtime_b200.ops import native
    native.call(module, fn, *args)
    torch.cuda.synchronize()


def _meta(segments, device):
    """segments: (first row, count, start position, slot) -> positions, segment_of_row, segment_info on the device."""
    positions, of_row = [], []
    for i, (first, count, start, slot) in enumerate(segments):
        positions += list(range(start, start + count))
        of_row += [i] * count
    as_int = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
    return as_int(positions), as_int(of_row), as_int(segments).reshape(-1, 4)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,groups", [(48, 3), (64, 1), (40, 40), (6000, 4)])
def test_grouped_norm_kernel(dtype, width, groups):
    from mini_llm_runtime_b200.ops import native
    dev = "cuda:0"
    g = torch.Generator().manual_seed(width)
    rows = 5
    h = torch.randn(rows, width, generator=g).to(dev)
    delta = (torch.randn(rows, width, generator=g) * 3).to(dev)
    bias, w_post, w_pre = (torch.randn(width, generator=g).to(dev) for _ in range(3))
    out = torch.empty(rows, width, dtype=dtype, device=dev)
    h0 = h.clone()
    _call("norm_grouped", "mlr_group_rmsnorm", h.data_ptr(), delta.data_ptr(), width, bias.data_ptr(), w_post.data_ptr(),
          w_pre.data_ptr(), out.data_ptr(), width, native.is_bf16(out), None, rows, width, groups, 1e-5, 1, native.stream())
    want_h = h0.double().cpu() + plain.group_rms_norm((delta + bias).double().cpu(), w_post.double().cpu(), groups, 1e-5)
    want = plain.group_rms_norm(want_h, w_pre.double().cpu(), groups, 1e-5)
    assert torch.allclose(h.cpu().double(), want_h, atol=1e-5, rtol=1e-5)
    tol = 1e-5 if dtype is torch.float32 else 2e-2
    assert torch.allclose(out.float().cpu().double(), want, atol=tol, rtol=tol)
    # Only chosen rows, nothing added: the stream stays as it is.
    index = torch.tensor([3, 0], dtype=torch.int32, device=dev)
    some = torch.empty(2, width, dtype=dtype, device=dev)
    before = h.clone()
    _call("norm_grouped", "mlr_group_rmsnorm", h.data_ptr(), None, 0, None, None, w_pre.data_ptr(), some.data_ptr(), width,
          native.is_bf16(some), index.data_ptr(), 2, width, groups, 1e-5, 0, native.stream())
    assert torch.equal(h, before)
    assert torch.allclose(some.float().cpu().double(), want[[3, 0]], atol=tol, rtol=tol)


@pytest.mark.gpu
@pytest.mark.parametrize("activation", [0, 1])
@pytest.mark.parametrize("inter", [37, 40, 1024])
def test_gated_bias_kernel(activation, inter):
    from mini_llm_runtime_b200.ops import native
    dev = "cuda:0"
    g = torch.Generator().manual_seed(3)
    rows = 7
    both = torch.randn(rows, 2 * inter, generator=g).to(dev)
    bg, bu = torch.randn(inter, generator=g).to(dev), torch.randn(inter, generator=g).to(dev)
    out = torch.empty(rows, inter, device=dev)
    _call("elementwise", "mlr_gated_bias", both.data_ptr(), 2 * inter, bg.data_ptr(), bu.data_ptr(), out.data_ptr(), inter, 0, rows,
          inter, activation, native.stream())
    z = (both[:, :inter] + bg).double().cpu()
    up = (both[:, inter:] + bu).double().cpu()
    act = plain.silu(z) if activation == 0 else 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
    assert torch.allclose(out.cpu().double(), act * up, atol=1e-5, rtol=1e-5)


def _attention_case(dtype, heads, kv_heads, dim, vdim, rot_dims, factor, chunk, window, sink, gate, T, page, boost=None, seed=0, tiled=0, split=None):
    """One request of T tokens written into a paged cache with shuffled pages, then every row's attention."""
    from mini_llm_runtime_b200.ops import native
    from mini_llm_runtime_b200.ops.specs import GATES, MaskedAttentionSpec
    dev = "cuda:0"
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, heads * dim, generator=g)
    k = torch.randn(T, kv_heads * dim, generator=g)
    v = torch.randn(T, kv_heads * vdim, generator=g)
    gates = torch.randn(T, heads * vdim, generator=g)
    if boost is not None:           # one far key whose score stands out for the last query, if it is seen at all
        j = boost
        k[j] = 0
        k[j, :dim][rot_dims:] = 6.0
        q[T - 1] = 0
        q[T - 1].view(heads, dim)[:, rot_dims:] = 6.0
    q, k, v, gates = (x.to(dtype).to(dev) for x in (q, k, v, gates))
    base = 300.0
    freq = torch.tensor([base ** (-2.0 * i / max(rot_dims, 1)) / factor for i in range(rot_dims // 2)], dtype=torch.float32, device=dev)
    spec = MaskedAttentionSpec(freq=freq.data_ptr() if rot_dims else None, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim,
                               rot_dims=rot_dims, window=window or 0, chunk=chunk or 0, sink=int(sink), gate_kind=GATES[gate],
                               scale=0.2, out_scale=0.75)
    n_pages = (T + page - 1) // page + 3
    order = torch.randperm(n_pages, generator=g)[:(T + page - 1) // page].to(torch.int32)
    table = order.reshape(1, -1).to(dev)
    cache = torch.full((n_pages, kv_heads * page * (dim + vdim)), float("nan"), dtype=dtype, device=dev)
    positions, of_row, _ = _meta([(0, T, 0, 0)], dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    is16 = native.is_bf16(q)
    _call("attention_masked", "mlr_kv_rope_cache", ctypes.addressof(spec), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), is16,
          cache.data_ptr(), n_pages, positions.data_ptr(), of_row.data_ptr(), table.data_ptr(), table.stride(0), page, T,
          status.data_ptr(), native.stream())
    out = torch.full((T, heads * vdim), float("nan"), dtype=dtype, device=dev)
    common = (ctypes.addressof(spec), q.data_ptr(), q.stride(0), gates.data_ptr() if gate else None, gates.stride(0) if gate else 0,
              out.data_ptr(), out.stride(0))
    if tiled:       # the request's rows in two steps' worth of tiles: a first portion of `tiled` rows, then the rest
        info = torch.tensor([[0, tiled, 0, 0], [tiled, T - tiled, tiled, 0]], dtype=torch.int32, device=dev)
        tiles = [(0, t) for t in range(0, tiled, 64)] + [(1, t) for t in range(0, T - tiled, 64)]
        tiles = torch.tensor(tiles, dtype=torch.int32, device=dev)
        two = torch.cat([table, table]).contiguous()
        _call("attention_masked", "mlr_attention_masked_tiles", *common, cache.data_ptr(), n_pages, tiles.data_ptr(), tiles.shape[0],
              info.data_ptr(), two.data_ptr(), two.stride(0), page, status.data_ptr(), native.stream())
    elif split:     # the last rows as a segment of few rows, its keys cut into ranges that are added up afterwards
        last, keys, most = split[:3]
        finer = split[3] if len(split) > 3 else 1
        info = torch.tensor([[T - last, last, T - last, 0]], dtype=torch.int32, device=dev)
        partial = torch.full((16 * kv_heads * most * finer * (vdim + 2),), float("nan"), device=dev)
        _call("attention_masked", "mlr_attention_masked", *common, is16, cache.data_ptr(), n_pages, positions.data_ptr(),
              of_row.data_ptr(), table.data_ptr(), table.stride(0), page, 0, None, 1, info.data_ptr(), keys, most, finer, partial.data_ptr(),
              status.data_ptr(), native.stream())
    else:
        _call("attention_masked", "mlr_attention_masked", *common, is16, cache.data_ptr(), n_pages, positions.data_ptr(),
              of_row.data_ptr(), table.data_ptr(), table.stride(0), page, T, None, 0, None, 0, 1, 1, None, status.data_ptr(), native.stream())
    assert int(status.item()) == 0
    pos = torch.arange(T)
    qd = plain.rotate_half(q.double().cpu().view(T, heads, dim), pos, rot_dims, base, factor) if rot_dims else q.double().cpu().view(T, heads, dim)
    kd = plain.rotate_half(k.double().cpu().view(T, kv_heads, dim), pos, rot_dims, base, factor) if rot_dims else k.double().cpu().view(T, kv_heads, dim)
    if dtype is torch.bfloat16:
        kd = kd.bfloat16().double()          # the cache holds the rotated keys in the activations' precision
    vd = v.double().cpu().view(T, kv_heads, vdim)
    if sink:
        want = plain.chunk_sink_attention(qd, kd, vd, pos, 0.2, chunk)
    else:
        want = torch.zeros(T, heads, vdim, dtype=torch.float64)
        for h in range(heads):
            s = (qd[:, h] @ kd[:, h // (heads // kv_heads)].T) * 0.2
            seen = pos[None, :] <= pos[:, None]
            if chunk:
                seen &= pos[None, :] // chunk == pos[:, None] // chunk
            want[:, h] = torch.softmax(s.masked_fill(~seen, -math.inf), dim=-1) @ vd[:, h // (heads // kv_heads)]
    if window:
        assert not chunk and not sink
        for h in range(heads):
            s = (qd[:, h] @ kd[:, h // (heads // kv_heads)].T) * 0.2
            seen = (pos[None, :] <= pos[:, None]) & (pos[None, :] > pos[:, None] - window)
            want[:, h] = torch.softmax(s.masked_fill(~seen, -math.inf), dim=-1) @ vd[:, h // (heads // kv_heads)]
    want = want.reshape(T, heads * vdim)
    if gate:
        gd = gates.double().cpu()
        want = want * (torch.sigmoid(gd) if gate == "sigmoid" else plain.silu(gd))
    if split:
        return out[T - split[0]:].float().cpu().double(), want[T - split[0]:] * 0.75
    return out.float().cpu().double(), want * 0.75


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [
    dict(heads=4, kv_heads=2, dim=24, vdim=16, rot_dims=8, factor=1.0, chunk=24, window=None, sink=True, gate="sigmoid", T=100, page=16),
    dict(heads=3, kv_heads=3, dim=8, vdim=40, rot_dims=8, factor=4.0, chunk=10, window=None, sink=True, gate=None, T=70, page=4),
    dict(heads=2, kv_heads=1, dim=20, vdim=12, rot_dims=0, factor=1.0, chunk=None, window=None, sink=False, gate="silu", T=150, page=16),
    dict(heads=2, kv_heads=2, dim=16, vdim=16, rot_dims=16, factor=1.0, chunk=None, window=33, sink=False, gate=None, T=90, page=8),
    dict(heads=1, kv_heads=1, dim=130, vdim=200, rot_dims=64, factor=2.0, chunk=64, window=None, sink=True, gate="sigmoid", T=200, page=16),
])
def test_masked_attention_kernel(dtype, case):
    got, want = _attention_case(dtype, **case)
    tol = 2e-5 if dtype is torch.float32 else 3e-2
    assert torch.allclose(got, want, atol=tol, rtol=tol), float((got - want).abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("case", [
    dict(heads=4, kv_heads=2, dim=32, vdim=16, rot_dims=8, factor=1.0, chunk=24, window=None, sink=True, gate="sigmoid", T=200, page=16, tiled=70),
    dict(heads=3, kv_heads=3, dim=16, vdim=40, rot_dims=16, factor=4.0, chunk=100, window=None, sink=True, gate=None, T=333, page=4, tiled=1),
    dict(heads=2, kv_heads=1, dim=96, vdim=96, rot_dims=0, factor=1.0, chunk=None, window=None, sink=False, gate="silu", T=150, page=16, tiled=64),
    dict(heads=2, kv_heads=2, dim=16, vdim=8, rot_dims=16, factor=1.0, chunk=None, window=33, sink=False, gate=None, T=190, page=8, tiled=129),
    dict(heads=1, kv_heads=1, dim=128, vdim=128, rot_dims=64, factor=2.0, chunk=64, window=None, sink=True, gate="sigmoid", T=260, page=16, tiled=100),
    dict(heads=1, kv_heads=1, dim=256, vdim=104, rot_dims=2, factor=1.0, chunk=130, window=None, sink=True, gate=None, T=270, page=16, tiled=5),
])
def test_masked_attention_in_tiles_on_the_tensor_cores(case):
    """Prompt portions in bfloat16: tiles of 64 rows of two portions of one request, the second continuing the first."""
    got, want = _attention_case(torch.bfloat16, **case)
    assert torch.allclose(got, want, atol=3e-2, rtol=3e-2), float((got - want).abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [
    dict(heads=4, kv_heads=2, dim=24, vdim=16, rot_dims=8, factor=1.0, chunk=None, window=None, sink=True, gate="sigmoid", T=700, page=16, split=(5, 128, 6)),
    dict(heads=2, kv_heads=2, dim=16, vdim=40, rot_dims=16, factor=2.0, chunk=300, window=None, sink=True, gate=None, T=650, page=8, split=(8, 64, 11)),
    dict(heads=3, kv_heads=1, dim=8, vdim=8, rot_dims=0, factor=1.0, chunk=None, window=None, sink=False, gate="silu", T=333, page=16, split=(1, 192, 2)),
    dict(heads=1, kv_heads=1, dim=32, vdim=200, rot_dims=4, factor=1.0, chunk=100, window=None, sink=True, gate=None, T=402, page=16, split=(16, 64, 7)),
    dict(heads=2, kv_heads=1, dim=16, vdim=24, rot_dims=8, factor=1.0, chunk=None, window=None, sink=True, gate="sigmoid", T=1500, page=16, split=(3, 512, 3, 4)),
    dict(heads=2, kv_heads=2, dim=8, vdim=8, rot_dims=0, factor=1.0, chunk=900, window=None, sink=False, gate=None, T=1000, page=16, split=(2, 384, 3, 4)),
])
def test_masked_attention_with_the_keys_cut_into_ranges(dtype, case):
    got, want = _attention_case(dtype, **case)
    tol = 2e-5 if dtype is torch.float32 else 3e-2
    assert torch.allclose(got, want, atol=tol, rtol=tol), float((got - want).abs().max())


@pytest.mark.gpu
def test_a_loud_key_at_the_chunk_border_in_tiles():
    for chunk, T in ((64, 200), (50, 230)):
        start = (T - 1) // chunk * chunk
        for key in (start, start - 1):
            got, want = _attention_case(torch.bfloat16, heads=2, kv_heads=1, dim=16, vdim=8, rot_dims=4, factor=1.0, chunk=chunk, window=None,
                                        sink=True, gate=None, T=T, page=16, boost=key, seed=key, tiled=T - 3)
            assert torch.allclose(got, want, atol=3e-2, rtol=3e-2), (chunk, key, float((got - want).abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("chunk,T", [(32, 100), (50, 230), (7, 67)])
def test_a_loud_key_just_inside_and_just_outside_the_chunk(chunk, T):
    """The last query's score with one chosen key stands far above all others: the result is that key's value if
    the key is the first of the query's chunk, and shows no trace of it if it is the last of the chunk before."""
    start = (T - 1) // chunk * chunk
    assert 0 < start < T - 1
    for key, inside in ((start, True), (start - 1, False), (0, False)):
        got, want = _attention_case(torch.float32, heads=2, kv_heads=1, dim=16, vdim=8, rot_dims=4, factor=1.0, chunk=chunk,
                                    window=None, sink=True, gate=None, T=T, page=16, boost=key, seed=key)
        assert torch.allclose(got, want, atol=2e-5, rtol=2e-5), (key, float((got - want).abs().max()))


def _recurrence_case(dtype, rule, heads, qk_heads, dim, vdim, rot_dims, segments, slots=4, taps=0, seed=0, weight=True, gate="silu", split=False):
    """`segments`: token counts of requests that share one launch; each request then runs a second step
    of 1 token (its state carried in its slot).  Returns engine and plain outputs for all rows of both steps."""
    from mini_llm_runtime_b200.ops import native
    from mini_llm_runtime_b200.ops.specs import GATES, RecurrenceSpec
    dev = "cuda:0"
    g = torch.Generator().manual_seed(seed)
    cq, ck, cv = 0, qk_heads * dim, 2 * qk_heads * dim
    cg = cv + heads * vdim
    cb, ca = cg + heads * vdim, cg + heads * vdim + heads
    width = ca + heads
    decay = (0.8 + 0.199 * torch.rand(heads, generator=g)).to(dev)
    a_log, dt_bias = torch.randn(heads, generator=g).to(dev), torch.randn(heads, generator=g).to(dev)
    out_w = (1 + 0.2 * torch.randn(vdim, generator=g)).to(dev)
    freq = torch.tensor([70.0 ** (-2.0 * i / max(rot_dims, 1)) for i in range(rot_dims // 2)], dtype=torch.float32, device=dev)
    spec = RecurrenceSpec(freq=freq.data_ptr() if rot_dims else None, decay=decay.data_ptr(), a_log=a_log.data_ptr(),
                          dt_bias=dt_bias.data_ptr(), out_weight=out_w.data_ptr() if weight else None, heads=heads, qk_heads=qk_heads,
                          dim=dim, vdim=vdim, prep=RecurrenceSpec.PREP["rotate" if rule == "decay" and rot_dims else ("unit" if rule == "delta" else None)],
                          rot_dims=rot_dims, rule=RecurrenceSpec.RULE[rule], gate_kind=GATES[gate], col_q=cq, col_k=ck, col_v=cv,
                          col_a=ca, col_b=cb, col_gate=cg, q_mult=1.0 if rule == "decay" else dim ** -0.5,
                          k_mult=dim ** -0.5 if rule == "decay" else 1.0, unit_eps=1e-6, eps=1e-5, out_scale=1.25)
    per_slot = heads * vdim * dim + 5
    state = torch.zeros(slots, per_slot, device=dev)
    use_slots = torch.randperm(slots, generator=g)[:len(segments)].tolist()
    projs = [torch.randn(n + 1, width, generator=g) for n in segments]
    got = [[] for _ in segments]
    for part in (0, 1):
        rows, info, first = [], [], 0
        for i, n in enumerate(segments):
            piece = projs[i][:n] if part == 0 else projs[i][n:]
            rows.append(piece)
            info.append((first, piece.shape[0], 0 if part == 0 else n, use_slots[i]))
            first += piece.shape[0]
        proj = torch.cat(rows).to(dtype).to(dev)
        _, _, seg_info = _meta(info, dev)
        out = torch.empty(proj.shape[0], heads * vdim, dtype=dtype, device=dev)
        if split and part == 0:      # the first step in three kernels, the second (one token each) in the fused one
            rows = proj.shape[0]
            positions, _, _ = _meta(info, dev)
            qf, kf = (torch.empty(rows, qk_heads * dim, device=dev) for _ in range(2))
            gb, obuf = torch.empty(rows, 2 * heads, device=dev), torch.empty(rows, heads * vdim, device=dev)
            _call("recurrence", "mlr_linear_recurrence_split", ctypes.addressof(spec), proj.data_ptr(), proj.stride(0), proj.data_ptr(),
                  proj.stride(0), native.is_bf16(proj), out.data_ptr(), out.stride(0), state.data_ptr(), state.stride(0),
                  seg_info.data_ptr(), len(segments), positions.data_ptr(), rows, qf.data_ptr(), kf.data_ptr(), gb.data_ptr(),
                  obuf.data_ptr(), native.stream())
        else:
            _call("recurrence", "mlr_linear_recurrence", ctypes.addressof(spec), proj.data_ptr(), proj.stride(0), proj.data_ptr(),
                  proj.stride(0), native.is_bf16(proj), out.data_ptr(), out.stride(0), state.data_ptr(), state.stride(0),
                  seg_info.data_ptr(), len(segments), 0, None, None, native.stream())
        for i, (f, c, _, _) in enumerate(info):
            got[i].append(out[f:f + c].float().cpu().double())
    wants = []
    for i, n in enumerate(segments):
        p = projs[i].to(dtype).double()
        T = n + 1
        q = p[:, cq:cq + qk_heads * dim].view(T, qk_heads, dim)
        k = p[:, ck:ck + qk_heads * dim].view(T, qk_heads, dim)
        v = p[:, cv:cv + heads * vdim].view(T, heads, vdim)
        gate_in = p[:, cg:cg + heads * vdim]
        if rule == "decay":
            if rot_dims:
                q, k = (plain.rotate_half(x, torch.arange(T), rot_dims, 70.0) for x in (q, k))
            o, _ = plain.retention(q, k * dim ** -0.5, v, decay.double().cpu().tolist())
        else:
            share = heads // qk_heads
            q = (plain.unit(q) * dim ** -0.5).repeat_interleave(share, dim=1)
            k = plain.unit(k).repeat_interleave(share, dim=1)
            beta = torch.sigmoid(p[:, cb:cb + heads])
            gg = torch.exp(-torch.exp(a_log.double().cpu()) * torch.nn.functional.softplus(p[:, ca:ca + heads] + dt_bias.double().cpu()))
            o = plain.gated_delta_rule(q, k, v, gg, beta)
        o = plain.group_rms_norm(o, out_w.double().cpu() if weight else None, 1, 1e-5).reshape(T, heads * vdim)
        o = o * (plain.silu(gate_in) if gate == "silu" else torch.sigmoid(gate_in) if gate else 1.0)
        wants.append(o * 1.25)
    # the padding behind every slot's matrix stays untouched
    assert float(state[:, heads * vdim * dim:].abs().max()) == 0.0
    return [torch.cat(x) for x in got], wants


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [
    dict(rule="decay", heads=3, qk_heads=3, dim=16, vdim=24, rot_dims=16, segments=[37, 1, 70]),
    dict(rule="decay", heads=2, qk_heads=2, dim=40, vdim=8, rot_dims=0, segments=[5], weight=False),
    dict(rule="decay", heads=1, qk_heads=1, dim=130, vdim=100, rot_dims=6, segments=[33, 2], gate="sigmoid"),
    dict(rule="delta", heads=4, qk_heads=2, dim=16, vdim=8, rot_dims=0, segments=[50, 3, 1, 18]),
    dict(rule="delta", heads=2, qk_heads=2, dim=64, vdim=200, rot_dims=0, segments=[40]),
    dict(rule="delta", heads=6, qk_heads=1, dim=8, vdim=33, rot_dims=0, segments=[2, 65]),
    dict(rule="delta", heads=2, qk_heads=1, dim=96, vdim=20, rot_dims=0, segments=[70, 9]),
    dict(rule="decay", heads=2, qk_heads=2, dim=128, vdim=128, rot_dims=64, segments=[100]),
    dict(rule="decay", heads=1, qk_heads=1, dim=32, vdim=7, rot_dims=32, segments=[3, 40]),
    dict(rule="delta", heads=1, qk_heads=1, dim=256, vdim=17, rot_dims=0, segments=[35]),
])
@pytest.mark.parametrize("split", [False, True])
def test_recurrence_kernel_with_state_carried_between_steps(dtype, case, split):
    got, want = _recurrence_case(dtype, split=split, **case)
    tol = 3e-5 if dtype is torch.float32 else 4e-2
    for i, (a, b) in enumerate(zip(got, want)):
        assert torch.allclose(a, b, atol=tol, rtol=tol), (i, float((a - b).abs().max()))
    if split and case["dim"] % 32:       # prepare / scan / read-out add in the order of the one kernel: the same bits
        fused, _ = _recurrence_case(dtype, split=False, **case)
        for a, b in zip(got, fused):
            assert torch.equal(a, b)


@pytest.mark.gpu
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_short_convolution_over_steps_of_any_size(taps):
    """Two requests in slots of their own, their tokens cut into steps of 1 to 9 (shorter and longer than the
    taps): every step reads the inputs the steps before left as state."""
    from mini_llm_runtime_b200.ops import native
    dev = "cuda:0"
    g = torch.Generator().manual_seed(taps)
    channels, T = 19, 40
    weights = torch.randn(channels, taps, generator=g).to(dev)
    xs = [torch.randn(T, channels, generator=g), torch.randn(T, channels, generator=g)]
    per_slot = 7 + max(taps - 1, 0) * channels
    state = torch.zeros(3, per_slot, device=dev)
    conv_state = state.data_ptr() + 4 * 7
    slots = [2, 0]
    outs, at = [[], []], 0
    sizes = [1, 2, 1, 9, 3, 1, 1, 5, 2, 8, 7]
    for n in sizes:
        n = min(n, T - at)
        if n <= 0:
            break
        x = torch.cat([xs[0][at:at + n], xs[1][at:at + n]]).to(dev)
        _, of_row, info = _meta([(0, n, at, slots[0]), (n, n, at, slots[1])], dev)
        out = torch.empty_like(x)
        _call("recurrence", "mlr_short_conv", x.data_ptr(), channels, out.data_ptr(), channels, 0, channels, taps, weights.data_ptr(),
              conv_state, per_slot, info.data_ptr(), of_row.data_ptr(), 2 * n, native.stream())
        _call("recurrence", "mlr_short_conv_state", x.data_ptr(), channels, 0, channels, taps, conv_state, per_slot, info.data_ptr(), 2,
              native.stream())
        outs[0].append(out[:n].cpu())
        outs[1].append(out[n:].cpu())
        at += n
    for i in range(2):
        want = plain.short_conv_silu(xs[i][:at].double(), weights.double().cpu())
        assert torch.allclose(torch.cat(outs[i]).double(), want, atol=1e-5, rtol=1e-5)
    assert float(state[:, :7].abs().max()) == 0.0 and float(state[1].abs().max()) == 0.0


# ----------------------------------------------------------------------------- whole models
@pytest.fixture(scope="module", params=sorted(gopevik_models.ALL))
def case(request, tmp_path_factory):
    config = gopevik_models.get(request.param)
    weights = gopevik_models.random_weights(config, seed=11)
    folder = str(tmp_path_factory.mktemp(request.param))
    write_model_folder(folder, config, weights)
    return folder, config, weights


def close(got, want, dtype, what):
    if dtype == "bfloat16":
        assert_rows_close(got, want, what, bounds=BF16)
    else:
        assert_close(got, want, dtype, what)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_portions_and_decoding_agree_with_the_plain_implementation(case, dtype):
    folder, config, weights = case
    model = engine_model(folder, dtype, num_pages=24, page_size=8, max_requests=2)
    assert model._native is not None, "the model must run in the native step executor"
    tokens = tokens_for(config, 150, 4)
    want = plain_logits(config, weights, tokens)
    whole = run_whole(model, tokens)
    close(whole, want, dtype, "whole")
    for sizes in ([1], [2], [3, 2, 7], [64, 1], [65, 2, 70], [149, 1], [11, 2, 2, 30, 1, 5]):      # [1]: decoding from the first token on
        got = run_portions(model, tokens, sizes)
        close(got, want, dtype, f"portions {sizes}")
        if dtype == "float32":      # how a prompt is cut changes nothing but the order of a few sums
            assert float((got - whole).abs().max()) <= 2e-5, sizes
    assert model.cache.free_slots() == 2


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_batch_of_unequal_requests_equals_each_alone_and_slots_are_used_again(case, dtype):
    from mini_llm_runtime_b200.engine.model import StepEntry
    folder, config, weights = case
    model = engine_model(folder, dtype, num_pages=40, page_size=8, max_requests=3)
    lengths = [70, 9, 33, 2, 51, 20, 64]
    requests = [tokens_for(config, n, 100 + n) for n in lengths]
    alone = [plain_logits(config, weights, t) for t in requests]
    got = [[] for _ in requests]
    # Three live requests at a time; a finished one gives its slot and pages to the next.
    waiting, live = list(range(len(requests))), {}
    sizes = [5, 1, 2, 13, 1, 1, 30, 3]
    turn = 0
    while waiting or live:
        while waiting and len(live) < 3:
            live[waiting.pop(0)] = [model.open_request(), 0]
        entries, who = [], []
        for i, (slot, at) in live.items():
            if (turn + i) % 4 == 3 and len(live) > 1:
                continue                                  # this request sits the step out
            n = min(sizes[(turn + i) % len(sizes)], len(requests[i]) - at)
            entries.append(StepEntry(slot, requests[i][at:at + n], list(range(n))))
            who.append((i, n))
        if entries:
            logits = model.step(entries).float().cpu()
            row = 0
            for i, n in who:
                got[i].append(logits[row:row + n])
                row += n
                live[i][1] += n
                if live[i][1] == len(requests[i]):
                    model.close_request(live.pop(i)[0])
        turn += 1
    model.check_status()
    for i in range(len(requests)):
        close(torch.cat(got[i]), alone[i], dtype, f"request {i}")
    assert model.cache.free_slots() == 3


@pytest.mark.gpu
def test_long_decoding_through_the_graphs_keeps_the_state_right(case):
    from mini_llm_runtime_b200.engine.model import StepEntry
    folder, config, weights = case
    model = engine_model(folder, "float32", num_pages=64, page_size=8, max_requests=2)
    a, b = tokens_for(config, 260, 1), tokens_for(config, 200, 2)
    sa, sb = model.open_request(), model.open_request()
    got_a, got_b = [], []
    for t in range(len(a)):
        entries = [StepEntry(sa, [a[t]], [0])] + ([StepEntry(sb, [b[t]], [0])] if t < len(b) else [])
        logits = model.step(entries).float().cpu()
        got_a.append(logits[0])
        if t < len(b):
            got_b.append(logits[1])
    model.check_status()
    assert model._graphs, "single-token steps did not reach the CUDA graphs"
    assert_close(torch.stack(got_a), plain_logits(config, weights, a), "float32", "a")
    assert_close(torch.stack(got_b), plain_logits(config, weights, b), "float32", "b")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(case, dtype):
    from mini_llm_runtime_b200 import LLM
    folder, config, weights = case
    prompts = [tokens_for(config, n, 50 + n) for n in (3, 41, 18, 77, 1)]
    llm = LLM(folder, dtype=dtype, max_model_len=128, max_requests=3, num_pages=48, page_size=8, max_batch_tokens=24, prefill_chunk=16)
    results = llm.generate(prompts, max_tokens=12, ignore_eos=True)
    for prompt, result in zip(prompts, results):
        assert len(result.token_ids) == 12
        tokens = list(prompt)
        for step, token in enumerate(result.token_ids):
            row = plain_logits(config, weights, tokens)[-1]
            best = int(torch.argmax(row))
            if token != best:       # two logits closer than the precision's rounding may change places; nothing else may
                margin = 1e-3 if dtype == "float32" else 2 * BF16["max"] * float(row.double().pow(2).mean().sqrt())
                assert float(row[best] - row[token]) <= margin, (len(prompt), step, token, best)
            tokens.append(token)
    assert llm.model.cache.free_slots() == 3


@pytest.mark.gpu
def test_trace_replay_with_a_pool_that_is_used_again(case, tmp_path):
    """Through `bin/trace_run` as a user runs it: up to four live requests in a pool sized for them, not for all."""
    import trace_tools
    folder, config, weights = case
    requests = {f"r{i}": tokens_for(config, n, 300 + i) for i, n in enumerate((90, 5, 130, 64, 31, 17, 100))}
    trace = trace_tools.mixed(requests, seed=9)
    logits = trace_tools.run_trace(folder, "float32", trace, str(tmp_path), config["vocab"])
    for name, tokens in requests.items():
        assert_close(trace_tools.stack(logits, name, len(tokens)), plain_logits(config, weights, tokens), "float32", name)
