"""Punilix (parallel-block family) on the GPU against the plain float64 restatement in tests/punilix_plain.py.

Kernel-level tests feed one mechanism through the C ABI; engine-level tests write a small random checkpoint (uzu_b200.synth), run it
through the engine's own passes / slots / decode graph and compare logits with the oracle. Engines run in true f32 (tight bounds: a
window or state fault is orders of magnitude above them) and in the serving precisions (bf16 products).
"""
import ctypes as C
import math

import numpy as np
import pytest
import torch

from tests import punilix_plain as P
from uzu_b200 import binding as B
from uzu_b200 import synth

pytestmark = pytest.mark.gpu
F64 = torch.float64


def t64(a):
    return torch.from_numpy(np.asarray(a)).to(F64)


def run(ctx, fn, *args):
    with ctx.command_buffer(fn) as cmd:
        cmd.encode(fn, *args)


def close(got, ref, tol, what=""):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    scale = max(float(np.sqrt((ref ** 2).mean())), 1e-6)
    err = float(np.abs(got - ref).max()) / scale
    assert err <= tol, f"{what}: max error {err:.3e} of the rms exceeds {tol:.1e}"


# ---- kernels, one mechanism each ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,n,groups", [(1, 96, 1), (5, 96, 3), (33, 130, 2), (3, 7, 7)])
def test_group_rms_norm(ctx, rows, n, groups):
    rng = np.random.default_rng(rows * n)
    x = rng.standard_normal((rows, n), dtype=np.float32) * 3
    w = rng.standard_normal(n, dtype=np.float32)
    bx, bw, bo = ctx.upload(x), ctx.upload(w), ctx.upload(np.zeros_like(x))
    a = B.GroupRmsNormArgs(input=bx.ptr, scales=bw.ptr, output=bo.ptr, rows=rows, n=n, groups=groups, in_stride=n, out_stride=n, epsilon=1e-3)
    run(ctx, "uzu_group_rms_norm_encode", C.byref(a))
    close(bo.numpy(np.float32, x.shape), P.group_rms(t64(x), t64(w), groups, 1e-3).numpy(), 2e-6, "group rms")


@pytest.mark.parametrize("limit", [0.5, 7.0])
def test_clamped_glu(ctx, limit):
    rng = np.random.default_rng(3)
    rows, f = 9, 37
    gu = rng.standard_normal((rows, 2 * f), dtype=np.float32) * 2
    bg, bo = ctx.upload(gu), ctx.upload(np.zeros((rows, f), np.float32))
    run(ctx, "uzu_clamped_glu_encode", bg.ptr, bo.ptr, rows, f, limit, 1.702)
    g = torch.clamp(t64(gu[:, :f]), max=limit)
    u = torch.clamp(t64(gu[:, f:]), -limit, limit)
    close(bo.numpy(np.float32, (rows, f)), (g * torch.sigmoid(1.702 * g) * (u + 1)).numpy(), 2e-6, "clamped glu")


def dense_linear(ctx, a, w, *, f32_weights, batch=1, a_z=0, w_z=0, d_z=0, lda=None, ldd=None, group_offsets=None, rows_map=None, d=None,
                 m=None, scale=1.0, accumulate=False):
    """w: f32 array [batch, n, k] (rounded to bf16 unless f32_weights)."""
    n, k = w.shape[-2], w.shape[-1]
    wb = ctx.upload(np.ascontiguousarray(w, np.float32) if f32_weights else synth.f32_to_bf16_bits(w))
    ab = ctx.upload(np.ascontiguousarray(a, np.float32))
    db = ctx.upload(d)
    go = ctx.upload(np.asarray(group_offsets, np.uint32)) if group_offsets is not None else None
    rm = ctx.upload(np.asarray(rows_map, np.uint32)) if rows_map is not None else None
    args = B.DenseLinearArgs(a=ab.ptr, w=wb.ptr, d=db.ptr, group_offsets=go.ptr if go else 0, rows_map=rm.ptr if rm else 0,
                             a_z_stride=a_z, w_z_stride=w_z, d_z_stride=d_z, m=m if m is not None else a.shape[0], n=n, k=k,
                             lda=lda or a.shape[-1], ldd=ldd or d.shape[-1], batch=batch, weights_dt=B.DT_F32 if f32_weights else B.DT_BF16,
                             accumulate=int(accumulate), scale=scale)
    run(ctx, "uzu_dense_linear_encode", C.byref(args))
    return db.numpy(np.float32, d.shape)


@pytest.mark.parametrize("m", [1, 3, 8, 9, 31, 32, 70, 96, 130, 257])
@pytest.mark.parametrize("f32_weights", [True, False])
def test_dense_linear_plain(ctx, m, f32_weights):
    rng = np.random.default_rng(m)
    n, k = 75, 203 if m % 2 else 96        # odd k takes the scalar loads
    a = rng.standard_normal((m, k), dtype=np.float32)
    w = synth.st_bits_to_f32(synth.f32_to_bf16_bits(rng.standard_normal((n, k), dtype=np.float32)))
    got = dense_linear(ctx, a, w[None], f32_weights=f32_weights, d=np.zeros((m, n), np.float32))
    if not f32_weights and m >= 32:          # the tensor-pipe kernel rounds the activations to bf16
        a = synth.st_bits_to_f32(synth.f32_to_bf16_bits(a))
    close(got, (t64(a) @ t64(w).T).numpy(), 3e-6, "dense linear")


@pytest.mark.parametrize("m,n,k", [(1, 40, 2048), (5, 40, 2048), (3, 2100, 1024), (2, 9, 1100), (8, 13, 4100)])
@pytest.mark.parametrize("f32_weights", [True, False])
def test_dense_linear_long_rows_shared_by_warps(ctx, m, n, k, f32_weights):
    """Few output features with a long k: several warps take slices of one weight row (also a k that is no multiple of a vector load)."""
    rng = np.random.default_rng(n + k)
    a = rng.standard_normal((m, k), dtype=np.float32)
    w = synth.st_bits_to_f32(synth.f32_to_bf16_bits(rng.standard_normal((n, k), dtype=np.float32)))
    got = dense_linear(ctx, a, w[None], f32_weights=f32_weights, d=np.zeros((m, n), np.float32))
    close(got, (t64(a) @ t64(w).T).numpy(), 3e-6, "dense linear, sliced k")


@pytest.mark.parametrize("m", [2, 40])
def test_dense_linear_heads_and_accumulate(ctx, m):
    """z-batches: head z reads its own column block of A and its own weight and writes its own column block of D."""
    rng = np.random.default_rng(7 + m)
    heads, k, n = 3, 20, 12
    a = rng.standard_normal((m, heads * k + 5), dtype=np.float32)      # rows are wider than the heads' blocks
    w = rng.standard_normal((heads, n, k), dtype=np.float32)
    d0 = rng.standard_normal((m, heads * n), dtype=np.float32)
    got = dense_linear(ctx, a, w, f32_weights=True, batch=heads, a_z=k, w_z=n * k, d_z=n, lda=a.shape[1], ldd=heads * n, d=d0.copy(),
                       scale=0.5, accumulate=True)
    ref = d0.astype(np.float64)
    for h in range(heads):
        ref[:, h * n:(h + 1) * n] += 0.5 * (a[:, h * k:(h + 1) * k].astype(np.float64) @ w[h].astype(np.float64).T)
    close(got, ref, 3e-6, "z-batched dense linear")


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (130, 200, 128), (257, 75, 192), (1024, 384, 1024), (300, 64, 2048)])
def test_dense_linear_tensor_memory_form(ctx, lib, m, n, k):
    """With a bf16 workspace, plain products of >= 128 rows run on tcgen05 (tile edges in m and n, 1 .. 32 K blocks, accumulate, gate, tanh)."""
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k + 4), dtype=np.float32)              # rows wider than k
    w = synth.st_bits_to_f32(synth.f32_to_bf16_bits(rng.standard_normal((n, k), dtype=np.float32)))
    d0 = rng.standard_normal((m, n + 5), dtype=np.float32)
    gate = rng.standard_normal((m, n), dtype=np.float32)
    ab, wb, db, gb = ctx.upload(a), ctx.upload(synth.f32_to_bf16_bits(w)), ctx.upload(d0), ctx.upload(gate)
    ws = ctx.buffer(m * k * 2, B.BUFFER_DEVICE)
    args = B.DenseLinearArgs(a=ab.ptr, w=wb.ptr, d=db.ptr, gate=gb.ptr, gate_ld=n, workspace=ws.ptr, m=m, n=n, k=k, lda=k + 4, ldd=n + 5, batch=1,
                             weights_dt=B.DT_BF16, accumulate=1, scale=0.5, a_op=1)
    with ctx.command_buffer("umma") as cmd:
        cmd.encode("uzu_dense_linear_encode", C.byref(args))
    assert cmd.launches == 2                                           # the conversion and the tensor-memory kernel, not the mma.sync form
    assert lib.uzu_debug_dense_umma_error() == 0
    ta = t64(synth.st_bits_to_f32(synth.f32_to_bf16_bits(np.tanh(a[:, :k].astype(np.float64)).astype(np.float32))))
    ref = d0.astype(np.float64)
    ref[:, :n] += (0.5 * (ta @ t64(w).T) * torch.sigmoid(t64(gate))).numpy()
    got = db.numpy(np.float32, d0.shape)
    assert np.array_equal(got[:, n:], d0[:, n:])                       # columns past n are untouched
    close(got[:, :n], ref[:, :n], 3e-3, "tensor-memory dense product")


@pytest.mark.parametrize("m", [1, 4, 8, 40, 130])
@pytest.mark.parametrize("f32_weights", [True, False])
def test_dense_linear_operand_and_epilogue_options(ctx, m, f32_weights):
    """tanh applied to A as it is read; the sigmoid gate on the product; the paired gated-unit form (<= 8 rows) against the two-launch form."""
    rng = np.random.default_rng(100 + m)
    n, k = 48, 64
    a = rng.standard_normal((m, k), dtype=np.float32)
    w = synth.st_bits_to_f32(synth.f32_to_bf16_bits(rng.standard_normal((2 * n, k), dtype=np.float32) / 4))
    gate = rng.standard_normal((m, n + 3), dtype=np.float32)
    wb = ctx.upload(np.ascontiguousarray(w) if f32_weights else synth.f32_to_bf16_bits(w))
    ab, gb = ctx.upload(a), ctx.upload(gate)
    dt = B.DT_F32 if f32_weights else B.DT_BF16
    rounds_a = (not f32_weights) and m >= 32             # the tensor-pipe kernels round the (transformed) activations to bf16
    bf = lambda x: synth.st_bits_to_f32(synth.f32_to_bf16_bits(np.asarray(x, np.float32)))
    # tanh on A + sigmoid gate on D
    db = ctx.upload(np.zeros((m, n), np.float32))
    args = B.DenseLinearArgs(a=ab.ptr, w=wb.ptr, d=db.ptr, gate=gb.ptr, gate_ld=n + 3, m=m, n=n, k=k, lda=k, ldd=n, batch=1, weights_dt=dt, scale=1.0, a_op=1)
    run(ctx, "uzu_dense_linear_encode", C.byref(args))
    ta = torch.tanh(t64(a))
    if rounds_a:
        ta = t64(bf(ta.numpy()))
    ref = (ta @ t64(w[:n]).T) * torch.sigmoid(t64(gate[:, :n]))
    close(db.numpy(np.float32, (m, n)), ref.numpy(), 3e-3 if rounds_a else 5e-6, "tanh operand + gate epilogue")   # a bf16 rounding of tanh may fall the other way
    # paired gated unit
    if m <= 8:
        db2 = ctx.upload(np.zeros((m, n), np.float32))
        args = B.DenseLinearArgs(a=ab.ptr, w=wb.ptr, d=db2.ptr, m=m, n=n, k=k, lda=k, ldd=n, batch=1, weights_dt=dt, scale=1.0, pair_rows=n,
                                 glu_limit=0.7, glu_alpha=1.702)
        run(ctx, "uzu_dense_linear_encode", C.byref(args))
        ref = P.clamped_glu(t64(a), t64(w[:n]), t64(w[n:]), torch.eye(n, dtype=F64), 0.7)
        close(db2.numpy(np.float32, (m, n)), ref.numpy(), 5e-6, "paired gated unit")


def test_unary_and_residual_add(ctx):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((7, 20), dtype=np.float32)
    bx, bo = ctx.upload(x), ctx.upload(np.zeros((7, 9), np.float32))
    run(ctx, "uzu_unary_f32_encode", bx.ptr + 4 * 3, 20, bo.ptr, 9, 7, 9, 0)          # tanh of columns 3..11
    close(bo.numpy(np.float32, (7, 9)), np.tanh(x[:, 3:12].astype(np.float64)), 2e-6, "tanh")
    r, a, b = (rng.standard_normal(150, dtype=np.float32) for _ in range(3))
    br, ba, bb = ctx.upload(r), ctx.upload(a), ctx.upload(b)
    run(ctx, "uzu_residual_add_encode", br.ptr, ba.ptr, bb.ptr, 150)
    run(ctx, "uzu_residual_add_encode", br.ptr, ba.ptr, 0, 150)
    close(br.numpy(np.float32, (150,)), r.astype(np.float64) + 2 * a.astype(np.float64) + b, 2e-6, "residual add")


@pytest.mark.parametrize("rows,top,experts", [(1, 1, 4), (5, 3, 7), (64, 2, 5), (200, 4, 16)])
def test_table_route_and_expert_products(ctx, rows, top, experts):
    """Router lists + grouped products + combine against a per-token loop; some experts get no token, some many."""
    rng = np.random.default_rng(rows + top)
    vocab, W, f = 50, 24, 10
    table = np.stack([rng.permutation(experts)[:top] for _ in range(vocab)]).astype(np.int32)
    tokens = rng.integers(0, vocab, rows).astype(np.uint32)
    h = rng.standard_normal((rows, W), dtype=np.float32)
    wg = rng.standard_normal((experts, f, W), dtype=np.float32) / 4
    wu = rng.standard_normal((experts, f, W), dtype=np.float32) / 4
    wd = rng.standard_normal((experts, W, f), dtype=np.float32) / 3
    bt, btab = ctx.upload(tokens), ctx.upload(table)
    off, rmap, ppos = ctx.upload(np.zeros(experts + 1, np.uint32)), ctx.upload(np.zeros(rows * top, np.uint32)), ctx.upload(np.zeros(rows * top, np.uint32))
    ra = B.TableRouteArgs(token_ids=bt.ptr, table=btab.ptr, group_offsets=off.ptr, rows_map=rmap.ptr, pair_pos=ppos.ptr, rows=rows, top=top,
                          experts=experts, vocab=vocab)
    run(ctx, "uzu_table_route_encode", C.byref(ra))
    offsets, rows_map, pair_pos = off.numpy(np.uint32, (experts + 1,)), rmap.numpy(np.uint32, (rows * top,)), ppos.numpy(np.uint32, (rows * top,))
    assert offsets[0] == 0 and offsets[-1] == rows * top and (np.diff(offsets.astype(np.int64)) >= 0).all()
    assert sorted(pair_pos.tolist()) == list(range(rows * top))
    for r in range(rows):
        for s in range(top):
            p = pair_pos[r * top + s]
            e = table[tokens[r], s]
            assert offsets[e] <= p < offsets[e + 1] and rows_map[p] == r
    gu = dense_linear(ctx, h, np.concatenate([wg, wu], axis=1), f32_weights=True, batch=experts, w_z=2 * f * W, group_offsets=offsets,
                      rows_map=rows_map, d=np.zeros((rows * top, 2 * f), np.float32), m=rows)
    bgu, bact = ctx.upload(gu), ctx.upload(np.zeros((rows * top, f), np.float32))
    run(ctx, "uzu_clamped_glu_encode", bgu.ptr, bact.ptr, rows * top, f, 1.5, 1.702)
    act = bact.numpy(np.float32, (rows * top, f))
    pairs = dense_linear(ctx, act, wd, f32_weights=True, batch=experts, w_z=W * f, group_offsets=offsets, d=np.zeros((rows * top, W), np.float32), m=rows)
    bp, bpp, bo = ctx.upload(pairs), ctx.upload(pair_pos), ctx.upload(np.zeros((rows, W), np.float32))
    run(ctx, "uzu_routed_combine_encode", bp.ptr, bpp.ptr, bo.ptr, rows, top, W, 1.0 / top, 0)
    ex = [(t64(wg[e]), t64(wu[e]), t64(wd[e])) for e in range(experts)]
    ref = P.table_moe(t64(h), tokens.tolist(), torch.from_numpy(table), ex, 1.5)
    close(bo.numpy(np.float32, (rows, W)), ref.numpy(), 5e-6, "table-routed experts")


def general_delta_gpu(ctx, r, k, v, rate, decay, rate_b, decay_b, state, heads, dim, prepared=False):
    rows = r.shape[0]
    bufs = [ctx.upload(np.ascontiguousarray(x, np.float32)) for x in (r, k, v, rate, decay, rate_b, decay_b, state)]
    out = ctx.upload(np.zeros((rows, heads * dim), np.float32))
    hd = heads * dim
    hd = heads * dim
    unit = ctx.upload(np.zeros((rows, hd), np.float32)) if prepared else None      # with it, passes of >= 4 rows form their vectors up front
    a = B.GeneralDeltaArgs(r=bufs[0].ptr, k=bufs[1].ptr, v=bufs[2].ptr, rate_logit=bufs[3].ptr, decay_logit=bufs[4].ptr, rate_bias=bufs[5].ptr,
                           decay_bias=bufs[6].ptr, unit=unit.ptr if unit else 0, state=bufs[7].ptr, out=out.ptr, r_stride=hd, k_stride=hd, v_stride=hd, rate_stride=hd,
                           decay_stride=hd, rows=rows, heads=heads, dim=dim)
    run(ctx, "uzu_general_delta_encode", C.byref(a))
    return out.numpy(np.float32, (rows, hd)), bufs[7].numpy(np.float32, state.shape)


def general_delta_plain(r, k, v, rate, decay, rate_b, decay_b, state, heads, dim):
    """The recurrence alone, from the raw projections (float64)."""
    T = r.shape[0]
    r, k, v = (t64(x).reshape(T, heads, dim) for x in (r, k, v))
    d = torch.exp(-math.exp(-0.5) * torch.sigmoid(t64(decay) + t64(decay_b))).reshape(T, heads, dim)
    a = torch.sigmoid(t64(rate) + t64(rate_b)).reshape(T, heads, dim)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    S = t64(state).clone()
    o = torch.zeros(T, heads, dim, dtype=F64)
    for t in range(T):
        for n in range(heads):
            z = u[t, n] @ S[n]
            S[n] = d[t, n][:, None] * S[n] - (a[t, n] * u[t, n])[:, None] * z[None, :] + k[t, n][:, None] * v[t, n][None, :]
            o[t, n] = S[n].T @ r[t, n]
    return o.reshape(T, heads * dim).numpy(), S.numpy()


@pytest.mark.parametrize("rows,heads,dim", [(1, 2, 16), (7, 3, 24), (40, 1, 48), (5, 2, 80), (3, 1, 130)])
def test_general_delta_kernel(ctx, rows, heads, dim):
    """State carried in (non-zero), several tokens in one launch, head sizes that do not fill the warps."""
    rng = np.random.default_rng(rows + dim)
    hd = heads * dim
    r, k, v, rate, decay = (rng.standard_normal((rows, hd), dtype=np.float32) for _ in range(5))
    rate_b, decay_b = rng.standard_normal(hd, dtype=np.float32), rng.standard_normal(hd, dtype=np.float32)
    state = rng.standard_normal((heads, dim, dim), dtype=np.float32)
    ref, ref_state = general_delta_plain(r, k, v, rate, decay, rate_b, decay_b, state, heads, dim)
    for prepared in (False, True):
        got, got_state = general_delta_gpu(ctx, r, k, v, rate, decay, rate_b, decay_b, state, heads, dim, prepared)
        close(got, ref, 1e-5, "generalized delta output")
        close(got_state, ref_state, 1e-5, "generalized delta state")


def test_general_delta_one_launch_equals_token_by_token(ctx):
    rng = np.random.default_rng(11)
    rows, heads, dim = 24, 2, 40
    hd = heads * dim
    r, k, v, rate, decay = (rng.standard_normal((rows, hd), dtype=np.float32) for _ in range(5))
    zb = np.zeros(hd, np.float32)
    state = np.zeros((heads, dim, dim), np.float32)
    whole, s_whole = general_delta_gpu(ctx, r, k, v, rate, decay, zb, zb, state, heads, dim)
    s, parts = state, []
    for t in range(rows):
        o, s = general_delta_gpu(ctx, r[t:t + 1], k[t:t + 1], v[t:t + 1], rate[t:t + 1], decay[t:t + 1], zb, zb, s, heads, dim)
        parts.append(o)
    assert np.array_equal(np.concatenate(parts), whole) and np.array_equal(s, s_whole)   # the same bits: partial sums meet in a fixed order


def test_general_delta_removal_reads_the_old_state(ctx):
    """With decay ~ 1, rate ~ 1 and a repeated unit key, the old content along that key is removed before the new pair is written:
    a reading r = k returns |k|^2 v_new exactly (a fault that reads the new state, or skips the removal, adds the old value)."""
    heads, dim = 1, 32
    k = np.zeros((2, dim), np.float32); k[:, 3] = 2.0
    v = np.stack([np.full(dim, 5.0, np.float32), np.arange(dim, dtype=np.float32)])
    big = np.full((2, dim), 40.0, np.float32)
    got, _ = general_delta_gpu(ctx, k.copy(), k, v, big, -big, np.zeros(dim, np.float32), np.zeros(dim, np.float32),
                               np.zeros((1, dim, dim), np.float32), heads, dim)
    close(got[1], 4.0 * v[1], 1e-5, "replace along a repeated key")


@pytest.mark.parametrize("rows,heads,dim", [(3, 2, 24), (6, 5, 70)])
def test_head_norm_gate(ctx, rows, heads, dim):
    rng = np.random.default_rng(dim)
    x, g = rng.standard_normal((rows, heads * dim), dtype=np.float32), rng.standard_normal((rows, heads * dim), dtype=np.float32)
    w = rng.standard_normal(heads * dim, dtype=np.float32)
    bx, bg, bw, bo = ctx.upload(x), ctx.upload(g), ctx.upload(w), ctx.upload(np.zeros_like(x))
    a = B.HeadNormGateArgs(x=bx.ptr, scales=bw.ptr, gate=bg.ptr, out=bo.ptr, rows=rows, heads=heads, dim=dim, normalize=1, epsilon=1e-4)
    run(ctx, "uzu_head_norm_gate_encode", C.byref(a))
    xh = t64(x).reshape(rows, heads, dim)
    ref = (xh / torch.sqrt((xh * xh).mean(-1, keepdim=True) + 1e-4)).reshape(rows, -1) * t64(w) * torch.sigmoid(t64(g))
    close(bo.numpy(np.float32, x.shape), ref.numpy(), 3e-6, "head norm + gate")


# ---- latent attention kernels: cache rows + rotated queries + causal softmax over the shared cache ----------------------------------
def rope_tables(rot, positions):
    f, mult = P.rotary_frequencies(rot)
    ang = (torch.arange(positions, dtype=torch.float32)[:, None] * f.to(torch.float32)[None, :]).to(F64)
    return (torch.cos(ang) * mult).to(torch.float32).numpy(), (torch.sin(ang) * mult).to(torch.float32).numpy()


def latent_gpu(ctx, q, kv, uk, norm_w, m, eps, prefix, cache, f32_cache=True, splits=0):
    """q [T, H, dim + rot], kv [T, rank + rot] raw projections; cache [capacity, rank + rot] holds the rows of earlier tokens.
    Returns the weighted latent sums [T, H, rank] and the cache."""
    T, H, dn, dr, R = q.shape[0], m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
    width = R + dr
    cos, sin = rope_tables(m["rot"], prefix + T)
    bq, bkv = ctx.upload(q.astype(np.float32)), ctx.upload(kv.astype(np.float32))
    bcache = ctx.upload(cache if f32_cache else synth.f32_to_bf16_bits(cache))
    bquery, bout = ctx.upload(np.zeros((T, H, width), np.float32)), ctx.upload(np.zeros((T, H, R), np.float32))
    bw, bcos, bsin = ctx.upload(norm_w.astype(np.float32)), ctx.upload(cos), ctx.upload(sin)
    dt = B.DT_F32 if f32_cache else B.DT_BF16
    pa = B.LatentPrepareArgs(kv=bkv.ptr, q=bq.ptr, query=bquery.ptr, cache=bcache.ptr, latent_scales=bw.ptr, cosines=bcos.ptr, sines=bsin.ptr,
                             rows=T, heads=H, dim=dn, rot_dim=dr, rank=R, rot_pairs=m["rot"]["dims"] // 2, kv_stride=width, q_stride=H * (dn + dr),
                             prefix=prefix, cache_dt=dt, epsilon=eps)
    run(ctx, "uzu_latent_prepare_encode", C.byref(pa))
    # absorbed key projection: query[:, h, :rank] = q[:, h, :dim] @ uk[h]  (uk[h] is [dim, rank])
    query = bquery.numpy(np.float32, (T, H, width))
    for h in range(H):
        query[:, h, :R] = (q[:, h, :dn].astype(np.float64) @ uk[h].astype(np.float64)).astype(np.float32)
    bquery2 = ctx.upload(query)
    bpart = ctx.upload(np.zeros(T * H * max(splits, 1) * (R + 2), np.float32))
    aa = B.LatentAttentionArgs(query=bquery2.ptr, cache=bcache.ptr, out=bout.ptr, partials=bpart.ptr, rows=T, heads=H, rank=R, rot_dim=dr,
                               prefix=prefix, cache_dt=dt, scale=m["scale"], splits=splits)
    run(ctx, "uzu_latent_attention_encode", C.byref(aa))
    new_cache = bcache.numpy(np.float32, cache.shape) if f32_cache else synth.st_bits_to_f32(bcache.numpy(np.uint16, cache.shape))
    return bout.numpy(np.float32, (T, H, R)), new_cache


def latent_plain(q, kv, uk, norm_w, m, eps, prefix, cache):
    """Same quantities in float64: scores through the per-head keys uk[h] c (not the absorbed form)."""
    T, H, dn, dr, R = q.shape[0], m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
    pos = torch.arange(prefix, prefix + T)
    c = P.plain_rms(t64(kv[:, :R]), t64(norm_w), eps)
    kr = P.rotate_pairs(t64(kv[:, R:]), pos, m["rot"])
    rows = torch.cat([t64(cache[:prefix]), torch.cat([c, kr], -1)])
    qq = t64(q)
    q_r = P.rotate_pairs(qq[..., dn:], pos, m["rot"])
    out = torch.zeros(T, H, R, dtype=F64)
    for h in range(H):
        keys = rows[:, :R] @ t64(uk[h]).T                   # [n, dim]
        s = (qq[:, h, :dn] @ keys.T + q_r[:, h] @ rows[:, R:].T) * m["scale"]
        mask = torch.arange(rows.shape[0])[None, :] <= pos[:, None]
        w = torch.softmax(s.masked_fill(~mask, float("-inf")), -1)
        out[:, h] = w @ rows[:, :R]
    return out.numpy(), rows.numpy()


def latent_sizes(heads, dim, rot_dim, rank, dims=None, scaling=None, base=10000.0):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "kv_rank": rank, "scale": 0.3,
            "rot": {"dims": dims or rot_dim, "base": base, "scaling": scaling}}


YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}


@pytest.mark.parametrize("T,prefix,heads,dim,rot,rank,dims,scaling", [
    (1, 0, 1, 8, 4, 16, None, None),          # the first token of a sequence
    (2, 0, 3, 12, 8, 40, None, YARN),
    (9, 31, 11, 16, 8, 24, 6, YARN),          # more heads than one CTA's group, rotation of a part of the rotated block, tile edge at 32 keys
    (33, 64, 2, 20, 16, 70, None, YARN),
    (1, 200, 9, 8, 32, 130, None, None),      # one decoded token far into the context
    (2, 300, 3, 8, 5, 20, 4, None),           # an odd row width: the tile is staged element by element
])
def test_latent_attention_kernels(ctx, T, prefix, heads, dim, rot, rank, dims, scaling):
    rng = np.random.default_rng(T + prefix)
    m = latent_sizes(heads, dim, rot, rank, dims, scaling)
    q = rng.standard_normal((T, heads, dim + rot), dtype=np.float32)
    kv = rng.standard_normal((T, rank + rot), dtype=np.float32)
    uk = rng.standard_normal((heads, dim, rank), dtype=np.float32) / 4
    norm_w = 1 + 0.1 * rng.standard_normal(rank, dtype=np.float32)
    cache = np.zeros((prefix + T + 3, rank + rot), np.float32)
    cache[:prefix] = rng.standard_normal((prefix, rank + rot), dtype=np.float32)
    cache[prefix + T:] = 1e4                    # rows beyond the causal bound must not be read
    ref, ref_rows = latent_plain(q, kv, uk, norm_w, m, 1e-5, prefix, cache)
    for splits in (0, 2, 5, 64):             # key ranges cut over several CTAs and merged: also more splits than tiles (empty parts)
        got, got_cache = latent_gpu(ctx, q, kv, uk, norm_w, m, 1e-5, prefix, cache.copy(), splits=splits)
        close(got_cache[:prefix + T], ref_rows, 3e-6, "cache rows")
        close(got, ref, 2e-5, f"latent attention, {splits} splits")


@pytest.mark.parametrize("far", [0, 1, 31, 32, 33, 500])
@pytest.mark.parametrize("f32_cache", [True, False])
def test_latent_attention_finds_one_far_key(ctx, far, f32_cache):
    """Among 600 cached rows exactly one has a latent that matches the query strongly: the output is that row's latent. Its place sweeps the
    first rows, the 32-key tile edge and the middle; the query is the last position (decode) or a few prompt rows."""
    rng = np.random.default_rng(far)
    heads, dim, rot, rank, n = 2, 8, 4, 24, 600
    m = latent_sizes(heads, dim, rot, rank)
    cache = synth.st_bits_to_f32(synth.f32_to_bf16_bits(0.05 * rng.standard_normal((n + 4, rank + rot), dtype=np.float32)))
    cache[far, :rank] = 0.0
    cache[far, 5] = 3.0
    uk = np.zeros((heads, dim, rank), np.float32)
    uk[:, 0, 5] = 1.0                                    # key channel 0 of every head reads latent channel 5
    for T in (1, 4):
        q = np.zeros((T, heads, dim + rot), np.float32)
        q[:, :, 0] = 40.0
        kv = 0.05 * rng.standard_normal((T, rank + rot), dtype=np.float32)
        kv[:, 5] = 0.0                                   # the new rows' own latents do not answer the query
        got, _ = latent_gpu(ctx, q, kv, uk, np.ones(rank, np.float32), m, 1e-5, n, cache.copy(), f32_cache, splits=7 if T == 1 else 0)
        want = np.zeros(rank); want[5] = 3.0
        for t in range(T):
            for h in range(heads):
                assert np.abs(got[t, h] - want).max() < 1e-3, (far, T, t, h)


# ---- whole models through the engine ----------------------------------------------------------------------------------------------
def config_a():
    """Every size differs from every other; three norm groups; experts with top 3; a layer without feed-forward; partial YaRN ramp."""
    S = synth
    return S.punilix_config(96, 211, [
        S.punilix_delta_layer(3, 24, S.punilix_dense_mlp(56, limit=1.0)),
        S.punilix_latent_layer(5, 16, 8, 20, 40, 48, S.punilix_moe_mlp(28, 6, 3, limit=0.8), scale=0.21, base=5000.0, scaling=dict(YARN)),
        S.punilix_latent_layer(2, 12, 6, 36, 24, 30, None, scale=0.4, base=100.0, scaling=None),
        S.punilix_delta_layer(2, 40, S.punilix_moe_mlp(44, 4, 1, limit=2.0)),
    ], norm_groups=3, eps=1e-4, logit_softcap=9.0)


def config_b():
    """One head, one group, one expert choice out of two, no soft cap, wide cache rows (few tokens per cache page)."""
    S = synth
    return S.punilix_config(64, 130, [
        S.punilix_latent_layer(1, 24, 16, 24, 500, 32, S.punilix_dense_mlp(40), scaling={"factor": 2.0, "original": 32, "fast": 4.0, "slow": 2.0}),
        S.punilix_delta_layer(1, 64, S.punilix_moe_mlp(20, 2, 1)),
        S.punilix_latent_layer(9, 8, 4, 8, 16, 20, S.punilix_moe_mlp(12, 5, 5, limit=0.5), base=3.0),
    ], norm_groups=1, eps=1e-6, logit_softcap=None)


def config_c():
    """Sizes that fit no vector width: width 90, an odd latent row (21 + 6), head sizes 18 (not a multiple of 4) and 20, odd feed-forwards."""
    S = synth
    return S.punilix_config(90, 77, [
        S.punilix_delta_layer(3, 18, S.punilix_moe_mlp(10, 3, 2, limit=1.5)),
        S.punilix_latent_layer(3, 7, 6, 9, 21, 11, S.punilix_dense_mlp(50, limit=3.0), scale=0.33, base=50.0,
                               scaling={"factor": 3.0, "original": 16, "fast": 2.0, "slow": 0.5}),
        S.punilix_delta_layer(2, 20, None),
    ], norm_groups=5, eps=1e-5, logit_softcap=4.0)


class Pair:
    """A checkpoint on disk, the engine on it and the oracle on the same (bf16-exact) tensors."""

    def __init__(self, ctx, tmp_path, config, seed=0, f32=True, tensors=None, max_context=4096, **kw):
        self.config = config
        self.tensors = tensors or synth.punilix_tensors(config, seed, decay_rank=5 + seed)
        self.tensors = {k: (v if np.issubdtype(np.asarray(v).dtype, np.integer) else synth.st_bits_to_f32(synth.f32_to_bf16_bits(v)))
                        for k, v in self.tensors.items()}           # what the checkpoint holds
        path = synth.write_punilix_model(config, tmp_path / f"m{seed}{int(f32)}", tensors=self.tensors)
        self.engine = B.Engine(ctx, path, max_context_length=max_context, storage_f32=f32, **kw)
        self.oracle = P.PlainModel(config, {k: torch.from_numpy(np.asarray(v)) for k, v in self.tensors.items()})
        self.tol = 2e-4 if f32 else 6e-2

    def reference(self, tokens):
        self.oracle.reset()
        return self.oracle.step(list(tokens)).numpy()

    def check(self, got, ref, what):
        got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
        d = (got - ref) - (got - ref).mean(-1, keepdims=True)
        err = np.sqrt((d * d).mean(-1)) / max(float(ref.std()), 1e-6)
        assert err.max() <= self.tol, f"{what}: row {int(err.argmax())} differs by {err.max():.3e} of the logits' spread (bound {self.tol:.0e})"

    def close(self):
        self.engine.close()


def tokens_for(config, n, seed=0):
    return np.random.default_rng(seed).integers(0, config["vocab"], n).tolist()


@pytest.mark.parametrize("make", [config_a, config_b, config_c])
@pytest.mark.parametrize("f32", [True, False])
def test_prompt_logits_and_layers(ctx, tmp_path, make, f32):
    pr = Pair(ctx, tmp_path, make(), seed=1, f32=f32)
    toks = tokens_for(pr.config, 70 if f32 else 130, 1)     # bf16: 130 rows take the large-tile tensor-pipe products (50 rows elsewhere: the small tiles)
    pr.engine.debug_layer_outputs(True)
    s = pr.engine.slot_acquire()
    got = pr.engine.forward_rows(toks, list(range(len(toks))), slot=s)
    layers = pr.engine.debug_layer_outputs(True)
    pr.oracle.reset()
    ref_layers = []
    ref = pr.oracle.step(toks, ref_layers).numpy()
    for i, (g, r) in enumerate(zip(layers, ref_layers)):
        close(g, r.numpy(), 1e-5 if f32 else 1e-1, f"residual after layer {i}")
    pr.check(got, ref, "prompt logits")
    pr.close()


@pytest.mark.parametrize("make", [config_a, config_b, config_c])
@pytest.mark.parametrize("f32", [True, False])
def test_decode_and_portions_match_the_whole_prompt(ctx, tmp_path, make, f32):
    """Prefill + token-by-token decoding, and portions of 2, 3, 1, 33, 2, ... tokens, give the logits of the whole prompt."""
    pr = Pair(ctx, tmp_path, make(), seed=2, f32=f32)
    n = 90
    toks = tokens_for(pr.config, n, 2)
    ref = pr.reference(toks)
    s = pr.engine.slot_acquire()
    parts = [pr.engine.forward_rows(toks[:50], list(range(50)), slot=s)]
    parts += [pr.engine.forward_rows(toks[p:p + 1], [0], slot=s) for p in range(50, n)]
    pr.check(np.concatenate(parts), ref, "prefill + decode")
    pr.engine.slot_release(s)
    s = pr.engine.slot_acquire()                 # the same slot again: its cache rows and states start over
    parts, p, k = [], 0, 0
    sizes = [2, 3, 1, 33, 2, 9, 32, 2]
    while p < n:
        c = min(sizes[k % len(sizes)], n - p)
        parts.append(pr.engine.forward_rows(toks[p:p + c], list(range(c)), slot=s))
        p, k = p + c, k + 1
    pr.check(np.concatenate(parts), ref, "portions")
    pr.close()


def test_slots_interleaved_and_reused(ctx, tmp_path):
    """Three unequal requests advance in turns in their own slots; one ends early and its slot serves a new request. Each equals its solo run."""
    pr = Pair(ctx, tmp_path, config_a(), seed=3, f32=True)
    reqs = {name: tokens_for(pr.config, n, 10 + i) for i, (name, n) in enumerate([("a", 41), ("b", 7), ("c", 64), ("d", 23)])}
    refs = {name: pr.reference(t) for name, t in reqs.items()}
    got = {name: [] for name in reqs}
    at = {name: 0 for name in reqs}
    slot = {}
    live, waiting = ["a", "b", "c"], ["d"]
    step = {"a": 5, "b": 2, "c": 1, "d": 4}
    while live:
        for name in list(live):
            if name not in slot:
                slot[name] = pr.engine.slot_acquire()
            c = min(step[name], len(reqs[name]) - at[name])
            got[name].append(pr.engine.forward_rows(reqs[name][at[name]:at[name] + c], list(range(c)), slot=slot[name]))
            at[name] += c
            if at[name] == len(reqs[name]):
                pr.engine.slot_release(slot[name])
                live.remove(name)
                if waiting:
                    live.append(waiting.pop())
    assert slot["d"] == slot["b"]                # the freed slot was handed out again
    for name in reqs:
        pr.check(np.concatenate(got[name]), refs[name], f"request {name}")
    pr.close()


def test_long_context_page_and_pass_edges(ctx, tmp_path):
    """1100 tokens: past the 1024-row pass and, with 516-wide f32 cache rows, past the first cache page; then 40 decoded tokens.
    Rows just before and after both edges are compared, in the prompt and decoded."""
    pr = Pair(ctx, tmp_path, config_b(), seed=4, f32=True)
    n = 1140
    toks = tokens_for(pr.config, n, 4)
    ref = pr.reference(toks)
    s = pr.engine.slot_acquire()
    rows = [0, 1, 2, 1014, 1015, 1016, 1017, 1022, 1023, 1024, 1025, 1099]
    got = pr.engine.forward_rows(toks[:1100], rows, slot=s)
    pr.check(got, ref[rows], "long prompt")
    dec = np.concatenate([pr.engine.forward_rows(toks[p:p + 1], [0], slot=s) for p in range(1100, n)])
    pr.check(dec, ref[1100:], "decoding after a long prompt")
    pr.engine.slot_release(s)
    s = pr.engine.slot_acquire()                 # decode across the pass edge: prompt of 1010, then one by one over 1016 and 1024
    pr.engine.forward_rows(toks[:1010], [], slot=s)
    dec = np.concatenate([pr.engine.forward_rows(toks[p:p + 1], [0], slot=s) for p in range(1010, 1030)])
    pr.check(dec, ref[1010:1030], "decoding over the edges")
    pr.close()


def marker_model(marker=7):
    """One latent-attention layer in which a marker token's cache row answers every query whose first latent entry is positive, far
    above the other rows: input coordinate 0 is non-zero for the marker only, latent channel 0 reads it, key channel 0 of every head reads
    latent channel 0 and query channel 0 reads the query latent's first entry."""
    S = synth
    cfg = S.punilix_config(48, 60, [S.punilix_latent_layer(2, 8, 4, 12, 16, 12, None, scale=1.0)], norm_groups=2, logit_softcap=None)
    t = S.punilix_tensors(cfg, 5)
    t["embed"][:, 0] = 0.0
    t["embed"][marker] = 0.0
    t["embed"][marker, 0] = 5.0
    t["l0.norm1"][:] = 1.0
    t["l0.mix.dkv.norm"][:] = 1.0
    t["l0.mix.dkv"][:, 0] = 0.0
    t["l0.mix.dkv"][0, :] = 0.0
    t["l0.mix.dkv"][0, 0] = 10.0
    t["l0.mix.uk"] *= 0.1
    t["l0.mix.uk"][:, 0] = 0.0
    for h in range(2):
        t["l0.mix.uk"][h * 8, 0] = 1.0
        t["l0.mix.uq"][h * 12, :] = 0.0
        t["l0.mix.uq"][h * 12, 0] = 6.0
    return cfg, t, marker


def test_far_token_decides_the_logits(ctx, tmp_path):
    """A marker token somewhere in a 700-token prompt (position 0, 1, 31, 32, 33, 400) changes the last logits strongly; the engine agrees
    with the oracle for each place, in the prompt's last row and in 10 decoded tokens."""
    cfg, t, marker = marker_model()
    pr = Pair(ctx, tmp_path, cfg, seed=5, f32=True, tensors=t)
    base = [x if x != marker else 8 for x in tokens_for(cfg, 700, 5)]
    without = pr.reference(base)
    for place in (0, 1, 31, 32, 33, 400):
        toks = list(base)
        toks[place] = marker
        ref = pr.reference(toks)
        moved = np.sqrt(((ref[689:] - without[689:]) ** 2).mean(-1)).max() / ref.std()
        assert moved > 0.3, "the marker must matter for this test to mean anything"
        s = pr.engine.slot_acquire()
        got = pr.engine.forward_rows(toks[:690], [689], slot=s)
        dec = np.concatenate([pr.engine.forward_rows(toks[p:p + 1], [0], slot=s) for p in range(690, 700)])
        pr.engine.slot_release(s)
        pr.check(got, ref[689:690], f"marker at {place}, prompt")
        pr.check(dec, ref[690:], f"marker at {place}, decoded")
    pr.close()


@pytest.mark.parametrize("graph", [True, False])
def test_greedy_generation_through_the_stream(ctx, tmp_path, graph):
    """prefill() + next()/flush() (the engine's generation entry point; CUDA-graph decode when `graph`), 300 tokens. The oracle is fed the
    engine's tokens: every chosen token must be the oracle's best within the rounding of the bf16 logits the sampler reads."""
    pr = Pair(ctx, tmp_path, config_a(), seed=6, f32=True, use_cuda_graph=graph)
    prompt = tokens_for(pr.config, 12, 6)
    steps = 300 if graph else 40
    out = pr.engine.generate(prompt, steps)
    assert len(out) == steps
    pr.oracle.reset()
    z = pr.oracle.step(prompt).numpy()[-1]
    for i, tok in enumerate(out):
        assert z[tok] >= z.max() - 2.0 ** -7 * np.abs(z).max() - 1e-3, f"token {i}: the engine chose {tok}, the oracle's best is {int(z.argmax())}"
        z = pr.oracle.step([tok]).numpy()[-1]
    # the stream's state is the context so far: feeding one more token gives the oracle's logits
    pr.check(pr.engine.forward_rows([out[-1]], [0]), z[None], "the stream's state after generation")
    pr.close()
