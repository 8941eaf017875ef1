"""Namalix's mechanisms alone, kernel by kernel, with inputs made so that a fault shows: one key among hundreds that fits the
query while every other weight is almost zero, that key at a page's last and first place and right behind the query (where
it must not be seen), a mixing matrix that moves weights between heads of different kv heads, values blended with another
layer's, a convolution whose record is shorter and longer than a portion, a delta rule that must give back the last value
written under a key after hundreds of tokens.  References: `plain_namalix.py`."""

import math

import numpy as np
import pytest
import torch

import plain_namalix as pn

pytestmark = pytest.mark.gpu
F64 = torch.float64

KERNELS = {"general-32": torch.float32, "general-16": torch.bfloat16, "the part's choice": torch.bfloat16}


def _dev(a, dtype):
    return torch.as_tensor(np.asarray(a, dtype=np.float64)).to("cuda", dtype)


def _rounded(a, dtype):
    return _dev(a, dtype).to(F64).cpu().numpy()


def _i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device="cuda")


def _paged(k, v, dtype, n_pages, order):
    """k [L, G, kd], v [L, G, vd] laid into pages in the given order of page ids; unused places hold finite junk."""
    L, G, kd = k.shape
    kp = torch.full((n_pages, G, 64, kd), 4.0, dtype=dtype, device="cuda")
    vp = torch.full((n_pages, G, 64, v.shape[2]), -3.0, dtype=dtype, device="cuda")
    for i in range((L + 63) // 64):
        n = min(64, L - 64 * i)
        kp[order[i], :, :n] = _dev(k[64 * i: 64 * i + n], dtype).transpose(0, 1)
        vp[order[i], :, :n] = _dev(v[64 * i: 64 * i + n], dtype).transpose(0, 1)
    return kp, vp, order[: (L + 63) // 64]


def plain_rows(q, k, v, p0, scale, softcap, pb, talk, gate):
    """Rows p0 .. p0 + n - 1 of the plain attention: q [n, H, kd] over keys k [L, G, kd], v [L, G, vd]; gate [n, H] or None."""
    n, H, kd = q.shape
    L, G = p0 + n, k.shape[1]
    full_q = torch.zeros(L, H, kd, dtype=F64)
    full_q[p0:] = torch.as_tensor(q)
    w = pn.attention_weights(full_q, torch.as_tensor(k[:L]), {"scale": scale, "softcap": softcap}, torch.as_tensor(pb), torch.as_tensor(talk))
    vv = torch.as_tensor(v[:L]).repeat_interleave(H // G, dim=1)
    o = torch.einsum("hij,jhv->ihv", w, vv)[p0:]
    if gate is not None:
        o = o * pn.logistic(torch.as_tensor(gate))[:, :, None]
    return o.numpy()


def attend(kernel, q, kp, vp, pages, p0, H, G, kd, vd, scale, softcap, pb, talk, gate, single=False):
    """q [n, H, kd] (already rounded) at positions p0 .. of ONE sequence whose pages are `pages` -> [n, H, vd] float64.
    single: every row as a sequence of its own that brings one token (a decode step of n sequences on the same pages)."""
    from rusty_llama_b200.kernels import ops

    dtype = KERNELS[kernel]
    n = q.shape[0]
    rows = torch.zeros((n, H * kd + 8 + H), dtype=dtype, device="cuda")  # rows longer than the queries, as a projection's are
    rows[:, : H * kd] = _dev(q.reshape(n, H * kd), dtype)
    g = None
    if gate is not None:
        rows[:, H * kd + 8 :] = _dev(gate, dtype)
        g = rows[:, H * kd + 8 :]
    pbd, mix = _dev(pb, torch.float32), _dev(talk, torch.float32)
    pos = _i32(np.arange(p0, p0 + n))
    if kernel.startswith("general"):
        table, seq = (_i32([pages] * n), _i32(np.arange(n))) if single else (_i32([pages]), _i32(np.zeros(n)))
        out = ops.sigmoid_attn(rows, kp, vp, table, seq, pos, H, G, kd, vd, scale, head_bias=pbd, mix=mix, gate=g, softcap=softcap)
    else:
        from types import SimpleNamespace

        from rusty_llama_b200.parts.attention import logistic_attention_runner

        if single:
            step = SimpleNamespace(tok_seq=_i32(np.arange(n)), tok_pos=pos, seq_start=_i32(np.arange(n + 1)), seq_pos0=pos, max_q_len=1, n_seqs=n,
                                   decode_only=True, plan_kv_len=p0 + n)
            table = _i32([pages] * n)
        else:
            step = SimpleNamespace(tok_seq=_i32(np.zeros(n)), tok_pos=pos, seq_start=_i32([0, n]), seq_pos0=_i32([p0]), max_q_len=n, n_seqs=1,
                                   decode_only=n == 1, plan_kv_len=p0 + n)
            table = _i32([pages])
        out = logistic_attention_runner(rows, g, kp, vp, table, step, H, G, kd, vd, scale, softcap, pbd, mix)()
    return out.to(F64).cpu().numpy().reshape(n, H, vd)


def _tol(kernel):
    return 2e-5 if KERNELS[kernel] == torch.float32 else 2.5e-2


SHAPES = [(6, 2, 20, 12), (4, 2, 64, 64), (8, 4, 48, 32), (1, 1, 24, 16), (3, 3, 128, 128)]


@pytest.mark.parametrize("single", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("kernel", list(KERNELS))
def test_one_key_among_hundreds(kernel, shape, single):
    """700 keys whose weights are almost zero (a bias of -12) but one per head, which fits the query so well that its weight is
    almost one: at the last place of a page, the first of the next, far back, and at the query's own position.  Then the same
    key ONE PLACE BEHIND the query, where it must not be seen at all."""
    H, G, kd, vd = shape
    dtype = KERNELS[kernel]
    rng = np.random.default_rng(H * 100 + kd)
    L, p0, n = 700, 660, 40
    for target in (63, 64, 5, 448, 699):
        k = _rounded(0.02 * rng.standard_normal((L, G, kd)), dtype)
        v = _rounded(rng.standard_normal((L, G, vd)), dtype)
        q = _rounded(0.5 * rng.standard_normal((n, H, kd)), dtype)
        unit = rng.standard_normal(kd)
        unit /= np.linalg.norm(unit)
        k[target] = _rounded(6.0 * unit, dtype)[None, :]
        q[:] += _rounded(6.0 * unit, dtype)[None, None, :]
        pb = np.full(H, -12.0)
        talk = np.eye(H) + 0.3 * rng.standard_normal((H, H))
        gate = _rounded(rng.standard_normal((n, H)), dtype)
        kp, vp, pages = _paged(k, v, dtype, 16, [9, 2, 14, 0, 7, 11, 5, 3, 12, 1, 8, 15, 4, 6, 10, 13])
        got = attend(kernel, q, kp, vp, pages, p0, H, G, kd, vd, 1.0, 30.0, pb, talk, gate, single)
        ref = plain_rows(q, k, v, p0, 1.0, 30.0, pb, talk, gate)
        scale = np.abs(ref).max()
        assert scale > 0.05  # the key is seen
        assert np.abs(got - ref).max() <= _tol(kernel) * scale, f"target {target}: {np.abs(got - ref).max() / scale:.2e}"
        # rows before the target must not see it: their results are tiny
        hidden = [i for i in range(n) if p0 + i < target]
        if hidden:
            assert np.abs(got[hidden]).max() <= 1e-2 * scale, f"target {target} is seen from before it"


@pytest.mark.parametrize("kernel", list(KERNELS))
def test_mixing_moves_weights_between_heads_of_different_kv_heads(kernel):
    """Head 0 (kv head 0) gets all of its weights from head 3 (kv head 1) and applies them to ITS OWN kv head's values."""
    H, G, kd, vd = 4, 2, 16, 16
    dtype = KERNELS[kernel]
    rng = np.random.default_rng(3)
    L = 130
    k = _rounded(rng.standard_normal((L, G, kd)), dtype)
    v = _rounded(rng.standard_normal((L, G, vd)), dtype)
    q = _rounded(rng.standard_normal((L, H, kd)), dtype)
    talk = np.zeros((H, H))
    talk[0, 3], talk[1, 1], talk[2, 0], talk[3, 2] = 1.0, 1.0, -0.5, 2.0
    pb = np.array([-1.0, 0.5, -2.0, 0.0])
    kp, vp, pages = _paged(k, v, dtype, 4, [2, 0, 3, 1])
    got = attend(kernel, q, kp, vp, pages, 0, H, G, kd, vd, 0.25, 0.0, pb, talk, None)
    ref = plain_rows(q, k, v, 0, 0.25, 0.0, pb, talk, None)
    assert np.abs(got - ref).max() <= _tol(kernel) * np.abs(ref).max()
    # by hand for head 0: head 3's weights (its own query, kv head 1's keys) on kv head 0's values
    s = np.einsum("id,jd->ij", q[:, 3], k[:, 1]) * 0.25
    w = np.tril(1 / (1 + np.exp(-(s + pb[3]))))
    assert np.abs(got[:, 0] - w @ v[:, 0]).max() <= _tol(kernel) * np.abs(ref).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(6, 2, 20, 12, 8), (4, 2, 64, 64, 32), (2, 1, 32, 8, 0)])
def test_values_are_blended_before_they_are_stored(dtype, sizes):
    """qkv_prep with another layer's values: the pages hold (1 - lambda) v + lambda v_first, keys are rotated as without."""
    from rusty_llama_b200.kernels import ops

    H, G, kd, vd, rot = sizes
    rng = np.random.default_rng(kd)
    T = 70
    cols = (H + G) * kd + G * vd
    for lam in (0.0, 0.375, 1.0):
        rows = _dev(rng.standard_normal((T, cols + 16)), dtype)
        first = _dev(rng.standard_normal((T, G * vd + 8)), dtype)[:, : G * vd]
        kp = torch.zeros((3, G, 64, kd), dtype=dtype, device="cuda")
        vp = torch.zeros((3, G, 64, vd), dtype=dtype, device="cuda")
        freq = _dev(0.3 ** np.arange(rot // 2), torch.float32) if rot else None
        before = rows.clone()
        ops.qkv_prep(rows, None, _i32(np.arange(T)), _i32(np.zeros(T)), _i32([[2, 0, 1]]), kp, vp, freq, 1.0, H, G, kd, vd, rot, True,
                     v_src=first, v_lambda=_dev([lam], torch.float32))
        v = before[:, (H + G) * kd : cols].to(F64).view(T, G, vd)
        want = (1 - lam) * v + lam * first.to(F64).view(T, G, vd)
        got = torch.cat([vp[2], vp[0]], dim=1)[:, :T].transpose(0, 1).to(F64)
        tol = 1e-6 if dtype == torch.float32 else 8e-3
        assert float((got - want).abs().max()) <= tol * float(want.abs().max())
        if lam in (0.0, 1.0):  # nothing of the other side leaks in
            other = first.to(F64).view(T, G, vd) if lam == 0.0 else v
            assert float((got - other).abs().max()) > 0.5
        plain = torch.zeros_like(vp)
        ops.qkv_prep(before.clone(), None, _i32(np.arange(T)), _i32(np.zeros(T)), _i32([[2, 0, 1]]), torch.zeros_like(kp), plain, freq, 1.0, H, G, kd, vd,
                     rot, True)
        if lam == 0.0:
            assert torch.equal(plain, vp)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_short_convolution_through_its_record(dtype, taps):
    """Two sequences in one step, cut into portions shorter and longer than the record; slots in another order than the batch."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(taps)
    C, lens = 37, (23, 9)
    w = _rounded(rng.standard_normal((C, taps)), torch.bfloat16)
    xs = [_rounded(rng.standard_normal((n, C)), dtype) for n in lens]
    want = [pn.silu(pn.short_convolution(torch.as_tensor(x), torch.as_tensor(w))).numpy() for x in xs]
    state = torch.zeros((4, max(taps - 1, 1), C), dtype=torch.float32, device="cuda")[:, : taps - 1] if taps > 1 else None
    if state is not None:
        state = torch.zeros((4, taps - 1, C), dtype=torch.float32, device="cuda")
    slots = _i32([3, 1])
    got = [[], []]
    at = [0, 0]
    for portion in ((1, 2), (2, 1), (5, 3), (1, 1), (14, 2)):
        parts = [xs[i][at[i] : at[i] + portion[i]] for i in range(2)]
        x = torch.zeros((sum(portion), C + 5), dtype=dtype, device="cuda")
        x[:, :C] = _dev(np.concatenate(parts), dtype)
        y = ops.short_conv(x[:, :C], _dev(w, torch.float32).t().contiguous(), state, slots, _i32([0, portion[0], sum(portion)]), _i32([0] * portion[0] + [1] * portion[1]))
        got[0].append(y[: portion[0]].to(F64).cpu().numpy())
        got[1].append(y[portion[0] :].to(F64).cpu().numpy())
        at = [at[i] + portion[i] for i in range(2)]
    assert at == list(lens)
    for i in range(2):
        g = np.concatenate(got[i])
        tol = 2e-6 if dtype == torch.float32 else 8e-3
        assert np.abs(g - want[i]).max() <= tol * max(1.0, np.abs(want[i]).max())
    if state is not None:  # the records hold the last inputs, oldest first, and the other slots were left alone
        assert np.allclose(state[3].cpu().numpy(), xs[0][-(taps - 1):]) and np.allclose(state[1].cpu().numpy(), xs[1][-(taps - 1):])
        assert float(state[0].abs().sum()) == 0.0 and float(state[2].abs().sum()) == 0.0


def _delta_inputs(rng, T, G, H, dim, vdim, dtype):
    qk = _rounded(rng.standard_normal((T, 2 * G * dim)), dtype)
    ba = _rounded(rng.standard_normal((T, 2 * H)), dtype)
    v = _rounded(rng.standard_normal((T, H * vdim)), dtype)
    a_log, dt = rng.standard_normal(H) - 1.0, rng.standard_normal(H)
    return qk, ba, v, a_log.astype(np.float32).astype(np.float64), dt.astype(np.float32).astype(np.float64)


def _plain_delta(qk, ba, v, a_log, dt, G, H, dim, vdim):
    T = qk.shape[0]
    q = pn.unit(torch.as_tensor(qk[:, : G * dim]).view(T, G, dim)) * dim ** -0.5
    k = pn.unit(torch.as_tensor(qk[:, G * dim :]).view(T, G, dim))
    beta = pn.logistic(torch.as_tensor(ba[:, :H]))
    g = torch.exp(-torch.exp(torch.as_tensor(a_log)) * pn.softplus(torch.as_tensor(ba[:, H:]) + torch.as_tensor(dt)))
    rep = H // G
    return pn.delta_recurrence(q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1), torch.as_tensor(v).view(T, H, vdim), beta, g).reshape(T, H * vdim).numpy()


def _run_delta(qk, ba, v, a_log, dt, G, H, dim, vdim, dtype, cuts, state, slot):
    from rusty_llama_b200.kernels import ops

    out, at = [], 0
    for n in cuts:
        rows = torch.zeros((n, 2 * G * dim + 2 * H + H * vdim + 3), dtype=dtype, device="cuda")
        a, b = 2 * G * dim, 2 * G * dim + 2 * H
        rows[:, :a], rows[:, a:b], rows[:, b : b + H * vdim] = _dev(qk[at : at + n], dtype), _dev(ba[at : at + n], dtype), _dev(v[at : at + n], dtype)
        qn, kn, kq, beta, decay = ops.delta_prep(rows[:, :a], rows[:, a:b], _dev(a_log, torch.float32), _dev(dt, torch.float32), G, H, dim, 1e-6, dim ** -0.5)
        out.append(ops.delta_rule(qn, kn, kq, rows[:, b : b + H * vdim], beta, decay, state, _i32([slot]), _i32([0, n]), H, G, dim, vdim).cpu())
        at += n
    return torch.cat(out).to(F64).numpy()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(2, 4, 24, 20), (1, 1, 40, 8), (2, 2, 36, 36), (1, 2, 128, 64), (1, 1, 200, 70)])
def test_delta_rule_against_the_plain_recurrence(dtype, sizes):
    """Whole, and cut into portions down to one token: the same bits, within 32-bit rounding of the plain recurrence."""
    G, H, dim, vdim = sizes
    rng = np.random.default_rng(dim)
    T = 150
    qk, ba, v, a_log, dt = _delta_inputs(rng, T, G, H, dim, vdim, dtype)
    ref = _plain_delta(qk, ba, v, a_log, dt, G, H, dim, vdim)
    state = torch.zeros((3, H, dim, vdim), dtype=torch.float32, device="cuda")
    whole = _run_delta(qk, ba, v, a_log, dt, G, H, dim, vdim, dtype, [T], state, 1)
    assert np.abs(whole - ref).max() <= 3e-5 * np.abs(ref).max()
    assert float(state[0].abs().sum()) == 0.0 and float(state[2].abs().sum()) == 0.0 and float(state[1].abs().sum()) > 0.0
    cut = _run_delta(qk, ba, v, a_log, dt, G, H, dim, vdim, dtype, [1, 2, 7, 8, 9, 64, 1, 58], state, 2)
    assert np.array_equal(cut, whole)
    assert torch.equal(state[1], state[2])


def test_delta_rule_gives_back_the_last_value_under_a_key_after_hundreds_of_tokens():
    """beta almost 1 and a decay of almost 1: 8 keys at right angles are written in turn for 400 tokens; the read-out with key j's
    direction gives the value last written under it, not an earlier one and not a sum."""
    G = H = 1
    dim, vdim, T = 8, 5, 400
    rng = np.random.default_rng(0)
    qk = np.zeros((T, 2 * dim))
    for t in range(T):
        qk[t, dim + t % dim] = 3.0  # the key
        qk[t, (t + 3) % dim] = 2.0  # the query reads another key's place
    ba = np.zeros((T, 2))
    ba[:, 0], ba[:, 1] = 30.0, -30.0  # beta = 1; softplus(-30) = 1e-13: no decay
    v = rng.standard_normal((T, vdim))
    state = torch.zeros((1, H, dim, vdim), dtype=torch.float32, device="cuda")
    got = _run_delta(qk, ba, v, np.zeros(1), np.zeros(1), G, H, dim, vdim, torch.float32, [300, 1, 1, 98], state, 0)
    for t in range(dim, T):
        j = (t + 3) % dim
        last = max(s for s in range(t + 1) if s % dim == j)
        assert np.abs(got[t] - v[last] * dim ** -0.5).max() <= 1e-5, t


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_logistic_router_against_the_plain_choice(dtype):
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(1)
    for T, d, E, top, scale in ((50, 96, 5, 2, 2.5), (7, 68, 6, 3, 1.5), (33, 128, 8, 8, 1.0), (4, 40, 1, 1, 0.7)):
        x = _rounded(rng.standard_normal((T, d)), dtype)
        w = _rounded(2.0 * rng.standard_normal((E, d)) / math.sqrt(d), torch.bfloat16)
        corr = _rounded(0.3 * rng.standard_normal(E), torch.bfloat16)
        W = {"r.router": torch.as_tensor(w), "r.correction": torch.as_tensor(corr)}
        chosen, weights = pn.route(torch.as_tensor(x), W, "r.", {"top": top, "scale": scale})
        ids, got, _ = ops.moe_router(_dev(x, dtype), _dev(w, torch.float32), _dev(corr, torch.float32), E, top, True, logistic=True, renorm_eps=1e-20,
                                     weight_scale=scale)
        s = pn.logistic(torch.as_tensor(x) @ torch.as_tensor(w).T) + torch.as_tensor(corr)
        for t in range(T):
            order = torch.sort(s[t], descending=True).values
            if top < E and float(order[top - 1] - order[top]) < 1e-4:
                continue  # (a close call is not a test)
            mine = dict(zip(ids[t].tolist(), got[t].tolist()))
            want = dict(zip(chosen[t].tolist(), weights[t].tolist()))
            assert set(mine) == set(want)
            for e in want:
                assert mine[e] == pytest.approx(want[e], rel=2e-5, abs=1e-7)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gelu_gate_in_every_product_that_fuses_it(dtype):
    """The dense feed-forward's gate/up product with the tanh-form gelu, at row counts that take the streaming, the small and
    the tensor-core product (bfloat16) and the plain one (32-bit), and at sizes that only the plain bfloat16 product takes."""
    from rusty_llama_b200.parts import FEED_FORWARDS, Runtime
    from rusty_llama_b200.spec import PartSpec

    rng = np.random.default_rng(2)
    for d, ff in ((128, 256), (68, 70), (256, 320)):
        rt = Runtime.create("cuda", dtype)
        part = FEED_FORWARDS.build(PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": ff, "activation": "gelu_tanh",
                                                          "names": {"gate": "gate", "up": "up", "down": "down"}}, "f."), rt)
        w = {n: _rounded(2.0 * rng.standard_normal(shape) / math.sqrt(shape[1]), torch.bfloat16) for n, shape in (("f.gate", (ff, d)), ("f.up", (ff, d)), ("f.down", (d, ff)))}
        part.load({n: _dev(t, dtype) for n, t in w.items()})
        for T in (1, 5, 20, 150):
            x = _rounded(rng.standard_normal((T, d)), dtype)
            got = part.forward(_dev(x, dtype), None).float()
            if got.dim() == 3:
                got = got.sum(dim=0)
            ref = pn.dense_ff(torch.as_tensor(x), {n: torch.as_tensor(t) for n, t in w.items()}, "f.").numpy()
            tol = 2e-5 if dtype == torch.float32 else 1.5e-2
            assert np.abs(got.cpu().numpy() - ref).max() <= tol * np.abs(ref).max(), (d, ff, T)


def test_embedding_scale_is_applied_in_32_bit():
    from rusty_llama_b200.kernels import ops

    table = _dev(np.random.default_rng(4).standard_normal((11, 20)), torch.bfloat16)
    out = ops.embed_gather(_i32([3, 0, 10]), table, scale=3.0)
    assert torch.equal(out, table[[3, 0, 10]].float() * 3.0)
    assert torch.equal(ops.embed_gather(_i32([3]), table), table[[3]].float())
